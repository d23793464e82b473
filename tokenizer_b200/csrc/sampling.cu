// Choosing the next token from 32-bit logits on the device, one block per row.
//
// temperature == 0: argmax with a strict ">" so equal logits keep the lower id.
// Otherwise: weights exp((l - max) / T); the candidates are ordered by logit
// descending (equal logits by lower id); nucleus sampling keeps the shortest
// prefix of that order whose share of the total weight reaches top_p (always at
// least one, everything when top_p >= 1); the draw u in [0,1) is scaled by the
// kept weight and the candidate whose interval holds it is returned.  The order
// is never materialised: the cut and the drawn candidate are found by bisection
// over the logits' bit patterns, every weight sum being a fixed-order block
// reduction, so a row's result is a function of (logits, T, top_p, u) alone.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned ordered_key(float v) {
  unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct BestPair { float value; int index; };

__device__ __forceinline__ BestPair better(BestPair a, BestPair b) {
  // higher value wins; equal values keep the lower index; index < 0 is "none"
  if (b.index < 0) return a;
  if (a.index < 0) return b;
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ int block_argmax(const float* __restrict__ row, int vocab, BestPair* pair_scratch) {
  BestPair best{-INFINITY, -1};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best.value) { best.value = v; best.index = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    BestPair other{__shfl_xor_sync(0xffffffffu, best.value, o),
                   __shfl_xor_sync(0xffffffffu, best.index, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) pair_scratch[warp] = best;
  __syncthreads();
  if (warp == 0) {
    BestPair w = lane < (int)(blockDim.x >> 5) ? pair_scratch[lane] : BestPair{-INFINITY, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      BestPair other{__shfl_xor_sync(0xffffffffu, w.value, o),
                     __shfl_xor_sync(0xffffffffu, w.index, o)};
      w = better(w, other);
    }
    if (lane == 0) pair_scratch[32] = w;
  }
  __syncthreads();
  const int result = pair_scratch[32].index;
  return result < 0 ? 0 : result;  // every logit NaN or -inf: id 0, as a scan from -inf finds nothing
}

// weight of the candidates whose key is >= `key_min`, and how many there are
__device__ __forceinline__ float mass_at_or_above(const float* __restrict__ row, int vocab,
                                                  float max_logit, float inv_t, unsigned key_min,
                                                  float* scratch) {
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (ordered_key(v) >= key_min) s += expf((v - max_logit) * inv_t);
  }
  return block_sum(s, scratch);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ BestPair pair_scratch[33];
  __shared__ int count_scratch[SAMPLE_THREADS];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const float temp = temperature ? temperature[r] : 0.f;
  const int greedy = block_argmax(row, vocab, pair_scratch);
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[r] = greedy;
    return;
  }
  const float max_logit = row[greedy];
  // weights are exp((l - max) / T), the division as the reference writes it
  const float inv_t = 1.0f / temp;
  const float p_keep = top_p ? top_p[r] : 1.f;
  const float total = mass_at_or_above(row, vocab, max_logit, inv_t, 0u, scratch);
  if (!(total > 0.f) || !isfinite(total)) {
    if (threadIdx.x == 0) out[r] = greedy;
    return;
  }

  // --- the nucleus: largest key `cut` with mass(key >= cut) >= top_p * total ---
  unsigned cut = 0u;          // keep everything
  float kept = total;
  if (p_keep < 1.f) {
    const float need = p_keep * total;
    unsigned lo = 0u, hi = ordered_key(max_logit);  // invariant: mass(>= lo) >= need
    // mass(>= hi) >= need may hold as well; find the largest such key
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1u) / 2u;
      const float mass = mass_at_or_above(row, vocab, max_logit, inv_t, mid, scratch);
      if (mass >= need) lo = mid; else hi = mid - 1u;
    }
    cut = lo;
    kept = mass_at_or_above(row, vocab, max_logit, inv_t, cut, scratch);
    // candidates exactly at the cut are equal logits: the walk takes them in id
    // order and stops as soon as the share is reached, so trailing ones drop out
    if (cut != 0xffffffffu) {
      const float above = mass_at_or_above(row, vocab, max_logit, inv_t, cut + 1u, scratch);
      const float each = expf((__uint_as_float((cut & 0x80000000u) ? (cut & 0x7fffffffu) : ~cut) -
                               max_logit) * inv_t);
      if (each > 0.f) {
        float n_ties = ceilf((need - above) / each);
        if (n_ties < 1.f) n_ties = 1.f;
        const float with_ties = above + n_ties * each;
        if (with_ties < kept) kept = with_ties;
      }
    }
  }

  // --- the draw: candidate whose interval [before, before + w) holds u * kept ---
  const float u = uniform ? uniform[r] : 0.f;
  const float threshold = u * kept;
  // largest key `sel` (>= cut) with mass(key >= sel) > threshold
  unsigned lo = cut, hi = ordered_key(max_logit);
  while (lo < hi) {
    const unsigned mid = lo + (hi - lo + 1u) / 2u;
    const float mass = mass_at_or_above(row, vocab, max_logit, inv_t, mid, scratch);
    if (mass > threshold) lo = mid; else hi = mid - 1u;
  }
  const unsigned sel = lo;
  const float sel_value = __uint_as_float((sel & 0x80000000u) ? (sel & 0x7fffffffu) : ~sel);
  const float each = expf((sel_value - max_logit) * inv_t);
  float above = 0.f;
  if (sel != 0xffffffffu) above = mass_at_or_above(row, vocab, max_logit, inv_t, sel + 1u, scratch);
  int skip = 0;  // equal logits before the drawn one, in id order
  if (each > 0.f && threshold > above) skip = (int)floorf((threshold - above) / each);

  // the (skip)-th id whose key equals `sel`, ids ascending; the last one if fewer
  const int per = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int begin = min(vocab, (int)threadIdx.x * per), end = min(vocab, begin + per);
  int mine = 0;
  for (int i = begin; i < end; ++i) mine += ordered_key(row[i]) == sel;
  count_scratch[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    int total_ties = 0;
    for (int i = 0; i < SAMPLE_THREADS; ++i) total_ties += count_scratch[i];
    int want = skip < total_ties ? skip : total_ties - 1;
    int chosen = greedy;
    if (total_ties > 0) {
      int owner = 0;
      while (want >= count_scratch[owner]) { want -= count_scratch[owner]; ++owner; }
      const int b = min(vocab, owner * per), e = min(vocab, b + per);
      for (int i = b; i < e; ++i) {
        if (ordered_key(row[i]) == sel) {
          if (want == 0) { chosen = i; break; }
          --want;
        }
      }
    }
    out[r] = chosen;
  }
}

// ----------------------------------------------------------------------------
// Greedy only: the vocabulary of a row is cut over ARGMAX_SPLITS blocks; each
// leaves its best (value, id) in scratch and the block that finishes last for the
// row picks among them, in index order (higher value, then lower id).
// scratch: [n_rows][ARGMAX_SPLITS] pairs; counters: [n_rows] ints, zero between
// launches.
// ----------------------------------------------------------------------------
#define ARGMAX_SPLITS 32
#define ARGMAX_THREADS 256

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out,
              BestPair* __restrict__ scratch, int* __restrict__ counters) {
  __shared__ BestPair pair_scratch[33];
  __shared__ int is_last;
  pdl_wait();
  pdl_launch();
  const int split = blockIdx.x, r = blockIdx.y;
  const float* row = logits + (size_t)r * vocab;
  const int per = (vocab + ARGMAX_SPLITS - 1) / ARGMAX_SPLITS;
  const int begin = min(vocab, split * per), end = min(vocab, begin + per);
  BestPair best{-INFINITY, -1};
  // four loads in flight per thread
  for (int i0 = begin + threadIdx.x; i0 < end; i0 += 4 * ARGMAX_THREADS) {
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = i0 + e * ARGMAX_THREADS;
      v[e] = i < end ? row[i] : -INFINITY;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (v[e] > best.value) { best.value = v[e]; best.index = i0 + e * ARGMAX_THREADS; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    BestPair other{__shfl_xor_sync(0xffffffffu, best.value, o),
                   __shfl_xor_sync(0xffffffffu, best.index, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) pair_scratch[warp] = best;
  __syncthreads();
  if (warp == 0) {
    BestPair w = lane < ARGMAX_THREADS / 32 ? pair_scratch[lane] : BestPair{-INFINITY, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      BestPair other{__shfl_xor_sync(0xffffffffu, w.value, o),
                     __shfl_xor_sync(0xffffffffu, w.index, o)};
      w = better(w, other);
    }
    if (lane == 0) {
      scratch[(size_t)r * ARGMAX_SPLITS + split] = w;
      __threadfence();
      const int done = atomicAdd(&counters[r], 1);
      is_last = done == ARGMAX_SPLITS - 1;
      if (is_last) counters[r] = 0;
    }
  }
  __syncthreads();
  if (!is_last || warp != 0) return;
  __threadfence();
  const BestPair* mine = scratch + (size_t)r * ARGMAX_SPLITS;
  BestPair w{__ldcg(&mine[lane].value), __ldcg(&mine[lane].index)};   // ARGMAX_SPLITS == 32 lanes
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    BestPair other{__shfl_xor_sync(0xffffffffu, w.value, o),
                   __shfl_xor_sync(0xffffffffu, w.index, o)};
    w = better(w, other);
  }
  if (lane == 0) out[r] = w.index < 0 ? 0 : w.index;
}

TOKB200_API long long tokb200_argmax_scratch_bytes(int n_rows) {
  return (long long)n_rows * ARGMAX_SPLITS * sizeof(BestPair);
}

TOKB200_API int tokb200_argmax(const float* logits, int n_rows, int vocab, int* out, void* scratch,
                               int* counters, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (vocab <= 0 || n_rows > 65535) return TOKB200_BAD_SIZE;
  return launch_dependent(argmax_kernel, dim3(ARGMAX_SPLITS, n_rows), dim3(ARGMAX_THREADS), 0,
                          stream, logits, vocab, out, (BestPair*)scratch, counters);
}

TOKB200_API int tokb200_sample(const float* logits, int n_rows, int vocab,
                               const float* temperature, const float* top_p,
                               const float* uniform, int* out, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (vocab <= 0) return TOKB200_BAD_SIZE;
  return launch_dependent(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits,
                          vocab, temperature, top_p, uniform, out);
}

// ----------------------------------------------------------------------------
// The greedy choice without any allocation: the scratch of argmax_kernel lives
// in this library (see no_alloc.h for who needs that and for the rules).
// ----------------------------------------------------------------------------
#include "no_alloc.h"

#define ARGMAX_NO_ALLOC_MAX_ROWS 256

struct ArgmaxStaticScratch {
  BestPair pairs[ARGMAX_NO_ALLOC_MAX_ROWS * ARGMAX_SPLITS];
  int counters[ARGMAX_NO_ALLOC_MAX_ROWS];
};

// In host code this name is only a handle for cudaGetSymbolAddress, never an
// address a kernel may be given.
static __device__ __align__(256) unsigned char argmax_static_scratch[sizeof(ArgmaxStaticScratch)];

TOKB200_API int tokb200_argmax_no_alloc_max_rows(void) { return ARGMAX_NO_ALLOC_MAX_ROWS; }

TOKB200_API const char* tokb200_no_alloc_error(int status) {
  switch (status) {
    case TOKB200_OK: return "ok";
    case TOKB200_BAD_SIZE:
      return "refused: rows beyond the built-in scratch (256), an empty vocabulary, or a null pointer";
    case TOKB200_BAD_ALIGNMENT: return "refused: logits and out must be 4-byte aligned";
    default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
  }
}

TOKB200_API int tokb200_argmax_no_alloc(const float* logits, int n_rows, int vocab, int* out,
                                        cudaStream_t stream) {
  if (n_rows == 0) return TOKB200_OK;
  if (n_rows < 0 || n_rows > ARGMAX_NO_ALLOC_MAX_ROWS || vocab <= 0 || !logits || !out)
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)logits | (uintptr_t)out) & 3) return TOKB200_BAD_ALIGNMENT;
  // set-up, once per device: the device address of the array, asked for with
  // that device current
  static void* scratch_of_device[64] = {};
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return (int)err;
  if (device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!scratch_of_device[device]) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, argmax_static_scratch);
    if (err != cudaSuccess) return (int)err;
    scratch_of_device[device] = address;
  }
  ArgmaxStaticScratch* scratch = static_cast<ArgmaxStaticScratch*>(scratch_of_device[device]);
  // the counters must start at zero whatever the last call left behind
  err = cudaMemsetAsync(scratch->counters, 0, sizeof(int) * n_rows, stream);
  if (err != cudaSuccess) return (int)err;
  return launch_dependent(argmax_kernel, dim3(ARGMAX_SPLITS, n_rows), dim3(ARGMAX_THREADS), 0,
                          stream, logits, vocab, out, scratch->pairs, scratch->counters);
}
