// Attention for rows that read far more keys than they bring: decoding.
//
// One block works on (a row, one kv head, one split of that row's keys) and
// serves all query heads of the kv head at once, so keys and values are read
// once per group.  A row's visible keys lo..pos are cut into n_splits pieces of
// `chunk` keys; chunk is 128 * 2^k, the smallest that needs at most MAX_SPLITS
// pieces, so the cut is a function of the row's own position and window and does
// not change with the batch around it.  Inside a block every warp walks its own
// keys, 32 at a time (a lane per key for the scores, a lane per pair of value
// lanes for the weighted sum), with its own running maximum and sum and without
// block-wide barriers; the warps are merged once at the end.  A step is bound by
// latency, not by arithmetic, so loads are issued in batches before their first
// use.  Pieces of several blocks meet in scratch memory; the block that finishes
// last for a (row, kv head) merges them in index order and writes the output.
// Scores, maxima, sums and the weighted values are 32-bit.
//
// HEAD_DIM is a compile-time size (a multiple of 16, at most 256), given with
// -DHEAD_DIM=...; the library is built per head size at first use.
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
#define DEC_WARPS 4
#define DEC_THREADS (DEC_WARPS * 32)
#define DEC_MAX_GROUP 8        // query heads per kv head served by one pass
#define DEC_MAX_SPLITS 32
#define DEC_BLOCK_KEYS (DEC_WARPS * 32)

static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size");

// value lanes owned by one lane of a warp in the weighted sum: the smallest even
// count that divides the head size and leaves at most 32 owners
constexpr int own_lanes(int d) {
  for (int n = 2; n <= 8; n += 2)
    if (d % n == 0 && d / n <= 32) return n;
  return 8;
}
constexpr int kOwn = own_lanes(HEAD_DIM);
constexpr int kOwners = HEAD_DIM / kOwn;             // lanes that own value lanes (<= 32)
static_assert(kOwn % 2 == 0 && HEAD_DIM % kOwn == 0 && kOwners <= 32, "value lanes per lane");

struct __align__(16) Bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ int split_chunk(int n_keys) {
  int chunk = DEC_BLOCK_KEYS;
  while ((n_keys + chunk - 1) / chunk > DEC_MAX_SPLITS) chunk <<= 1;
  return chunk;
}

__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ row_req, const int* __restrict__ pos, int nh,
                        int nkv, int page, int window, float scale,
                        float* __restrict__ scratch, int* __restrict__ counters) {
  pdl_wait();
  pdl_launch();
  const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int r = row_req[t];
  if (r < 0) return;
  const int p = pos[t];
  const int lo = (window >= 0 && p - window > 0) ? p - window : 0;
  const int n_keys = p - lo + 1;
  const int chunk = split_chunk(n_keys);
  const int n_splits = (n_keys + chunk - 1) / chunk;
  if (split >= n_splits) return;
  const int group = nh / nkv;                       // <= DEC_MAX_GROUP, checked by the launcher
  const int first = lo + split * chunk;
  const int last = min(p, first + chunk - 1);
  const int* table = block_table + (size_t)r * table_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  __shared__ float q_s[DEC_MAX_GROUP][HEAD_DIM];
  __shared__ float acc_s[DEC_WARPS][DEC_MAX_GROUP][HEAD_DIM];
  __shared__ float m_s[DEC_WARPS][DEC_MAX_GROUP], l_s[DEC_WARPS][DEC_MAX_GROUP];
  __shared__ int is_last;

  for (int i = tid; i < group * HEAD_DIM; i += DEC_THREADS) {
    const int h = i / HEAD_DIM, c = i % HEAD_DIM;
    q_s[h][c] = __bfloat162float(q[((size_t)t * nh + kvh * group + h) * HEAD_DIM + c]);
  }
  __syncthreads();

  float m_run[DEC_MAX_GROUP], l_run[DEC_MAX_GROUP], acc[DEC_MAX_GROUP][kOwn];
#pragma unroll
  for (int h = 0; h < DEC_MAX_GROUP; ++h) {
    m_run[h] = -INFINITY;
    l_run[h] = 0.f;
#pragma unroll
    for (int e = 0; e < kOwn; ++e) acc[h][e] = 0.f;
  }

  for (int k0 = first + warp * 32; k0 <= last; k0 += DEC_BLOCK_KEYS) {
    // ---- scores: a lane per key ----
    const int key = k0 + lane;
    const bool live = key <= last;
    const int key_ok = live ? key : k0;                 // idle lanes read the first key again
    const int slot = table[key_ok / page] * page + key_ok % page;
    const Bf16x8* row = reinterpret_cast<const Bf16x8*>(k_pool + ((size_t)slot * nkv + kvh) * HEAD_DIM);
    Bf16x8 kreg[HEAD_DIM / 8];
#pragma unroll
    for (int c = 0; c < HEAD_DIM / 8; ++c) kreg[c] = row[c];
    float s[DEC_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < DEC_MAX_GROUP; ++h) s[h] = 0.f;
#pragma unroll
    for (int c = 0; c < HEAD_DIM / 8; ++c) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 kf = __bfloat1622float2(kreg[c].v[e]);
#pragma unroll
        for (int h = 0; h < DEC_MAX_GROUP; ++h)
          if (h < group) s[h] += q_s[h][c * 8 + e * 2] * kf.x + q_s[h][c * 8 + e * 2 + 1] * kf.y;
      }
    }
    // ---- running softmax of this warp ----
    float corr[DEC_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < DEC_MAX_GROUP; ++h) {
      if (h < group) {
        const float sh = live ? s[h] * scale : -INFINITY;
        const float m_new = fmaxf(m_run[h], warp_max(sh));      // finite: lane 0's key is live
        const float e = expf(sh - m_new);                        // exp(-inf) = 0 for idle lanes
        corr[h] = expf(m_run[h] - m_new);                        // 0 on the first pass
        l_run[h] = l_run[h] * corr[h] + warp_sum(e);
        m_run[h] = m_new;
        s[h] = e;
      }
    }
    // ---- weighted values: a lane per kOwn value lanes, keys one after another ----
#pragma unroll
    for (int h = 0; h < DEC_MAX_GROUP; ++h) {
      if (h < group) {
#pragma unroll
        for (int e = 0; e < kOwn; ++e) acc[h][e] *= corr[h];
      }
    }
    const int n = min(32, last - k0 + 1);
    const int own = (lane < kOwners ? lane : 0) * kOwn;
#pragma unroll 8
    for (int j = 0; j < 32; ++j) {
      const int slot_j = __shfl_sync(0xffffffffu, slot, j);      // idle keys carry weight 0
      float vals[kOwn];
      const __nv_bfloat16* vrow = v_pool + ((size_t)slot_j * nkv + kvh) * HEAD_DIM + own;
#pragma unroll
      for (int e = 0; e < kOwn; e += 2) {
        const float2 vf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vrow + e));
        vals[e] = vf.x;
        vals[e + 1] = vf.y;
      }
#pragma unroll
      for (int h = 0; h < DEC_MAX_GROUP; ++h) {
        if (h < group) {
          const float w = __shfl_sync(0xffffffffu, s[h], j);
#pragma unroll
          for (int e = 0; e < kOwn; ++e) acc[h][e] += w * vals[e];
        }
      }
      if (j + 1 >= n && ((j + 1) & 7) == 0) break;                // whole batches of 8 keys only
    }
  }

  // ---- merge the warps of the block ----
#pragma unroll
  for (int h = 0; h < DEC_MAX_GROUP; ++h) {
    if (h < group) {
      if (lane < kOwners) {
#pragma unroll
        for (int e = 0; e < kOwn; ++e) acc_s[warp][h][lane * kOwn + e] = acc[h][e];
      }
      if (lane == 0) { m_s[warp][h] = m_run[h]; l_s[warp][h] = l_run[h]; }
    }
  }
  __syncthreads();

  // scratch layout per (row, head): [split][HEAD_DIM + 2] = weighted values, max, sum
  const size_t per_head = (size_t)DEC_MAX_SPLITS * (HEAD_DIM + 2);
  float* base = scratch + ((size_t)t * nh + kvh * group) * per_head;
  for (int i = tid; i < group * HEAD_DIM; i += DEC_THREADS) {
    const int h = i / HEAD_DIM, c = i % HEAD_DIM;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, m_s[w][h]);   // a warp without keys has -inf
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float f = expf(m_s[w][h] - m);
      num += f * acc_s[w][h][c];
      den += f * l_s[w][h];
    }
    if (n_splits == 1) {
      out[((size_t)t * nh + kvh * group + h) * HEAD_DIM + c] = __float2bfloat16_rn(num / den);
    } else {
      float* piece = base + h * per_head + (size_t)split * (HEAD_DIM + 2);
      piece[c] = num;
      if (c == 0) { piece[HEAD_DIM] = m; piece[HEAD_DIM + 1] = den; }
    }
  }
  if (n_splits == 1) return;
  // ---- the last block to finish merges the pieces, in index order ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int done = atomicAdd(&counters[t * nkv + kvh], 1);
    is_last = done == n_splits - 1;
    if (is_last) counters[t * nkv + kvh] = 0;   // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int i = tid; i < group * HEAD_DIM; i += DEC_THREADS) {
    const int h = i / HEAD_DIM, c = i % HEAD_DIM;
    const float* piece = base + h * per_head;
    float ms[DEC_MAX_SPLITS], ls[DEC_MAX_SPLITS], vs[DEC_MAX_SPLITS];
#pragma unroll
    for (int sp = 0; sp < DEC_MAX_SPLITS; ++sp) {
      const bool on = sp < n_splits;
      ms[sp] = on ? __ldcg(&piece[(size_t)sp * (HEAD_DIM + 2) + HEAD_DIM]) : -INFINITY;
      ls[sp] = on ? __ldcg(&piece[(size_t)sp * (HEAD_DIM + 2) + HEAD_DIM + 1]) : 0.f;
      vs[sp] = on ? __ldcg(&piece[(size_t)sp * (HEAD_DIM + 2) + c]) : 0.f;
    }
    float m = -INFINITY;
#pragma unroll
    for (int sp = 0; sp < DEC_MAX_SPLITS; ++sp) m = fmaxf(m, ms[sp]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int sp = 0; sp < DEC_MAX_SPLITS; ++sp) {
      const float f = expf(ms[sp] - m);
      num += f * vs[sp];
      den += f * ls[sp];
    }
    out[((size_t)t * nh + kvh * group + h) * HEAD_DIM + c] = __float2bfloat16_rn(num / den);
  }
}

// floats of scratch and ints of counters a launch over n_rows needs
TOKB200_API long long tokb200_decode_attention_scratch_floats(int n_rows, int nh) {
  return (long long)n_rows * nh * DEC_MAX_SPLITS * (HEAD_DIM + 2);
}

TOKB200_API int tokb200_decode_attention_head_dim() { return HEAD_DIM; }

// `counters` holds n_rows * nkv ints, zero before the first launch; every launch
// leaves them zero again.
TOKB200_API int tokb200_decode_attention(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* block_table,
    int table_stride, const int* row_req, const int* pos, int n_rows, int nh, int nkv, int d,
    int page, int window, float scale, float* scratch, int* counters, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (d != HEAD_DIM || nh <= 0 || nkv <= 0 || nh % nkv || nh / nkv > DEC_MAX_GROUP || page <= 0 ||
      nkv > 65535 || n_rows > 65535)
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15)
    return TOKB200_BAD_ALIGNMENT;
  dim3 grid(DEC_MAX_SPLITS, nkv, n_rows);
  return launch_dependent(decode_attention_kernel, grid, dim3(DEC_THREADS), 0, stream,
                          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
                          (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, block_table,
                          table_stride, row_req, pos, nh, nkv, page, window, scale, scratch,
                          counters);
}
