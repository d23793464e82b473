// Attention for rows that read far more keys than they bring: decoding.
//
// One block works on (a row, one kv head, one split of that row's keys) and
// serves all query heads of the kv head at once, so keys and values are read
// once per group.  A row's visible keys lo..pos are cut into n_splits pieces of
// `chunk` keys; chunk is 64 * 2^k, the smallest that needs at most MAX_SPLITS
// pieces, so the cut is a function of the row's own position and window and does
// not change with the batch around it.  Each block runs an online softmax over
// its piece in tiles of 64 keys and leaves (max, sum, weighted values) in
// scratch memory; the block that finishes last for a (row, kv head) merges the
// pieces in index order and writes the output.  Scores, maxima, sums and the
// weighted values are 32-bit.
//
// HEAD_DIM is a compile-time size (a multiple of 16, at most 256), given with
// -DHEAD_DIM=...; the library is built per head size at first use.
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
#define DEC_THREADS 128
#define DEC_TILE 64            // keys per tile: two threads share a key in the score phase
#define DEC_MAX_GROUP 8        // query heads per kv head served by one pass
#define DEC_MAX_SPLITS 32

static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size");

constexpr int kPairs = HEAD_DIM / 2;                 // value lanes are handled in pairs
constexpr int kKeyGroups = DEC_THREADS / kPairs;     // key groups in the value phase (>= 1)
constexpr int kHalf = HEAD_DIM / 2;                  // lanes per thread in the score phase

struct __align__(16) Bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ int split_chunk(int n_keys) {
  int chunk = DEC_TILE;
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
  const int tid = threadIdx.x;

  __shared__ float q_s[DEC_MAX_GROUP][HEAD_DIM];
  __shared__ float p_s[DEC_MAX_GROUP][DEC_TILE];
  __shared__ int slot_s[DEC_TILE];
  __shared__ float red_s[kKeyGroups][DEC_MAX_GROUP][HEAD_DIM];
  __shared__ float m_s[DEC_MAX_GROUP], l_s[DEC_MAX_GROUP], corr_s[DEC_MAX_GROUP];
  __shared__ int is_last;

  for (int i = tid; i < group * HEAD_DIM; i += DEC_THREADS) {
    const int h = i / HEAD_DIM, c = i % HEAD_DIM;
    q_s[h][c] = __bfloat162float(q[((size_t)t * nh + kvh * group + h) * HEAD_DIM + c]);
  }
  if (tid < DEC_MAX_GROUP) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
  float acc[DEC_MAX_GROUP][2];
#pragma unroll
  for (int h = 0; h < DEC_MAX_GROUP; ++h) acc[h][0] = acc[h][1] = 0.f;
  __syncthreads();

  const int key_in_tile = tid >> 1, half = tid & 1;      // score phase: 2 threads per key
  const int pair = tid % kPairs, kgroup = tid / kPairs;  // value phase

  for (int k0 = first; k0 <= last; k0 += DEC_TILE) {
    const int n = min(DEC_TILE, last - k0 + 1);
    // ---- scores of this tile: every thread takes half a key ----
    float s[DEC_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < DEC_MAX_GROUP; ++h) s[h] = 0.f;
    if (key_in_tile < n) {
      const int key = k0 + key_in_tile;
      const int slot = table[key / page] * page + key % page;
      if (half == 0) slot_s[key_in_tile] = slot;
      const Bf16x8* row = reinterpret_cast<const Bf16x8*>(
          k_pool + ((size_t)slot * nkv + kvh) * HEAD_DIM + half * kHalf);
#pragma unroll
      for (int c = 0; c < kHalf / 8; ++c) {
        const Bf16x8 kv8 = row[c];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 kf = __bfloat1622float2(kv8.v[e]);
          const int lane = half * kHalf + c * 8 + e * 2;
#pragma unroll
          for (int h = 0; h < DEC_MAX_GROUP; ++h)
            if (h < group) s[h] += q_s[h][lane] * kf.x + q_s[h][lane + 1] * kf.y;
        }
      }
    }
#pragma unroll
    for (int h = 0; h < DEC_MAX_GROUP; ++h) {
      s[h] += __shfl_xor_sync(0xffffffffu, s[h], 1);
      if (half == 0 && h < group) p_s[h][key_in_tile] = key_in_tile < n ? s[h] * scale : -INFINITY;
    }
    __syncthreads();
    // ---- online softmax: warp w looks after heads w, w + 4 ----
    for (int h = tid >> 5; h < group; h += DEC_THREADS / 32) {
      const int lane = tid & 31;
      const float s0 = p_s[h][lane], s1 = p_s[h][lane + 32];
      const float m_old = m_s[h];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
      const float e0 = expf(s0 - m_new), e1 = expf(s1 - m_new);   // exp(-inf) = 0 for unused keys
      p_s[h][lane] = e0;
      p_s[h][lane + 32] = e1;
      const float sum = warp_sum(e0 + e1);
      if (lane == 0) {
        const float corr = expf(m_old - m_new);                     // 0 on the first tile
        corr_s[h] = corr;
        l_s[h] = l_s[h] * corr + sum;
        m_s[h] = m_new;
      }
    }
    __syncthreads();
    // ---- weighted values: thread (pair, key group) takes keys kgroup, kgroup + G, ... ----
    if (kgroup < kKeyGroups) {
#pragma unroll
      for (int h = 0; h < DEC_MAX_GROUP; ++h) {
        if (h < group) { acc[h][0] *= corr_s[h]; acc[h][1] *= corr_s[h]; }
      }
      for (int j = kgroup; j < n; j += kKeyGroups) {
        const float2 vf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(
            v_pool + ((size_t)slot_s[j] * nkv + kvh) * HEAD_DIM + pair * 2));
#pragma unroll
        for (int h = 0; h < DEC_MAX_GROUP; ++h) {
          if (h < group) {
            const float w = p_s[h][j];
            acc[h][0] += w * vf.x;
            acc[h][1] += w * vf.y;
          }
        }
      }
    }
    __syncthreads();   // p_s, slot_s and corr_s are rewritten by the next tile
  }

  // ---- sum the key groups ----
  if (kgroup < kKeyGroups) {
#pragma unroll
    for (int h = 0; h < DEC_MAX_GROUP; ++h) {
      if (h < group) {
        red_s[kgroup][h][pair * 2] = acc[h][0];
        red_s[kgroup][h][pair * 2 + 1] = acc[h][1];
      }
    }
  }
  __syncthreads();

  // scratch layout per (row, head): [split][HEAD_DIM + 2] = weighted values, max, sum
  const size_t per_head = (size_t)DEC_MAX_SPLITS * (HEAD_DIM + 2);
  float* base = scratch + ((size_t)t * nh + kvh * group) * per_head;
  if (n_splits == 1) {
    for (int i = tid; i < group * HEAD_DIM; i += DEC_THREADS) {
      const int h = i / HEAD_DIM, c = i % HEAD_DIM;
      float v = 0.f;
#pragma unroll
      for (int g = 0; g < kKeyGroups; ++g) v += red_s[g][h][c];
      out[((size_t)t * nh + kvh * group + h) * HEAD_DIM + c] = __float2bfloat16_rn(v / l_s[h]);
    }
    return;
  }
  for (int i = tid; i < group * HEAD_DIM; i += DEC_THREADS) {
    const int h = i / HEAD_DIM, c = i % HEAD_DIM;
    float v = 0.f;
#pragma unroll
    for (int g = 0; g < kKeyGroups; ++g) v += red_s[g][h][c];
    base[h * per_head + (size_t)split * (HEAD_DIM + 2) + c] = v;
  }
  if (tid < group) {
    base[tid * per_head + (size_t)split * (HEAD_DIM + 2) + HEAD_DIM] = m_s[tid];
    base[tid * per_head + (size_t)split * (HEAD_DIM + 2) + HEAD_DIM + 1] = l_s[tid];
  }
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
    float m = -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) m = fmaxf(m, __ldcg(&piece[(size_t)sp * (HEAD_DIM + 2) + HEAD_DIM]));
    float num = 0.f, den = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) {
      const float w = expf(__ldcg(&piece[(size_t)sp * (HEAD_DIM + 2) + HEAD_DIM]) - m);
      num += w * __ldcg(&piece[(size_t)sp * (HEAD_DIM + 2) + c]);
      den += w * __ldcg(&piece[(size_t)sp * (HEAD_DIM + 2) + HEAD_DIM + 1]);
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
  decode_attention_kernel<<<grid, DEC_THREADS, 0, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
      (__nv_bfloat16*)out, block_table, table_stride, row_req, pos, nh, nkv, page, window, scale,
      scratch, counters);
  return tokb200_launch_status();
}
