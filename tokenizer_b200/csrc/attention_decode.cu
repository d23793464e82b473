// Attention for rows that read far more keys than they bring: decoding.
//
// A decoding step is bound by latency, not by arithmetic or bytes: few rows, a few
// hundred keys each.  So the work is spread over as many short, independent warps
// as possible.  One block works on (a row, one kv head, one split of that row's
// keys); each of its warps takes ONE query head of the kv head's group, so the
// keys and values of the split are fetched from L2 once and met again in L1 by the
// other warps.  A warp walks its keys 32 at a time: a lane per key for the scores
// (q is read from shared memory, broadcast), a lane per few value lanes for the
// weighted sum, its own running maximum and sum, no block-wide barrier.
//
// A row's visible keys lo..pos are cut into n_splits pieces of `chunk` keys; chunk
// is 32 * 2^k, the smallest that needs at most MAX_SPLITS pieces, so the cut is a
// function of the row's own position and window and does not change with the
// batch around it.  Pieces meet in scratch memory (max, sum, weighted values per
// (row, head, split)); the block that finishes last for a (row, kv head) merges
// them in index order and writes the output.  Everything but q, k, v and the
// output is 32-bit.
//
// HEAD_DIM is a compile-time size (a multiple of 16, at most 256), given with
// -DHEAD_DIM=...; the library is built per head size at first use.
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
#define DEC_MAX_GROUP 8        // query heads per kv head: one warp each
#define DEC_MAX_SPLITS 32
#define DEC_TILE 32            // keys a warp takes per pass

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
constexpr int kBatch = 64 / kOwn;                   // keys whose values a lane holds at once (32, 16, 8)

struct __align__(16) Bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ int split_chunk(int n_keys) {
  int chunk = DEC_TILE;
  while ((n_keys + chunk - 1) / chunk > DEC_MAX_SPLITS) chunk <<= 1;
  return chunk;
}

__global__ void __launch_bounds__(DEC_MAX_GROUP * 32)
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
  const int group = nh / nkv;                       // == warps of the block
  const int first = lo + split * chunk;
  const int last = min(p, first + chunk - 1);
  const int* table = block_table + (size_t)r * table_stride;
  const int tid = threadIdx.x, h = tid >> 5, lane = tid & 31;   // h: this warp's head in the group
  const int head = kvh * group + h;

  __shared__ float q_s[DEC_MAX_GROUP][HEAD_DIM];
  __shared__ int is_last;

  // each warp stages its own head's q: no block-wide barrier is needed
  for (int c = lane; c < HEAD_DIM; c += 32)
    q_s[h][c] = __bfloat162float(q[((size_t)t * nh + head) * HEAD_DIM + c]);
  __syncwarp();

  float m_run = -INFINITY, l_run = 0.f, acc[kOwn];
#pragma unroll
  for (int e = 0; e < kOwn; ++e) acc[e] = 0.f;
  const int own = (lane < kOwners ? lane : 0) * kOwn;

  for (int k0 = first; k0 <= last; k0 += DEC_TILE) {
    // ---- scores: a lane per key ----
    const int key = k0 + lane;
    const bool live = key <= last;
    const int key_ok = live ? key : k0;                 // idle lanes read the first key again
    const int slot = table[key_ok / page] * page + key_ok % page;
    const Bf16x8* row = reinterpret_cast<const Bf16x8*>(k_pool + ((size_t)slot * nkv + kvh) * HEAD_DIM);
    Bf16x8 kreg[HEAD_DIM / 8];
#pragma unroll
    for (int c = 0; c < HEAD_DIM / 8; ++c) kreg[c] = row[c];
    // the values do not wait for the scores: the first batch is requested together
    // with the keys, so one trip to memory serves both
    const int n = min(DEC_TILE, last - k0 + 1);
    __nv_bfloat162 vreg[kBatch][kOwn / 2];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int slot_j = __shfl_sync(0xffffffffu, slot, j);
      const __nv_bfloat162* vrow = reinterpret_cast<const __nv_bfloat162*>(
          v_pool + ((size_t)slot_j * nkv + kvh) * HEAD_DIM + own);
#pragma unroll
      for (int e = 0; e < kOwn / 2; ++e) vreg[j][e] = vrow[e];
    }
    float dot[4] = {0.f, 0.f, 0.f, 0.f};                // four chains instead of one
#pragma unroll
    for (int c = 0; c < HEAD_DIM / 8; ++c) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 kf = __bfloat1622float2(kreg[c].v[e]);
        const float2 qf = *reinterpret_cast<const float2*>(&q_s[h][c * 8 + e * 2]);
        dot[e] += qf.x * kf.x + qf.y * kf.y;
      }
    }
    const float s = live ? ((dot[0] + dot[1]) + (dot[2] + dot[3])) * scale : -INFINITY;
    // ---- running softmax of this warp ----
    const float m_new = fmaxf(m_run, warp_max(s));      // finite: lane 0's key is live
    const float w = expf(s - m_new);                     // exp(-inf) = 0 for idle lanes
    const float corr = expf(m_run - m_new);              // 0 on the first pass
    l_run = l_run * corr + warp_sum(w);
    m_run = m_new;
#pragma unroll
    for (int e = 0; e < kOwn; ++e) acc[e] *= corr;
    // ---- weighted values: a lane per kOwn value lanes; idle keys carry weight 0 ----
#pragma unroll
    for (int j0 = 0; j0 < DEC_TILE; j0 += kBatch) {
      if (j0 > 0 && j0 < n) {
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const int slot_j = __shfl_sync(0xffffffffu, slot, j0 + j);
          const __nv_bfloat162* vrow = reinterpret_cast<const __nv_bfloat162*>(
              v_pool + ((size_t)slot_j * nkv + kvh) * HEAD_DIM + own);
#pragma unroll
          for (int e = 0; e < kOwn / 2; ++e) vreg[j][e] = vrow[e];
        }
      }
      if (j0 < n) {
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const float wj = __shfl_sync(0xffffffffu, w, j0 + j);
#pragma unroll
          for (int e = 0; e < kOwn / 2; ++e) {
            const float2 vf = __bfloat1622float2(vreg[j][e]);
            acc[2 * e] += wj * vf.x;
            acc[2 * e + 1] += wj * vf.y;
          }
        }
      }
    }
  }

  // scratch layout per (row, head): [split][HEAD_DIM + 2] = weighted values, max, sum
  const size_t per_head = (size_t)DEC_MAX_SPLITS * (HEAD_DIM + 2);
  if (n_splits == 1) {
    if (lane < kOwners) {
      const float inv = 1.0f / l_run;
      __nv_bfloat16* dst = out + ((size_t)t * nh + head) * HEAD_DIM + own;
#pragma unroll
      for (int e = 0; e < kOwn; e += 2)
        *reinterpret_cast<__nv_bfloat162*>(dst + e) = __floats2bfloat162_rn(acc[e] * inv, acc[e + 1] * inv);
    }
    return;
  }
  float* piece = scratch + ((size_t)t * nh + head) * per_head + (size_t)split * (HEAD_DIM + 2);
  if (lane < kOwners) {
#pragma unroll
    for (int e = 0; e < kOwn; ++e) piece[own + e] = acc[e];
  }
  if (lane == 0) { piece[HEAD_DIM] = m_run; piece[HEAD_DIM + 1] = l_run; }
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
  // warp h merges head h: lane s holds split s's maximum and sum
  const float* pieces = scratch + ((size_t)t * nh + head) * per_head;
  const bool on = lane < n_splits;
  const float m_s = on ? __ldcg(&pieces[(size_t)lane * (HEAD_DIM + 2) + HEAD_DIM]) : -INFINITY;
  const float l_s = on ? __ldcg(&pieces[(size_t)lane * (HEAD_DIM + 2) + HEAD_DIM + 1]) : 0.f;
  const float m_all = warp_max(m_s);
  const float f = expf(m_s - m_all);                    // 0 for lanes without a split
  const float den = warp_sum(f * l_s);
  for (int c0 = 0; c0 < HEAD_DIM; c0 += 32) {
    const int c = c0 + lane;
    float num = 0.f;
    if (c < HEAD_DIM) {
      float v[DEC_MAX_SPLITS];
#pragma unroll
      for (int sp = 0; sp < DEC_MAX_SPLITS; ++sp)
        v[sp] = sp < n_splits ? __ldcg(&pieces[(size_t)sp * (HEAD_DIM + 2) + c]) : 0.f;
#pragma unroll
      for (int sp = 0; sp < DEC_MAX_SPLITS; ++sp) num += __shfl_sync(0xffffffffu, f, sp) * v[sp];
    } else {
#pragma unroll
      for (int sp = 0; sp < DEC_MAX_SPLITS; ++sp) (void)__shfl_sync(0xffffffffu, f, sp);
    }
    if (c < HEAD_DIM) out[((size_t)t * nh + head) * HEAD_DIM + c] = __float2bfloat16_rn(num / den);
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
  return launch_dependent(decode_attention_kernel, grid, dim3(32 * (nh / nkv)), 0, stream,
                          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
                          (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, block_table,
                          table_stride, row_req, pos, nh, nkv, page, window, scale, scratch,
                          counters);
}
