// Attention over the paged cache for any batch of rows: portions of prompts and
// single decoded tokens alike.  Row t belongs to request row_req[t] and sits at
// absolute position pos[t]; it attends to the keys of its request at positions
// lo..pos[t] (lo = 0, or pos - window when the layer has a window: a key is
// hidden when key + window < query), all read from the cache, where this step's
// own keys were written before the launch.
//
// This is the general kernel: any head size, any number of heads and groups,
// both precisions.  One block per (row, query head); keys are processed in
// fixed chunks of ATT_CHUNK counted from lo, so a row's arithmetic depends only on
// its own position and window, never on the batch around it.  Scores, the
// running maximum, the exponentials and the weighted sum are 32-bit.
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_CHUNK 128
#define ATT_MAX_HEAD_DIM 512

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                               const T* __restrict__ v_pool, T* __restrict__ out,
                               const int* __restrict__ block_table, int table_stride,
                               const int* __restrict__ row_req, const int* __restrict__ pos,
                               int nh, int nkv, int d, int page, int window, float scale) {
  extern __shared__ float smem[];
  float* q_s = smem;                 // d
  float* p_s = smem + d;             // ATT_CHUNK
  int* slot_s = (int*)(p_s + ATT_CHUNK);  // ATT_CHUNK
  __shared__ float scratch[33];

  const int t = blockIdx.x, h = blockIdx.y;
  const int r = row_req[t];
  if (r < 0) return;
  const int p = pos[t];
  const int kvh = h / (nh / nkv);
  const int lo = (window >= 0 && p - window > 0) ? p - window : 0;
  const int* table = block_table + (size_t)r * table_stride;

  const T* q_row = q + ((size_t)t * nh + h) * d;
  for (int i = threadIdx.x; i < d; i += ATT_THREADS) q_s[i] = to_float(q_row[i]);
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_HEAD_DIM / ATT_THREADS];
#pragma unroll
  for (int i = 0; i < ATT_MAX_HEAD_DIM / ATT_THREADS; ++i) acc[i] = 0.f;

  for (int c0 = lo; c0 <= p; c0 += ATT_CHUNK) {
    const int key = c0 + threadIdx.x;
    float s = -INFINITY;
    int slot = -1;
    if (key <= p) {
      const int pg = table[key / page];
      slot = pg * page + key % page;
      const T* k_row = k_pool + ((size_t)slot * nkv + kvh) * d;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot += q_s[i] * to_float(k_row[i]);
      s = dot * scale;
    }
    const float c_max = block_max(s, scratch);
    const float m_new = fmaxf(m, c_max);
    const float e = key <= p ? expf(s - m_new) : 0.f;
    p_s[threadIdx.x] = e;
    slot_s[threadIdx.x] = slot;
    const float c_sum = block_sum(e, scratch);  // contains the barrier that publishes p_s
    const float corr = expf(m - m_new);         // 0 on the first chunk (m = -inf)
    l = l * corr + c_sum;
    m = m_new;
    const int n = min(ATT_CHUNK, p - c0 + 1);
#pragma unroll
    for (int i = 0; i < ATT_MAX_HEAD_DIM / ATT_THREADS; ++i) {
      const int dim = threadIdx.x + i * ATT_THREADS;
      if (dim < d) {
        float a = acc[i] * corr;
        for (int j = 0; j < n; ++j)
          a += p_s[j] * to_float(v_pool[((size_t)slot_s[j] * nkv + kvh) * d + dim]);
        acc[i] = a;
      }
    }
    __syncthreads();  // p_s and slot_s are rewritten by the next chunk
  }
  T* o_row = out + ((size_t)t * nh + h) * d;
#pragma unroll
  for (int i = 0; i < ATT_MAX_HEAD_DIM / ATT_THREADS; ++i) {
    const int dim = threadIdx.x + i * ATT_THREADS;
    if (dim < d) o_row[dim] = from_float<T>(acc[i] / l);
  }
}

TOKB200_API int tokb200_paged_attention_generic(
    const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
    const int* block_table, int table_stride, const int* row_req, const int* pos, int n_rows,
    int nh, int nkv, int d, int page, int window, float scale, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (d <= 0 || d > ATT_MAX_HEAD_DIM || nh <= 0 || nkv <= 0 || nh % nkv || page <= 0 ||
      nh > 65535)
    return TOKB200_BAD_SIZE;
  const size_t smem = (size_t)(d + 2 * ATT_CHUNK) * sizeof(float);
  dim3 grid(n_rows, nh);
  if (dtype == TOKB200_F32)
    paged_attention_generic_kernel<float><<<grid, ATT_THREADS, smem, stream>>>(
        (const float*)q, (const float*)k_pool, (const float*)v_pool, (float*)out, block_table,
        table_stride, row_req, pos, nh, nkv, d, page, window, scale);
  else if (dtype == TOKB200_BF16)
    paged_attention_generic_kernel<__nv_bfloat16><<<grid, ATT_THREADS, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
        (__nv_bfloat16*)out, block_table, table_stride, row_req, pos, nh, nkv, d, page, window,
        scale);
  else
    return TOKB200_BAD_DTYPE;
  return tokb200_launch_status();
}
