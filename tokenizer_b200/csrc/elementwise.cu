// Memory-bound parts of the step: embedding gather, RMSNorm with the residual
// add folded in, rotary encoding fused with the bias add and the write of K and
// V into cache pages, the gated activation, row gathers.  The residual stream is
// 32-bit in both precisions; `T` is the type of the matrix-product operands
// (float for the 32-bit path, bfloat16 for serving).  Statistics, angles and
// sums are 32-bit throughout.
#include "common.cuh"

// ----------------------------------------------------------------------------
// embedding gather: x[t, :] = table[ids[t], :], widened to 32-bit
// ----------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ x, int hidden, int vocab) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // ids are validated on the host; never read outside
  const T* row = table + (size_t)id * hidden;
  float* out = x + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_float(row[i]);
}

TOKB200_API int tokb200_embed(const int* ids, const void* table, int table_dtype, float* x,
                              int n_tokens, int hidden, int vocab, cudaStream_t stream) {
  if (n_tokens <= 0) return TOKB200_OK;
  if (table_dtype == TOKB200_F32)
    return launch_dependent(embed_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, ids,
                            (const float*)table, x, hidden, vocab);
  if (table_dtype == TOKB200_BF16)
    return launch_dependent(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, ids,
                            (const __nv_bfloat16*)table, x, hidden, vocab);
  return TOKB200_BAD_DTYPE;
}

// ----------------------------------------------------------------------------
// RMSNorm, optionally after x += delta (the pending residual):
//   x <- x + delta (stored back, 32-bit);  y = x / sqrt(mean(x^2) + eps) * gain
// One block per row.  `rows` optionally names the rows to read (a gather of the
// wanted rows before the final norm); y is then dense [n_rows, hidden].
// ----------------------------------------------------------------------------
// Each thread keeps its elements in registers between the two passes (up to
// RMS_MAX_PER_THREAD of them; wider rows fall back to re-reading), and all loads
// of a pass are issued before the first use, so a row costs one round trip to
// memory, not one per element.
#define RMS_MAX_PER_THREAD 8

template <typename TD, typename TO>
__global__ void __launch_bounds__(1024) rms_norm_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                const float* __restrict__ gain, TO* __restrict__ y,
                                const int* __restrict__ rows, int hidden, float eps,
                                int n_partials, size_t partial_stride) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * hidden;
  const TD* dr = delta ? delta + (size_t)src * hidden : nullptr;
  TO* yr = y + (size_t)r * hidden;
  const bool in_registers = hidden <= RMS_MAX_PER_THREAD * (int)blockDim.x;
  float v[RMS_MAX_PER_THREAD];
  float ss = 0.f;
  if (in_registers) {
#pragma unroll
    for (int e = 0; e < RMS_MAX_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      v[e] = i < hidden ? xr[i] : 0.f;
    }
    if (dr) {
      // the pending residual may come as partial sums of a product cut along k; four of
      // them are asked for at a time (a trip to memory per group, not per partial sum) and
      // added in index order
      for (int s0 = 0; s0 < n_partials; s0 += 4) {
        float d[4][RMS_MAX_PER_THREAD];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int e = 0; e < RMS_MAX_PER_THREAD; ++e) {
            const int i = threadIdx.x + e * blockDim.x;
            d[u][e] = (s0 + u < n_partials && i < hidden) ? to_float(dr[(size_t)(s0 + u) * partial_stride + i]) : 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int e = 0; e < RMS_MAX_PER_THREAD; ++e) v[e] += d[u][e];
        }
      }
#pragma unroll
      for (int e = 0; e < RMS_MAX_PER_THREAD; ++e) {
        const int i = threadIdx.x + e * blockDim.x;
        if (i < hidden) xr[i] = v[e];
      }
    }
#pragma unroll
    for (int e = 0; e < RMS_MAX_PER_THREAD; ++e) ss += v[e] * v[e];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float a = xr[i];
      if (dr) {
        for (int s = 0; s < n_partials; ++s) a += to_float(dr[(size_t)s * partial_stride + i]);
        xr[i] = a;
      }
      ss += a * a;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  if (in_registers) {
#pragma unroll
    for (int e = 0; e < RMS_MAX_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < hidden) yr[i] = from_float<TO>(v[e] * inv * gain[i]);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      yr[i] = from_float<TO>(xr[i] * inv * gain[i]);
  }
}

// Many rows (portions of prompts), bfloat16 residual and output, width a multiple
// of 8 up to 8192: one block a row, eight elements (16 bytes of bfloat16) a thread,
// values kept in registers between the sum and the scaling.
__global__ void rms_norm_rows_bf16_kernel(float* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                                          const float* __restrict__ gain, __nv_bfloat16* __restrict__ y,
                                          int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const size_t base = (size_t)blockIdx.x * hidden;
  const int c = threadIdx.x * 8;
  const bool on = c < hidden;
  float v[8];
  float ss = 0.f;
  if (on) {
    const float4 a = *reinterpret_cast<const float4*>(x + base + c);
    const float4 b = *reinterpret_cast<const float4*>(x + base + c + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    if (delta) {
      const uint4 d4 = *reinterpret_cast<const uint4*>(delta + base + c);
      const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d4);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 d = __bfloat1622float2(d2[e]);
        v[2 * e] += d.x;
        v[2 * e + 1] += d.y;
      }
      *reinterpret_cast<float4*>(x + base + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(x + base + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  if (on) {
    const float4 ga = *reinterpret_cast<const float4*>(gain + c);
    const float4 gb = *reinterpret_cast<const float4*>(gain + c + 4);
    const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e)
      o2[e] = __floats2bfloat162_rn(v[2 * e] * inv * g[2 * e], v[2 * e + 1] * inv * g[2 * e + 1]);
    *reinterpret_cast<uint4*>(y + base + c) = o4;
  }
}

// The same for a pending residual that comes as float32 partial sums [n_partials, rows, hidden]
// of a product cut along k: all planes of a thread's eight elements are asked for at once and
// added in index order.
__global__ void rms_norm_rows_partials_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                              const float* __restrict__ gain, __nv_bfloat16* __restrict__ y,
                                              int hidden, float eps, int n_partials, size_t partial_stride) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const size_t base = (size_t)blockIdx.x * hidden;
  const int c = threadIdx.x * 8;
  const bool on = c < hidden;
  float v[8];
  float ss = 0.f;
  if (on) {
    const float4 a = *reinterpret_cast<const float4*>(x + base + c);
    const float4 b = *reinterpret_cast<const float4*>(x + base + c + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    for (int s0 = 0; s0 < n_partials; s0 += 4) {
      float4 lo[4], hi[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u < n_partials) {
          const float* plane = delta + (size_t)(s0 + u) * partial_stride + base + c;
          lo[u] = *reinterpret_cast<const float4*>(plane);
          hi[u] = *reinterpret_cast<const float4*>(plane + 4);
        } else {
          lo[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          hi[u] = lo[u];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v[0] += lo[u].x; v[1] += lo[u].y; v[2] += lo[u].z; v[3] += lo[u].w;
        v[4] += hi[u].x; v[5] += hi[u].y; v[6] += hi[u].z; v[7] += hi[u].w;
      }
    }
    *reinterpret_cast<float4*>(x + base + c) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(x + base + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  if (on) {
    const float4 ga = *reinterpret_cast<const float4*>(gain + c);
    const float4 gb = *reinterpret_cast<const float4*>(gain + c + 4);
    const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e)
      o2[e] = __floats2bfloat162_rn(v[2 * e] * inv * g[2 * e], v[2 * e + 1] * inv * g[2 * e + 1]);
    *reinterpret_cast<uint4*>(y + base + c) = o4;
  }
}

TOKB200_API int tokb200_rms_norm(float* x, const void* delta, int delta_dtype, int n_partials,
                                 long long partial_stride, const float* gain, void* y,
                                 int y_dtype, const int* rows, int n_rows, int hidden, float eps,
                                 cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0 || n_partials < 1) return TOKB200_BAD_SIZE;
  if (n_rows >= 64 && !rows && n_partials == 1 && y_dtype == TOKB200_BF16 &&
      (!delta || delta_dtype == TOKB200_BF16) && hidden % 8 == 0 && hidden <= 8192 &&
      (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)gain | (uintptr_t)y) & 15) == 0) {
    const int threads8 = ((hidden / 8 + 31) / 32) * 32;
    return launch_dependent(rms_norm_rows_bf16_kernel, dim3(n_rows), dim3(threads8), 0, stream, x,
                            (const __nv_bfloat16*)delta, gain, (__nv_bfloat16*)y, hidden, eps);
  }
  if (n_rows > 16 && !rows && delta && delta_dtype == TOKB200_F32 && y_dtype == TOKB200_BF16 &&
      hidden % 8 == 0 && hidden <= 8192 && partial_stride % 4 == 0 &&
      (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)gain | (uintptr_t)y) & 15) == 0) {
    const int threads8 = ((hidden / 8 + 31) / 32) * 32;
    return launch_dependent(rms_norm_rows_partials_kernel, dim3(n_rows), dim3(threads8), 0, stream, x,
                            (const float*)delta, gain, (__nv_bfloat16*)y, hidden, eps, n_partials,
                            (size_t)partial_stride);
  }
  int threads = 128;   // rows of up to 8 elements a thread stay in registers
  while (threads < 1024 && hidden > threads * 4) threads *= 2;
#define LAUNCH(TD, TO)                                                                        \
  return launch_dependent(rms_norm_kernel<TD, TO>, dim3(n_rows), dim3(threads), 0, stream, x, \
                          (const TD*)delta, gain, (TO*)y, rows, hidden, eps, n_partials,     \
                          (size_t)partial_stride)
  if (delta_dtype == TOKB200_F32 && y_dtype == TOKB200_F32) LAUNCH(float, float);
  if (delta_dtype == TOKB200_F32 && y_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (delta_dtype == TOKB200_BF16 && y_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
  if (delta_dtype == TOKB200_BF16 && y_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}

// x += delta, elementwise (a pending residual that no norm follows)
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n,
                                    int n_partials) {
  pdl_wait();
  pdl_launch();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float v = x[i];
    for (int s = 0; s < n_partials; ++s) v += to_float(delta[(size_t)s * n + i]);
    x[i] = v;
  }
}

TOKB200_API int tokb200_residual_add(float* x, const void* delta, int delta_dtype, int n_partials,
                                     long long n, cudaStream_t stream) {
  if (n <= 0) return TOKB200_OK;
  if (n_partials < 1) return TOKB200_BAD_SIZE;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (delta_dtype == TOKB200_F32)
    residual_add_kernel<float><<<blocks, 256, 0, stream>>>(x, (const float*)delta, (size_t)n, n_partials);
  else if (delta_dtype == TOKB200_BF16)
    residual_add_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(x, (const __nv_bfloat16*)delta, (size_t)n, n_partials);
  else
    return TOKB200_BAD_DTYPE;
  return tokb200_launch_status();
}

// ----------------------------------------------------------------------------
// rotary tables: cos/sin of float(position) * inv_freq[i], 32-bit
// ----------------------------------------------------------------------------
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float* __restrict__ cos_t,
                                  float* __restrict__ sin_t, int n_positions, int half) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_positions * half) return;
  const int p = (int)(i / half), f = (int)(i % half);
  const float angle = (float)p * inv_freq[f];
  cos_t[i] = cosf(angle);
  sin_t[i] = sinf(angle);
}

TOKB200_API int tokb200_rope_table(const float* inv_freq, float* cos_t, float* sin_t,
                                   int n_positions, int half, cudaStream_t stream) {
  const size_t n = (size_t)n_positions * half;
  if (n == 0) return TOKB200_OK;
  rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(inv_freq, cos_t, sin_t,
                                                                    n_positions, half);
  return tokb200_launch_status();
}

// ----------------------------------------------------------------------------
// bias + rotary encoding + cache write.
// qkv is [T, (nh + 2 nkv) d]: query heads, then key heads, then value heads.
// Per token: q and k get their bias and are rotated by the half-split rule over
// the first `rotary` lanes of each head (pairs (i, i + rotary/2)); v gets its
// bias.  q goes to q_out [T, nh d]; k and v go to the cache at slot[t]
// (page * page_size + offset), pool layout [slots, nkv, d].  A negative slot, or
// no pool, skips the write (a layer that reads another layer's cache).
// ----------------------------------------------------------------------------
template <typename T>
__global__ void rope_store_kernel(const T* __restrict__ qkv, const float* __restrict__ bias,
                                  const int* __restrict__ pos, const int* __restrict__ slot,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  T* __restrict__ q_out, T* __restrict__ k_pool,
                                  T* __restrict__ v_pool, int nh, int nkv, int d, int rotary,
                                  int table_half) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const int p = pos[t];
  const int s = slot ? slot[t] : -1;
  const int width = (nh + 2 * nkv) * d;
  const T* row = qkv + (size_t)t * width;
  const int half_d = d / 2;            // work items per head: pairs (j, j + d/2)
  const int rot_half = rotary / 2;
  const int items = (nh + 2 * nkv) * half_d;
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int head = it / half_d, j = it % half_d;
    // the two lanes this item owns.  Inside the rotary width lanes pair up as
    // (j, j + rot_half); outside it they are copied.  Items cover lanes j and
    // j + half_d, so remap: item j < rot_half rotates (j, j + rot_half); the
    // remaining lanes are passed through in pairs.
    int a, b;
    bool rotate;
    if (j < rot_half) { a = j; b = j + rot_half; rotate = true; }
    else { a = rotary + (j - rot_half) * 2; b = a + 1; rotate = false; }
    float va = to_float(row[head * d + a]);
    float vb = to_float(row[head * d + b]);
    if (bias) { va += bias[head * d + a]; vb += bias[head * d + b]; }
    T* dst;
    if (head < nh) {
      dst = q_out + (size_t)t * nh * d + head * d;
    } else if (head < nh + nkv) {
      if (s < 0 || !k_pool) continue;
      dst = k_pool + ((size_t)s * nkv + (head - nh)) * d;
    } else {
      if (s < 0 || !v_pool) continue;
      dst = v_pool + ((size_t)s * nkv + (head - nh - nkv)) * d;
      rotate = false;
    }
    if (rotate) {
      const float c = cos_t[(size_t)p * table_half + j], sn = sin_t[(size_t)p * table_half + j];
      const float ra = va * c - vb * sn;
      const float rb = vb * c + va * sn;
      va = ra; vb = rb;
    }
    dst[a] = from_float<T>(va);
    dst[b] = from_float<T>(vb);
  }
}

// The same for many rows in bfloat16 when the whole head is rotated and the head
// size is a multiple of 16: a thread takes 8 lanes of a head and their 8 partners
// (two 16-byte loads, two 16-byte stores).
__global__ void rope_store_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ bias,
                                         const int* __restrict__ pos, const int* __restrict__ slot,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool,
                                         __nv_bfloat16* __restrict__ v_pool, int n_tokens, int nh, int nkv,
                                         int d) {
  pdl_wait();
  pdl_launch();
  const int heads = nh + 2 * nkv, half = d / 2, per_head = d / 16, per_token = heads * per_head;
  const size_t item = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (size_t)n_tokens * per_token) return;
  const int t = (int)(item / per_token), rest = (int)(item % per_token);
  const int head = rest / per_head, j = (rest % per_head) * 8;
  const __nv_bfloat16* src = qkv + (size_t)t * heads * d + head * d + j;
  const uint4 a4 = *reinterpret_cast<const uint4*>(src);
  const uint4 b4 = *reinterpret_cast<const uint4*>(src + half);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a4);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b4);
  float a[8], b[8];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 fa = __bfloat1622float2(a2[e]), fb = __bfloat1622float2(b2[e]);
    a[2 * e] = fa.x; a[2 * e + 1] = fa.y; b[2 * e] = fb.x; b[2 * e + 1] = fb.y;
  }
  // eight consecutive floats as two 16-byte loads (j, half and d are multiples of 8; the tables and the bias
  // are 16-byte aligned, checked by the launcher)
  auto load8 = [](const float* p, float (&v)[8]) {
    const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
  };
  if (bias) {
    float ba[8], bb[8];
    load8(bias + head * d + j, ba);
    load8(bias + head * d + j + half, bb);
#pragma unroll
    for (int e = 0; e < 8; ++e) { a[e] += ba[e]; b[e] += bb[e]; }
  }
  __nv_bfloat16* dst;
  if (head < nh) {
    dst = q_out + ((size_t)t * nh + head) * d;
  } else {
    const int s = slot ? slot[t] : -1;
    const bool is_key = head < nh + nkv;
    __nv_bfloat16* pool = is_key ? k_pool : v_pool;
    if (s < 0 || !pool) return;
    dst = pool + ((size_t)s * nkv + (head - nh - (is_key ? 0 : nkv))) * d;
  }
  if (head < nh + nkv) {
    float c[8], sn[8];
    load8(cos_t + (size_t)pos[t] * half + j, c);
    load8(sin_t + (size_t)pos[t] * half + j, sn);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ra = a[e] * c[e] - b[e] * sn[e], rb = b[e] * c[e] + a[e] * sn[e];
      a[e] = ra;
      b[e] = rb;
    }
  }
  uint4 oa, ob;
  __nv_bfloat162* oa2 = reinterpret_cast<__nv_bfloat162*>(&oa);
  __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    oa2[e] = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
    ob2[e] = __floats2bfloat162_rn(b[2 * e], b[2 * e + 1]);
  }
  *reinterpret_cast<uint4*>(dst + j) = oa;
  *reinterpret_cast<uint4*>(dst + j + half) = ob;
}

// The same from float32 partial sums [S, T, heads d] of a product that was cut along k: the
// pieces are added in index order, then bias, rotation and the cache write as above.
__global__ void rope_store_partials_kernel(const float* __restrict__ parts, int n_partials, size_t stride,
                                           const float* __restrict__ bias, const int* __restrict__ pos,
                                           const int* __restrict__ slot, const float* __restrict__ cos_t,
                                           const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ q_out,
                                           __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                                           int n_tokens, int nh, int nkv, int d) {
  pdl_wait();
  pdl_launch();
  const int heads = nh + 2 * nkv, half = d / 2, per_head = d / 16, per_token = heads * per_head;
  const size_t item = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (size_t)n_tokens * per_token) return;
  const int t = (int)(item / per_token), rest = (int)(item % per_token);
  const int head = rest / per_head, j = (rest % per_head) * 8;
  const float* src = parts + (size_t)t * heads * d + head * d + j;
  float a[8], b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) a[e] = b[e] = 0.f;
  for (int s = 0; s < n_partials; ++s) {
    const float4 a0 = *reinterpret_cast<const float4*>(src + s * stride);
    const float4 a1 = *reinterpret_cast<const float4*>(src + s * stride + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(src + s * stride + half);
    const float4 b1 = *reinterpret_cast<const float4*>(src + s * stride + half + 4);
    a[0] += a0.x; a[1] += a0.y; a[2] += a0.z; a[3] += a0.w; a[4] += a1.x; a[5] += a1.y; a[6] += a1.z; a[7] += a1.w;
    b[0] += b0.x; b[1] += b0.y; b[2] += b0.z; b[3] += b0.w; b[4] += b1.x; b[5] += b1.y; b[6] += b1.z; b[7] += b1.w;
  }
  if (bias) {
#pragma unroll
    for (int e = 0; e < 8; ++e) { a[e] += bias[head * d + j + e]; b[e] += bias[head * d + j + half + e]; }
  }
  __nv_bfloat16* dst;
  if (head < nh) {
    dst = q_out + ((size_t)t * nh + head) * d;
  } else {
    const int sl = slot ? slot[t] : -1;
    const bool is_key = head < nh + nkv;
    __nv_bfloat16* pool = is_key ? k_pool : v_pool;
    if (sl < 0 || !pool) return;
    dst = pool + ((size_t)sl * nkv + (head - nh - (is_key ? 0 : nkv))) * d;
  }
  if (head < nh + nkv) {
    const float* c = cos_t + (size_t)pos[t] * half + j;
    const float* sn = sin_t + (size_t)pos[t] * half + j;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ra = a[e] * c[e] - b[e] * sn[e], rb = b[e] * c[e] + a[e] * sn[e];
      a[e] = ra;
      b[e] = rb;
    }
  }
  uint4 oa, ob;
  __nv_bfloat162* oa2 = reinterpret_cast<__nv_bfloat162*>(&oa);
  __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    oa2[e] = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
    ob2[e] = __floats2bfloat162_rn(b[2 * e], b[2 * e + 1]);
  }
  *reinterpret_cast<uint4*>(dst + j) = oa;
  *reinterpret_cast<uint4*>(dst + j + half) = ob;
}

// parts: float32 [n_partials, n_tokens, (nh + 2 nkv) d]; outputs bfloat16; the whole head is
// rotated (d a multiple of 16).
TOKB200_API int tokb200_rope_store_partials(const float* parts, int n_partials, const float* bias,
                                            const int* pos, const int* slot, const float* cos_t,
                                            const float* sin_t, void* q_out, void* k_pool, void* v_pool,
                                            int n_tokens, int nh, int nkv, int d, cudaStream_t stream) {
  if (n_tokens <= 0) return TOKB200_OK;
  if (d <= 0 || d % 16 || n_partials < 1) return TOKB200_BAD_SIZE;
  if (((uintptr_t)parts | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15)
    return TOKB200_BAD_ALIGNMENT;
  const size_t total = (size_t)n_tokens * (nh + 2 * nkv) * (d / 16);
  const size_t stride = (size_t)n_tokens * (nh + 2 * nkv) * d;
  return launch_dependent(rope_store_partials_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                          stream, parts, n_partials, stride, bias, pos, slot, cos_t, sin_t,
                          (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_tokens,
                          nh, nkv, d);
}

TOKB200_API int tokb200_rope_store(const void* qkv, const float* bias, const int* pos,
                                   const int* slot, const float* cos_t, const float* sin_t,
                                   void* q_out, void* k_pool, void* v_pool, int dtype,
                                   int n_tokens, int nh, int nkv, int d, int rotary,
                                   cudaStream_t stream) {
  if (n_tokens <= 0) return TOKB200_OK;
  if (d <= 0 || (d & 1) || rotary < 0 || rotary > d || (rotary & 1) || ((d - rotary) & 1))
    return TOKB200_BAD_SIZE;
  if (dtype == TOKB200_BF16 && rotary == d && d % 16 == 0 && n_tokens >= 64 &&
      (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)bias |
        (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) == 0) {
    const size_t total = (size_t)n_tokens * (nh + 2 * nkv) * (d / 16);
    return launch_dependent(rope_store_bf16x8_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                            stream, (const __nv_bfloat16*)qkv, bias, pos, slot, cos_t, sin_t,
                            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                            n_tokens, nh, nkv, d);
  }
  const int items = (nh + 2 * nkv) * (d / 2);
  int threads = items < 256 ? ((items + 31) / 32) * 32 : 256;
  if (dtype == TOKB200_F32)
    return launch_dependent(rope_store_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream,
                            (const float*)qkv, bias, pos, slot, cos_t, sin_t, (float*)q_out,
                            (float*)k_pool, (float*)v_pool, nh, nkv, d, rotary, rotary / 2);
  if (dtype == TOKB200_BF16)
    return launch_dependent(rope_store_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0,
                            stream, (const __nv_bfloat16*)qkv, bias, pos, slot, cos_t, sin_t,
                            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                            nh, nkv, d, rotary, rotary / 2);
  return TOKB200_BAD_DTYPE;
}

// ----------------------------------------------------------------------------
// gated activation: out[t, i] = act(gu[t, i]) * gu[t, inner + i], `act` by its tag
// (silu(z) = z * sigmoid(z) = z / (1 + exp(-z)) for the architecture served), in 32-bit
// ----------------------------------------------------------------------------
template <typename T>
__global__ void silu_gate_kernel(const T* __restrict__ gu, T* __restrict__ out, int inner, int act) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.y;
  const T* row = gu + (size_t)t * 2 * inner;
  T* orow = out + (size_t)t * inner;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inner; i += gridDim.x * blockDim.x) {
    const float g = to_float(row[i]), u = to_float(row[inner + i]);
    orow[i] = from_float<T>(gate_activation(act, g) * u);
  }
}

// bfloat16 rows whose width is a multiple of 8: eight elements (16 bytes) a thread
__global__ void silu_gate_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu,
                                        __nv_bfloat16* __restrict__ out, int inner, int n_rows, int act) {
  pdl_wait();
  pdl_launch();
  const int per_row = inner / 8;
  const size_t total = (size_t)n_rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inner + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inner + inner + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
      o2[e] = __floats2bfloat162_rn(gate_activation(act, g.x) * u.x, gate_activation(act, g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * inner + c) = o4;
  }
}

// the same for the interleaved layout of the gated kernels: for every 128 outputs,
// 128 gate values followed by their 128 up values
__global__ void silu_gate_interleaved_kernel(const __nv_bfloat16* __restrict__ gu,
                                             __nv_bfloat16* __restrict__ out, int inner, int n_rows, int act) {
  pdl_wait();
  pdl_launch();
  const int per_row = inner / 8;
  const size_t total = (size_t)n_rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row;
    const int c = (int)(i % per_row) * 8;                   // output column
    const size_t at = t * 2 * inner + (size_t)(c / 128) * 256 + c % 128;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + at);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + at + 128);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
      o2[e] = __floats2bfloat162_rn(gate_activation(act, g.x) * u.x, gate_activation(act, g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * inner + c) = o4;
  }
}

TOKB200_API int tokb200_silu_gate_interleaved(const void* gu, void* out, int n_tokens, int inner,
                                              int act, cudaStream_t stream) {
  if (n_tokens <= 0) return TOKB200_OK;
  if (inner <= 0 || inner % 128 || act < 0 || act >= TOKB200_ACT_COUNT) return TOKB200_BAD_SIZE;
  if (((uintptr_t)gu | (uintptr_t)out) & 15) return TOKB200_BAD_ALIGNMENT;
  const size_t total = (size_t)n_tokens * (inner / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return launch_dependent(silu_gate_interleaved_kernel, dim3(blocks), dim3(256), 0, stream,
                          (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inner, n_tokens, act);
}

TOKB200_API int tokb200_silu_gate(const void* gu, void* out, int dtype, int n_tokens, int inner,
                                  int act, cudaStream_t stream) {
  if (n_tokens <= 0) return TOKB200_OK;
  if (inner <= 0 || n_tokens > 65535 * 1024 || act < 0 || act >= TOKB200_ACT_COUNT) return TOKB200_BAD_SIZE;
  if (dtype == TOKB200_BF16 && inner % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
    const size_t total = (size_t)n_tokens * (inner / 8);
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    return launch_dependent(silu_gate_bf16x8_kernel, dim3(blocks), dim3(256), 0, stream,
                            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inner, n_tokens, act);
  }
  // grid.y is limited to 65535 rows; tile rows over several launches beyond it
  for (int row0 = 0; row0 < n_tokens; row0 += 65535) {
    const int rows = n_tokens - row0 < 65535 ? n_tokens - row0 : 65535;
    dim3 grid((inner + 255) / 256 < 64 ? (inner + 255) / 256 : 64, rows);
    int status;
    if (dtype == TOKB200_F32)
      status = launch_dependent(silu_gate_kernel<float>, grid, dim3(256), 0, stream,
                                (const float*)gu + (size_t)row0 * 2 * inner,
                                (float*)out + (size_t)row0 * inner, inner, act);
    else if (dtype == TOKB200_BF16)
      status = launch_dependent(silu_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream,
                                (const __nv_bfloat16*)gu + (size_t)row0 * 2 * inner,
                                (__nv_bfloat16*)out + (size_t)row0 * inner, inner, act);
    else
      return TOKB200_BAD_DTYPE;
    if (status != TOKB200_OK) return status;
  }
  return TOKB200_OK;
}

// ----------------------------------------------------------------------------
// Decoding several steps without the host: after a step's ids were drawn, make
// the next step's metadata in place.  For each live row r: the drawn id becomes
// the next input, its position and stored length grow by one, its cache slot is
// looked up in its block table (pages were reserved ahead), and the id is
// appended to `history[step, r]`; `step_counter` counts the steps.
// ----------------------------------------------------------------------------
struct AdvanceGroups {
  int* slots[4];
  const int* tables[4];
  int widths[4];
  int count;
};

__global__ void advance_decode_kernel(int* __restrict__ ids, const int* __restrict__ drawn,
                                      int* __restrict__ pos, int* __restrict__ kv_len,
                                      const int* __restrict__ row_req, AdvanceGroups groups,
                                      int page, int n_rows, int* __restrict__ history,
                                      int* __restrict__ step_counter) {
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const int step = *step_counter;
  if (r < n_rows && row_req[r] >= 0) {
    const int id = drawn[r];
    ids[r] = id;
    history[(size_t)step * n_rows + r] = id;
    const int p = pos[r] + 1;
    pos[r] = p;
    kv_len[r] += 1;
    for (int g = 0; g < groups.count; ++g) {
      // after the last step of a burst the next position may lie one block past the row's
      // table (a length of exactly width * page): nothing will be written there
      const int block = p / page;
      const int pg = block < groups.widths[g] ? groups.tables[g][(size_t)r * groups.widths[g] + block] : -1;
      groups.slots[g][r] = pg < 0 ? -1 : pg * page + p % page;
    }
  }
}

__global__ void bump_counter_kernel(int* counter) {
  pdl_wait();
  pdl_launch();
  *counter += 1;
}

TOKB200_API int tokb200_advance_decode(int* ids, const int* drawn, int* pos, int* kv_len,
                                       const int* row_req, int n_groups, int** slots,
                                       const int** tables, const int* widths, int page,
                                       int n_rows, int* history, int* step_counter,
                                       cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (n_groups < 0 || n_groups > 4) return TOKB200_BAD_SIZE;
  AdvanceGroups groups;
  groups.count = n_groups;
  for (int g = 0; g < n_groups; ++g) {
    groups.slots[g] = slots[g];
    groups.tables[g] = tables[g];
    groups.widths[g] = widths[g];
  }
  int status = launch_dependent(advance_decode_kernel, dim3((n_rows + 127) / 128), dim3(128), 0,
                                stream, ids, drawn, pos, kv_len, row_req, groups, page, n_rows,
                                history, step_counter);
  if (status != TOKB200_OK) return status;
  return launch_dependent(bump_counter_kernel, dim3(1), dim3(1), 0, stream, step_counter);
}

// ---- bringing weights into L2 ahead of their use ------------------------------------
// While a decoding step's kernels each wait on a short chain of loads, DRAM is mostly
// idle.  This kernel asks the memory system to bring `bytes` at `base` into L2 and
// returns at once; it runs on a second stream beside the layer that comes before the
// one whose weights it names, so that layer's kernels then read L2 and not DRAM.
constexpr int kPrefetchChunk = 8192;

__global__ void prefetch_l2_kernel(const char* __restrict__ base, long long bytes) {
  long long chunk = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long step = (long long)gridDim.x * blockDim.x;
  for (long long at = chunk * kPrefetchChunk; at < bytes; at += step * kPrefetchChunk) {
    long long left = bytes - at;
    unsigned size = (unsigned)(left < kPrefetchChunk ? (left & ~15ll) : kPrefetchChunk);
    if (size)
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + at), "r"(size) : "memory");
  }
}

TOKB200_API int tokb200_prefetch_l2(const void* base, long long bytes, cudaStream_t stream) {
  if (bytes <= 0) return TOKB200_OK;
  if (reinterpret_cast<uintptr_t>(base) % 16) return TOKB200_BAD_ALIGNMENT;
  long long chunks = (bytes + kPrefetchChunk - 1) / kPrefetchChunk;
  int blocks = (int)((chunks + 127) / 128);
  if (blocks > 16) blocks = 16;
  prefetch_l2_kernel<<<blocks, 128, 0, stream>>>(static_cast<const char*>(base), bytes);
  return (int)cudaGetLastError();
}
