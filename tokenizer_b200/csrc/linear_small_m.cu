// y[M,N] = x[M,K] W[N,K]^T (+ bias) for few rows (decoding: M <= 64), bfloat16
// operands, 32-bit accumulation.  The product is bound by reading W once, so the
// kernel is built around that stream: the weight rows play the M side of the
// tensor-core instruction (mma.sync m16n8k16, 16 weight rows per warp) and the
// batch plays its N side (8 rows of x per instruction), and every thread feeds
// its fragments straight from 16-byte global loads, with no staging of W in
// shared memory.  That works because a dot product does not care about the
// order of k: within a step of 64 k, thread t of a quad loads k = 16t .. 16t+15 of
// its weight row, and the same 16 of its x row, and both are handed to the four
// instructions of the step under the same (permuted) k slots.
//
// Work is cut three ways: row tiles of 16 over the grid's x, the warps of a block
// share a row tile by interleaved k steps and add up in shared memory in warp
// order, and (for matrices with few rows) K is also cut over the grid's y into
// `k_splits` pieces whose 32-bit partial results [k_splits, M, N] the consumer
// adds in index order.  Every sum has a fixed order: results are reproducible.
#include "common.cuh"

#define LSM_WARPS 8
#define LSM_THREADS (LSM_WARPS * 32)
#define LSM_PRE 4            // steps of 32 k of weights in flight per thread (the q/k/v kernel)
#define LSM_DENSE_ELEMENTS 9000000LL    // the largest weight (elements) that takes the DENSE form (3584 x 3584: 9.0 -> 11.2 us with it)
#define LSM_WIDE_PRE 2       // steps of 64 k of weights in flight per thread (the plain and the gated product)

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2,
                                               unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load16(const __nv_bfloat16* p, bool ok) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (ok) v = __ldg(reinterpret_cast<const uint4*>(p));
  return v;
}

// MT: tiles of 8 rows of x (M <= 8 MT).  TPB: row tiles of W per block; the
// block's warps split into TPB teams of LSM_WARPS / TPB warps, a team per row tile.
// GATED: w [N, K] holds, for every 128 outputs, their 128 "gate" rows followed by
// their 128 "up" rows; a row tile is then 8 gate rows and the 8 up rows of the same
// outputs, and the result is act(gate) * up, [M, N / 2] (`act`: the activation's tag).
// DENSE (9 to 16 rows, a weight of up to LSM_DENSE_ELEMENTS): the kernel is held to 80 registers so
// that three blocks fit a multiprocessor.  A small matrix gains from the loads in flight (hidden
// 896, 16 rows: 0.86 -> 0.80 ms a decoding step); a large one loses (3584 x 18944: 38 -> 55 us).
template <int MT, int TPB, bool GATED, bool DENSE = false>
__global__ void __launch_bounds__(LSM_THREADS, DENSE ? 3 : 1)
linear_small_m_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                      const float* __restrict__ bias, void* __restrict__ out, int out_is_f32,
                      int M, int N, int K, int k_per_split, int act) {
  constexpr int TEAM = LSM_WARPS / TPB;
  __shared__ float part[LSM_WARPS][16][8 * MT + 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int team = warp / TEAM, member = warp % TEAM;
  const int row0 = (blockIdx.x * TPB + team) * 16;
  const int k_begin = blockIdx.y * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);

  float acc[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  // the weight rows behind rows g and g + 8 of the tile
  int row_a = row0 + g, row_b = row0 + g + 8;
  if (GATED) {
    const int out0 = (blockIdx.x * TPB + team) * 8;           // 8 outputs a tile
    row_a = (out0 / 128) * 256 + out0 % 128 + g;
    row_b = row_a + 128;
  }
  const bool row_a_ok = row_a < N, row_b_ok = row_b < N;
  const __nv_bfloat16* wa = w + (size_t)row_a * K + 16 * t;
  const __nv_bfloat16* wb = w + (size_t)row_b * K + 16 * t;

  // A step is 64 k: thread t of a quad takes k = 16t .. 16t+15 of its two weight rows as two
  // 16-byte loads next to each other, so that a quad asks for a whole 128-byte line of a row
  // (with half a line per request, the other half asked for by another warp, the gate/up product
  // of a wide model took 64 us instead of 44; the loads alone: 3.8 against 4.6 TB/s at two blocks a
  // multiprocessor).  A ring of
  // LSM_WIDE_PRE steps of weights is requested before the wait on the predecessor (weights are
  // written by no kernel of the step); x, which the predecessor produced, is read after it.
  constexpr int step = TEAM * 64;
  const int k_first = k_begin + member * 64;
  uint4 a_ring[LSM_WIDE_PRE][2], b_ring[LSM_WIDE_PRE][2];
#pragma unroll
  for (int i = 0; i < LSM_WIDE_PRE; ++i) {
    const int kk = k_first + i * step + 16 * t;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const bool k_ok = kk + 8 * h + 8 <= k_end;
      a_ring[i][h] = load16(wa + k_first + i * step + 8 * h, row_a_ok && k_ok);
      b_ring[i][h] = load16(wb + k_first + i * step + 8 * h, row_b_ok && k_ok);
    }
  }
  // The successor may start now, before this kernel has even waited for its own predecessor:
  // the kernels that follow a plain product (a norm, the fused feed-forward, the sampler) touch
  // only weights before their own wait, and that wait still covers this kernel whole.  The
  // feed-forward thus streams its weights while the attention before this product still runs.
  pdl_launch();
  pdl_wait();
  for (int k = k_first; k < k_end; k += LSM_WIDE_PRE * step) {
#pragma unroll
    for (int i = 0; i < LSM_WIDE_PRE; ++i) {
      const int kk = k + i * step;
      uint4 a[2], b[2];
      const int kn = kk + LSM_WIDE_PRE * step;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        a[h] = a_ring[i][h];
        b[h] = b_ring[i][h];
        const bool next_ok = kn + 16 * t + 8 * h + 8 <= k_end;
        a_ring[i][h] = load16(wa + kn + 8 * h, row_a_ok && next_ok);
        b_ring[i][h] = load16(wb + kn + 8 * h, row_b_ok && next_ok);
      }
      if (kk < k_end) {
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const int m = 8 * j + g;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const bool k_ok = kk + 16 * t + 8 * h + 8 <= k_end;
            // (x a round ahead like the weights costs 16 registers and a resident block: slower)
            const uint4 xv = load16(x + (size_t)m * K + kk + 16 * t + 8 * h, m < M && k_ok);
            mma_bf16_16816(acc[j], a[h].x, b[h].x, a[h].y, b[h].y, xv.x, xv.y);
            mma_bf16_16816(acc[j], a[h].z, b[h].z, a[h].w, b[h].w, xv.z, xv.w);
          }
        }
      }
    }
  }

  // accumulator layout: c0,c1 -> (row g, columns 2t, 2t+1); c2,c3 -> (row g + 8, same)
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    part[warp][g][8 * j + 2 * t] = acc[j][0];
    part[warp][g][8 * j + 2 * t + 1] = acc[j][1];
    part[warp][g + 8][8 * j + 2 * t] = acc[j][2];
    part[warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();

  if (GATED) {
    const int half = N / 2;
    for (int i = threadIdx.x; i < TPB * 8 * M; i += LSM_THREADS) {
      const int tm = i / (8 * M);
      const int m = (i / 8) % M, rr = i % 8;
      const int n = (blockIdx.x * TPB + tm) * 8 + rr;
      if (n >= half) continue;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int s = 0; s < TEAM; ++s) {
        gate += part[tm * TEAM + s][rr][m];
        up += part[tm * TEAM + s][rr + 8][m];
      }
      reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * half + n] =
          __float2bfloat16_rn(gate_activation(act, gate) * up);
    }
    return;
  }
  // each team's 16 x M results: consecutive threads take consecutive weight rows (n)
  const bool partial = gridDim.y > 1;
  for (int i = threadIdx.x; i < TPB * 16 * M; i += LSM_THREADS) {
    const int tm = i / (16 * M);
    const int m = (i / 16) % M, rr = i % 16;
    const int n = (blockIdx.x * TPB + tm) * 16 + rr;
    if (n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < TEAM; ++s) v += part[tm * TEAM + s][rr][m];
    if (partial) {
      reinterpret_cast<float*>(out)[((size_t)blockIdx.y * M + m) * N + n] = v;
    } else {
      if (bias) v += bias[n];
      if (out_is_f32) reinterpret_cast<float*>(out)[(size_t)m * N + n] = v;
      else reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * N + n] = __float2bfloat16_rn(v);
    }
  }
}

template <int MT>
static int launch_small_m_gated(const void* x, const void* w, void* out, int M, int N, int K,
                                int act, cudaStream_t stream) {
  const int tiles = (N / 2 + 7) / 8;
  const int k_per_split = (K + 31) / 32 * 32;
  // two row tiles a block from 300 tiles on: with one, a feed-forward of a few thousand
  // outputs needs more blocks than the device holds at once and runs a second, short wave
  if constexpr (MT == 2) {
    if ((long long)N * K <= LSM_DENSE_ELEMENTS) {
      if (tiles >= 300)
        return launch_dependent(linear_small_m_kernel<MT, 2, true, true>, dim3((tiles + 1) / 2), dim3(LSM_THREADS),
                                0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                (const float*)nullptr, out, 0, M, N, K, k_per_split, act);
      return launch_dependent(linear_small_m_kernel<MT, 1, true, true>, dim3(tiles), dim3(LSM_THREADS), 0, stream,
                              (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const float*)nullptr, out,
                              0, M, N, K, k_per_split, act);
    }
  }
  if (tiles >= 300) {
    return launch_dependent(linear_small_m_kernel<MT, 2, true>, dim3((tiles + 1) / 2), dim3(LSM_THREADS),
                            0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                            (const float*)nullptr, out, 0, M, N, K, k_per_split, act);
  }
  return launch_dependent(linear_small_m_kernel<MT, 1, true>, dim3(tiles), dim3(LSM_THREADS), 0, stream,
                          (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const float*)nullptr, out,
                          0, M, N, K, k_per_split, act);
}

template <int MT>
static int launch_small_m(const void* x, const void* w, const float* bias, void* out,
                          int out_is_f32, int M, int N, int K, int k_splits,
                          cudaStream_t stream) {
  const int tiles = (N + 15) / 16;
  int k_per_split = (K + k_splits - 1) / k_splits;
  k_per_split = (k_per_split + 31) / 32 * 32;
  // many row tiles: two per block (teams of 4 warps); few: one per block (8 warps on its k)
  if constexpr (MT == 2) {
    if ((long long)N * K <= LSM_DENSE_ELEMENTS) {
      if (tiles >= 1024)
        return launch_dependent(linear_small_m_kernel<MT, 2, false, true>, dim3((tiles + 1) / 2, k_splits),
                                dim3(LSM_THREADS), 0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                bias, out, out_is_f32, M, N, K, k_per_split, 0);
      return launch_dependent(linear_small_m_kernel<MT, 1, false, true>, dim3(tiles, k_splits), dim3(LSM_THREADS),
                              0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, out, out_is_f32,
                              M, N, K, k_per_split, 0);
    }
  }
  if (tiles >= 1024) {
    dim3 grid((tiles + 1) / 2, k_splits);
    return launch_dependent(linear_small_m_kernel<MT, 2, false>, grid, dim3(LSM_THREADS), 0, stream,
                            (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, out, out_is_f32,
                            M, N, K, k_per_split, 0);
  }
  dim3 grid(tiles, k_splits);
  return launch_dependent(linear_small_m_kernel<MT, 1, false>, grid, dim3(LSM_THREADS), 0, stream,
                          (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, out, out_is_f32,
                          M, N, K, k_per_split, 0);
}

// out: [M, N] bfloat16 or float32 when k_splits == 1 (bias added); float32
// partial sums [k_splits, M, N] otherwise (no bias: the consumer adds them up).
TOKB200_API int tokb200_linear_small_m(const void* x, const void* w, const float* bias, void* out,
                                       int out_is_f32, int M, int N, int K, int k_splits,
                                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return TOKB200_OK;
  if (M > 64 || K <= 0 || K % 8 || k_splits < 1 || k_splits > 64) return TOKB200_BAD_SIZE;
  if (k_splits > 1 && (bias || !out_is_f32)) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TOKB200_BAD_ALIGNMENT;
  if (M <= 8) return launch_small_m<1>(x, w, bias, out, out_is_f32, M, N, K, k_splits, stream);
  if (M <= 16) return launch_small_m<2>(x, w, bias, out, out_is_f32, M, N, K, k_splits, stream);
  if (M <= 32) return launch_small_m<4>(x, w, bias, out, out_is_f32, M, N, K, k_splits, stream);
  return launch_small_m<8>(x, w, bias, out, out_is_f32, M, N, K, k_splits, stream);
}

// out[M, N/2] (bfloat16) = act(x Wg^T) * (x Wu^T), w in the 128-gate / 128-up row
// blocks described at the kernel (N a multiple of 256); `act` is the activation's tag.
TOKB200_API int tokb200_linear_small_m_gated(const void* x, const void* w, void* out, int M, int N,
                                             int K, int act, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return TOKB200_OK;
  if (M > 64 || K <= 0 || K % 8 || N % 256 || act < 0 || act >= TOKB200_ACT_COUNT) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TOKB200_BAD_ALIGNMENT;
  if (M <= 8) return launch_small_m_gated<1>(x, w, out, M, N, K, act, stream);
  if (M <= 16) return launch_small_m_gated<2>(x, w, out, M, N, K, act, stream);
  if (M <= 32) return launch_small_m_gated<4>(x, w, out, M, N, K, act, stream);
  return launch_small_m_gated<8>(x, w, out, M, N, K, act, stream);
}

// ----------------------------------------------------------------------------
// The query/key/value projection of a decoding step with everything that follows
// it folded into the epilogue: bias, the rotary encoding of q and k at each row's
// position, and the write of k and v into the row's cache slot.  w is the stacked
// [q heads; k heads; v heads] x K weight.  A row tile is 8 lanes j0 .. j0 + 7 of a
// head and their rotation partners j0 + d/2 .. (rows g and g + 8 of the mma), so a
// thread of the epilogue holds both halves of a pair.  The rotary width must be
// the whole head (d), d a multiple of 16.
// ----------------------------------------------------------------------------
// The residual sum and the norm in front of a projection, for kernels that compute them
// themselves (every block for all rows: a few KB): x' = x + pending (float32; the pending
// part is [M, K] bfloat16 or float32, or float32 partial sums [S, M, K], added in index order),
// h = x' / sqrt(mean(x'^2) + eps) * gain as bfloat16 rows in shared memory.
struct NormInput {
  const float* x;          // [M, K]
  float* x_out;            // [M, K]: x' (written by block 0)
  const void* delta;       // may be null
  int delta_is_f32, n_partials;
  long long partial_stride;
  const float* gain;
  float eps;
  int h_pitch;             // bytes between rows of h in shared memory
};

// One warp, one row of up to 1024 elements (K a multiple of 4): the row goes in two halves; a
// half's loads of x and of up to three partial sums are all asked for before the first is used.
__device__ __forceinline__ void norm_row_to_shared(const NormInput& in, int m, int K, int lane,
                                                   bool write_x, __nv_bfloat16* hrow) {
  constexpr int kVec = 8;
  const float* xr = in.x + (size_t)m * K;
  const float* df = reinterpret_cast<const float*>(in.delta) + (size_t)m * K;
  const __nv_bfloat16* dh = reinterpret_cast<const __nv_bfloat16*>(in.delta) + (size_t)m * K;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[kVec];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    constexpr int kHalf = kVec / 2;
    float4 a[3][kHalf];
    uint2 raw[kHalf];
#pragma unroll
    for (int e = 0; e < kHalf; ++e) {
      const int i = (lane + 32 * (half * kHalf + e)) * 4;
      const bool inside = i < K;
      v[half * kHalf + e] = inside ? *reinterpret_cast<const float4*>(xr + i) : zero4;
      raw[e] = make_uint2(0u, 0u);
      if (in.delta && !in.delta_is_f32 && inside) raw[e] = *reinterpret_cast<const uint2*>(dh + i);
#pragma unroll
      for (int s = 0; s < 3; ++s)
        a[s][e] = (in.delta && in.delta_is_f32 && s < in.n_partials && inside)
                      ? *reinterpret_cast<const float4*>(df + (size_t)s * in.partial_stride + i) : zero4;
    }
#pragma unroll
    for (int e = 0; e < kHalf; ++e) {
      float4& t4 = v[half * kHalf + e];
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[e].x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[e].y));
      t4.x += lo.x; t4.y += lo.y; t4.z += hi.x; t4.w += hi.y;
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        t4.x += a[s][e].x; t4.y += a[s][e].y; t4.z += a[s][e].z; t4.w += a[s][e].w;
      }
    }
    if (in.delta && in.delta_is_f32) {
      for (int s = 3; s < in.n_partials; ++s) {
#pragma unroll
        for (int e = 0; e < kHalf; ++e) {
          const int i = (lane + 32 * (half * kHalf + e)) * 4;
          if (i < K) {
            const float4 more = *reinterpret_cast<const float4*>(df + (size_t)s * in.partial_stride + i);
            float4& t4 = v[half * kHalf + e];
            t4.x += more.x; t4.y += more.y; t4.z += more.z; t4.w += more.w;
          }
        }
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < kVec; ++e) {
    ss += v[e].x * v[e].x + v[e].y * v[e].y + v[e].z * v[e].z + v[e].w * v[e].w;
    const int i = (lane + 32 * e) * 4;
    if (write_x && i < K) *reinterpret_cast<float4*>(in.x_out + (size_t)m * K + i) = v[e];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = 1.0f / sqrtf(ss / (float)K + in.eps);
#pragma unroll
  for (int e = 0; e < kVec; ++e) {
    const int i = (lane + 32 * e) * 4;
    if (i < K) {
      const float4 gn = *reinterpret_cast<const float4*>(in.gain + i);
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[e].x * inv * gn.x, v[e].y * inv * gn.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v[e].z * inv * gn.z, v[e].w * inv * gn.w);
      uint2 packed;
      packed.x = *reinterpret_cast<unsigned*>(&lo);
      packed.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(hrow + i) = packed;
    }
  }
}

// NORM: the kernel is handed the residual stream instead of normed rows and computes the
// norm itself (`x` is then unused): one launch and one trip through memory less per layer.
template <int MT, bool NORM>
__global__ void __launch_bounds__(LSM_THREADS)
qkv_rope_small_m_kernel(const NormInput norm, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                        const float* __restrict__ bias, const int* __restrict__ pos,
                        const int* __restrict__ slot, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ q_out,
                        __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int M,
                        int nh, int nkv, int d, int K) {
  __shared__ float part[LSM_WARPS][16][8 * MT + 1];
  extern __shared__ __align__(16) unsigned char qkv_h[];        // NORM: [8 MT][norm.h_pitch]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tiles_per_head = d / 16;
  const int head = blockIdx.x / tiles_per_head, j0 = (blockIdx.x % tiles_per_head) * 8;
  const int row_a = head * d + j0 + g, row_b = row_a + d / 2;

  float acc[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const __nv_bfloat16* wa = w + (size_t)row_a * K + 16 * t;
  const __nv_bfloat16* wb = w + (size_t)row_b * K + 16 * t;

  // steps of 64 k, a whole 128-byte line of a row per quad (see linear_small_m_kernel)
  constexpr int step = LSM_WARPS * 64;
  const int k_first = warp * 64;
  uint4 a_ring[LSM_WIDE_PRE][2], b_ring[LSM_WIDE_PRE][2];
#pragma unroll
  for (int i = 0; i < LSM_WIDE_PRE; ++i) {
    const int kk = k_first + i * step;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const bool k_ok = kk + 16 * t + 8 * h + 8 <= K;
      a_ring[i][h] = load16(wa + kk + 8 * h, k_ok);
      b_ring[i][h] = load16(wb + kk + 8 * h, k_ok);
    }
  }
  // What the epilogue needs from memory is asked for now, so that it has arrived by then
  // (thread i of the epilogue serves row m = i / 8 and lane pair j0 + i % 8), and before the
  // wait: positions and slots were written before the predecessor (the norm) started.
  constexpr int kEpi = (64 * MT + LSM_THREADS - 1) / LSM_THREADS;
  const int half = d / 2;
  float e_bias_a[kEpi], e_bias_b[kEpi], e_cos[kEpi], e_sin[kEpi];
  int e_slot[kEpi];
#pragma unroll
  for (int e = 0; e < kEpi; ++e) {
    const int i = threadIdx.x + e * LSM_THREADS;
    const int m = i / 8, j = j0 + i % 8;
    e_bias_a[e] = e_bias_b[e] = 0.f;
    e_cos[e] = 1.f;
    e_sin[e] = 0.f;
    e_slot[e] = -1;
    if (i < 8 * M) {
      if (bias) {
        e_bias_a[e] = bias[head * d + j];
        e_bias_b[e] = bias[head * d + j + half];
      }
      if (head >= nh && slot) e_slot[e] = slot[m];
      if (head < nh + nkv) {
        const int p = pos[m];
        e_cos[e] = cos_t[(size_t)p * half + j];
        e_sin[e] = sin_t[(size_t)p * half + j];
      }
    }
  }
  if (NORM && (int)threadIdx.x * 32 < K)       // the gain, first touched here in this step: towards L2 before the wait
    asm volatile("prefetch.global.L2 [%0];" ::"l"(norm.gain + threadIdx.x * 32));
  pdl_wait();
  pdl_launch();
  if (NORM) {
    for (int m = warp; m < 8 * MT; m += LSM_WARPS) {
      __nv_bfloat16* hrow = reinterpret_cast<__nv_bfloat16*>(qkv_h + (size_t)m * norm.h_pitch);
      if (m < M) norm_row_to_shared(norm, m, K, lane, blockIdx.x == 0, hrow);
      else for (int i = lane * 2; i < K; i += 64) *reinterpret_cast<unsigned*>(hrow + i) = 0u;
    }
    __syncthreads();
  }
  constexpr bool kXRing = MT <= 2 && !NORM;
  uint4 x_ring[kXRing ? LSM_WIDE_PRE : 1][MT][2];
  if (kXRing) {
#pragma unroll
    for (int i = 0; i < LSM_WIDE_PRE; ++i) {
      const int kk = k_first + i * step;
#pragma unroll
      for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          x_ring[i][j][h] = load16(x + (size_t)(8 * j + g) * K + kk + 16 * t + 8 * h,
                                   8 * j + g < M && kk + 16 * t + 8 * h + 8 <= K);
    }
  }
  for (int k = k_first; k < K; k += LSM_WIDE_PRE * step) {
#pragma unroll
    for (int i = 0; i < LSM_WIDE_PRE; ++i) {
      const int kk = k + i * step;
      const int kn = kk + LSM_WIDE_PRE * step;
      uint4 a[2], b[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        a[h] = a_ring[i][h];
        b[h] = b_ring[i][h];
        const bool next_ok = kn + 16 * t + 8 * h + 8 <= K;
        a_ring[i][h] = load16(wa + kn + 8 * h, next_ok);
        b_ring[i][h] = load16(wb + kn + 8 * h, next_ok);
      }
      if (kk < K) {
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const int m = 8 * j + g;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const bool k_ok = kk + 16 * t + 8 * h + 8 <= K;
            uint4 xv = make_uint4(0u, 0u, 0u, 0u);
            if (NORM) {
              if (k_ok) xv = *reinterpret_cast<const uint4*>(qkv_h + (size_t)m * norm.h_pitch + (kk + 16 * t + 8 * h) * 2);
            } else if (kXRing) {
              xv = x_ring[i][j][h];
              x_ring[i][j][h] = load16(x + (size_t)m * K + kn + 16 * t + 8 * h,
                                       m < M && kn + 16 * t + 8 * h + 8 <= K);
            } else {
              xv = load16(x + (size_t)m * K + kk + 16 * t + 8 * h, m < M && k_ok);
            }
            mma_bf16_16816(acc[j], a[h].x, b[h].x, a[h].y, b[h].y, xv.x, xv.y);
            mma_bf16_16816(acc[j], a[h].z, b[h].z, a[h].w, b[h].w, xv.z, xv.w);
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    part[warp][g][8 * j + 2 * t] = acc[j][0];
    part[warp][g][8 * j + 2 * t + 1] = acc[j][1];
    part[warp][g + 8][8 * j + 2 * t] = acc[j][2];
    part[warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();

#pragma unroll
  for (int e = 0; e < kEpi; ++e) {
    const int i = threadIdx.x + e * LSM_THREADS;
    if (i >= 8 * M) break;
    const int m = i / 8, rr = i % 8;
    const int j = j0 + rr;
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int s = 0; s < LSM_WARPS; ++s) {
      a += part[s][rr][m];
      b += part[s][rr + 8][m];
    }
    a += e_bias_a[e];
    b += e_bias_b[e];
    __nv_bfloat16* dst;
    if (head < nh) {
      dst = q_out + ((size_t)m * nh + head) * d;
    } else {
      const int s = e_slot[e];
      if (s < 0) continue;                                    // no cache write for this row
      const bool is_key = head < nh + nkv;
      __nv_bfloat16* pool = is_key ? k_pool : v_pool;
      if (!pool) continue;
      dst = pool + ((size_t)s * nkv + (head - nh - (is_key ? 0 : nkv))) * d;
    }
    if (head < nh + nkv) {                                    // values are not rotated: cos 1, sin 0
      const float ra = a * e_cos[e] - b * e_sin[e], rb = b * e_cos[e] + a * e_sin[e];
      a = ra;
      b = rb;
    }
    dst[j] = __float2bfloat16_rn(a);
    dst[j + half] = __float2bfloat16_rn(b);
  }
}

TOKB200_API int tokb200_qkv_rope_small_m(const void* x, const void* w, const float* bias, const int* pos,
                                         const int* slot, const float* cos_t, const float* sin_t,
                                         void* q_out, void* k_pool, void* v_pool, int M, int nh, int nkv,
                                         int d, int K, cudaStream_t stream) {
  if (M <= 0) return TOKB200_OK;
  if (M > 64 || K <= 0 || K % 8 || d <= 0 || d % 16 || nh <= 0 || nkv <= 0) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TOKB200_BAD_ALIGNMENT;
  const dim3 grid((nh + 2 * nkv) * (d / 16));
  const NormInput none = {};
#define LAUNCH_QKV(MT)                                                                              \
  return launch_dependent(qkv_rope_small_m_kernel<MT, false>, grid, dim3(LSM_THREADS), 0, stream,  \
                          none, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, pos, slot, cos_t, \
                          sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, \
                          M, nh, nkv, d, K)
  if (M <= 8) LAUNCH_QKV(1);
  if (M <= 16) LAUNCH_QKV(2);
  if (M <= 32) LAUNCH_QKV(4);
  LAUNCH_QKV(8);
#undef LAUNCH_QKV
}

// The same with the residual add and the RMS norm in front computed by the kernel itself:
// x_out = x + delta (delta as for the norm kernel: [M, K] or float32 partial sums [S, M, K], or
// null); the projection is taken of norm(x_out) * gain.  Up to 16 rows, K a multiple of 32 up to
// 1024.
TOKB200_API int tokb200_qkv_norm_rope_small_m(const float* x, float* x_out, const void* delta,
                                              int delta_is_f32, int n_partials, long long partial_stride,
                                              const float* gain, float eps, const void* w,
                                              const float* bias, const int* pos, const int* slot,
                                              const float* cos_t, const float* sin_t, void* q_out,
                                              void* k_pool, void* v_pool, int M, int nh, int nkv, int d,
                                              int K, cudaStream_t stream) {
  if (M <= 0) return TOKB200_OK;
  if (M > 16 || K <= 0 || K % 32 || K > 1024 || d <= 0 || d % 16 || nh <= 0 || nkv <= 0) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)x_out | (uintptr_t)w | (uintptr_t)delta | (uintptr_t)gain) & 15)
    return TOKB200_BAD_ALIGNMENT;
  NormInput norm;
  norm.x = x; norm.x_out = x_out; norm.delta = delta; norm.delta_is_f32 = delta_is_f32;
  norm.n_partials = n_partials; norm.partial_stride = partial_stride; norm.gain = gain; norm.eps = eps;
  norm.h_pitch = (2 * K + 127) / 128 * 128 + 64;      // 64 mod 128: rows g and g + 1 miss each other's banks
  const dim3 grid((nh + 2 * nkv) * (d / 16));
  const int MT = M <= 8 ? 1 : 2;
  const size_t smem = (size_t)8 * MT * norm.h_pitch;
  if (MT == 1)
    return launch_dependent(qkv_rope_small_m_kernel<1, true>, grid, dim3(LSM_THREADS), smem, stream, norm,
                            (const __nv_bfloat16*)nullptr, (const __nv_bfloat16*)w, bias, pos, slot, cos_t,
                            sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                            M, nh, nkv, d, K);
  return launch_dependent(qkv_rope_small_m_kernel<2, true>, grid, dim3(LSM_THREADS), smem, stream, norm,
                          (const __nv_bfloat16*)nullptr, (const __nv_bfloat16*)w, bias, pos, slot, cos_t,
                          sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                          M, nh, nkv, d, K);
}
