// The whole gated feed-forward of a decoding step in ONE kernel, for few rows
// (M <= 16, bfloat16 weights, 32-bit sums):
//
//   x' = x + pending                      (the residual sum, 32-bit)
//   h  = rms_norm(x') * gain              (bfloat16)
//   a  = act(h Wg^T) * (h Wu^T)           (bfloat16, [M, I]; act by its tag, silu for the model served)
//   y  = a Wd^T as S partial sums over k  (32-bit, [S, M, H]; the next norm adds them)
//
// As separate kernels these are three launches whose time is mostly waiting: each
// starts cold, asks for its weights, waits a trip to memory, multiplies for a
// microsecond and leaves.  Here one block per SM stays for the whole feed-forward:
//   * a producer warp streams the block's share of BOTH weight matrices, in the order
//     they will be used, through a ring of shared-memory stages with bulk asynchronous
//     copies (cp.async.bulk, completion on an mbarrier).  It starts at once and never
//     waits for the arithmetic, so the weights of the second product are already
//     arriving while the first is computed and while the blocks meet at the barrier;
//   * eight consumer warps first compute the norm of all M rows (every block does this
//     for itself: M rows are a few KB), then multiply their row tiles of the gate/up
//     matrix out of the ring (mma.sync m16n8k16 with the weight rows as the M side, as
//     in the kernel for single products), apply the activation and write `a`;
//   * all blocks meet at a barrier in global memory (one block per SM: all are resident),
//     then multiply their (row tile, k range) units of the down
//     matrix and write the partial sums.
// Sums have a fixed order: results are reproducible.  Every wait (mbarrier, grid
// barrier) is bounded; when one gives up an error flag is set, the role goes on to
// the end without touching the ring again, and the host reads the flag.
//
// The gate/up matrix is in the row order of the gated kernels: for every 128 outputs,
// their 128 gate rows, then their 128 up rows.
#include "common.cuh"

#define FFN_WARPS 8                          // consumer warps
#define FFN_CONSUMERS (FFN_WARPS * 32)
#define FFN_THREADS (FFN_CONSUMERS + 32)     // + the producer warp
#define FFN_KC 1024                          // k elements of a stage: row pieces of up to 2 KB (the copy
                                             // engine takes some 45 cycles a copy, whatever its size)
#define FFN_ROW_PITCH (FFN_KC * 2 + 64)      // bytes between a stage's rows: 64 mod 128, so that
                                             // 16-byte reads of 8 rows x 4 pieces miss each other's banks
#define FFN_STAGE_BYTES (16 * FFN_ROW_PITCH)
// the bounds of the waits; a test build makes them small so that a wait that nothing ends runs out quickly
#ifndef FFN_WAIT_LIMIT
#define FFN_WAIT_LIMIT (1u << 16)            // polls of up to 20 us
#endif
#ifndef FFN_GRID_WAIT_LIMIT
#define FFN_GRID_WAIT_LIMIT (1u << 22)
#endif

__device__ int ffn_error_flag = 0;

__device__ __forceinline__ unsigned ffn_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ffn_mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ffn_smem(bar)), "r"(count));
}
__device__ __forceinline__ void ffn_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ffn_smem(bar)) : "memory");
}
__device__ __forceinline__ void ffn_mbar_expect(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ffn_smem(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool ffn_mbar_wait(unsigned long long* bar, unsigned parity) {
  const unsigned addr = ffn_smem(bar);
  const unsigned suspend_ns = 20000u;
  for (unsigned spin = 0; spin < FFN_WAIT_LIMIT; ++spin) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity), "r"(suspend_ns) : "memory");
    if (done) return true;
  }
  atomicExch(&ffn_error_flag, 1);
  tokb200_report_error(TOKB200_LIB_FFN_SMALL_M, 1);
  return false;
}
__device__ __forceinline__ void ffn_bulk_copy(void* dst, const void* src, unsigned bytes,
                                              unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(ffn_smem(dst)), "l"(src), "r"(bytes), "r"(ffn_smem(bar)) : "memory");
}
__device__ __forceinline__ void ffn_consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(FFN_CONSUMERS) : "memory");
}
__device__ __forceinline__ void ffn_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                        unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct FfnParams {
  const float* x_in;            // [M, H]
  float* x_out;                 // [M, H]: x + pending (written by block 0)
  const void* delta;            // pending: [M, H] bfloat16 or float32, or float32 [S, M, H]; may be null
  int delta_is_f32;
  int n_partials;
  long long partial_stride;     // elements between partial sums
  const float* gain;            // [H]
  float eps;
  const __nv_bfloat16* w_gu;    // [2 I, H], 128 gate rows / 128 up rows interleaved
  const __nv_bfloat16* w_d;     // [H, I]
  __nv_bfloat16* act;           // [M, I] scratch
  float* out;                   // [S_d, M, H] partial sums
  int M, H, I;
  int s_down, k_per_split;      // the down product's cut along k (k_per_split a multiple of 32)
  int n_stages;
  int act_pitch;                // bytes between rows of the activation tile in shared memory
  int activation;               // the gate's activation, by its tag
  int* sync;                    // [2] zero before the first launch; every launch leaves them zero
};

template <int MT>
__global__ void __launch_bounds__(FFN_THREADS, 1)
ffn_small_m_kernel(const FfnParams p) {
  extern __shared__ __align__(128) unsigned char ffn_raw[];
  unsigned char* ring = ffn_raw;
  unsigned char* h_s = ring + (size_t)p.n_stages * FFN_STAGE_BYTES;       // [8 MT][act_pitch]: h, later pieces of a
  float* part = reinterpret_cast<float*>(h_s + (size_t)8 * MT * p.act_pitch);   // [2][warps][16][8 MT + 1]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(part + 2 * FFN_WARPS * 16 * (8 * MT + 1));
  unsigned long long* empty = full + p.n_stages;
  __shared__ int grid_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int n_tiles_a = p.I / 8;                 // 8 outputs (8 gate rows + 8 up rows) a tile
  const int n_row_tiles_b = p.H / 16;
  // the down product: a block owns ONE k range (split = block mod S) and walks the row tiles
  // of that range with the other blocks of the same split, so it stages its columns of the
  // activation once
  const int split = cta % p.s_down;
  const int my_first_rt = cta / p.s_down;
  const int my_rt_step = (G - split + p.s_down - 1) / p.s_down;   // blocks that share this split
  const int k_begin = split * p.k_per_split, k_end = min(p.I, k_begin + p.k_per_split);

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.n_stages; ++i) {
      ffn_mbar_init(&full[i], 1);
      ffn_mbar_init(&empty[i], FFN_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    grid_ok = 1;
  }
  __syncthreads();

  if (warp == FFN_WARPS) {
    // ------------------------------ producer ------------------------------
    int c = 0;                                   // stages filled so far
    bool ok = true;
    auto fill = [&](const __nv_bfloat16* rows_lo, const __nv_bfloat16* rows_hi, int K, int k0, int kn) {
      // rows_lo: 8 consecutive rows of K elements (stage rows 0..7), rows_hi: stage rows 8..15
      const int stage = c % p.n_stages, use = c / p.n_stages;
      if (use > 0) ok = ok && __all_sync(0xffffffffu, ffn_mbar_wait(&empty[stage], (use - 1) & 1));
      if (ok) {
        const unsigned bytes = (unsigned)kn * 2u;
        if (lane == 0) ffn_mbar_expect(&full[stage], 16u * bytes);
        __syncwarp();
        if (lane < 16) {
          const __nv_bfloat16* src = (lane < 8 ? rows_lo + (size_t)lane * K : rows_hi + (size_t)(lane - 8) * K) + k0;
          ffn_bulk_copy(ring + (size_t)stage * FFN_STAGE_BYTES + lane * FFN_ROW_PITCH, src, bytes, &full[stage]);
        }
      }
      ++c;
    };
    for (int tile = cta; tile < n_tiles_a && ok; tile += G) {
      const int out0 = tile * 8;
      const __nv_bfloat16* gate = p.w_gu + (size_t)((out0 / 128) * 256 + out0 % 128) * p.H;
      for (int k0 = 0; k0 < p.H && ok; k0 += FFN_KC) fill(gate, gate + (size_t)128 * p.H, p.H, k0, min(FFN_KC, p.H - k0));
    }
    for (int rt = my_first_rt; rt < n_row_tiles_b && ok; rt += my_rt_step) {
      const __nv_bfloat16* rows = p.w_d + (size_t)rt * 16 * p.I;
      for (int k0 = k_begin; k0 < k_end && ok; k0 += FFN_KC)
        fill(rows, rows + (size_t)8 * p.I, p.I, k0, min(FFN_KC, k_end - k0));
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  // the gain is a constant of the layer, first touched here in this step: asked towards L2
  // before the wait, so that the norm does not pay a trip to DRAM after it
  if ((int)threadIdx.x * 32 < p.H) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.gain + threadIdx.x * 32));
  pdl_wait();          // x and the pending sums come from the predecessor; the weights above do not
  pdl_launch();
  const int g = lane >> 2, t = lane & 3;
  // ---- the norm of all rows: a warp per row, twice over the row (sum of squares, then values) ----
  for (int m = warp; m < 8 * MT; m += FFN_WARPS) {
    __nv_bfloat16* hrow = reinterpret_cast<__nv_bfloat16*>(h_s + (size_t)m * p.act_pitch);
    if (m >= p.M) {
      for (int i = lane * 2; i < p.H; i += 64) *reinterpret_cast<unsigned*>(hrow + i) = 0u;
      continue;
    }
    const float* xr = p.x_in + (size_t)m * p.H;
    constexpr int kVec = 8;                      // rows up to 32 * 4 * kVec wide stay in registers
    if (p.H <= 128 * kVec) {
      // a row goes in two halves; a half's loads of x and of up to three partial sums are
      // all asked for before the first is used (one trip to L2 a half, not one per array)
      float4 v[kVec];
      const float* df = reinterpret_cast<const float*>(p.delta) + (size_t)m * p.H;
      const __nv_bfloat16* dh = reinterpret_cast<const __nv_bfloat16*>(p.delta) + (size_t)m * p.H;
      const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        constexpr int kHalf = kVec / 2;
        float4 a[3][kHalf];
        uint2 raw[kHalf];
#pragma unroll
        for (int e = 0; e < kHalf; ++e) {
          const int i = (lane + 32 * (half * kHalf + e)) * 4;
          const bool in = i < p.H;
          v[half * kHalf + e] = in ? *reinterpret_cast<const float4*>(xr + i) : zero4;
          raw[e] = make_uint2(0u, 0u);
          if (p.delta && !p.delta_is_f32 && in) raw[e] = *reinterpret_cast<const uint2*>(dh + i);
#pragma unroll
          for (int s = 0; s < 3; ++s)
            a[s][e] = (p.delta && p.delta_is_f32 && s < p.n_partials && in)
                          ? *reinterpret_cast<const float4*>(df + (size_t)s * p.partial_stride + i) : zero4;
        }
#pragma unroll
        for (int e = 0; e < kHalf; ++e) {
          float4& t4 = v[half * kHalf + e];
          const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[e].x));
          const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[e].y));
          t4.x += lo.x; t4.y += lo.y; t4.z += hi.x; t4.w += hi.y;
#pragma unroll
          for (int s = 0; s < 3; ++s) {          // in index order, as the separate norm adds them
            t4.x += a[s][e].x; t4.y += a[s][e].y; t4.z += a[s][e].z; t4.w += a[s][e].w;
          }
        }
        // further partial sums, if a product was cut in more than three
        if (p.delta && p.delta_is_f32) {
          for (int s = 3; s < p.n_partials; ++s) {
#pragma unroll
            for (int e = 0; e < kHalf; ++e) {
              const int i = (lane + 32 * (half * kHalf + e)) * 4;
              if (i < p.H) {
                const float4 more = *reinterpret_cast<const float4*>(df + (size_t)s * p.partial_stride + i);
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
        if (cta == 0 && i < p.H) *reinterpret_cast<float4*>(p.x_out + (size_t)m * p.H + i) = v[e];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = 1.0f / sqrtf(ss / (float)p.H + p.eps);
#pragma unroll
      for (int e = 0; e < kVec; ++e) {
        const int i = (lane + 32 * e) * 4;
        if (i < p.H) {
          const float4 gn = *reinterpret_cast<const float4*>(p.gain + i);
          __nv_bfloat162 lo = __floats2bfloat162_rn(v[e].x * inv * gn.x, v[e].y * inv * gn.y);
          __nv_bfloat162 hi = __floats2bfloat162_rn(v[e].z * inv * gn.z, v[e].w * inv * gn.w);
          uint2 packed;
          packed.x = *reinterpret_cast<unsigned*>(&lo);
          packed.y = *reinterpret_cast<unsigned*>(&hi);
          *reinterpret_cast<uint2*>(hrow + i) = packed;
        }
      }
      continue;
    }
    auto value = [&](int i) {
      float a = xr[i];
      if (p.delta) {
        if (p.delta_is_f32) {
          const float* d = reinterpret_cast<const float*>(p.delta) + (size_t)m * p.H + i;
          for (int s = 0; s < p.n_partials; ++s) a += d[(size_t)s * p.partial_stride];
        } else {
          a += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.delta)[(size_t)m * p.H + i]);
        }
      }
      return a;
    };
    float ss = 0.f;
    for (int i = lane; i < p.H; i += 32) {
      const float a = value(i);
      ss += a * a;
      if (cta == 0) p.x_out[(size_t)m * p.H + i] = a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)p.H + p.eps);
    for (int i = lane; i < p.H; i += 32) hrow[i] = __float2bfloat16_rn(value(i) * inv * p.gain[i]);
  }
  ffn_consumer_sync();

  int c = 0;                                     // stages consumed so far
  bool ok = true;
  float acc[MT][4];
  // one stage: the warp takes the steps of 32 k that are its own (warp, warp + 8, ...)
  auto multiply = [&](int k_local0, int kn) {
    const int stage = c % p.n_stages, use = c / p.n_stages;
    ok = ok && __all_sync(0xffffffffu, ffn_mbar_wait(&full[stage], use & 1));
    if (ok) {
      const unsigned char* st = ring + (size_t)stage * FFN_STAGE_BYTES;
      for (int s = warp; s * 32 < kn; s += FFN_WARPS) {
        const uint4 a = *reinterpret_cast<const uint4*>(st + g * FFN_ROW_PITCH + (s * 32 + 8 * t) * 2);
        const uint4 b = *reinterpret_cast<const uint4*>(st + (g + 8) * FFN_ROW_PITCH + (s * 32 + 8 * t) * 2);
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const uint4 xv = *reinterpret_cast<const uint4*>(
              h_s + (size_t)(8 * j + g) * p.act_pitch + (k_local0 + s * 32 + 8 * t) * 2);
          ffn_mma(acc[j], a.x, b.x, a.y, b.y, xv.x, xv.y);
          ffn_mma(acc[j], a.z, b.z, a.w, b.w, xv.z, xv.w);
        }
      }
      __syncwarp();
      if (lane == 0) ffn_mbar_arrive(&empty[stage]);
    }
    ++c;
  };
  auto clear = [&]() {
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  };
  // accumulator layout: c0,c1 -> (row g, columns 2t, 2t+1 of rows 8 j ..); c2,c3 -> row g + 8
  // The warps' sums of a tile meet in one of two buffers, in turn: a thread that reads buffer
  // b for tile i has, by the barrier of tile i + 1, finished reading it, so tile i + 2 may
  // write it again, and one barrier a tile is enough.
  int turn = 0;
  constexpr int kPart = FFN_WARPS * 16 * (8 * MT + 1);
  auto spill = [&]() {
    float* mine = part + (size_t)turn * kPart + (size_t)warp * 16 * (8 * MT + 1);
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      mine[g * (8 * MT + 1) + 8 * j + 2 * t] = acc[j][0];
      mine[g * (8 * MT + 1) + 8 * j + 2 * t + 1] = acc[j][1];
      mine[(g + 8) * (8 * MT + 1) + 8 * j + 2 * t] = acc[j][2];
      mine[(g + 8) * (8 * MT + 1) + 8 * j + 2 * t + 1] = acc[j][3];
    }
  };
  auto summed = [&](int row, int m) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < FFN_WARPS; ++w) v += part[(size_t)turn * kPart + ((size_t)w * 16 + row) * (8 * MT + 1) + m];
    return v;
  };

  // ---- gate and up, activation ----
  for (int tile = cta; tile < n_tiles_a; tile += G) {
    clear();
    for (int k0 = 0; k0 < p.H; k0 += FFN_KC) multiply(k0, min(FFN_KC, p.H - k0));
    spill();
    ffn_consumer_sync();
    for (int i = threadIdx.x; i < 8 * p.M; i += FFN_CONSUMERS) {
      const int m = i / 8, rr = i % 8;
      const float gate = summed(rr, m), up = summed(rr + 8, m);
      p.act[(size_t)m * p.I + tile * 8 + rr] = __float2bfloat16_rn(gate_activation(p.activation, gate) * up);
    }
    turn ^= 1;
  }

  // ---- all blocks have written their part of the activation ----
  // (every consumer's writes of the activation are ordered before the arrival: a block barrier
  // first, then one thread's fence and atomic, whose release is cumulative over what it has seen)
  ffn_consumer_sync();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(&p.sync[0], 1);
    bool met = false;
    for (unsigned spin = 0; spin < FFN_GRID_WAIT_LIMIT; ++spin) {
      int seen;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.sync) : "memory");
      if (seen >= G) { met = true; break; }
      __nanosleep(64);
    }
    if (!met) {
      atomicExch(&ffn_error_flag, 2);
      tokb200_report_error(TOKB200_LIB_FFN_SMALL_M, 2);
      grid_ok = 0;
    }
    __threadfence();
  }
  ffn_consumer_sync();
  ok = ok && grid_ok;

  // ---- down: this block's k range of the activation, all rows, into shared memory (rows past M: zeros) ----
  if (my_first_rt < n_row_tiles_b) {
    for (int i = threadIdx.x; i < 8 * MT * (p.k_per_split / 8); i += FFN_CONSUMERS) {
      const int m = i / (p.k_per_split / 8), piece = i % (p.k_per_split / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (m < p.M && k_begin + piece * 8 < k_end)
        v = __ldcg(reinterpret_cast<const uint4*>(p.act + (size_t)m * p.I + k_begin + piece * 8));
      *reinterpret_cast<uint4*>(h_s + (size_t)m * p.act_pitch + piece * 16) = v;
    }
  }
  ffn_consumer_sync();
  for (int rt = my_first_rt; rt < n_row_tiles_b; rt += my_rt_step) {
    clear();
    for (int k0 = k_begin; k0 < k_end; k0 += FFN_KC) multiply(k0 - k_begin, min(FFN_KC, k_end - k0));
    spill();
    ffn_consumer_sync();
    for (int i = threadIdx.x; i < 16 * p.M; i += FFN_CONSUMERS) {
      const int m = i / 16, rr = i % 16;
      p.out[((size_t)split * p.M + m) * p.H + rt * 16 + rr] = summed(rr, m);
    }
    turn ^= 1;
  }

  // ---- the last block to leave makes the barrier ready for the next launch ----
  if (threadIdx.x == 0) {
    const int left = atomicAdd(&p.sync[1], 1);
    if (left == G - 1) {
      p.sync[0] = 0;
      p.sync[1] = 0;
      __threadfence();
    }
  }
}

TOKB200_API int tokb200_ffn_small_m_error(void) {
  int flag = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&flag, ffn_error_flag, sizeof(int)) != cudaSuccess) return -1;
  if (flag) cudaMemcpyToSymbol(ffn_error_flag, &zero, sizeof(int));
  return flag;
}

// The plan for sizes (M, H, I) on this device: blocks, cut of the down product, stages and
// shared memory; 0 blocks if the kernel does not take the sizes.
struct FfnPlan {
  int blocks, s_down, k_per_split, n_stages, act_pitch, smem_max;
  size_t smem;
};

static FfnPlan ffn_plan(int M, int H, int I) {
  FfnPlan plan = {};
  if (M <= 0 || M > 16 || H <= 0 || I <= 0 || H % 32 || I % 128) return plan;
  int device = 0, sms = 0, smem_max = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return plan;
  const int MT = M <= 8 ? 1 : 2;
  const int row_tiles = H / 16;
  // about two units of the down product a block
  int s = (2 * sms + row_tiles / 2) / row_tiles;
  if (s < 1) s = 1;
  if (s > 16) s = 16;
  int kps = ((I + s - 1) / s + 31) / 32 * 32;
  s = (I + kps - 1) / kps;
  const int widest = H > kps ? H : kps;
  const int pitch = (2 * widest + 127) / 128 * 128 + 64;
  const size_t fixed = (size_t)8 * MT * pitch + (size_t)2 * FFN_WARPS * 16 * (8 * MT + 1) * 4 + 1024;
  const long long room = (long long)smem_max - 2048 - (long long)fixed;
  int stages = (int)(room / FFN_STAGE_BYTES);
  if (stages > 8) stages = 8;
  // TOKB200_FFN_STAGES caps the ring (fewer stages leave shared memory for the blocks of the
  // kernels before this one, so that this kernel's blocks become resident, and its weights start
  // to stream, while those still run)
  static const int cap = [] {
    const char* v = getenv("TOKB200_FFN_STAGES");
    return v ? atoi(v) : 0;
  }();
  if (cap >= 3 && stages > cap) stages = cap;
  if (stages < 3) return plan;
  plan.blocks = sms;
  plan.s_down = s;
  plan.k_per_split = kps;
  plan.n_stages = stages;
  plan.act_pitch = pitch;
  plan.smem_max = smem_max;
  plan.smem = fixed + (size_t)stages * FFN_STAGE_BYTES;
  return plan;
}

// How many partial sums the output holds for these sizes (0: sizes not taken).
TOKB200_API int tokb200_ffn_small_m_splits(int M, int H, int I) { return ffn_plan(M, H, I).s_down; }

// x_out = x_in + delta; out[S, M, H] = partial sums of the feed-forward of norm(x_out).
// `sync` is two ints, zero before the first launch.  `act` is [M, I] bfloat16 scratch.
TOKB200_API int tokb200_ffn_small_m(const float* x_in, float* x_out, const void* delta, int delta_is_f32,
                                    int n_partials, long long partial_stride, const float* gain,
                                    float eps, const void* w_gu, const void* w_d, void* act, float* out,
                                    int M, int H, int I, int activation, int* sync, cudaStream_t stream) {
  const FfnPlan plan = ffn_plan(M, H, I);
  if (plan.blocks == 0 || activation < 0 || activation >= TOKB200_ACT_COUNT) return TOKB200_BAD_SIZE;
  if (((uintptr_t)w_gu | (uintptr_t)w_d | (uintptr_t)act) & 15) return TOKB200_BAD_ALIGNMENT;
  FfnParams p;
  p.x_in = x_in; p.x_out = x_out; p.delta = delta; p.delta_is_f32 = delta_is_f32;
  p.n_partials = n_partials; p.partial_stride = partial_stride; p.gain = gain; p.eps = eps;
  p.w_gu = (const __nv_bfloat16*)w_gu; p.w_d = (const __nv_bfloat16*)w_d;
  p.act = (__nv_bfloat16*)act; p.out = out; p.M = M; p.H = H; p.I = I;
  p.s_down = plan.s_down; p.k_per_split = plan.k_per_split; p.n_stages = plan.n_stages;
  p.act_pitch = plan.act_pitch; p.sync = sync; p.activation = activation;
  void (*kernel)(const FfnParams) = M <= 8 ? ffn_small_m_kernel<1> : ffn_small_m_kernel<2>;
  static bool configured[64][2] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!configured[device][M <= 8 ? 0 : 1]) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_max - 1024);
    if (err != cudaSuccess) return (int)err;
    configured[device][M <= 8 ? 0 : 1] = true;
  }
  // One block per SM, each with most of an SM's shared memory: all blocks become resident as
  // the predecessor's blocks leave (they wait for nothing of ours), so the barrier between
  // the products is met; its wait is bounded all the same.  Launched like the step's other
  // kernels: it may start, and stream weights, while its predecessor still runs.
  return launch_dependent(kernel, dim3(plan.blocks), dim3(FFN_THREADS), plan.smem, stream, p);
}
