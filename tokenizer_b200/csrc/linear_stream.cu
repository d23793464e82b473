// y[M,N] = x[M,K] W[N,K]^T (+ bias) for few rows (M <= 16) and MANY weight rows (the
// vocabulary projection of a decoding step: a quarter of all bytes the step reads).
//
// One block per SM stays for the whole product.  A producer warp streams the block's
// tiles of 16 weight rows through a ring of shared-memory stages with bulk asynchronous
// copies (cp.async.bulk, completion on an mbarrier), always as far ahead as the stages
// allow; each consumer warp owns whole tiles (tile j of the block goes to warp j mod 7)
// and stages of its own, multiplies its tile out of the ring (mma.sync m16n8k16 with the weight rows as the M
// side, fragments by 16-byte shared loads under a permuted k, as in the kernel for single
// products) and writes the tile's results straight from its accumulators.  No two warps
// share a sum, so there is no barrier after the activations are staged, and the weight
// stream never drains between tiles.  Every wait is bounded; when one gives up an error
// flag is set, the role goes on to the end without touching the ring again, and the host
// reads the flag.
#include "common.cuh"

#define LS_WARPS 7                          // consumer warps (the host may let fewer multiply: p.warps)
#define LS_CONSUMERS (LS_WARPS * 32)
#define LS_THREADS (LS_CONSUMERS + 32)      // + the producer warp
#define LS_KC_MAX 1024                      // k elements of a stage: row pieces of up to 2 KB
#define LS_WAIT_LIMIT (1u << 16)            // polls of up to 20 us

__device__ int ls_error_flag = 0;

__device__ __forceinline__ unsigned ls_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ls_mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ls_smem(bar)), "r"(count));
}
__device__ __forceinline__ void ls_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ls_smem(bar)) : "memory");
}
__device__ __forceinline__ void ls_mbar_expect(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ls_smem(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool ls_mbar_wait(unsigned long long* bar, unsigned parity) {
  const unsigned addr = ls_smem(bar);
  const unsigned suspend_ns = 20000u;
  for (unsigned spin = 0; spin < LS_WAIT_LIMIT; ++spin) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity), "r"(suspend_ns) : "memory");
    if (done) return true;
  }
  atomicExch(&ls_error_flag, 1);
  tokb200_report_error(TOKB200_LIB_LINEAR_STREAM, 1);
  return false;
}
__device__ __forceinline__ void ls_bulk_copy(void* dst, const void* src, unsigned bytes,
                                             unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(ls_smem(dst)), "l"(src), "r"(bytes), "r"(ls_smem(bar)) : "memory");
}
__device__ __forceinline__ void ls_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct LsParams {
  const __nv_bfloat16* x;       // [M, K]
  const __nv_bfloat16* w;       // [N, K]
  const float* bias;            // [N] or null
  void* out;                    // [M, N] float32 or bfloat16
  int out_is_f32;
  int M, N, K;
  int n_stages, per_warp, warps, kc, row_pitch, stage_bytes, x_pitch;   // warps that multiply; n_stages = warps * per_warp
};

template <int MT>
__global__ void __launch_bounds__(LS_THREADS, 1)
linear_stream_kernel(const LsParams p) {
  extern __shared__ __align__(128) unsigned char ls_raw[];
  unsigned char* ring = ls_raw;
  unsigned char* x_s = ring + (size_t)p.n_stages * p.stage_bytes;        // [8 MT][x_pitch]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(x_s + (size_t)8 * MT * p.x_pitch);
  unsigned long long* empty = full + p.n_stages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int n_tiles = (p.N + 15) / 16;
  const int slabs = (p.K + p.kc - 1) / p.kc;
  // the block's tiles are a contiguous run: the weight stream of a block is one piece of memory
  const int per = (n_tiles + G - 1) / G;
  const int tile_first = cta * per, tile_last = min(n_tiles, tile_first + per);

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.n_stages; ++i) {
      ls_mbar_init(&full[i], 1);
      ls_mbar_init(&empty[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == LS_WARPS) {
    // ------------------------------ producer ------------------------------
    // Every consumer warp has stages of its own (p.per_warp of them), which only it waits on,
    // one use after the other: a barrier's parity tells two consecutive uses apart, no more,
    // so a stage must not be waited on by a warp that has not seen its uses before.
    // The order of the copies: a round of tiles (one per consumer warp), and within the round
    // slab by slab across the warps, so that every warp's stages are filled as it frees them
    // and all warps multiply at the same time (tile after tile, a tile of several slabs would
    // keep all warps but its owner waiting).
    bool ok = true;
    const int n_mine = tile_last - tile_first;
    for (int j0 = 0; j0 < n_mine && ok; j0 += p.warps) {
      for (int sl = 0; sl < slabs && ok; ++sl) {
        const int c = (j0 / p.warps) * slabs + sl;                    // an owner's stages filled so far
        const int k0 = sl * p.kc, kn = min(p.kc, p.K - k0);
        const unsigned bytes = (unsigned)kn * 2u;
        for (int owner = 0; owner < p.warps && j0 + owner < n_mine; ++owner) {
          const int tile = tile_first + j0 + owner;
          const int rows = min(16, p.N - tile * 16);
          const int stage = owner * p.per_warp + c % p.per_warp, use = c / p.per_warp;
          if (use > 0) ok = __all_sync(0xffffffffu, ls_mbar_wait(&empty[stage], (use - 1) & 1));
          if (!ok) break;
          if (lane == 0) ls_mbar_expect(&full[stage], (unsigned)rows * bytes);
          __syncwarp();
          if (lane < rows)
            ls_bulk_copy(ring + (size_t)stage * p.stage_bytes + lane * p.row_pitch,
                         p.w + (size_t)(tile * 16 + lane) * p.K + k0, bytes, &full[stage]);
        }
      }
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  pdl_wait();          // x comes from the predecessor; the weights above do not
  pdl_launch();
  const int g = lane >> 2, t = lane & 3;
  for (int i = threadIdx.x; i < 8 * MT * (p.K / 8); i += LS_CONSUMERS) {
    const int m = i / (p.K / 8), piece = i % (p.K / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (m < p.M) v = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + piece * 8);
    *reinterpret_cast<uint4*>(x_s + (size_t)m * p.x_pitch + piece * 16) = v;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(LS_CONSUMERS) : "memory");

  bool ok = true;
  for (int j = warp; warp < p.warps && tile_first + j < tile_last; j += p.warps) {
    const int tile = tile_first + j;
    float acc[MT][4];
#pragma unroll
    for (int q = 0; q < MT; ++q) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
    for (int sl = 0; sl < slabs; ++sl) {
      const int c = (j / p.warps) * slabs + sl;                       // this warp's stages used so far
      const int stage = warp * p.per_warp + c % p.per_warp, use = c / p.per_warp;
      ok = ok && __all_sync(0xffffffffu, ls_mbar_wait(&full[stage], use & 1));
      if (!ok) break;
      const unsigned char* st = ring + (size_t)stage * p.stage_bytes;
      const int k0 = sl * p.kc, kn = min(p.kc, p.K - k0);
      // rows of the tile past N were not copied: their sums are never written
#pragma unroll 4
      for (int s = 0; s * 32 < kn; ++s) {
        const uint4 a = *reinterpret_cast<const uint4*>(st + g * p.row_pitch + (s * 32 + 8 * t) * 2);
        const uint4 b = *reinterpret_cast<const uint4*>(st + (g + 8) * p.row_pitch + (s * 32 + 8 * t) * 2);
#pragma unroll
        for (int q = 0; q < MT; ++q) {
          const uint4 xv = *reinterpret_cast<const uint4*>(
              x_s + (size_t)(8 * q + g) * p.x_pitch + (k0 + s * 32 + 8 * t) * 2);
          ls_mma(acc[q], a.x, b.x, a.y, b.y, xv.x, xv.y);
          ls_mma(acc[q], a.z, b.z, a.w, b.w, xv.z, xv.w);
        }
      }
      __syncwarp();
      if (lane == 0) ls_mbar_arrive(&empty[stage]);
    }
    if (!ok) break;
    // accumulator layout: c0,c1 -> (weight row g, rows 2t, 2t+1 of x in tile q); c2,c3 -> weight row g + 8
#pragma unroll
    for (int q = 0; q < MT; ++q) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = tile * 16 + g + (e >> 1) * 8, m = 8 * q + 2 * t + (e & 1);
        if (n < p.N && m < p.M) {
          const float v = acc[q][e] + (p.bias ? p.bias[n] : 0.f);
          if (p.out_is_f32) reinterpret_cast<float*>(p.out)[(size_t)m * p.N + n] = v;
          else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

TOKB200_API int tokb200_linear_stream_error(void) {
  int flag = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&flag, ls_error_flag, sizeof(int)) != cudaSuccess) return -1;
  if (flag) cudaMemcpyToSymbol(ls_error_flag, &zero, sizeof(int));
  return flag;
}

struct LsPlan {
  int blocks, n_stages, per_warp, warps, kc, row_pitch, stage_bytes, x_pitch, smem_max;
  size_t smem;
};

static LsPlan ls_plan(int M, int N, int K) {
  LsPlan plan = {};
  if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K % 32 || K > 8192) return plan;
  int device = 0, sms = 0, smem_max = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return plan;
  const int MT = M <= 8 ? 1 : 2;
  const int x_pitch = (2 * K + 127) / 128 * 128 + 64;
  const size_t fixed = (size_t)8 * MT * x_pitch + 1024;
  const long long room = (long long)smem_max - 2048 - (long long)fixed;
  // the longest row piece (up to 2 KB) and the most consumer warps such that every warp has a
  // stage of its own, two if a tile takes more than one stage (else the warp would wait a whole
  // trip to memory between the pieces of a tile)
  int kc = (K + 63) / 64 * 64;
  if (kc > LS_KC_MAX) kc = LS_KC_MAX;
  int row_pitch = 0, stage_bytes = 0, per_warp = 0, warps = 0;
  for (;; kc = (kc / 2 + 63) / 64 * 64) {
    row_pitch = 2 * kc + 64;                  // 64 mod 128: 16-byte reads of 8 rows x 4 pieces miss each other's banks
    stage_bytes = 16 * row_pitch;
    const int fit = (int)(room / stage_bytes), slabs = (K + kc - 1) / kc;
    for (warps = LS_WARPS; warps >= 4; --warps) {
      per_warp = fit / warps;
      if (per_warp >= (slabs > 1 ? 2 : 1)) break;
    }
    if (warps >= 4 || kc == 64) break;
  }
  if (warps < 4 || per_warp < 1) return plan;
  if (per_warp > 4) per_warp = 4;
  const int stages = per_warp * warps;
  const int tiles = (N + 15) / 16;
  plan.blocks = tiles < sms ? tiles : sms;
  plan.n_stages = stages;
  plan.per_warp = per_warp;
  plan.warps = warps;
  plan.kc = kc;
  plan.row_pitch = row_pitch;
  plan.stage_bytes = stage_bytes;
  plan.x_pitch = x_pitch;
  plan.smem_max = smem_max;
  plan.smem = fixed + (size_t)stages * stage_bytes;
  return plan;
}

// 1 when the kernel takes the sizes on this device (M <= 16, K a multiple of 32 up to 8192).
TOKB200_API int tokb200_linear_stream_supported(int M, int N, int K) { return ls_plan(M, N, K).blocks > 0; }

TOKB200_API int tokb200_linear_stream(const void* x, const void* w, const float* bias, void* out,
                                      int out_is_f32, int M, int N, int K, cudaStream_t stream) {
  const LsPlan plan = ls_plan(M, N, K);
  if (plan.blocks == 0) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TOKB200_BAD_ALIGNMENT;
  LsParams p;
  p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = bias; p.out = out;
  p.out_is_f32 = out_is_f32; p.M = M; p.N = N; p.K = K;
  p.n_stages = plan.n_stages; p.per_warp = plan.per_warp; p.warps = plan.warps; p.kc = plan.kc; p.row_pitch = plan.row_pitch;
  p.stage_bytes = plan.stage_bytes; p.x_pitch = plan.x_pitch;
  void (*kernel)(const LsParams) = M <= 8 ? linear_stream_kernel<1> : linear_stream_kernel<2>;
  static bool configured[64][2] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!configured[device][M <= 8 ? 0 : 1]) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           plan.smem_max - 1024);
    if (err != cudaSuccess) return (int)err;
    configured[device][M <= 8 ? 0 : 1] = true;
  }
  return launch_dependent(kernel, dim3(plan.blocks), dim3(LS_THREADS), plan.smem, stream, p);
}
