// y[M,N] = x[M,K] W[N,K]^T (+ bias) for many rows (portions of prompts), bfloat16
// operands, 32-bit accumulation, on the fifth-generation tensor cores of sm_100a:
//
//   * TMA (cp.async.bulk.tensor) brings 128 x 64 tiles of x and BLOCK_N x 64 tiles
//     of W into shared memory in the 128-byte swizzled layout, STAGES deep, each
//     stage guarded by a "full" mbarrier (armed with the bytes to arrive) and an
//     "empty" mbarrier;
//   * one thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BLOCK_N,
//     K = 16, both operands K-major from shared-memory descriptors); the 128 x
//     BLOCK_N float accumulator lives in tensor memory (TMEM); tcgen05.commit
//     releases a stage when the instructions that read it have finished, and
//     signals the epilogue after the last one;
//   * four epilogue warps read the accumulator back with tcgen05.ld (each warp its
//     quarter of the 128 lanes), add the bias, convert and store.
//
// Warp roles: warp 0 loads, warp 1 allocates TMEM and issues the products, warps
// 2..5 are the epilogue.  In these forms no operand tile is shared between CTAs; the
// persistent kernel further down also has a form in which two CTAs of a cluster work
// on one tile (cta_group::2), each loading half of the W tile - still without any
// multicast load.  Rows and columns past M, N or K are zero-filled by TMA and masked
// at the store.  Every wait on an mbarrier is bounded: when it runs out the
// thread records an error flag, and all roles fall through to the common exit,
// where TMEM is given back.
#include <cuda.h>

#include "common.cuh"

#define TC_BLOCK_M 128
#define TC_BLOCK_K 64          // 64 bfloat16 = 128 bytes = one swizzle row
#define TC_UMMA_K 16
#define TC_THREADS 192
#define TC_WAIT_LIMIT (1u << 17)      // polls of up to 20 us each: seconds in all

__device__ int tc_error_flag = 0;   // set when a bounded wait gave up

__device__ __forceinline__ unsigned tc_smem(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem(bar)), "r"(bytes)
               : "memory");
}
// Waits for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
  const unsigned addr = tc_smem(bar);
  // the thread sleeps in hardware until the phase completes or the hint runs out, so
  // waiting warps do not take issue slots from working ones
  const unsigned suspend_ns = 20000u;
  for (unsigned spin = 0; spin < TC_WAIT_LIMIT; ++spin) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity), "r"(suspend_ns) : "memory");
    if (done) return true;
  }
  atomicExch(&tc_error_flag, 1);
  tokb200_report_error(TOKB200_LIB_GEMM_TCGEN05, 1);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, unsigned long long* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(tc_smem(dst)), "l"(map), "r"(tc_smem(bar)), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptor: K-major tile with 128-byte swizzle, rows of 128
// bytes, 8-row groups 1024 bytes apart (sm_100 descriptor version 1).
__device__ __forceinline__ unsigned long long umma_desc(const void* tile) {
  const unsigned long long addr = (tc_smem(tile) & 0x3FFFFu) >> 4;
  return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long a_desc,
                                          unsigned long long b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(tc_smem(bar)) : "memory");
}
__device__ __forceinline__ void tmem_wait_loads() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// the same load without the wait: the caller waits once for several loads
__device__ __forceinline__ void tmem_load_32_async(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
      "%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_load_32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
      "%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int BLOCK_N, int STAGES>
struct TcSmem {
  static constexpr int kABytes = TC_BLOCK_M * TC_BLOCK_K * 2;
  static constexpr int kBBytes = BLOCK_N * TC_BLOCK_K * 2;
  static constexpr int kStage = kABytes + kBBytes;
  static constexpr int kTotal = STAGES * kStage + 1024 /* alignment slack */ + 256 /* barriers */;
};

template <int BLOCK_N, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, void* __restrict__ out, int out_is_f32, int M,
                    int N, int K) {
  using S = TcSmem<BLOCK_N, STAGES>;
  extern __shared__ unsigned char tc_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);        // swizzle atoms: 1024-aligned
  unsigned long long* full = reinterpret_cast<unsigned long long*>(tiles + STAGES * S::kStage);
  unsigned long long* empty = full + STAGES;
  unsigned long long* accum_ready = empty + STAGES;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(accum_ready + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * TC_BLOCK_M, n0 = blockIdx.y * BLOCK_N;
  const int k_blocks = (K + TC_BLOCK_K - 1) / TC_BLOCK_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(accum_ready, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // one warp allocates the accumulator's columns of tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(tc_smem(tmem_slot)), "r"((unsigned)BLOCK_N) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  pdl_wait();      // x may be the predecessor's output

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: fill the ring ----
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1)) break;
        unsigned char* a_tile = tiles + s * S::kStage;
        mbar_expect_tx(&full[s], S::kStage);
        tma_load_2d(a_tile, &map_x, &full[s], kb * TC_BLOCK_K, m0);
        tma_load_2d(a_tile + S::kABytes, &map_w, &full[s], kb * TC_BLOCK_K, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- products: D[128 x BLOCK_N] (+)= A[128 x 16] B[BLOCK_N x 16]^T, four per stage ----
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BLOCK_N >> 3) << 17) |
                             ((unsigned)(TC_BLOCK_M >> 4) << 24);
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(&full[s], (kb / STAGES) & 1)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* a_tile = tiles + s * S::kStage;
        const unsigned long long a_desc = umma_desc(a_tile), b_desc = umma_desc(a_tile + S::kABytes);
#pragma unroll
        for (int k = 0; k < TC_BLOCK_K / TC_UMMA_K; ++k) {
          // 16 bfloat16 = 32 bytes along K inside the swizzled row: +2 in units of 16 bytes
          umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
        }
        umma_commit(&empty[s]);            // the stage is free once these products have read it
      }
      umma_commit(accum_ready);            // all products done: the accumulator is complete
    }
  } else {
    // ---- epilogue: warp w reads lanes 32 (w % 4) .. + 31 of the accumulator ----
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    if (mbar_wait(accum_ready, 0)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < BLOCK_N; c0 += 32) {
        unsigned v[32];
        tmem_load_32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, v);
        const int col0 = n0 + c0;
        if (row < M && col0 < N) {
          if (out_is_f32) {
            float* dst = reinterpret_cast<float*>(out) + (size_t)row * N + col0;
            if (col0 + 32 <= N && (N & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o;
                o.x = __uint_as_float(v[j]) + (bias ? bias[col0 + j] : 0.f);
                o.y = __uint_as_float(v[j + 1]) + (bias ? bias[col0 + j + 1] : 0.f);
                o.z = __uint_as_float(v[j + 2]) + (bias ? bias[col0 + j + 2] : 0.f);
                o.w = __uint_as_float(v[j + 3]) + (bias ? bias[col0 + j + 3] : 0.f);
                *reinterpret_cast<float4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j)
                dst[j] = __uint_as_float(v[j]) + (bias ? bias[col0 + j] : 0.f);
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + col0;
            if (col0 + 32 <= N && (N & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                unsigned* ow = reinterpret_cast<unsigned*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float lo = __uint_as_float(v[j + 2 * e]) + (bias ? bias[col0 + j + 2 * e] : 0.f);
                  const float hi = __uint_as_float(v[j + 2 * e + 1]) + (bias ? bias[col0 + j + 2 * e + 1] : 0.f);
                  __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
                  ow[e] = *reinterpret_cast<unsigned*>(&pair);
                }
                *reinterpret_cast<uint4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j)
                dst[j] = __float2bfloat16_rn(__uint_as_float(v[j]) + (bias ? bias[col0 + j] : 0.f));
            }
          }
        }
      }
    }
  }
  // ---- common exit: everybody arrives, then tensor memory is given back ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  pdl_launch();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((unsigned)BLOCK_N) : "memory");
  }
}

// ----------------------------------------------------------------------------
// The persistent form, for outputs whose row pitch is a multiple of 16 bytes: one
// CTA per SM walks output tiles (tile t = blockIdx.x + i * gridDim.x, m fastest so
// that CTAs running side by side share a tile of W in L2).  The accumulator is
// double-buffered in tensor memory (2 x BLOCK_N columns), so the epilogue of a
// tile overlaps the products of the next; the epilogue stages the tile in shared
// memory (128-byte swizzled slabs) and writes it with TMA stores, which also clip
// what lies past M and N.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(bar)) : "memory");
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(tc_smem(src)), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(tc_smem(src)), "r"(x), "r"(y), "r"(z) : "memory");
}

// ---- two CTAs on one tile (cta_group::2) ----------------------------------------
// A pair of CTAs (a cluster of two, on the two SMs of one TPC) works on a tile of 256 rows x
// BLOCK_N columns: each CTA loads its 128 rows of x and HALF of the tile's rows of W, the even
// CTA's thread issues products of M = 256 that read both halves of W, and each CTA's tensor
// memory gets the accumulator of its own 128 rows.  A k block then costs each SM 32 KB of
// shared-memory fill for 512 cycles of products (BLOCK_N = 256) where a lone CTA needs 48 KB,
// which is what the fill rate from L2 allows.
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's window, of the same shared-memory location in CTA 0 of the pair
__device__ __forceinline__ unsigned leader_address(const void* p) {
  unsigned a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(tc_smem(p)), "r"(0u));
  return a;
}
// a load into this CTA's shared memory whose bytes are counted on a barrier of the pair's CTA 0
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, unsigned leader_bar,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(tc_smem(dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long a_desc,
                                               unsigned long long b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this offset in BOTH CTAs of the pair once the products issued so far are done
__device__ __forceinline__ void umma_commit_pair(unsigned long long* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(tc_smem(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}
// the bounded wait, acquiring at cluster scope (arrivals come from the other CTA of the pair)
__device__ __forceinline__ bool mbar_wait_cluster(unsigned long long* bar, unsigned parity) {
  const unsigned addr = tc_smem(bar);
  const unsigned suspend_ns = 20000u;
  for (unsigned spin = 0; spin < TC_WAIT_LIMIT; ++spin) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity), "r"(suspend_ns) : "memory");
    if (done) return true;
  }
  atomicExch(&tc_error_flag, 2);
  tokb200_report_error(TOKB200_LIB_GEMM_TCGEN05, 2);
  return false;
}

template <int BLOCK_N, int STAGES, bool OUT_F32, bool GATED = false, bool PAIR = false>
struct TcPersistentSmem {
  static constexpr int kABytes = TC_BLOCK_M * TC_BLOCK_K * 2;
  static constexpr int kBBytes = (PAIR ? BLOCK_N / 2 : BLOCK_N) * TC_BLOCK_K * 2;
  static constexpr int kStage = kABytes + kBBytes;
  static constexpr int kSlabCols = OUT_F32 ? 32 : 64;                  // 128 bytes of output
  // slabs staged at a time: the gated tile has 128 output columns; the pair's 256-column
  // 32-bit tile goes out in two passes of 128 columns
  static constexpr int kSlabs = GATED ? 2 : ((PAIR && OUT_F32 && BLOCK_N == 256) ? 4 : BLOCK_N / kSlabCols);
  static constexpr int kPassCols = GATED ? BLOCK_N : kSlabs * kSlabCols;   // accumulator columns a pass
  static constexpr int kSlabBytes = TC_BLOCK_M * 128;
  static constexpr int kOutBytes = kSlabs * kSlabBytes;
  static constexpr int kTotal = STAGES * kStage + kOutBytes + 1024 + 256;
};

// What the epilogues need besides the product.  QKV: each row's position and cache slot, the
// rotary tables, the key/value pools and the head geometry.  GATED: the activation's tag.
struct QkvEpilogue {
  int activation;               // the gated epilogue's activation (TOKB200_ACT_*)
  const int* pos;
  const int* slot;              // may be null: no cache write
  const float* cos_t;
  const float* sin_t;           // [positions, d / 2]
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;        // [slots, nkv, d]; may be null
  int nh, nkv, d;
};

// GATED: the weight rows come in blocks of 256 = 128 "gate" rows followed by the 128
// "up" rows of the same outputs; the epilogue writes silu(gate) * up, 128 columns a
// tile, and the 2 N wide product never goes to memory.
// QKV: w is the stacked [q heads; k heads; v heads] weight; the epilogue adds the bias, rotates
// q and k by each row's position (half-split pairs (j, j + d/2), the whole head) and writes q to
// its matrix (TMA store) and k and v to the rows' cache slots, so the stacked product never goes
// to memory.  Tiles of 128 columns hold whole heads (d = 64 or 128) of one kind.
template <int BLOCK_N, int STAGES, bool OUT_F32, bool GATED, bool QKV = false, bool PAIR = false>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_x,
                               const __grid_constant__ CUtensorMap map_w,
                               const __grid_constant__ CUtensorMap map_out,
                               const float* __restrict__ bias, int M, int N, int K, int k_splits,
                               const QkvEpilogue qkv) {
  static_assert(!QKV || (BLOCK_N == 128 && !OUT_F32 && !GATED), "the QKV epilogue works on 128-column bfloat16 tiles");
  // k_splits > 1 (32-bit output only): a unit of work is (tile, piece of k); the output is
  // [k_splits, M, N] partial sums that the consumer adds in index order, written through a
  // three-dimensional map so that a tile's rows past M fall outside its piece's plane.
  using S = TcPersistentSmem<BLOCK_N, STAGES, OUT_F32, GATED, PAIR>;
  static_assert(!GATED || (BLOCK_N == 256 && !OUT_F32), "the gated epilogue pairs two halves of a 256 tile");
  static_assert(!PAIR || !QKV, "the QKV epilogue has no pair form");
  // PAIR: the grid is clusters of two CTAs; a tile has 256 rows, of which this CTA owns 128
  constexpr int kTileM = PAIR ? 2 * TC_BLOCK_M : TC_BLOCK_M;
  const int rank = PAIR ? (int)cluster_rank() : 0;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ unsigned char tc_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* staging = tiles + STAGES * S::kStage;                 // 1024-aligned as well
  unsigned long long* full = reinterpret_cast<unsigned long long*>(staging + S::kOutBytes);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_full = empty + STAGES;
  unsigned long long* acc_empty = acc_full + 2;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + kTileM - 1) / kTileM;
  const int n_tiles = (N + BLOCK_N - 1) / BLOCK_N;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + TC_BLOCK_K - 1) / TC_BLOCK_K;
  const int kb_per_split = (k_blocks + k_splits - 1) / k_splits;
  const int total_units = total_tiles * k_splits;

  if (threadIdx.x == 0) {
    // PAIR: the loads of both CTAs count on CTA 0's "full"; a commit arrives on "empty" and
    // "acc_full" of both; the epilogue warps of both CTAs arrive on CTA 0's "acc_empty"
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], PAIR ? 8 : 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {      // the warps of both CTAs take part: the same columns in both tensor memories
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(tc_smem(tmem_slot)), "r"((unsigned)(2 * BLOCK_N)) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(tc_smem(tmem_slot)), "r"((unsigned)(2 * BLOCK_N)) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if (PAIR) cluster_sync_all();        // the other CTA's barriers are ready before anything arrives there
  else __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;                                   // k blocks issued so far, over all tiles
      bool ok = true;
      for (int unit = worker; ok && unit < total_units; unit += workers) {
        const int tile = unit % total_tiles, split = unit / total_tiles;
        const int m0 = (tile % m_tiles) * kTileM + rank * TC_BLOCK_M;
        const int n0 = (tile / m_tiles) * BLOCK_N + (PAIR ? rank * (BLOCK_N / 2) : 0);
        const int kb_end = min(k_blocks, (split + 1) * kb_per_split);
        for (int kb = split * kb_per_split; kb < kb_end; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) { ok = false; break; }   // fresh barriers pass
          unsigned char* a_tile = tiles + s * S::kStage;
          if (PAIR) {
            if (rank == 0) mbar_expect_tx(&full[s], 2 * S::kStage);      // the bytes of both CTAs
            const unsigned bar = leader_address(&full[s]);
            tma_load_2d_pair(a_tile, &map_x, bar, kb * TC_BLOCK_K, m0);
            tma_load_2d_pair(a_tile + S::kABytes, &map_w, bar, kb * TC_BLOCK_K, n0);
          } else {
            mbar_expect_tx(&full[s], S::kStage);
            tma_load_2d(a_tile, &map_x, &full[s], kb * TC_BLOCK_K, m0);
            tma_load_2d(a_tile + S::kABytes, &map_w, &full[s], kb * TC_BLOCK_K, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {        // PAIR: CTA 0's thread issues for both
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BLOCK_N >> 3) << 17) |
                             ((unsigned)(kTileM >> 4) << 24);
      int it = 0, round = 0;
      bool ok = true;
      for (int unit = worker; ok && unit < total_units; unit += workers, ++round) {
        const int split = unit / total_tiles;
        const int kb_begin = split * kb_per_split, kb_end = min(k_blocks, kb_begin + kb_per_split);
        const int buf = round & 1;
        // the epilogue (of both CTAs) has drained it
        if (!(PAIR ? mbar_wait_cluster(&acc_empty[buf], ((round >> 1) & 1) ^ 1)
                   : mbar_wait(&acc_empty[buf], ((round >> 1) & 1) ^ 1))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned tmem_d = tmem_base + (unsigned)(buf * BLOCK_N);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % STAGES;
          if (!(PAIR ? mbar_wait_cluster(&full[s], (it / STAGES) & 1) : mbar_wait(&full[s], (it / STAGES) & 1))) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* a_tile = tiles + s * S::kStage;
          const unsigned long long a_desc = umma_desc(a_tile), b_desc = umma_desc(a_tile + S::kABytes);
#pragma unroll
          for (int k = 0; k < TC_BLOCK_K / TC_UMMA_K; ++k) {
            if (PAIR) umma_bf16_pair(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, ((kb - kb_begin) | k) != 0);
            else umma_bf16(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, ((kb - kb_begin) | k) != 0);
          }
          if (PAIR) umma_commit_pair(&empty[s]);
          else umma_commit(&empty[s]);
        }
        if (PAIR) umma_commit_pair(&acc_full[buf]);
        else umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;              // this thread's row of the tile
    const bool issuer = warp == 2 && lane == 0;     // the thread that issues the TMA stores
    int round = 0;
    for (int unit = worker; unit < total_units; unit += workers, ++round) {
      const int tile = unit % total_tiles, split = unit / total_tiles;
      const int m0 = (tile % m_tiles) * kTileM + rank * TC_BLOCK_M, n0 = (tile / m_tiles) * BLOCK_N;
      const int buf = round & 1;
      if (!mbar_wait(&acc_full[buf], (round >> 1) & 1)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c_base = 0; c_base < BLOCK_N; c_base += S::kPassCols) {    // the tile in passes of staged columns
      // the stores of the previous pass or tile must have read the staging area
      if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      epilogue_barrier();
      if (QKV) {
        const int row = m0 + r;
        const bool row_ok = row < M;
        const int d = qkv.d, half = d / 2;
        const int q_cols = qkv.nh * d, k_cols = qkv.nkv * d;
        const int kind = n0 < q_cols ? 0 : (n0 < q_cols + k_cols ? 1 : 2);      // q, k, v
        const int p = row_ok ? qkv.pos[row] : 0;
        const int sl = (row_ok && qkv.slot) ? qkv.slot[row] : -1;
        const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BLOCK_N);
#pragma unroll 1
        for (int h0 = 0; h0 < 128; h0 += d) {                 // the heads of this tile
#pragma unroll 1
          for (int j0 = 0; j0 < half; j0 += 32) {             // 32 lanes and their partners
            unsigned a[32], b[32];
            tmem_load_32_async(lane_base + (unsigned)(h0 + j0), a);
            tmem_load_32_async(lane_base + (unsigned)(h0 + half + j0), b);
            tmem_wait_loads();
            float fa[32], fb[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              fa[i] = __uint_as_float(a[i]) + (bias ? bias[n0 + h0 + j0 + i] : 0.f);
              fb[i] = __uint_as_float(b[i]) + (bias ? bias[n0 + h0 + half + j0 + i] : 0.f);
            }
            if (kind != 2 && row_ok) {
              const float4* c4 = reinterpret_cast<const float4*>(qkv.cos_t + (size_t)p * half + j0);
              const float4* s4 = reinterpret_cast<const float4*>(qkv.sin_t + (size_t)p * half + j0);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 c = c4[i], sn = s4[i];
                const float cs[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float ra = fa[4 * i + e] * cs[e] - fb[4 * i + e] * ss[e];
                  const float rb = fb[4 * i + e] * cs[e] + fa[4 * i + e] * ss[e];
                  fa[4 * i + e] = ra;
                  fb[4 * i + e] = rb;
                }
              }
            }
            uint4 oa[4], ob[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              unsigned* wa = reinterpret_cast<unsigned*>(&oa[j]);
              unsigned* wb = reinterpret_cast<unsigned*>(&ob[j]);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 pa = __floats2bfloat162_rn(fa[8 * j + 2 * e], fa[8 * j + 2 * e + 1]);
                __nv_bfloat162 pb = __floats2bfloat162_rn(fb[8 * j + 2 * e], fb[8 * j + 2 * e + 1]);
                wa[e] = *reinterpret_cast<unsigned*>(&pa);
                wb[e] = *reinterpret_cast<unsigned*>(&pb);
              }
            }
            if (kind == 0) {
              // into the staging slabs (64 columns each, 128-byte swizzled rows) for the TMA store
              const int ca = h0 + j0, cb = h0 + half + j0;
              unsigned char* slab_a = staging + (ca / 64) * S::kSlabBytes + r * 128;
              unsigned char* slab_b = staging + (cb / 64) * S::kSlabBytes + r * 128;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                *reinterpret_cast<uint4*>(slab_a + ((((ca / 32) % 2) * 4 + j) ^ (r & 7)) * 16) = oa[j];
                *reinterpret_cast<uint4*>(slab_b + ((((cb / 32) % 2) * 4 + j) ^ (r & 7)) * 16) = ob[j];
              }
            } else {
              __nv_bfloat16* pool = kind == 1 ? qkv.k_pool : qkv.v_pool;
              if (row_ok && sl >= 0 && pool) {
                const int kv_head = (n0 + h0 - q_cols - (kind == 2 ? k_cols : 0)) / d;
                __nv_bfloat16* dst = pool + ((size_t)sl * qkv.nkv + kv_head) * d;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  *reinterpret_cast<uint4*>(dst + j0 + 8 * j) = oa[j];
                  *reinterpret_cast<uint4*>(dst + half + j0 + 8 * j) = ob[j];
                }
              }
            }
          }
        }
      } else if (GATED) {
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
          unsigned gate[32], up[32];
          const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BLOCK_N);
          tmem_load_32_async(lane_base + (unsigned)c0, gate);
          tmem_load_32_async(lane_base + (unsigned)(128 + c0), up);
          tmem_wait_loads();
          unsigned char* slab = staging + (c0 / 64) * S::kSlabBytes + r * 128;
          const int piece0 = (c0 / 32 % 2) * 4;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            unsigned* ow = reinterpret_cast<unsigned*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float g0 = __uint_as_float(gate[8 * j + 2 * e]), g1 = __uint_as_float(gate[8 * j + 2 * e + 1]);
              const float u0 = __uint_as_float(up[8 * j + 2 * e]), u1 = __uint_as_float(up[8 * j + 2 * e + 1]);
              // silu in 32-bit with the fast exponential and reciprocal (a few ulp,
              // far below the bfloat16 rounding of the result); another activation by its tag
              const bool silu = qkv.activation == TOKB200_ACT_SILU;     // uniform over the grid
              const float a0 = silu ? __fdividef(g0, 1.0f + __expf(-g0)) : gate_activation(qkv.activation, g0);
              const float a1 = silu ? __fdividef(g1, 1.0f + __expf(-g1)) : gate_activation(qkv.activation, g1);
              __nv_bfloat162 pair = __floats2bfloat162_rn(a0 * u0, a1 * u1);
              ow[e] = *reinterpret_cast<unsigned*>(&pair);
            }
            *reinterpret_cast<uint4*>(slab + (((piece0 + j) ^ (r & 7)) << 4)) = o;
          }
        }
      } else {
#pragma unroll 1
      for (int c0 = c_base; c0 < c_base + S::kPassCols; c0 += 32) {
        unsigned v[32];
        tmem_load_32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BLOCK_N + c0), v);
        if (OUT_F32) {
          // a slab is 32 columns: row r holds 8 pieces of 16 bytes, piece j at (j ^ (r % 8))
          unsigned char* slab = staging + ((c0 - c_base) / 32) * S::kSlabBytes + r * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o;
            o.x = __uint_as_float(v[4 * j]) + (bias && n0 + c0 + 4 * j < N ? bias[n0 + c0 + 4 * j] : 0.f);
            o.y = __uint_as_float(v[4 * j + 1]) + (bias && n0 + c0 + 4 * j + 1 < N ? bias[n0 + c0 + 4 * j + 1] : 0.f);
            o.z = __uint_as_float(v[4 * j + 2]) + (bias && n0 + c0 + 4 * j + 2 < N ? bias[n0 + c0 + 4 * j + 2] : 0.f);
            o.w = __uint_as_float(v[4 * j + 3]) + (bias && n0 + c0 + 4 * j + 3 < N ? bias[n0 + c0 + 4 * j + 3] : 0.f);
            *reinterpret_cast<float4*>(slab + ((j ^ (r & 7)) << 4)) = o;
          }
        } else {
          // a slab is 64 columns: these 32 are pieces 4 * (c0 / 32 % 2) .. + 3 of row r
          unsigned char* slab = staging + ((c0 - c_base) / 64) * S::kSlabBytes + r * 128;
          const int piece0 = (c0 / 32 % 2) * 4;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            unsigned* ow = reinterpret_cast<unsigned*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int col = n0 + c0 + 8 * j + 2 * e;
              const float lo = __uint_as_float(v[8 * j + 2 * e]) + (bias && col < N ? bias[col] : 0.f);
              const float hi = __uint_as_float(v[8 * j + 2 * e + 1]) + (bias && col + 1 < N ? bias[col + 1] : 0.f);
              __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
              ow[e] = *reinterpret_cast<unsigned*>(&pair);
            }
            *reinterpret_cast<uint4*>(slab + (((piece0 + j) ^ (r & 7)) << 4)) = o;
          }
        }
      }
      }
      if (c_base + S::kPassCols >= BLOCK_N) {
        // the accumulator buffer is free for the products of the tile after next
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (lane == 0) {
          if (PAIR) mbar_arrive_cluster(leader_address(&acc_empty[buf]));
          else mbar_arrive(&acc_empty[buf]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // staging writes -> TMA reads
      epilogue_barrier();
      if (issuer && m0 < M) {
        if (GATED) {   // the tile's 128 output columns start at n0 / 2
#pragma unroll 1
          for (int sl = 0; sl < 2; ++sl)
            if (n0 / 2 + sl * 64 < N / 2)
              tma_store_2d(&map_out, staging + sl * S::kSlabBytes, n0 / 2 + sl * 64, m0);
        } else if (!QKV || n0 < qkv.nh * qkv.d) {
#pragma unroll 1
          for (int sl = 0; sl < S::kSlabs; ++sl) {
            const int col = n0 + c_base + sl * S::kSlabCols;
            if (col < (QKV ? qkv.nh * qkv.d : N)) {
              if (OUT_F32) tma_store_3d(&map_out, staging + sl * S::kSlabBytes, col, m0, split);
              else tma_store_2d(&map_out, staging + sl * S::kSlabBytes, col, m0);
            }
          }
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
      }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // before the CTA's memory goes
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  if (PAIR) cluster_sync_all();       // neither CTA's shared or tensor memory goes while the other may use it
  else __syncthreads();
  pdl_launch();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"((unsigned)(2 * BLOCK_N)) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"((unsigned)(2 * BLOCK_N)) : "memory");
  }
}

// ---- host side ----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// A map over a row-major [rows, K] bfloat16 matrix, boxes of box_rows x 64, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return TOKB200_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {TC_BLOCK_K, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                  elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TOKB200_OK : TOKB200_BAD_ALIGNMENT;
}

// A map over the row-major [M, N] output, boxes of 128 rows x 128 bytes, 128-byte swizzle.
static int make_out_map(CUtensorMap* map, void* base, long long M, long long N, bool f32, int planes = 1) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return TOKB200_BAD_SIZE;
  if (f32) {   // [planes, M, N]: a plane per piece of k (one plane for a whole product)
    const cuuint64_t dims3[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)planes};
    const cuuint64_t strides3[2] = {(cuuint64_t)N * 4, (cuuint64_t)M * (cuuint64_t)N * 4};
    const cuuint32_t box3[3] = {32, TC_BLOCK_M, 1};
    const cuuint32_t elem3[3] = {1, 1, 1};
    CUresult r3 = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims3, strides3, box3, elem3,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r3 == CUDA_SUCCESS ? TOKB200_OK : TOKB200_BAD_ALIGNMENT;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)N * (f32 ? 4 : 2)};
  const cuuint32_t box[2] = {(cuuint32_t)(f32 ? 32 : 64), TC_BLOCK_M};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base,
                  dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TOKB200_OK : TOKB200_BAD_ALIGNMENT;
}

template <int BLOCK_N, int STAGES, bool OUT_F32, bool GATED = false, bool QKV = false, bool PAIR = false>
static int launch_tc_persistent(const void* x, const void* w, const float* bias, void* out, int M, int N,
                                int K, cudaStream_t stream, int k_splits = 1,
                                const QkvEpilogue* qkv_in = nullptr, int activation = TOKB200_ACT_SILU) {
  using S = TcPersistentSmem<BLOCK_N, STAGES, OUT_F32, GATED, PAIR>;
  static_assert(S::kTotal <= 227 * 1024, "shared memory of one CTA");
  CUtensorMap map_x, map_w, map_out;
  int status = make_map(&map_x, x, M, K, TC_BLOCK_M);
  if (status != TOKB200_OK) return status;
  status = make_map(&map_w, w, N, K, PAIR ? BLOCK_N / 2 : BLOCK_N);      // a pair's CTA loads half the rows
  if (status != TOKB200_OK) return status;
  if (k_splits < 1 || (k_splits > 1 && (!OUT_F32 || bias))) return TOKB200_BAD_SIZE;
  QkvEpilogue qkv = {};
  if (QKV) qkv = *qkv_in;
  qkv.activation = activation;
  status = make_out_map(&map_out, out, M, GATED ? N / 2 : (QKV ? (long long)qkv.nh * qkv.d : N), OUT_F32, k_splits);
  if (status != TOKB200_OK) return status;
  static bool configured[64] = {};
  static int sm_count[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  auto kernel = gemm_tcgen05_persistent_kernel<BLOCK_N, STAGES, OUT_F32, GATED, QKV, PAIR>;
  if (!configured[device]) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (err != cudaSuccess) return (int)err;
    err = cudaDeviceGetAttribute(&sm_count[device], cudaDevAttrMultiProcessorCount, device);
    if (err != cudaSuccess) return (int)err;
    configured[device] = true;
  }
  const int tile_m = PAIR ? 2 * TC_BLOCK_M : TC_BLOCK_M;
  const int tiles = ((M + tile_m - 1) / tile_m) * ((N + BLOCK_N - 1) / BLOCK_N) * k_splits;
  if (!PAIR) {
    dim3 grid(tiles < sm_count[device] ? tiles : sm_count[device]);
    return launch_dependent(kernel, grid, dim3(TC_THREADS), (size_t)S::kTotal, stream, map_x, map_w, map_out,
                            bias, M, N, K, k_splits, qkv);
  }
  // clusters of two CTAs, one cluster per pair of SMs at most
  const int pairs = sm_count[device] / 2;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * (tiles < pairs ? tiles : pairs));
  config.blockDim = dim3(TC_THREADS);
  config.dynamicSmemBytes = (size_t)S::kTotal;
  config.stream = stream;
  static const int overlap = [] {
    const char* v = getenv("TOKB200_PDL");
    return (v && v[0] == '0') ? 0 : 1;
  }();
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = overlap;
  attribute[1].id = cudaLaunchAttributeClusterDimension;
  attribute[1].val.clusterDim.x = 2;
  attribute[1].val.clusterDim.y = 1;
  attribute[1].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 2;
  cudaError_t err = cudaLaunchKernelEx(&config, kernel, map_x, map_w, map_out, bias, M, N, K, k_splits, qkv);
  return err == cudaSuccess ? TOKB200_OK : (int)err;
}

template <int BLOCK_N, int STAGES>
static int launch_tc(const void* x, const void* w, const float* bias, void* out, int out_is_f32, int M,
                     int N, int K, cudaStream_t stream) {
  using S = TcSmem<BLOCK_N, STAGES>;
  CUtensorMap map_x, map_w;
  int status = make_map(&map_x, x, M, K, TC_BLOCK_M);
  if (status != TOKB200_OK) return status;
  status = make_map(&map_w, w, N, K, BLOCK_N);
  if (status != TOKB200_OK) return status;
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!configured[device]) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BLOCK_N, STAGES>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (err != cudaSuccess) return (int)err;
    configured[device] = true;
  }
  dim3 grid((M + TC_BLOCK_M - 1) / TC_BLOCK_M, (N + BLOCK_N - 1) / BLOCK_N);
  return launch_dependent(gemm_tcgen05_kernel<BLOCK_N, STAGES>, grid, dim3(TC_THREADS),
                          (size_t)S::kTotal, stream, map_x, map_w, bias, out, out_is_f32, M, N, K);
}

// 1 when some launch since the last call recorded a wait that ran out; clears the flag.
TOKB200_API int tokb200_gemm_tcgen05_error(void) {
  int flag = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&flag, tc_error_flag, sizeof(int)) != cudaSuccess) return -1;
  if (flag) cudaMemcpyToSymbol(tc_error_flag, &zero, sizeof(int));
  return flag;
}

TOKB200_API int tokb200_gemm_tcgen05(const void* x, const void* w, const float* bias, void* out,
                                     int out_is_f32, int M, int N, int K, int block_n,
                                     cudaStream_t stream) {
  if (M <= 0 || N <= 0) return TOKB200_OK;
  if (K <= 0 || K % 8) return TOKB200_BAD_SIZE;          // TMA: row pitch a multiple of 16 bytes
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TOKB200_BAD_ALIGNMENT;
  if (((uintptr_t)out) & 15) return TOKB200_BAD_ALIGNMENT;
  if (M > 128 * 65535) return TOKB200_BAD_SIZE;
  // block_n + 1000 asks for the persistent kernel (TMA-stored output): the output's
  // row pitch must then be a multiple of 16 bytes
  if (block_n >= 1000) {
    if ((out_is_f32 ? N % 4 : N % 8) != 0) return TOKB200_BAD_SIZE;
    switch (block_n - 1000) {
      case 128:
        return out_is_f32 ? launch_tc_persistent<128, 4, true>(x, w, bias, out, M, N, K, stream)
                          : launch_tc_persistent<128, 5, false>(x, w, bias, out, M, N, K, stream);
      case 256:
        return out_is_f32 ? TOKB200_BAD_SIZE
                          : launch_tc_persistent<256, 3, false>(x, w, bias, out, M, N, K, stream);
      default: return TOKB200_BAD_SIZE;
    }
  }
  switch (block_n) {
    case 64: return launch_tc<64, 4>(x, w, bias, out, out_is_f32, M, N, K, stream);
    case 128: return launch_tc<128, 3>(x, w, bias, out, out_is_f32, M, N, K, stream);
    case 256: return launch_tc<256, 4>(x, w, bias, out, out_is_f32, M, N, K, stream);
    default: return TOKB200_BAD_SIZE;
  }
}

// out[k_splits, M, N] (float32) = partial sums of x w^T over k_splits pieces of k (of whole
// 64-element blocks; every piece must get at least one), for products with too few output
// tiles to fill the device; the consumer adds the pieces in index order.
TOKB200_API int tokb200_gemm_tcgen05_partials(const void* x, const void* w, void* out, int M, int N, int K,
                                              int k_splits, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return TOKB200_OK;
  if (K <= 0 || K % 8 || N % 4 || k_splits < 1) return TOKB200_BAD_SIZE;
  const int k_blocks = (K + TC_BLOCK_K - 1) / TC_BLOCK_K;
  const int per = (k_blocks + k_splits - 1) / k_splits;
  if ((k_splits - 1) * per >= k_blocks) return TOKB200_BAD_SIZE;        // an empty piece
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return TOKB200_BAD_ALIGNMENT;
  if (M > 128 * 65535) return TOKB200_BAD_SIZE;
  return launch_tc_persistent<128, 4, true>(x, w, nullptr, out, M, N, K, stream, k_splits);
}

// The pair form (two CTAs a tile of 256 rows x 256 columns; see the kernel).  kind 0: out [M,N]
// bfloat16 (+ bias); kind 1: the gated product, out [M, N/2] bfloat16 (N a multiple of 256, no
// bias); kind 2: float32 partial sums out [k_splits, M, N] (no bias); kind 3: as kind 0 with
// 128-column tiles.  `activation`: the gated product's activation tag (kind 1 only).
TOKB200_API int tokb200_gemm_tcgen05_pair(const void* x, const void* w, const float* bias, void* out,
                                          int kind, int M, int N, int K, int k_splits, int activation,
                                          cudaStream_t stream) {
  if (M <= 0 || N <= 0) return TOKB200_OK;
  if (K <= 0 || K % 8 || k_splits < 1 || activation < 0 || activation >= TOKB200_ACT_COUNT) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return TOKB200_BAD_ALIGNMENT;
  if (M > 128 * 65535) return TOKB200_BAD_SIZE;
  const int k_blocks = (K + TC_BLOCK_K - 1) / TC_BLOCK_K;
  const int per = (k_blocks + k_splits - 1) / k_splits;
  if ((k_splits - 1) * per >= k_blocks) return TOKB200_BAD_SIZE;        // an empty piece
  switch (kind) {
    case 0:
      if (N % 8 || k_splits != 1) return TOKB200_BAD_SIZE;
      return launch_tc_persistent<256, 5, false, false, false, true>(x, w, bias, out, M, N, K, stream);
    case 1:
      if (N % 256 || k_splits != 1 || bias) return TOKB200_BAD_SIZE;
      return launch_tc_persistent<256, 6, false, true, false, true>(x, w, nullptr, out, M, N, K, stream, 1,
                                                                    nullptr, activation);
    case 2:
      if (N % 4 || bias) return TOKB200_BAD_SIZE;
      return launch_tc_persistent<256, 5, true, false, false, true>(x, w, nullptr, out, M, N, K, stream, k_splits);
    case 3:
      if (N % 8 || k_splits != 1) return TOKB200_BAD_SIZE;
      return launch_tc_persistent<128, 6, false, false, false, true>(x, w, bias, out, M, N, K, stream);
    default: return TOKB200_BAD_SIZE;
  }
}

// out[M, N/2] = act(x Wg^T) * (x Wu^T) where w [N, K] holds, for every 128 outputs,
// their 128 gate rows followed by their 128 up rows (N a multiple of 256); act by its tag.
TOKB200_API int tokb200_gemm_tcgen05_gated(const void* x, const void* w, void* out, int M, int N, int K,
                                           int activation, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return TOKB200_OK;
  if (K <= 0 || K % 8 || N % 256 || activation < 0 || activation >= TOKB200_ACT_COUNT) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return TOKB200_BAD_ALIGNMENT;
  if (M > 128 * 65535) return TOKB200_BAD_SIZE;
  return launch_tc_persistent<256, 3, false, true>(x, w, nullptr, out, M, N, K, stream, 1, nullptr, activation);
}

// The stacked q/k/v projection of many rows with bias, rotary encoding (the whole head, half-split
// pairs) and the cache write in the epilogue: q_out [M, nh d] bfloat16; k and v go to
// pool[slot[row], kv head, :] (a negative slot, a null slot array or a null pool skip the write).
// Head size 64 or 128, and both nh d and nkv d multiples of 128, so that a tile holds whole heads
// of one kind.
TOKB200_API int tokb200_gemm_tcgen05_qkv_rope(const void* x, const void* w, const float* bias,
                                              const int* pos, const int* slot, const float* cos_t,
                                              const float* sin_t, void* q_out, void* k_pool, void* v_pool,
                                              int M, int nh, int nkv, int d, int K, cudaStream_t stream) {
  if (M <= 0) return TOKB200_OK;
  if (K <= 0 || K % 8 || (d != 64 && d != 128) || nh <= 0 || nkv <= 0 || (nh * d) % 128 || (nkv * d) % 128)
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool |
       (uintptr_t)cos_t | (uintptr_t)sin_t) & 15)
    return TOKB200_BAD_ALIGNMENT;
  if (M > 128 * 65535) return TOKB200_BAD_SIZE;
  QkvEpilogue qkv;
  qkv.pos = pos; qkv.slot = slot; qkv.cos_t = cos_t; qkv.sin_t = sin_t;
  qkv.k_pool = (__nv_bfloat16*)k_pool; qkv.v_pool = (__nv_bfloat16*)v_pool;
  qkv.nh = nh; qkv.nkv = nkv; qkv.d = d;
  return launch_tc_persistent<128, 5, false, false, true>(x, w, bias, q_out, M, (nh + 2 * nkv) * d, K, stream,
                                                          1, &qkv);
}
