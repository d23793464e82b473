// Attention for portions of prompts on the fifth-generation tensor cores
// (bfloat16, tcgen05 with the scores and the weighted values in tensor memory).
//
// A block takes one (tile of up to 128 consecutive rows of one request, query head)
// and walks the request's keys in blocks of 128; it owns its SM (all 512 columns of
// tensor memory: two score buffers and SPLITS output accumulators):
//   * loader warps gather a block's keys and values from their cache pages with
//     16-byte asynchronous copies into shared memory, in the 128-byte swizzled layout
//     the tensor core reads (any page size works), several blocks ahead of their use;
//   * one thread issues S = Q K^T (tcgen05.mma, M = 128 rows, N = 128 keys, both
//     operands K-major) into one of two score buffers, one block ahead, so the
//     scores of block b + 1 are ready while the softmax of block b runs;
//   * the softmax is cut by key columns: SPLITS threads share a row (thread = row r,
//     columns 128/SPLITS * q ...), each with its OWN running maximum, sum and output
//     accumulator in tensor memory, so no value crosses threads inside the walk; a
//     thread reads its scores once (one tcgen05.ld), writes the probabilities as
//     bfloat16 into shared memory (the A operand of the second product) and moves on;
//   * the same issuing thread adds P V of each column split into that split's
//     accumulator (M = 128, N = head size; V is the B operand in MN-major form, which
//     is how the cache stores it: a key per row).  The accumulators stay in tensor
//     memory over the whole walk.  A thread's reference maximum follows the true
//     maximum lazily: only when the maximum has grown by more than 2^8 since it was
//     set are the sum and the accumulator rescaled (read, multiplied, written back),
//     which happens a few times per row, not per block; probabilities stay below 2^8;
//   * at the end the SPLITS partial results of a row are merged: maxima and sums go
//     through shared memory, and each thread reads its slice of the head from all
//     accumulators.
// Everything but q, k, v, p and the output is 32-bit.  Every wait is bounded; when
// one runs out an error flag is set and all roles fall through to the common exit,
// where tensor memory is given back.
//
// HEAD_DIM is a compile-time size (64 or 128), -DHEAD_DIM=...
#include <cuda.h>

#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "head size");

#define FA_ROWS 128
#define FA_KEYS 128
#define FA_SPLITS (HEAD_DIM == 64 ? 4 : 2)        // threads (and accumulators) per row
#define FA_SOFTMAX_THREADS (128 * FA_SPLITS)
#define FA_LOADER_THREADS 64            // two rows a thread: 19 warps in all leave 96 registers a thread
#define FA_THREADS (FA_SOFTMAX_THREADS + FA_LOADER_THREADS + 32)
#define FA_KV_BUFFERS (HEAD_DIM == 64 ? 4 : 2)
#define FA_WAIT_LIMIT (1u << 17)      // polls of up to 20 us each: seconds in all
#define FA_RESCALE_AT 8.0f            // log2 units the maximum may lead its reference by
constexpr int kDBlocks = HEAD_DIM / 64;           // 64-lane pieces of the head (128 bytes a row)
constexpr int kSubTile = 128 * 128;               // bytes of a [128 x 64] bfloat16 swizzled tile
constexpr int kTmemCols = 512;                    // S0, S1: 128 columns each; SPLITS accumulators of HEAD_DIM
constexpr int kSplitKeys = FA_KEYS / FA_SPLITS;   // key columns a softmax thread owns (32 or 64)
constexpr int kSlice = HEAD_DIM / FA_SPLITS;      // output lanes a thread writes at the end (16 or 64)
static_assert(256 + FA_SPLITS * HEAD_DIM == kTmemCols, "tensor memory plan");

__device__ int fa_error_flag = 0;


__device__ __forceinline__ unsigned fa_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fa_smem(bar)), "r"(count));
}
__device__ __forceinline__ void fa_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fa_smem(bar)) : "memory");
}
__device__ __forceinline__ bool fa_mbar_wait(unsigned long long* bar, unsigned parity) {
  const unsigned addr = fa_smem(bar);
  // the thread sleeps in hardware until the phase completes or the hint runs out, so
  // waiting warps do not take issue slots from working ones
  const unsigned suspend_ns = 20000u;
  for (unsigned spin = 0; spin < FA_WAIT_LIMIT; ++spin) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity), "r"(suspend_ns) : "memory");
    if (done) return true;
  }
  atomicExch(&fa_error_flag, 1);
  tokb200_report_error(TOKB200_LIB_ATTENTION_TCGEN05, 1);
  return false;
}
__device__ __forceinline__ void fa_cp16(void* dst, const void* src, bool ok) {
  const int bytes = ok ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(fa_smem(dst)), "l"(src), "r"(bytes));
}
// byte offset of element (row, 16-byte piece c) in a [rows x 64] bfloat16 tile with 128-byte swizzle
__device__ __forceinline__ int swz(int row, int c) {
  return (row >> 3) * 1024 + (row & 7) * 128 + ((c ^ (row & 7)) << 4);
}
// K-major operand (q, k, p): rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ unsigned long long desc_k_major(const void* tile) {
  const unsigned long long addr = (fa_smem(tile) & 0x3FFFFu) >> 4;
  return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (v: a key per 128-byte row of 64 lanes): 8-key groups 1024 bytes
// apart (stride offset), 64-lane pieces of the head one sub-tile apart (leading offset)
__device__ __forceinline__ unsigned long long desc_mn_major(const void* tile) {
  const unsigned long long addr = (fa_smem(tile) & 0x3FFFFu) >> 4;
  return addr | ((unsigned long long)(kSubTile >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void fa_mma(unsigned tmem_d, unsigned long long a, unsigned long long b,
                                       unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fa_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(fa_smem(bar)) : "memory");
}
__device__ __forceinline__ void fa_tmem_load32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
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
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fa_tmem_load16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fa_tmem_store32(unsigned taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,"
      "%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
        "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
        "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
        "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
        "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
// two 32-bit values in one 64-bit register, for the packed arithmetic of sm_100
__device__ __forceinline__ unsigned long long fa_pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void fa_unpack2(unsigned long long v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long fa_fma2(unsigned long long a, unsigned long long b,
                                                      unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long fa_add2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// shared memory: q | k[buffers] | v[buffers] | p[2]   (each a whole number of 16 KB sub-tiles),
// then the rows' maxima and sums for the final merge, then the barriers
constexpr int kQBytes = kDBlocks * kSubTile;
constexpr int kKVBytes = kDBlocks * kSubTile;
constexpr int kPBytes = 2 * kSubTile;
constexpr int kStatBytes = FA_SPLITS * FA_ROWS * 2 * 4;
constexpr int kFaSmem = kQBytes + 2 * FA_KV_BUFFERS * kKVBytes + 2 * kPBytes + kStatBytes + 256;
static_assert(kFaSmem > 116 * 1024, "one block an SM: it takes all of tensor memory");

__global__ void __launch_bounds__(FA_THREADS, 1)
attention_tcgen05_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ row_req, const int* __restrict__ pos,
                         const int* __restrict__ tiles, int n_tiles, int nh, int nkv, int page, int window,
                         float scale_log2) {
  extern __shared__ __align__(1024) unsigned char fa_raw[];      // swizzle atoms: 1024-byte aligned
  unsigned char* q_s = fa_raw;
  unsigned char* k_s = q_s + kQBytes;                            // FA_KV_BUFFERS buffers
  unsigned char* v_s = k_s + FA_KV_BUFFERS * kKVBytes;           // FA_KV_BUFFERS buffers
  unsigned char* p_s = v_s + FA_KV_BUFFERS * kKVBytes;           // two buffers, blocks in turn
  float* stat_s = reinterpret_cast<float*>(p_s + 2 * kPBytes);   // [split][row][max, sum]
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(p_s + 2 * kPBytes + kStatBytes);
  unsigned long long* kv_full = bars;                            // [buffers], an arrival per loader warp
  unsigned long long* kv_empty = bars + FA_KV_BUFFERS;           // [buffers], commit of the block's P V
  unsigned long long* s_full = bars + 2 * FA_KV_BUFFERS;         // [2], commit of Q K^T
  unsigned long long* p_ready = s_full + 2;                      // an arrival per softmax warp
  unsigned long long* pv_done = s_full + 3;                      // commit of P V
  unsigned long long* q_full = s_full + 4;                       // an arrival per loader warp
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(s_full + 5);

  // heads run fastest over the grid so that the tiles with the most keys (first in
  // `tiles`) of all heads are placed first
  const int h = blockIdx.x, tile = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = tiles[2 * tile], n_rows = tiles[2 * tile + 1];
  const int r_id = row_req[row0];
  // uniform over the block; a misaligned base (never seen) is reported instead of used
  const bool aligned = (fa_smem(fa_raw) & 1023u) == 0;
  if (!aligned && threadIdx.x == 0) {
    atomicExch(&fa_error_flag, 2);
    tokb200_report_error(TOKB200_LIB_ATTENTION_TCGEN05, 2);
  }
  const bool live = aligned && tile < n_tiles && r_id >= 0 && n_rows > 0;
  const int kvh = h / (nh / nkv);
  const int pos0 = live ? pos[row0] : 0;
  const int pos_last = pos0 + n_rows - 1;
  const int lo_first = (window >= 0 && pos0 - window > 0) ? pos0 - window : 0;
  const int kb_first = lo_first / FA_KEYS * FA_KEYS;
  const int n_blocks = live ? (pos_last - kb_first) / FA_KEYS + 1 : 0;
  const int* table = block_table + (size_t)(live ? r_id : 0) * table_stride;
  constexpr int kSoftmaxWarps = FA_SOFTMAX_THREADS / 32;
  constexpr int kMmaWarp = kSoftmaxWarps + FA_LOADER_THREADS / 32;

  if (threadIdx.x == 0) {
    for (int i = 0; i < FA_KV_BUFFERS; ++i) {
      fa_mbar_init(&kv_full[i], FA_LOADER_THREADS / 32);
      fa_mbar_init(&kv_empty[i], 1);
    }
    fa_mbar_init(&s_full[0], 1);
    fa_mbar_init(&s_full[1], 1);
    fa_mbar_init(p_ready, FA_SOFTMAX_THREADS / 32);
    fa_mbar_init(pv_done, 1);
    fa_mbar_init(q_full, FA_LOADER_THREADS / 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(fa_smem(tmem_slot)), "r"((unsigned)kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;           // scores: columns 0..127 and 128..255
  const unsigned tmem_o = tmem_base + 256;         // accumulator of split j: columns 256 + j * HEAD_DIM ...
  pdl_wait();

  if (live && warp >= kSoftmaxWarps && warp < kMmaWarp) {
    // ---------------- loaders: a thread brings rows t0, t0 + 64 of q, then those keys of every block ----------------
    const int t0 = threadIdx.x - FA_SOFTMAX_THREADS;
#pragma unroll
    for (int t = t0; t < FA_ROWS; t += FA_LOADER_THREADS) {
      const bool ok = t < n_rows;
      const __nv_bfloat16* src = q + ((size_t)(row0 + (ok ? t : 0)) * nh + h) * HEAD_DIM;
#pragma unroll
      for (int c = 0; c < HEAD_DIM / 8; ++c)
        fa_cp16(q_s + (c / 8) * kSubTile + swz(t, c % 8), src + c * 8, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    // kLag blocks are in flight at a time: before block b is asked for, block b - kLag is
    // waited for and announced (q rides with block 0)
    constexpr int kLag = FA_KV_BUFFERS / 2;
    // a warp's copies have all landed once each of its lanes has waited: one arrival a warp
    auto announce = [&](int e) {
      __syncwarp();
      if (lane == 0) {
        if (e == 0) fa_mbar_arrive(q_full);
        fa_mbar_arrive(&kv_full[e % FA_KV_BUFFERS]);
      }
    };
    bool ok = true;
    for (int b = 0; b < n_blocks; ++b) {
      const int buf = b % FA_KV_BUFFERS, use = b / FA_KV_BUFFERS;
      if (b >= kLag) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kLag - 1) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        announce(b - kLag);
      }
      // the buffer is free once the P V of the block that held it has read it
      if (use > 0 && !__all_sync(0xffffffffu, fa_mbar_wait(&kv_empty[buf], (use - 1) & 1))) { ok = false; break; }   // a warp gives up together
#pragma unroll
      for (int t = t0; t < FA_KEYS; t += FA_LOADER_THREADS) {
        const int key = kb_first + b * FA_KEYS + t;
        const bool in = key >= lo_first && key <= pos_last;
        size_t offset = 0;
        if (in) offset = ((size_t)(table[key / page] * page + key % page) * nkv + kvh) * HEAD_DIM;
#pragma unroll
        for (int c = 0; c < HEAD_DIM / 8; ++c) {
          fa_cp16(k_s + buf * kKVBytes + (c / 8) * kSubTile + swz(t, c % 8), k_pool + offset + c * 8, in);
          fa_cp16(v_s + buf * kKVBytes + (c / 8) * kSubTile + swz(t, c % 8), v_pool + offset + c * 8, in);
        }
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (ok)
      for (int e = n_blocks > kLag ? n_blocks - kLag : 0; e < n_blocks; ++e) announce(e);
  } else if (live && warp == kMmaWarp) {
    // ---------------- products ----------------
    if (lane == 0) {
      const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(FA_KEYS >> 3) << 17) |
                               ((unsigned)(FA_ROWS >> 4) << 24);
      const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /* v is MN-major */ |
                               ((unsigned)(HEAD_DIM >> 3) << 17) | ((unsigned)(FA_ROWS >> 4) << 24);
      // S = Q K^T of block b into score buffer b & 1, 16 lanes of the head at a time
      auto scores = [&](int b) {
        const int buf = b % FA_KV_BUFFERS;
#pragma unroll
        for (int kk = 0; kk < HEAD_DIM / 16; ++kk) {
          const unsigned long long a = desc_k_major(q_s + (kk / 4) * kSubTile) + 2 * (kk % 4);
          const unsigned long long bd = desc_k_major(k_s + buf * kKVBytes + (kk / 4) * kSubTile) + 2 * (kk % 4);
          fa_mma(tmem_base + (unsigned)((b & 1) * 128), a, bd, idesc_s, kk != 0);
        }
        fa_commit(&s_full[b & 1]);
      };
      bool ok = fa_mbar_wait(q_full, 0) && fa_mbar_wait(&kv_full[0], 0);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        scores(0);
      }
      for (int b = 0; ok && b < n_blocks; ++b) {
        const int buf = b % FA_KV_BUFFERS;
        if (b + 1 < n_blocks) {
          // the other score buffer held block b - 1, whose readers all arrived at p_ready(b - 1)
          if (!fa_mbar_wait(&kv_full[(b + 1) % FA_KV_BUFFERS], ((b + 1) / FA_KV_BUFFERS) & 1)) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          scores(b + 1);
        }
        if (!fa_mbar_wait(p_ready, b & 1)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // P V over the block's keys, 16 at a time, each column split into its own accumulator:
        // p advances 32 bytes in its row (a new sub-tile after 64 keys), v two 8-key groups
        constexpr int kStepsPerSplit = (FA_KEYS / 16) / FA_SPLITS;
#pragma unroll
        for (int kk = 0; kk < FA_KEYS / 16; ++kk) {
          const unsigned long long a = desc_k_major(p_s + (b & 1) * kPBytes + (kk / 4) * kSubTile) + 2 * (kk % 4);
          const unsigned long long bd = desc_mn_major(v_s + buf * kKVBytes) + (unsigned long long)(kk * 128);
          fa_mma(tmem_o + (unsigned)((kk / kStepsPerSplit) * HEAD_DIM), a, bd, idesc_o,
                 (b > 0 || kk % kStepsPerSplit != 0) ? 1u : 0u);
        }
        fa_commit(pv_done);
        fa_commit(&kv_empty[buf]);
      }
    }
  } else if (live && warp < kSoftmaxWarps) {
    // ---------------- softmax: thread (r, split) owns columns split * kSplitKeys ... of row r ----------------
    const int split = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int p_row = pos0 + min(r, n_rows - 1);            // rows past the tile repeat its last row
    const int lo_row = (window >= 0 && p_row - window > 0) ? p_row - window : 0;
    const unsigned lane_base = ((unsigned)((warp & 3) * 32) << 16);
    const unsigned my_o = tmem_o + lane_base + (unsigned)(split * HEAD_DIM);
    float m_ref = -INFINITY, l_run = 0.f;     // reference maximum (raw score units) and running sum
    bool ok = true;
    for (int b = 0; b < n_blocks; ++b) {
      const int kb = kb_first + b * FA_KEYS + split * kSplitKeys;
      if (!__all_sync(0xffffffffu, fa_mbar_wait(&s_full[b & 1], (b >> 1) & 1))) { ok = false; break; }

      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float s[kSplitKeys];
#pragma unroll
      for (int c0 = 0; c0 < kSplitKeys; c0 += 32)
        fa_tmem_load32(tmem_base + lane_base + (unsigned)((b & 1) * 128 + split * kSplitKeys + c0),
                       *reinterpret_cast<float(*)[32]>(&s[c0]));
      const bool needs_mask = kb + kSplitKeys - 1 > pos0 || (window >= 0 && kb < pos_last - window);
      float m_blk = -INFINITY;
      if (needs_mask) {
#pragma unroll
        for (int j = 0; j < kSplitKeys; ++j) {
          const int key = kb + j;
          s[j] = (key <= p_row && key >= lo_row) ? s[j] : -INFINITY;
          m_blk = fmaxf(m_blk, s[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < kSplitKeys; ++j) m_blk = fmaxf(m_blk, s[j]);
      }
      // the reference moves only when the maximum has run away from it
      const bool move = m_blk > -INFINITY &&
                        (m_ref == -INFINITY || (m_blk - m_ref) * scale_log2 > FA_RESCALE_AT);
      float factor = 1.f;
      if (move) {
        factor = m_ref == -INFINITY ? 0.f : fa_exp2((m_ref - m_blk) * scale_log2);
        m_ref = m_blk;
        l_run *= factor;
      }
      // The probabilities of blocks b and b - 1 have buffers of their own, and the scores of
      // block b were committed after the P V of block b - 2 was issued, so p's buffer is free
      // by now.  Only a rescaling has to wait for the last block's P V, which writes the
      // accumulator.
      if (b > 0 && __any_sync(0xffffffffu, move)) {
        if (!__all_sync(0xffffffffu, fa_mbar_wait(pv_done, (b - 1) & 1))) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c0 = 0; c0 < HEAD_DIM; c0 += 32) {
          float acc[32];
          fa_tmem_load32(my_o + (unsigned)c0, acc);
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] *= factor;
          fa_tmem_store32(my_o + (unsigned)c0, acc);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      // probabilities, their sum, and the bfloat16 copy for the second product
      const float m_scaled = m_ref == -INFINITY ? 0.f : m_ref * scale_log2;
      // two columns an instruction where the hardware has it (scale and shift, the sum); the
      // exponential is one column each.  Masked scores are -inf: probability 0.
      const unsigned long long scale2 = fa_pack2(scale_log2, scale_log2), shift2 = fa_pack2(-m_scaled, -m_scaled);
      unsigned long long sum2 = fa_pack2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < kSplitKeys; j += 2) {
        float x0, x1;
        fa_unpack2(fa_fma2(fa_pack2(s[j], s[j + 1]), scale2, shift2), x0, x1);
        s[j] = fa_exp2(x0);
        s[j + 1] = fa_exp2(x1);
        sum2 = fa_add2(sum2, fa_pack2(s[j], s[j + 1]));
      }
      float sum_even, sum_odd;
      fa_unpack2(sum2, sum_even, sum_odd);
      l_run += sum_even + sum_odd;
#pragma unroll
      for (int c = 0; c < kSplitKeys / 8; ++c) {            // 16-byte pieces of 8 keys
        uint4 piece;
        unsigned* w = reinterpret_cast<unsigned*>(&piece);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 pair = __floats2bfloat162_rn(s[8 * c + 2 * e], s[8 * c + 2 * e + 1]);
          w[e] = *reinterpret_cast<unsigned*>(&pair);
        }
        const int chunk = split * (kSplitKeys / 8) + c;     // 0 .. 15 over the 128 keys
        *reinterpret_cast<uint4*>(p_s + (b & 1) * kPBytes + (chunk / 8) * kSubTile + swz(r, chunk % 8)) = piece;
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // p in shared memory -> the tensor core
      __syncwarp();
      if (lane == 0) fa_mbar_arrive(p_ready);                          // one arrival a warp
    }
    // ---------------- merge the row's splits ----------------
    if (ok && n_blocks > 0) ok = fa_mbar_wait(pv_done, (n_blocks - 1) & 1);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    stat_s[(split * FA_ROWS + r) * 2] = m_ref;
    stat_s[(split * FA_ROWS + r) * 2 + 1] = l_run;
    asm volatile("bar.sync 1, %0;" ::"n"(FA_SOFTMAX_THREADS) : "memory");
    float m_all = -INFINITY;
#pragma unroll
    for (int j = 0; j < FA_SPLITS; ++j) m_all = fmaxf(m_all, stat_s[(j * FA_ROWS + r) * 2]);
    float weight[FA_SPLITS], den = 0.f;
#pragma unroll
    for (int j = 0; j < FA_SPLITS; ++j) {
      const float m_j = stat_s[(j * FA_ROWS + r) * 2];
      weight[j] = m_j == -INFINITY ? 0.f : fa_exp2((m_j - m_all) * scale_log2);
      den += weight[j] * stat_s[(j * FA_ROWS + r) * 2 + 1];
    }
    if (ok) {
      const float inv = 1.0f / den;
      __nv_bfloat16* dst = out + ((size_t)(row0 + min(r, n_rows - 1)) * nh + h) * HEAD_DIM + split * kSlice;
#pragma unroll 1
      for (int c0 = 0; c0 < kSlice; c0 += 16) {
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll
        for (int j = 0; j < FA_SPLITS; ++j) {
          float part[16];
          fa_tmem_load16(tmem_o + lane_base + (unsigned)(j * HEAD_DIM + split * kSlice + c0), part);
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = fmaf(weight[j], part[i], acc[i]);
        }
        if (r < n_rows) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint4 piece;
            unsigned* w = reinterpret_cast<unsigned*>(&piece);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 pair = __floats2bfloat162_rn(acc[8 * c + 2 * e] * inv, acc[8 * c + 2 * e + 1] * inv);
              w[e] = *reinterpret_cast<unsigned*>(&pair);
            }
            *reinterpret_cast<uint4*>(dst + c0 + c * 8) = piece;
          }
        }
      }
    }
  }
  // ---------------- common exit ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  pdl_launch();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((unsigned)kTmemCols) : "memory");
  }
}

TOKB200_API int tokb200_attention_tcgen05_head_dim() { return HEAD_DIM; }

TOKB200_API int tokb200_attention_tcgen05_error(void) {
  int flag = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&flag, fa_error_flag, sizeof(int)) != cudaSuccess) return -1;
  if (flag) cudaMemcpyToSymbol(fa_error_flag, &zero, sizeof(int));
  return flag;
}

// tiles: [n_tiles][2] = (first row, rows) of consecutive rows of one request, rows <= 128
TOKB200_API int tokb200_attention_tcgen05(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* block_table,
    int table_stride, const int* row_req, const int* pos, const int* tiles, int n_tiles, int nh,
    int nkv, int d, int page, int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return TOKB200_OK;
  if (d != HEAD_DIM || nh <= 0 || nkv <= 0 || nh % nkv || page <= 0)
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15)
    return TOKB200_BAD_ALIGNMENT;
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!configured[device]) {
    cudaError_t err = cudaFuncSetAttribute(attention_tcgen05_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmem);
    if (err != cudaSuccess) return (int)err;
    configured[device] = true;
  }
  if (n_tiles > 65535) return TOKB200_BAD_SIZE;
  dim3 grid(nh, n_tiles);
  // This kernel starts strictly after its predecessor.  Started early (its blocks allocating tensor
  // memory and waiting while the rotary kernel before it still runs), with the product after it
  // started early as well, about one step in a hundred of some 1,800 prompt tokens came out with
  // a few rows wrong (bitwise comparison of repeated identical steps; never with either of the
  // two early starts taken away, nor with this kernel alone or between two products).  The cause
  // has not been found; the early start saved about two microseconds a layer.
  return launch_ordered(false, attention_tcgen05_kernel, grid, dim3(FA_THREADS), (size_t)kFaSmem, stream,
                          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
                          (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, block_table, table_stride,
                          row_req, pos, tiles, n_tiles, nh, nkv, page, window,
                          scale * 1.4426950408889634f);
}
