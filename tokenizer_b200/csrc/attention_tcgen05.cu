// Attention for portions of prompts on the fifth-generation tensor cores
// (bfloat16, tcgen05 with the scores and the weighted values in tensor memory).
//
// A block takes one (tile of up to 128 consecutive rows of one request, query head)
// and walks the request's keys in blocks of 128:
//   * loader warps gather the block's keys and values from their cache pages with
//     16-byte asynchronous copies into shared memory, in the 128-byte swizzled layout
//     the tensor core reads (any page size works), one block ahead of its use;
//   * one thread issues S = Q K^T (tcgen05.mma, M = 128 rows, N = 128 keys, both
//     operands K-major) into tensor memory;
//   * four softmax warps own one row per thread (thread r = row r = lane r of tensor
//     memory): they read the row's scores, keep the running maximum and sum, write the
//     probabilities as bfloat16 into shared memory (the A operand of the second
//     product), and fold the block's P V (read back from tensor memory) into the
//     row's output, which stays in registers: o = o * exp(m_old - m_new) + P V;
//   * the same thread issues P V (M = 128, N = head size, K = 128 keys; V is the B
//     operand in MN-major form, which is how the cache stores it: a key per row).
// No row reduction crosses threads, so the softmax needs no shuffles.  Everything
// but q, k, v, p and the output is 32-bit.  Every wait is bounded; when one runs
// out an error flag is set and all roles fall through to the common exit, where
// tensor memory is given back.
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
#define FA_SOFTMAX_THREADS 128
#define FA_LOADER_THREADS 128
#define FA_THREADS (FA_SOFTMAX_THREADS + FA_LOADER_THREADS + 32)
#define FA_WAIT_LIMIT (1u << 17)      // polls of up to 20 us each: seconds in all
constexpr int kDBlocks = HEAD_DIM / 64;           // 64-lane pieces of the head (128 bytes a row)
constexpr int kSubTile = 128 * 128;               // bytes of a [128 x 64] bfloat16 swizzled tile
constexpr int kTmemCols = 256;                    // S: 128 columns, P V: up to 128

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
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// shared memory: q | k[2] | v[2] | p   (each a whole number of 16 KB sub-tiles), then barriers
constexpr int kQBytes = kDBlocks * kSubTile;
constexpr int kKVBytes = kDBlocks * kSubTile;
constexpr int kPBytes = 2 * kSubTile;
constexpr int kFaSmem = kQBytes + 4 * kKVBytes + kPBytes + 128;   // tiles, then the barriers

__global__ void __launch_bounds__(FA_THREADS, HEAD_DIM == 64 ? 2 : 1)
attention_tcgen05_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ row_req, const int* __restrict__ pos,
                         const int* __restrict__ tiles, int n_tiles, int nh, int nkv, int page, int window,
                         float scale_log2) {
  extern __shared__ __align__(1024) unsigned char fa_raw[];      // swizzle atoms: 1024-byte aligned
  unsigned char* base = fa_raw;
  unsigned char* q_s = base;
  unsigned char* k_s = q_s + kQBytes;                      // 2 buffers
  unsigned char* v_s = k_s + 2 * kKVBytes;                 // 2 buffers
  unsigned char* p_s = v_s + 2 * kKVBytes;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(p_s + kPBytes);
  unsigned long long* kv_full = bars;                      // [2], 128 loader arrivals
  unsigned long long* kv_empty = bars + 2;                 // [2], commit of the block's P V
  unsigned long long* s_full = bars + 4;                   // commit of Q K^T
  unsigned long long* p_ready = bars + 5;                  // 128 softmax arrivals
  unsigned long long* o_full = bars + 6;                   // commit of P V
  unsigned long long* q_full = bars + 7;                   // 128 loader arrivals
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 8);

  const int tile = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = tiles[2 * tile], n_rows = tiles[2 * tile + 1];
  const int r_id = row_req[row0];
  // uniform over the block; a misaligned base (never seen) is reported instead of used
  const bool aligned = (fa_smem(fa_raw) & 1023u) == 0;
  if (!aligned && threadIdx.x == 0) atomicExch(&fa_error_flag, 2);
  const bool live = aligned && tile < n_tiles && r_id >= 0 && n_rows > 0;
  const int kvh = h / (nh / nkv);
  const int pos0 = live ? pos[row0] : 0;
  const int pos_last = pos0 + n_rows - 1;
  const int lo_first = (window >= 0 && pos0 - window > 0) ? pos0 - window : 0;
  const int kb_first = lo_first / FA_KEYS * FA_KEYS;
  const int n_blocks = live ? (pos_last - kb_first) / FA_KEYS + 1 : 0;
  const int* table = block_table + (size_t)(live ? r_id : 0) * table_stride;

  if (threadIdx.x == 0) {
    fa_mbar_init(&kv_full[0], FA_LOADER_THREADS);
    fa_mbar_init(&kv_full[1], FA_LOADER_THREADS);
    fa_mbar_init(&kv_empty[0], 1);
    fa_mbar_init(&kv_empty[1], 1);
    fa_mbar_init(s_full, 1);
    fa_mbar_init(p_ready, FA_SOFTMAX_THREADS);
    fa_mbar_init(o_full, 1);
    fa_mbar_init(q_full, FA_LOADER_THREADS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(fa_smem(tmem_slot)), "r"((unsigned)kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_s = *tmem_slot;              // scores: columns 0 .. 127
  const unsigned tmem_o = tmem_s + 128;            // the block's P V: columns 128 .. 128 + HEAD_DIM - 1
  pdl_wait();

  if (live && warp >= 4 && warp < 8) {
    // ---------------- loaders: thread t brings row t of q, then key t of every block ----------------
    const int t = threadIdx.x - FA_SOFTMAX_THREADS;
    {
      const bool ok = t < n_rows;
      const __nv_bfloat16* src = q + ((size_t)(row0 + (ok ? t : 0)) * nh + h) * HEAD_DIM;
#pragma unroll
      for (int c = 0; c < HEAD_DIM / 8; ++c)
        fa_cp16(q_s + (c / 8) * kSubTile + swz(t, c % 8), src + c * 8, ok);
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    for (int b = 0; b < n_blocks; ++b) {
      const int buf = b & 1;
      // the buffer is free once the P V of block b - 2 has read it
      if (b >= 2 && !fa_mbar_wait(&kv_empty[buf], ((b >> 1) - 1) & 1)) break;
      const int key = kb_first + b * FA_KEYS + t;
      const bool ok = key >= lo_first && key <= pos_last;
      size_t offset = 0;
      if (ok) offset = ((size_t)(table[key / page] * page + key % page) * nkv + kvh) * HEAD_DIM;
#pragma unroll
      for (int c = 0; c < HEAD_DIM / 8; ++c) {
        fa_cp16(k_s + buf * kKVBytes + (c / 8) * kSubTile + swz(t, c % 8), k_pool + offset + c * 8, ok);
        fa_cp16(v_s + buf * kKVBytes + (c / 8) * kSubTile + swz(t, c % 8), v_pool + offset + c * 8, ok);
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
      // say so as soon as the block has landed (q rides with block 0): the copies of
      // block b run while block b - 1 is multiplied, so this wait is short
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (b == 0) fa_mbar_arrive(q_full);
      fa_mbar_arrive(&kv_full[buf]);
    }
  } else if (live && warp == 8) {
    // ---------------- products ----------------
    if (lane == 0) {
      const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(FA_KEYS >> 3) << 17) |
                               ((unsigned)(FA_ROWS >> 4) << 24);
      const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /* v is MN-major */ |
                               ((unsigned)(HEAD_DIM >> 3) << 17) | ((unsigned)(FA_ROWS >> 4) << 24);
      bool ok = fa_mbar_wait(q_full, 0);
      for (int b = 0; ok && b < n_blocks; ++b) {
        const int buf = b & 1;
        if (!fa_mbar_wait(&kv_full[buf], (b >> 1) & 1)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // S = Q K^T over the head's lanes, 16 at a time (32 bytes inside a swizzled row)
#pragma unroll
        for (int kk = 0; kk < HEAD_DIM / 16; ++kk) {
          const unsigned long long a = desc_k_major(q_s + (kk / 4) * kSubTile) + 2 * (kk % 4);
          const unsigned long long bd = desc_k_major(k_s + buf * kKVBytes + (kk / 4) * kSubTile) + 2 * (kk % 4);
          fa_mma(tmem_s, a, bd, idesc_s, kk != 0);
        }
        fa_commit(s_full);
        if (!fa_mbar_wait(p_ready, b & 1)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // P V over the block's keys, 16 at a time: p advances 32 bytes in its row (a new
        // sub-tile after 64 keys), v advances two 8-key groups (2048 bytes)
#pragma unroll
        for (int kk = 0; kk < FA_KEYS / 16; ++kk) {
          const unsigned long long a = desc_k_major(p_s + (kk / 4) * kSubTile) + 2 * (kk % 4);
          const unsigned long long bd = desc_mn_major(v_s + buf * kKVBytes) + (unsigned long long)(kk * 128);
          fa_mma(tmem_o, a, bd, idesc_o, kk != 0);
        }
        fa_commit(o_full);
        fa_commit(&kv_empty[buf]);
      }
    }
  } else if (live && warp < 4) {
    // ---------------- softmax: thread r owns row r ----------------
    const int r = threadIdx.x;
    const int p_row = pos0 + min(r, n_rows - 1);            // rows past the tile repeat its last row
    const int lo_row = (window >= 0 && p_row - window > 0) ? p_row - window : 0;
    const unsigned lane_base = ((unsigned)(warp * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f;
    float o[HEAD_DIM];
#pragma unroll
    for (int i = 0; i < HEAD_DIM; ++i) o[i] = 0.f;
    for (int b = 0; b < n_blocks; ++b) {
      const int kb = kb_first + b * FA_KEYS;
      if (!fa_mbar_wait(s_full, b & 1)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool needs_mask = kb + FA_KEYS - 1 > pos0 || (window >= 0 && kb < pos_last - window);
      // first pass: the row's maximum over the block
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_KEYS; c0 += 32) {
        float s[32];
        fa_tmem_load32(tmem_s + lane_base + (unsigned)c0, s);
        if (needs_mask) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = kb + c0 + j;
            m_blk = fmaxf(m_blk, (key <= p_row && key >= lo_row) ? s[j] : -INFINITY);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) m_blk = fmaxf(m_blk, s[j]);
        }
      }
      const float m_new = fmaxf(m_run, m_blk);
      const float m_scaled = m_new == -INFINITY ? 0.f : m_new * scale_log2;
      const float corr = fa_exp2(m_run * scale_log2 - m_scaled);      // 0 on the first block
      m_run = m_new;
      // second pass: probabilities, their sum, and the bfloat16 copy for the second product
      float sum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_KEYS; c0 += 32) {
        float s[32];
        fa_tmem_load32(tmem_s + lane_base + (unsigned)c0, s);
        if (needs_mask) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = kb + c0 + j;
            s[j] = (key <= p_row && key >= lo_row) ? fa_exp2(fmaf(s[j], scale_log2, -m_scaled)) : 0.f;
            sum += s[j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            s[j] = fa_exp2(fmaf(s[j], scale_log2, -m_scaled));
            sum += s[j];
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {                     // four 16-byte pieces of 8 keys
          uint4 piece;
          unsigned* w = reinterpret_cast<unsigned*>(&piece);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 pair = __floats2bfloat162_rn(s[8 * c + 2 * e], s[8 * c + 2 * e + 1]);
            w[e] = *reinterpret_cast<unsigned*>(&pair);
          }
          const int chunk = c0 / 8 + c;                   // 0 .. 15 over the 128 keys
          *reinterpret_cast<uint4*>(p_s + (chunk / 8) * kSubTile + swz(r, chunk % 8)) = piece;
        }
      }
      l_run = l_run * corr + sum;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // p in shared memory -> the tensor core
      fa_mbar_arrive(p_ready);
      // fold the block's P V into the row's output
      if (!fa_mbar_wait(o_full, b & 1)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < HEAD_DIM; c0 += 32) {
        float pv[32];
        fa_tmem_load32(tmem_o + lane_base + (unsigned)c0, pv);
#pragma unroll
        for (int j = 0; j < 32; ++j) o[c0 + j] = o[c0 + j] * corr + pv[j];
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (r < n_rows) {
      const float inv = 1.0f / l_run;
      __nv_bfloat16* dst = out + ((size_t)(row0 + r) * nh + h) * HEAD_DIM;
#pragma unroll
      for (int c = 0; c < HEAD_DIM / 8; ++c) {
        uint4 piece;
        unsigned* w = reinterpret_cast<unsigned*>(&piece);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 pair = __floats2bfloat162_rn(o[8 * c + 2 * e] * inv, o[8 * c + 2 * e + 1] * inv);
          w[e] = *reinterpret_cast<unsigned*>(&pair);
        }
        *reinterpret_cast<uint4*>(dst + c * 8) = piece;
      }
    }
  }
  // ---------------- common exit ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  pdl_launch();
  if (warp == 8) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s),
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
  if (d != HEAD_DIM || nh <= 0 || nkv <= 0 || nh % nkv || page <= 0 || nh > 65535)
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
  dim3 grid(n_tiles, nh);
  return launch_dependent(attention_tcgen05_kernel, grid, dim3(FA_THREADS), (size_t)kFaSmem, stream,
                          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
                          (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, block_table, table_stride,
                          row_req, pos, tiles, n_tiles, nh, nkv, page, window,
                          scale * 1.4426950408889634f);
}
