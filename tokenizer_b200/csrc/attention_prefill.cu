// Attention for portions of prompts: many rows of one request at once, over the
// paged cache (bfloat16, tensor cores, 32-bit softmax).
//
// The rows of a step are cut on the host into tiles of up to 64 consecutive rows
// of one request.  A block takes one (tile, query head): its four warps hold 16
// rows each, walk the request's keys in blocks of 64 from the first key any row of
// the tile can see to the tile's last position, and keep a running maximum, sum
// and weighted value per row (the flash-attention recurrence).  Keys and values
// are gathered from their pages into shared memory with 16-byte asynchronous
// copies, a ring of three blocks deep (the look-up in the block table runs one block
// further ahead), so any page size works.  q k^T and p v run on mma.sync m16n8k16 with fragments read by
// ldmatrix from rows padded by 16 bytes (conflict-free for every head size that
// is a multiple of 16).  A row's arithmetic depends on its position, its window
// and its place in its 64-row tile only.
//
// HEAD_DIM is a compile-time size (multiple of 16, at most 128), -DHEAD_DIM=...
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 128, "head size");

#define PF_ROWS 64          // rows of a tile (4 warps x 16)
#define PF_KEYS 64          // keys of a block
#define PF_THREADS 128
#define PF_STAGES 3         // key/value blocks in flight
constexpr int kStride = HEAD_DIM + 8;          // elements between rows in shared memory
constexpr int kChunks = HEAD_DIM / 8;          // 16-byte pieces of a row
constexpr int kTile = PF_KEYS * kStride;       // elements of one staged tile

__device__ __forceinline__ unsigned smem_addr(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool ok) {
  const int bytes = ok ? 16 : 0;   // 0: the 16 bytes are filled with zeros, src is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src),
               "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (one instruction; relative error about 2^-22,
// far inside the bfloat16 rounding the probabilities get next)
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Staging of the keys and the values key0 .. key0 + 63 of one kv head.  Two threads
// share a key: one look-up in the block table serves the key's and the value's row.
// The look-up (a dependent load) is made one block ahead of the copies that use it,
// so the copies of a block are issued without waiting.  Keys outside [first_ok,
// last_ok] are zero-filled and their pages are not touched (offset -1).
// The page of this thread's key in the block starting at key0 (-1: the key is not to
// be read).  Only the load is issued here; `kv_row_offset` turns it into an offset
// when the copies are issued, one block later, so nothing waits for the load.
__device__ __forceinline__ int kv_page(const int* __restrict__ table, int page, int key0, int first_ok,
                                       int last_ok) {
  static_assert(PF_THREADS == 2 * PF_KEYS && kChunks % 2 == 0, "two threads a key");
  const int key = key0 + (threadIdx.x >> 1);
  if (key < first_ok || key > last_ok) return -1;
  return table[key / page];
}
__device__ __forceinline__ long long kv_row_offset(int pg, int page, int nkv, int kvh, int key0) {
  if (pg < 0) return -1;
  const int key = key0 + (threadIdx.x >> 1);
  return ((long long)(pg * page + key % page) * nkv + kvh) * HEAD_DIM;
}
__device__ __forceinline__ void stage_kv(__nv_bfloat16* k_dst, __nv_bfloat16* v_dst,
                                         const __nv_bfloat16* __restrict__ k_pool,
                                         const __nv_bfloat16* __restrict__ v_pool, long long offset) {
  const int j = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * (kChunks / 2);
  const bool ok = offset >= 0;
  const size_t at = ok ? (size_t)offset : 0;
#pragma unroll
  for (int c = 0; c < kChunks / 2; ++c) {
    cp_async16(k_dst + j * kStride + (c0 + c) * 8, k_pool + at + (c0 + c) * 8, ok);
    cp_async16(v_dst + j * kStride + (c0 + c) * 8, v_pool + at + (c0 + c) * 8, ok);
  }
}

__global__ void __launch_bounds__(PF_THREADS)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ row_req, const int* __restrict__ pos,
                         const int* __restrict__ tiles, int n_tiles, int nh, int nkv, int page,
                         int window, float scale_log2) {
  extern __shared__ __align__(16) __nv_bfloat16 smem[];
  __nv_bfloat16* q_s = smem;                       // [64][kStride]
  __nv_bfloat16* k_s = q_s + kTile;                // PF_STAGES tiles
  __nv_bfloat16* v_s = k_s + PF_STAGES * kTile;    // PF_STAGES tiles

  // The host orders the tiles by the number of key blocks they walk, most first, so
  // the blocks that run longest start first and the short ones fill in behind them.
  const int h = blockIdx.y;
  const int tile = blockIdx.x;
  if (tile >= n_tiles) return;
  const int row0 = tiles[2 * tile], n_rows = tiles[2 * tile + 1];
  const int r = row_req[row0];
  if (r < 0 || n_rows <= 0) return;
  const int kvh = h / (nh / nkv);
  const int pos0 = pos[row0];
  const int pos_last = pos0 + n_rows - 1;
  const int lo_first = (window >= 0 && pos0 - window > 0) ? pos0 - window : 0;  // first key any row sees
  const int* table = block_table + (size_t)r * table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  // ---- stage q and the first key/value block ----
  for (int i = threadIdx.x; i < PF_ROWS * kChunks; i += PF_THREADS) {
    const int j = i / kChunks, c = i % kChunks;
    const bool ok = j < n_rows;
    const __nv_bfloat16* src = ok ? q + ((size_t)(row0 + j) * nh + h) * HEAD_DIM + c * 8 : q;
    cp_async16(q_s + j * kStride + c * 8, src, ok);
  }
  const int kb_first = lo_first / PF_KEYS * PF_KEYS;
  const int n_blocks = (pos_last - kb_first) / PF_KEYS + 1;
  // fill the ring: blocks 0 .. PF_STAGES - 2 (q rides in the first group); a group is
  // committed for every block, existing or not, so that group counts stay in step
#pragma unroll
  for (int b = 0; b < PF_STAGES - 1; ++b) {
    if (b < n_blocks) {
      const int key0 = kb_first + b * PF_KEYS;
      stage_kv(k_s + b * kTile, v_s + b * kTile, k_pool, v_pool,
               kv_row_offset(kv_page(table, page, key0, lo_first, pos_last), page, nkv, kvh, key0));
    }
    cp_async_commit();
  }
  int next_page = PF_STAGES - 1 < n_blocks
      ? kv_page(table, page, kb_first + (PF_STAGES - 1) * PF_KEYS, lo_first, pos_last) : -1;

  // per thread: rows g and g + 8 of the warp's 16
  const int my_row[2] = {warp * 16 + g, warp * 16 + g + 8};
  int p_row[2], lo_row[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    p_row[i] = pos0 + min(my_row[i], n_rows - 1);       // rows past the tile repeat its last row
    lo_row[i] = (window >= 0 && p_row[i] - window > 0) ? p_row[i] - window : 0;
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HEAD_DIM / 8][4];
#pragma unroll
  for (int i = 0; i < HEAD_DIM / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  unsigned q_frag[HEAD_DIM / 16][4];

  for (int b = 0; b < n_blocks; ++b) {
    const int kb = kb_first + b * PF_KEYS;
    const int stage = b % PF_STAGES;
    cp_async_wait<PF_STAGES - 2>();                 // block b has landed (for this thread)
    __syncthreads();                                // ... for all; and block b - 1 is no longer read
    {
      const int nb = b + PF_STAGES - 1;             // goes where block b - 1 was
      if (nb < n_blocks)
        stage_kv(k_s + (nb % PF_STAGES) * kTile, v_s + (nb % PF_STAGES) * kTile, k_pool, v_pool,
                 kv_row_offset(next_page, page, nkv, kvh, kb_first + nb * PF_KEYS));
      cp_async_commit();
      next_page = nb + 1 < n_blocks
          ? kv_page(table, page, kb_first + (nb + 1) * PF_KEYS, lo_first, pos_last) : -1;
    }
    if (b == 0) {
#pragma unroll
      for (int ks = 0; ks < HEAD_DIM / 16; ++ks)
        ldmatrix_x4(q_frag[ks], q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kStride +
                                    ks * 16 + (lane >> 4) * 8);
    }
    const __nv_bfloat16* kt = k_s + stage * kTile;
    const __nv_bfloat16* vt = v_s + stage * kTile;

    // ---- scores s[16 x 64] = q k^T ----
    float s[PF_KEYS / 8][4];
#pragma unroll
    for (int i = 0; i < PF_KEYS / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    // the fragments of step ks + 1 are read while the products of step ks run
    {
      unsigned kf[2][PF_KEYS / 16][4];
      const __nv_bfloat16* k_lane = kt + ((lane & 7) + (lane >> 4) * 8) * kStride + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int np = 0; np < PF_KEYS / 16; ++np) ldmatrix_x4(kf[0][np], k_lane + np * 16 * kStride);
#pragma unroll
      for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
        if (ks + 1 < HEAD_DIM / 16) {
#pragma unroll
          for (int np = 0; np < PF_KEYS / 16; ++np)
            ldmatrix_x4(kf[(ks + 1) & 1][np], k_lane + np * 16 * kStride + (ks + 1) * 16);
        }
#pragma unroll
        for (int np = 0; np < PF_KEYS / 16; ++np) {
          mma16816(s[2 * np], q_frag[ks], kf[ks & 1][np][0], kf[ks & 1][np][1]);
          mma16816(s[2 * np + 1], q_frag[ks], kf[ks & 1][np][2], kf[ks & 1][np][3]);
        }
      }
    }
    // ---- mask (only in blocks that reach past a row's position or before its window),
    // running softmax on the raw scores: exp2(s * c - max * c), c = scale * log2(e) ----
    const bool needs_mask = kb + PF_KEYS - 1 > pos0 || (window >= 0 && kb < pos_last - window);
    if (needs_mask) {
#pragma unroll
      for (int nt = 0; nt < PF_KEYS / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kb + nt * 8 + 2 * t + (e & 1);
          if (key > p_row[e >> 1] || key < lo_row[e >> 1]) s[nt][e] = -INFINITY;
        }
      }
    }
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < PF_KEYS / 8; ++nt) {
      m_new[0] = fmaxf(m_new[0], fmaxf(s[nt][0], s[nt][1]));
      m_new[1] = fmaxf(m_new[1], fmaxf(s[nt][2], s[nt][3]));
    }
    float corr[2], m_scaled[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
      // nothing seen yet (all keys of the block hidden from this row): keep exp2() finite
      m_scaled[i] = m_new[i] == -INFINITY ? 0.f : m_new[i] * scale_log2;
      corr[i] = exp2_approx(m_run[i] * scale_log2 - m_scaled[i]);     // exp2(-inf) = 0 on the first block
      m_run[i] = m_new[i];
    }
#pragma unroll
    for (int nt = 0; nt < PF_KEYS / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pe = exp2_approx(fmaf(s[nt][e], scale_log2, -m_scaled[e >> 1]));
        s[nt][e] = pe;
        sum[e >> 1] += pe;
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
      l_run[i] = l_run[i] * corr[i] + sum[i];
    }
#pragma unroll
    for (int i = 0; i < HEAD_DIM / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    // ---- o += p v ----
    {
      // value fragments are read in groups of four (64 lanes of the head) ahead of their products
      constexpr int kGroups = (HEAD_DIM / 16 + 3) / 4;
      const __nv_bfloat16* v_lane = vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * kStride + (lane >> 4) * 8;
#pragma unroll
      for (int ks = 0; ks < PF_KEYS / 16; ++ks) {
        unsigned pf[4];
        pf[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
        pf[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
        pf[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
        pf[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
        for (int grp = 0; grp < kGroups; ++grp) {
          unsigned vf[4][4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int dp = grp * 4 + i;
            if (dp < HEAD_DIM / 16) ldmatrix_x4_trans(vf[i], v_lane + ks * 16 * kStride + dp * 16);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int dp = grp * 4 + i;
            if (dp < HEAD_DIM / 16) {
              mma16816(o[2 * dp], pf, vf[i][0], vf[i][1]);
              mma16816(o[2 * dp + 1], pf, vf[i][2], vf[i][3]);
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- write the rows that exist ----
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (my_row[i] >= n_rows) continue;
    const float inv = 1.0f / l_run[i];
    __nv_bfloat16* dst = out + ((size_t)(row0 + my_row[i]) * nh + h) * HEAD_DIM;
#pragma unroll
    for (int nt = 0; nt < HEAD_DIM / 8; ++nt) {
      *reinterpret_cast<unsigned*>(dst + nt * 8 + 2 * t) =
          pack_bf16(o[nt][2 * i] * inv, o[nt][2 * i + 1] * inv);
    }
  }
}

TOKB200_API int tokb200_prefill_attention_head_dim() { return HEAD_DIM; }

// tiles: [n_tiles][2] = (first row, rows) of consecutive rows of one request, rows <= 64
TOKB200_API int tokb200_prefill_attention(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* block_table,
    int table_stride, const int* row_req, const int* pos, const int* tiles, int n_tiles, int nh,
    int nkv, int d, int page, int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return TOKB200_OK;
  if (d != HEAD_DIM || nh <= 0 || nkv <= 0 || nh % nkv || page <= 0 || nh > 65535)
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15)
    return TOKB200_BAD_ALIGNMENT;
  const size_t smem = (size_t)(1 + 2 * PF_STAGES) * kTile * sizeof(__nv_bfloat16);
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!configured[device]) {   // the larger shared memory is granted per device
    cudaError_t err = cudaFuncSetAttribute(prefill_attention_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured[device] = true;
  }
  dim3 grid(n_tiles, nh);
  const float scale_log2 = scale * 1.4426950408889634f;
  prefill_attention_kernel<<<grid, PF_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
      (__nv_bfloat16*)out, block_table, table_stride, row_req, pos, tiles, n_tiles, nh, nkv, page,
      window, scale_log2);
  return tokb200_launch_status();
}
