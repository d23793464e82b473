// Attention for rows that read far more keys than they bring: decoding
// (bfloat16, tensor cores, 32-bit softmax).
//
// One block works on (a row, one kv head, one split of that row's keys) and
// serves all query heads of the kv head's group at once: the group is the M side
// of mma.sync m16n8k16 (up to 16 heads), the keys are its N side, so keys and
// values are read once per group and a 32-key tile costs a warp a few dozen
// instructions.  q k^T takes its fragments straight from 16-byte global loads (a
// dot product does not care about the order of the head's lanes, so a thread's 8
// consecutive lanes are handed to two instructions under permuted k slots, the
// same permutation for q and k); p v needs v transposed, so each warp stages its
// tile's values in shared memory and reads them with ldmatrix.trans.
//
// A row's visible keys lo..pos are cut into n_splits pieces of `chunk` keys; chunk is
// min_chunk * 2^k, the smallest that needs at most MAX_SPLITS pieces.  The launcher picks
// min_chunk (256 .. 2048) for the launch as a whole from the number of (row, kv head) pairs
// and the table's reach: with few pairs, short pieces on many blocks win (a block's time is
// a chain of dependent loads per pass); with many pairs, long pieces win (fewer blocks than
// the device holds at once cost no second wave, and fewer pieces cost less merging).  The
// cut thus changes with the batch, which changes the order of the 32-bit merge, nothing else.  The eight warps of a block take tiles of 32 keys in turn, each with its
// own running maximum, sum and weighted values; they are merged once at the end.  Pieces of several blocks meet in scratch memory (max, sum, weighted
// values per (row, head, split)); the block that finishes last for a (row, kv
// head) merges them in index order and writes the output.
//
// HEAD_DIM is a compile-time size (a multiple of 16, at most 256), given with
// -DHEAD_DIM=...; the library is built per head size at first use.
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
#define DEC_WARPS 8
#define DEC_THREADS (DEC_WARPS * 32)
#define DEC_MAX_GROUP 16       // query heads per kv head: the rows of one mma
#define DEC_MAX_SPLITS 32
#define DEC_TILE 32            // keys a warp takes per pass
#define DEC_BLOCK_KEYS (DEC_WARPS * DEC_TILE)   // keys a block takes per pass
#define DEC_MIN_CHUNK 256      // one pass of a block's warps: the shortest piece a launch may choose

static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size");
constexpr int kSteps32 = HEAD_DIM / 32;              // steps of 32 lanes: one 16-byte load, two mma
constexpr bool kTail16 = HEAD_DIM % 32 != 0;         // one more step of 16 lanes: an 8-byte load
// Where lane t of a quad reads its 8 elements of step `st` in a row of q or of keys.  Steps go in
// pairs over 64 elements, in which a lane's two pieces lie next to each other (32 bytes), so
// that a quad's two loads ask for one whole 128-byte line of the row; a last step without a
// partner takes 8t.  q and the keys use the same places, which is all a dot product needs.
__device__ __forceinline__ int dec_k_offset(int st, int t) {
  return (st | 1) < kSteps32 ? (st >> 1) * 64 + 16 * t + 8 * (st & 1) : st * 32 + 8 * t;
}
constexpr int kVStride = HEAD_DIM + 8;               // elements between staged value rows
constexpr int kVBuffers = HEAD_DIM <= 128 ? 2 : 1;   // staging buffers of values a warp (two fit up to 128)

__device__ __forceinline__ int split_chunk(int n_keys, int min_chunk) {
  int chunk = min_chunk;
  while ((n_keys + chunk - 1) / chunk > DEC_MAX_SPLITS) chunk <<= 1;
  return chunk;
}
__device__ __forceinline__ void dec_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void dec_ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ unsigned dec_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ uint4 dec_load16(const __nv_bfloat16* p, bool ok) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (ok) v = *reinterpret_cast<const uint4*>(p);
  return v;
}
__device__ __forceinline__ uint2 dec_load8(const __nv_bfloat16* p, bool ok) {
  uint2 v = make_uint2(0u, 0u);
  if (ok) v = *reinterpret_cast<const uint2*>(p);
  return v;
}

#define DEC_CLUSTER_MAX 8      // pieces that can meet through distributed shared memory

__device__ __forceinline__ void dec_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// a float of block `rank` of this cluster, at the place `local` has in this block's shared memory
__device__ __forceinline__ float dec_peer_load(const float* local, unsigned rank) {
  const unsigned mine = (unsigned)__cvta_generic_to_shared(local);
  unsigned theirs;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(theirs) : "r"(mine), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(theirs) : "memory");
  return v;
}

// CLUSTER: the grid's x (the pieces of a row) is one thread-block cluster; the pieces meet in
// the first block through distributed shared memory instead of scratch memory, a fence and a
// counter.
// EARLY: the warps' first tiles are asked for before the wait on the predecessor (short pieces,
// where a trip to memory is a good part of the kernel's time; in a long piece it only costs registers).
template <bool CLUSTER, bool EARLY>
__global__ void __launch_bounds__(DEC_THREADS, HEAD_DIM <= 64 ? 2 : 1)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ row_req, const int* __restrict__ pos, int nh,
                        int nkv, int page, int window, float scale,
                        float* __restrict__ scratch, int* __restrict__ counters, int min_chunk,
                        const int* __restrict__ rows) {
  extern __shared__ __align__(16) unsigned char dec_smem[];
  __shared__ int is_last;
  // The rows' requests, positions and block tables were written before the predecessor (the
  // projection that writes q and the newest key) started, so they are read while it still
  // runs; q, keys and values only after the wait.
  // `rows` (optional): the batch rows this launch serves, one per z (-1: none); scratch and
  // counters are indexed by z, q, out, positions and requests by the row
  const int split = blockIdx.x, kvh = blockIdx.y, z = blockIdx.z;
  const int row = rows ? rows[z] : z;
  const int r = row < 0 ? -1 : row_req[row];
  const int p = r < 0 ? 0 : pos[row];
  const int lo = (window >= 0 && p - window > 0) ? p - window : 0;
  const int n_keys = p - lo + 1;
  const int chunk = split_chunk(n_keys, min_chunk);
  const int n_splits = (n_keys + chunk - 1) / chunk;
  const bool idle = r < 0 || split >= n_splits;
  if (!idle) {
    // the block's table entries, into L1 for the lookups below
    const int first_page = (lo + split * chunk) / page, last_page = min(p, lo + split * chunk + chunk - 1) / page;
    for (int e = first_page + (int)threadIdx.x * 32; e <= last_page; e += DEC_THREADS * 32)
      asm volatile("prefetch.global.L1 [%0];" ::"l"(block_table + (size_t)r * table_stride + e));
    // ... and the keys and values of the block's first pass towards L2: all but the row's newest
    // key were written by earlier steps, so they can be asked for while the projection before
    // this kernel runs.  Only the first pass: asking for a long piece at once made the kernel
    // slower (268 MB at 64 rows of 8,192 keys: 76 us against 68 without).
    {
      const int* tb = block_table + (size_t)r * table_stride;
      const int k_first = lo + split * chunk, k_last = min(p, k_first + min(chunk, DEC_BLOCK_KEYS) - 1);
      for (int key = k_first + (int)threadIdx.x; key <= k_last; key += DEC_THREADS) {
        const size_t at = ((size_t)(tb[key / page] * page + key % page) * nkv + kvh) * HEAD_DIM;
#pragma unroll
        for (int c = 0; c < HEAD_DIM; c += 64) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(k_pool + at + c));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(v_pool + at + c));
        }
      }
    }
  }
  const int group = nh / nkv;                       // <= DEC_MAX_GROUP, checked by the launcher
  const int first = lo + split * chunk;
  const int last = min(p, first + chunk - 1);
  const int* table = block_table + (size_t)(r < 0 ? 0 : r) * table_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;

  // two staging buffers of values a warp: the next tile's values are on their way while this
  // tile is computed
  __nv_bfloat16* v_buf = reinterpret_cast<__nv_bfloat16*>(dec_smem) + (size_t)warp * kVBuffers * DEC_TILE * kVStride;

  // A tile's values go straight to a staging buffer (asynchronous 16-byte copies, zeros for idle
  // keys); its keys come as mma fragments in registers.  Both are asked for one tile AHEAD: the
  // next tile's values when this tile starts, the next tile's keys as soon as this tile's scores
  // are computed (the registers are free then), so that their trip to memory runs beside the
  // softmax and the weighted sum of this tile.  Lane l looks up the place of a tile's key l in
  // the block table, once for the keys and the values; the loads get a row's place from the
  // lane that looked it up.
  const int page_shift = (page & (page - 1)) == 0 ? __ffs(page) - 1 : -1;
  auto tile_slots = [&](int k0) {
    const int key = k0 + lane;
    if (key > last) return -1;
    const int pg = page_shift >= 0 ? key >> page_shift : key / page;
    return table[pg] * page + (key - pg * page);
  };
  auto stage_values = [&](int my_slot, __nv_bfloat16* dst_rows) {
    // the copies run over the tile's 16-byte pieces in order: neighbouring lanes take
    // neighbouring pieces of one row, so that every 32-byte sector is asked for once
    constexpr int kPieces = HEAD_DIM / 8;   // 16-byte pieces a row
#pragma unroll
    for (int c = 0; c < kPieces; ++c) {
      const int i = c * 32 + lane;
      const int row = i / kPieces, piece = i % kPieces;
      const int slot = __shfl_sync(0xffffffffu, my_slot, row);
      const __nv_bfloat16* src = v_pool + ((size_t)max(slot, 0) * nkv + kvh) * HEAD_DIM + piece * 8;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(dst_rows + row * kVStride + piece * 8);
      const int bytes = slot < 0 ? 0 : 16;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  uint4 kf[DEC_TILE / 8][kSteps32 > 0 ? kSteps32 : 1];
  uint2 kt[DEC_TILE / 8];
  auto load_keys = [&](int my_slot) {
#pragma unroll
    for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
      const int slot = __shfl_sync(0xffffffffu, my_slot, nt * 8 + g);
      const bool ok = slot >= 0;
      const __nv_bfloat16* krow = k_pool + ((size_t)max(slot, 0) * nkv + kvh) * HEAD_DIM;
#pragma unroll
      for (int st = 0; st < kSteps32; ++st) kf[nt][st] = dec_load16(krow + dec_k_offset(st, t), ok);
      if (kTail16) kt[nt] = dec_load8(krow + kSteps32 * 32 + 4 * t, ok);
    }
  };
  // The warp's first tile is asked for BEFORE the wait on the predecessor when none of its keys
  // is the row's newest (the only one the predecessor writes; all others are from earlier steps):
  // after the wait only q is still to come.
  int turn = 0, slots_now = -1;
  const int k_mine = first + warp * DEC_TILE;
  const bool have_tile = !idle && k_mine <= last;
  const bool early = EARLY && have_tile && k_mine + DEC_TILE - 1 < p;
  if (early) {
    slots_now = tile_slots(k_mine);
    if (kVBuffers == 2) stage_values(slots_now, v_buf);
    load_keys(slots_now);
  }
  pdl_wait();
  pdl_launch();
  if (idle) {
    // in a cluster whose row is live, a block without keys still keeps the two appointments
    if (CLUSTER && r >= 0) {
      dec_cluster_sync();
      dec_cluster_sync();
    }
    return;
  }
  // ---- q fragments: heads g and g + 8 of the group, lanes in the permuted order ----
  unsigned qa[kSteps32 > 0 ? kSteps32 : 1][2][4];
  unsigned qt[4];
  {
    const bool ok_a = g < group, ok_b = g + 8 < group;
    const __nv_bfloat16* qa_row = q + ((size_t)row * nh + kvh * group + g) * HEAD_DIM;
    const __nv_bfloat16* qb_row = qa_row + (size_t)8 * HEAD_DIM;
#pragma unroll
    for (int st = 0; st < kSteps32; ++st) {
      const uint4 a = dec_load16(qa_row + dec_k_offset(st, t), ok_a);
      const uint4 b = dec_load16(qb_row + dec_k_offset(st, t), ok_b);
      qa[st][0][0] = a.x; qa[st][0][1] = b.x; qa[st][0][2] = a.y; qa[st][0][3] = b.y;
      qa[st][1][0] = a.z; qa[st][1][1] = b.z; qa[st][1][2] = a.w; qa[st][1][3] = b.w;
    }
    if (kTail16) {
      const uint2 a = dec_load8(qa_row + kSteps32 * 32 + 4 * t, ok_a);
      const uint2 b = dec_load8(qb_row + kSteps32 * 32 + 4 * t, ok_b);
      qt[0] = a.x; qt[1] = b.x; qt[2] = a.y; qt[3] = b.y;
    }
  }

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HEAD_DIM / 8][4];
#pragma unroll
  for (int i = 0; i < HEAD_DIM / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const float scale_log2 = scale * 1.4426950408889634f;
  if (have_tile && !early) {
    slots_now = tile_slots(k_mine);
    if (kVBuffers == 2) stage_values(slots_now, v_buf);
    load_keys(slots_now);
  }
  for (int k0 = first + warp * DEC_TILE; k0 <= last; k0 += DEC_BLOCK_KEYS, turn ^= 1) {
    __nv_bfloat16* v_s = v_buf + (size_t)(kVBuffers == 2 ? turn : 0) * DEC_TILE * kVStride;
    const bool more = k0 + DEC_BLOCK_KEYS <= last;
    const int slots_next = more ? tile_slots(k0 + DEC_BLOCK_KEYS) : -1;
    if (kVBuffers == 1) stage_values(slots_now, v_s);   // the last tile's sum is done (the __syncwarp below)
    else if (more) stage_values(slots_next, v_buf + (size_t)(turn ^ 1) * DEC_TILE * kVStride);
    slots_now = slots_next;
    float s[DEC_TILE / 8][4];
#pragma unroll
    for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int st = 0; st < kSteps32; ++st) {
        dec_mma(s[nt], qa[st][0], kf[nt][st].x, kf[nt][st].y);
        dec_mma(s[nt], qa[st][1], kf[nt][st].z, kf[nt][st].w);
      }
      if (kTail16) dec_mma(s[nt], qt, kt[nt].x, kt[nt].y);
    }
    if (more) load_keys(slots_next);
    // ---- scale, mask, running softmax: rows g (heads 0..7) and g + 8 (heads 8..15) ----
    float m_new[2] = {m_run[0], m_run[1]};
    if (k0 + DEC_TILE - 1 <= last) {          // a whole tile (every tile of a piece but its last): no key to mask
#pragma unroll
      for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] *= scale_log2;
          m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nt][e]);
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = k0 + nt * 8 + 2 * t + (e & 1);
          s[nt][e] = key <= last ? s[nt][e] * scale_log2 : -INFINITY;
          m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nt][e]);
        }
      }
    }
    float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));   // finite: key k0 is live
      corr[i] = exp2f(m_run[i] - m_new[i]);                                   // 0 on the first pass
      m_run[i] = m_new[i];
    }
#pragma unroll
    for (int nt = 0; nt < DEC_TILE / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pe = exp2f(s[nt][e] - m_new[e >> 1]);
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
    if (kVBuffers == 2 && more) asm volatile("cp.async.wait_group 1;\n" ::: "memory");   // this tile's values have landed (the next tile's may not)
    else asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncwarp();
    // ---- o += p v ----
#pragma unroll
    for (int ks = 0; ks < DEC_TILE / 16; ++ks) {
      unsigned pf[4];
      pf[0] = dec_pack(s[2 * ks][0], s[2 * ks][1]);
      pf[1] = dec_pack(s[2 * ks][2], s[2 * ks][3]);
      pf[2] = dec_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pf[3] = dec_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int dp = 0; dp < HEAD_DIM / 16; ++dp) {
        unsigned vf[4];
        dec_ldmatrix_x4_trans(vf, v_s + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kVStride +
                                      dp * 16 + (lane >> 4) * 8);
        dec_mma(o[2 * dp], pf, vf[0], vf[1]);
        dec_mma(o[2 * dp + 1], pf, vf[2], vf[3]);
      }
    }
    __syncwarp();   // the staged values are overwritten by the next tile
  }

  // ---- merge the warps of the block (the merge buffer takes the place of the staging area) ----
  __syncthreads();
  float* acc_s = reinterpret_cast<float*>(dec_smem);           // [warp][head][HEAD_DIM + 2]
  constexpr int kRow = HEAD_DIM + 2;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int head = g + 8 * i;
    if (head < group) {
      float* dst = acc_s + ((size_t)warp * group + head) * kRow;
#pragma unroll
      for (int nt = 0; nt < HEAD_DIM / 8; ++nt) {
        dst[nt * 8 + 2 * t] = o[nt][2 * i];
        dst[nt * 8 + 2 * t + 1] = o[nt][2 * i + 1];
      }
      if (t == 0) { dst[HEAD_DIM] = m_run[i]; dst[HEAD_DIM + 1] = l_run[i]; }
    }
  }
  __syncthreads();

  // scratch layout per (row, head): [split][HEAD_DIM + 2] = weighted values, max (log2 units), sum
  const size_t per_head = (size_t)DEC_MAX_SPLITS * kRow;
  float* base = scratch + ((size_t)z * nh + kvh * group) * per_head;
  float* piece_s = acc_s + (size_t)DEC_WARPS * group * kRow;     // CLUSTER: this block's piece, [head][kRow]
  for (int i = tid; i < group * HEAD_DIM; i += DEC_THREADS) {
    const int head = i / HEAD_DIM, c = i % HEAD_DIM;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, acc_s[((size_t)w * group + head) * kRow + HEAD_DIM]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float* src = acc_s + ((size_t)w * group + head) * kRow;
      const float f = exp2f(src[HEAD_DIM] - m);          // a warp without keys has max -inf: weight 0
      num += f * src[c];
      den += f * src[HEAD_DIM + 1];
    }
    if (CLUSTER) {
      float* piece = piece_s + (size_t)head * kRow;
      piece[c] = num;
      if (c == 0) { piece[HEAD_DIM] = m; piece[HEAD_DIM + 1] = den; }
    } else if (n_splits == 1) {
      out[((size_t)row * nh + kvh * group + head) * HEAD_DIM + c] = __float2bfloat16_rn(num / den);
    } else {
      float* piece = base + head * per_head + (size_t)split * kRow;
      piece[c] = num;
      if (c == 0) { piece[HEAD_DIM] = m; piece[HEAD_DIM + 1] = den; }
    }
  }
  if (CLUSTER) {
    // ---- the pieces meet in the first block, read from their blocks' shared memory ----
    dec_cluster_sync();
    if (split == 0) {
      for (int head = warp; head < group; head += DEC_WARPS) {
        const float* piece = piece_s + (size_t)head * kRow;
        const bool on = lane < n_splits;
        const float m_s = on ? dec_peer_load(piece + HEAD_DIM, (unsigned)lane) : -INFINITY;
        const float l_s = on ? dec_peer_load(piece + HEAD_DIM + 1, (unsigned)lane) : 0.f;
        const float m_all = warp_max(m_s);
        const float f = exp2f(m_s - m_all);                 // 0 for lanes without a piece
        const float den = warp_sum(f * l_s);
        for (int c0 = 0; c0 < HEAD_DIM; c0 += 32) {
          const int c = c0 + lane;
          const bool have = c < HEAD_DIM;
          float v[DEC_CLUSTER_MAX];
#pragma unroll
          for (int sp = 0; sp < DEC_CLUSTER_MAX; ++sp)
            v[sp] = (have && sp < n_splits) ? dec_peer_load(piece + c, (unsigned)sp) : 0.f;
          float num = 0.f;
#pragma unroll
          for (int sp = 0; sp < DEC_CLUSTER_MAX; ++sp) num += __shfl_sync(0xffffffffu, f, sp) * v[sp];
          if (have) out[((size_t)row * nh + kvh * group + head) * HEAD_DIM + c] = __float2bfloat16_rn(num / den);
        }
      }
    }
    dec_cluster_sync();            // nobody leaves while its piece may still be read
    return;
  }
  if (n_splits == 1) return;
  // ---- the last block to finish merges the pieces, in index order ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int done = atomicAdd(&counters[z * nkv + kvh], 1);
    is_last = done == n_splits - 1;
    if (is_last) counters[z * nkv + kvh] = 0;     // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // a warp per head: lane s holds split s's maximum and sum
  for (int head = warp; head < group; head += DEC_WARPS) {
    const float* pieces = base + head * per_head;
    const bool on = lane < n_splits;
    const float m_s = on ? __ldcg(&pieces[(size_t)lane * kRow + HEAD_DIM]) : -INFINITY;
    const float l_s = on ? __ldcg(&pieces[(size_t)lane * kRow + HEAD_DIM + 1]) : 0.f;
    const float m_all = warp_max(m_s);
    const float f = exp2f(m_s - m_all);                   // 0 for lanes without a split
    const float den = warp_sum(f * l_s);
    for (int c0 = 0; c0 < HEAD_DIM; c0 += 32) {
      const int c = c0 + lane;
      const bool have = c < HEAD_DIM;
      float v[DEC_MAX_SPLITS];
#pragma unroll
      for (int sp = 0; sp < DEC_MAX_SPLITS; ++sp)
        v[sp] = (have && sp < n_splits) ? __ldcg(&pieces[(size_t)sp * kRow + c]) : 0.f;
      float num = 0.f;
#pragma unroll
      for (int sp = 0; sp < DEC_MAX_SPLITS; ++sp) num += __shfl_sync(0xffffffffu, f, sp) * v[sp];
      if (have) out[((size_t)row * nh + kvh * group + head) * HEAD_DIM + c] = __float2bfloat16_rn(num / den);
    }
  }
}

// floats of scratch and ints of counters a launch over n_rows needs
TOKB200_API long long tokb200_decode_attention_scratch_floats(int n_rows, int nh) {
  return (long long)n_rows * nh * DEC_MAX_SPLITS * (HEAD_DIM + 2);
}

TOKB200_API int tokb200_decode_attention_head_dim() { return HEAD_DIM; }

// `counters` holds n_rows * nkv ints, zero before the first launch; every launch
// leaves them zero again.  `rows` (optional, n_rows ints): the batch rows to serve, -1 for none;
// without it the launch serves rows 0 .. n_rows - 1.
TOKB200_API int tokb200_decode_attention(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* block_table,
    int table_stride, const int* row_req, const int* pos, int n_rows, int nh, int nkv, int d,
    int page, int window, float scale, float* scratch, int* counters, const int* rows,
    cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (d != HEAD_DIM || nh <= 0 || nkv <= 0 || nh % nkv || nh / nkv > DEC_MAX_GROUP || page <= 0 ||
      nkv > 65535 || n_rows > 65535)
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15)
    return TOKB200_BAD_ALIGNMENT;
  const int group = nh / nkv;
  const size_t stage = (size_t)kVBuffers * DEC_WARPS * DEC_TILE * kVStride * sizeof(__nv_bfloat16);
  const size_t merge = (size_t)(DEC_WARPS + 1) * group * (HEAD_DIM + 2) * sizeof(float);
  const size_t smem = stage > merge ? stage : merge;
  // no row sees more keys than its table reaches (or its window holds), so no row has
  // more pieces than this; blocks beyond would only find that out and leave
  long long reach = (long long)table_stride * page;
  if (window >= 0 && window + 1 < reach) reach = window + 1;
  // The shortest piece for this launch: the candidate (a whole number of passes of 256 keys)
  // with the least estimated time, from a block's fixed cost (3), 2 per pass of 256 keys at head
  // size 64 (in proportion for others), 3 for a merge across blocks, and as many waves as the
  // blocks need at the number of blocks a multiprocessor holds (figures in microseconds, fitted
  // to measurements at 8 and 64 rows, contexts of 600 to 16,000).  Pieces need not be powers of
  // two: 64 rows of 8,192 keys with 4 kv heads of size 128 take 213 us in pieces of 2,816 keys
  // (768 blocks, 5.2 waves of 148) against 266 us in pieces of 2,048 (1,024 blocks, 6.9 waves).
  static int slots = 0;      // blocks the device holds at once
  const long long pairs = (long long)n_rows * nkv;
  int min_chunk = DEC_MIN_CHUNK;
  {
    int& have = slots;
    if (!have) {
      int device = 0, sms = 148, per_sm = 0;
      if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(decode_attention_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_attention_kernel<false, false>, DEC_THREADS, smem) !=
              cudaSuccess || per_sm < 1)
        per_sm = 1;
      have = per_sm * sms;
    }
    const double per_pass = 2.0 * HEAD_DIM / 64.0;
    double best = 1e30;
    for (int c = DEC_MIN_CHUNK; c <= 4096; c += DEC_BLOCK_KEYS) {
      int chunk = c;
      while ((reach + chunk - 1) / chunk > DEC_MAX_SPLITS) chunk <<= 1;
      const long long pieces = (reach + chunk - 1) / chunk;
      const long long passes = ((reach < chunk ? reach : chunk) + DEC_BLOCK_KEYS - 1) / DEC_BLOCK_KEYS;
      const long long waves = (pairs * pieces + have - 1) / have;
      const double t = (double)waves * (3.0 + per_pass * (double)passes + (pieces > 1 ? 3.0 : 0.0));
      if (t < best - 1e-9) { best = t; min_chunk = c; }
    }
  }
  // no row has more pieces than this (a row a little shorter than the reach may be cut finer
  // than the reach itself would be: its pieces are counted from min_chunk, not from the
  // reach's chunk)
  long long most = (reach + min_chunk - 1) / min_chunk;
  if (most > DEC_MAX_SPLITS) most = DEC_MAX_SPLITS;
  if (most < 1) most = 1;
  // up to DEC_CLUSTER_MAX pieces: one cluster a (row, kv head), pieces merged through
  // distributed shared memory; more: scratch memory and the last block.  TOKB200_DECODE_MERGE
  // = scratch always takes the second way.
  static const bool clusters_allowed = [] {
    const char* v = getenv("TOKB200_DECODE_MERGE");
    return !(v && v[0] == 's');
  }();
  // ... and only while all blocks are resident at once: a block of a cluster whose row has fewer
  // pieces than the grid stays until its siblings are done, which costs nothing in a single wave
  // and a quarter of the device's block slots in a long run of uneven rows (64 rows of 4,900 to
  // 8,192 keys, head size 128: 227 us with clusters, 172 us through scratch memory)
  const bool cluster = clusters_allowed && most <= DEC_CLUSTER_MAX && pairs * most <= slots;
  // pieces of up to two passes: the first tiles before the wait (see EARLY)
  const bool early = min_chunk <= 2 * DEC_BLOCK_KEYS;
  void (*kernel)(const __nv_bfloat16*, const __nv_bfloat16*, const __nv_bfloat16*, __nv_bfloat16*, const int*,
                 int, const int*, const int*, int, int, int, int, float, float*, int*, int, const int*) =
      early ? (cluster ? decode_attention_kernel<true, true> : decode_attention_kernel<false, true>)
            : (cluster ? decode_attention_kernel<true, false> : decode_attention_kernel<false, false>);
  if (smem > 48 * 1024) {   // the larger shared memory is granted per device, once
    static bool configured[64][4] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
    if (!configured[device][2 * early + cluster]) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (err != cudaSuccess) return (int)err;
      configured[device][2 * early + cluster] = true;
    }
  }
  dim3 grid((unsigned)most, nkv, n_rows);
  if (!cluster)
    return launch_dependent(kernel, grid, dim3(DEC_THREADS), smem, stream,
                            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
                            (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, block_table,
                            table_stride, row_req, pos, nh, nkv, page, window, scale, scratch,
                            counters, min_chunk, rows);
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(DEC_THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  static const int overlap = [] {
    const char* v = getenv("TOKB200_PDL");
    return (v && v[0] == '0') ? 0 : 1;
  }();
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = overlap;
  attribute[1].id = cudaLaunchAttributeClusterDimension;
  attribute[1].val.clusterDim.x = (unsigned)most;
  attribute[1].val.clusterDim.y = 1;
  attribute[1].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 2;
  cudaError_t err = cudaLaunchKernelEx(&config, kernel, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
                                       (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, block_table,
                                       table_stride, row_req, pos, nh, nkv, page, window, scale, scratch,
                                       counters, min_chunk, rows);
  return err == cudaSuccess ? TOKB200_OK : (int)err;
}
