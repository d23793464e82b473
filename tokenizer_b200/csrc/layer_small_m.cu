// A whole decoder layer of a decoding step in ONE kernel, for few rows (M <= 32, bfloat16
// weights and cache, 32-bit sums): pre-norm residual arrangement, grouped-query attention with
// biases on q/k/v and a half-split rotary encoding over the paged cache, gated feed-forward.
//
//   x1 = x + pending                                   (32-bit residual sum; pending: the layer before)
//   h  = rms_norm(x1) * gain1                          (bfloat16)
//   q,k,v = h Wqkv^T + b; q,k rotated at the row's position; k,v -> the row's cache slot
//   a  = softmax(q k^T / sqrt(d)) v over the row's visible keys (window), per query head
//   x2 = x1 + a Wo^T
//   h2 = rms_norm(x2) * gain2
//   y  = (act(h2 Wg^T) * (h2 Wu^T)) Wd^T  as S partial sums over k (the next norm adds them)
//
// As separate kernels these are four launches whose time is mostly waiting (each starts cold,
// asks for a few hundred KB per SM, waits a trip to memory, computes for a microsecond).  Here
// one block per SM stays for the whole layer:
//   * a producer warp streams the block's share of ALL four weight matrices, in the order
//     they will be used, through a ring of shared-memory stages with bulk asynchronous copies
//     (cp.async.bulk, completion on an mbarrier).  It never waits for the arithmetic or for the
//     other blocks, only for a free stage, so the weights of a later product are already in
//     shared memory when the blocks come out of the barrier before it;
//   * eight consumer warps run the phases: norm (every block for itself: M rows are a few
//     KB), q/k/v row tiles out of the ring (mma.sync m16n8k16 with the weight rows as the M
//     side; a row tile is 8 lanes of a head and their 8 rotation partners, so a thread of the
//     epilogue holds both halves of a pair), attention over (row, kv head, piece of the keys)
//     units with the group's query heads as the M side of the mma, the pieces of a (row, kv
//     head) merged by the block that finishes last, then the output projection, the second
//     norm, gate/up with the activation, and down;
//   * between phases that need each other's results all blocks meet at a barrier in global
//     memory (one block per SM: all are resident).
// Sums have a fixed order: results are reproducible.  Every wait (mbarrier, grid barrier) is
// bounded; when one gives up an error flag is set, the block goes on to the end without
// touching the ring again and skips the later barriers' waits, and the host reads the flag.
//
// HEAD_DIM is a compile-time size (64 or 128 are built; any multiple of 32 up to 128 compiles).
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
static_assert(HEAD_DIM % 32 == 0 && HEAD_DIM >= 32 && HEAD_DIM <= 128, "head size of the layer kernel");

#define LAY_WARPS 8                          // consumer warps
#define LAY_CONSUMERS (LAY_WARPS * 32)
#define LAY_THREADS (LAY_CONSUMERS + 32)     // + the producer warp
#define LAY_KC 1024                          // k elements of a stage
#define LAY_ROW_PITCH (LAY_KC * 2 + 64)      // bytes between a stage's rows (64 mod 128: no bank conflicts)
#define LAY_STAGE_BYTES (16 * LAY_ROW_PITCH)
#ifndef LAY_WAIT_LIMIT
#define LAY_WAIT_LIMIT (1u << 16)            // polls of up to 20 us
#endif
#ifndef LAY_GRID_WAIT_LIMIT
#define LAY_GRID_WAIT_LIMIT (1u << 22)
#endif
#define LAY_MAX_SPLITS 32                    // pieces of a row's keys (a lane each in the merge)
#define LAY_TILE 32                          // keys a warp takes per pass
#define LAY_MAX_GROUP 16                     // query heads per kv head: the rows of one mma
#define LAY_TABLE_ENTRIES 256                // pages of a block's first attention unit kept in shared memory

constexpr int kVStride = HEAD_DIM + 8;       // elements between staged value rows
constexpr int kPieceRow = HEAD_DIM + 2;      // a piece: weighted values, max (log2 units), sum

__device__ int lay_error_flag = 0;

__device__ __forceinline__ unsigned lay_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lay_mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(lay_smem(bar)), "r"(count));
}
__device__ __forceinline__ void lay_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(lay_smem(bar)) : "memory");
}
__device__ __forceinline__ void lay_mbar_expect(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(lay_smem(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool lay_mbar_wait(unsigned long long* bar, unsigned parity) {
  const unsigned addr = lay_smem(bar);
  const unsigned suspend_ns = 20000u;
  for (unsigned spin = 0; spin < LAY_WAIT_LIMIT; ++spin) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity), "r"(suspend_ns) : "memory");
    if (done) return true;
  }
  atomicExch(&lay_error_flag, 1);
  tokb200_report_error(TOKB200_LIB_LAYER_SMALL_M, 1);
  return false;
}
__device__ __forceinline__ void lay_bulk_copy(void* dst, const void* src, unsigned bytes,
                                              unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(lay_smem(dst)), "l"(src), "r"(bytes), "r"(lay_smem(bar)) : "memory");
}
__device__ __forceinline__ void lay_consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(LAY_CONSUMERS) : "memory");
}
__device__ __forceinline__ void lay_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                        unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lay_ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(lay_smem(p)));
}
__device__ __forceinline__ unsigned lay_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
// data that another block of this launch wrote: read past L1, which is not coherent between SMs
__device__ __forceinline__ uint4 lay_load16_cg(const void* p, bool ok) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (ok) v = __ldcg(reinterpret_cast<const uint4*>(p));
  return v;
}

struct LayerParams {
  // ---- the layer's constants ----
  const __nv_bfloat16* w_qkv;   // [(nh + 2 nkv) d, H]
  const float* b_qkv;           // [(nh + 2 nkv) d] or null
  const __nv_bfloat16* w_o;     // [H, nh d]
  const float* gain1;           // [H]
  const float* gain2;           // [H]
  const __nv_bfloat16* w_gu;    // [2 I, H], 128 gate rows / 128 up rows interleaved
  const __nv_bfloat16* w_d;     // [H, I]
  __nv_bfloat16* k_pool;        // [slots, nkv, d]; null: this call reads another call's cache
  __nv_bfloat16* v_pool;
  const __nv_bfloat16* k_read;  // the pools attention reads (== k_pool where the call writes)
  const __nv_bfloat16* v_read;
  const float* cos_t;           // [positions, d / 2]
  const float* sin_t;
  float eps1, eps2, scale;
  int window, activation;
  // ---- the step ----
  const float* x_in;            // [M, H]
  const void* delta;            // pending: [M, H] bfloat16 or float32, or float32 [S, M, H]; may be null
  int delta_is_f32, n_partials;
  long long partial_stride;
  float* x_mid;                 // [M, H]: x_in + pending (written by block 0)
  float* x_out;                 // [M, H]: x_mid + the attention's output (written by block 0)
  float* out;                   // [s_down, M, H] partial sums of the feed-forward
  const int* pos;               // [M]
  const int* slot;              // [M] or null
  const int* row_req;           // [M], -1: idle row
  const int* block_table;       // [R, table_stride]
  int table_stride, page;
  // ---- scratch (global memory; all of it is written before it is read within a launch) ----
  __nv_bfloat16* q_buf;         // [M, nh d]
  float* att_part;              // [M, nh, LAY_MAX_SPLITS, d + 2]
  int* att_count;               // [M, nkv] zero between launches
  __nv_bfloat16* att_out;       // [M, nh d]
  float* o_part;                // [M, H]: the output projection
  __nv_bfloat16* act;           // [M, I]
  int* sync;                    // [2] zero between launches
  // ---- sizes and the plan ----
  int M, H, I, nh, nkv;
  int n_stages, h_pitch;        // h_pitch: bytes between rows of the activation tile in shared memory
  int s_down, k_per_split_d;    // the down projection's cut along k (k_per_split_d a multiple of 32)
  int att_splits;               // pieces a row's keys are cut into at most
  long long* stamps;            // null, or [blocks, 32]: the time (ns) at which a block's consumers pass each phase
  const __nv_bfloat16* next_w;  // null, or the q/k/v weight (same shape) of the layer that runs next: brought into L2
  const float* next_gain;       // ... its first norm's gain [H] and its q/k/v bias, likewise
  const float* next_bias;
  int repeat;                   // 1; more (profiling only): the same layer that many times in one launch
};

// One warp, one row of up to 128 KVEC elements kept in registers: x' = x + pending (the pending
// part is [M, H] bfloat16 or float32, or float32 partial sums [S, M, H], added in index order),
// h = x' / sqrt(mean(x'^2) + eps) * gain as a bfloat16 row in shared memory.  The loads of four
// 16-byte pieces of x and of up to three partial sums each are all asked for before the first is
// used (one trip to L2 per group, not one per array), and go past L1: another block of this
// launch may have written them.
template <int KVEC>
__device__ __forceinline__ void lay_norm_row(const float* __restrict__ xr, const void* delta, int delta_is_f32,
                                             int n_partials, long long stride, const float* __restrict__ gain,
                                             float eps, float* x_store, __nv_bfloat16* hrow, int H, int lane) {
  const float* df = reinterpret_cast<const float*>(delta);
  const __nv_bfloat16* dh = reinterpret_cast<const __nv_bfloat16*>(delta);
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr bool kGainEarly = KVEC <= 8;         // rows of up to 1024: the gain in the same trip as x
  float4 v[KVEC], gn[kGainEarly ? KVEC : 1];
#pragma unroll
  for (int grp = 0; grp < KVEC / 4; ++grp) {
    float4 a[3][4];
    uint2 raw[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = (lane + 32 * (grp * 4 + e)) * 4;
      const bool in = i < H;
      v[grp * 4 + e] = in ? __ldcg(reinterpret_cast<const float4*>(xr + i)) : zero4;
      if (kGainEarly) gn[grp * 4 + e] = in ? *reinterpret_cast<const float4*>(gain + i) : zero4;
      raw[e] = make_uint2(0u, 0u);
      if (delta && !delta_is_f32 && in) raw[e] = __ldcg(reinterpret_cast<const uint2*>(dh + i));
#pragma unroll
      for (int s = 0; s < 3; ++s)
        a[s][e] = (delta && delta_is_f32 && s < n_partials && in)
                      ? __ldcg(reinterpret_cast<const float4*>(df + (size_t)s * stride + i)) : zero4;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float4& t4 = v[grp * 4 + e];
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[e].x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[e].y));
      t4.x += lo.x; t4.y += lo.y; t4.z += hi.x; t4.w += hi.y;
#pragma unroll
      for (int s = 0; s < 3; ++s) {              // in index order
        t4.x += a[s][e].x; t4.y += a[s][e].y; t4.z += a[s][e].z; t4.w += a[s][e].w;
      }
    }
    if (delta && delta_is_f32) {
      for (int s0 = 3; s0 < n_partials; s0 += 3) {      // further partial sums, three at a time
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = (lane + 32 * (grp * 4 + e)) * 4;
#pragma unroll
          for (int s = 0; s < 3; ++s)
            a[s][e] = (s0 + s < n_partials && i < H)
                          ? __ldcg(reinterpret_cast<const float4*>(df + (size_t)(s0 + s) * stride + i)) : zero4;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float4& t4 = v[grp * 4 + e];
#pragma unroll
          for (int s = 0; s < 3; ++s) {
            t4.x += a[s][e].x; t4.y += a[s][e].y; t4.z += a[s][e].z; t4.w += a[s][e].w;
          }
        }
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < KVEC; ++e) {
    ss += v[e].x * v[e].x + v[e].y * v[e].y + v[e].z * v[e].z + v[e].w * v[e].w;
    const int i = (lane + 32 * e) * 4;
    if (x_store && i < H) *reinterpret_cast<float4*>(x_store + i) = v[e];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int e = 0; e < KVEC; ++e) {
    const int i = (lane + 32 * e) * 4;
    if (i < H) {
      const float4 g4 = kGainEarly ? gn[kGainEarly ? e : 0] : *reinterpret_cast<const float4*>(gain + i);
      const __nv_bfloat162 lo = __floats2bfloat162_rn(v[e].x * inv * g4.x, v[e].y * inv * g4.y);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(v[e].z * inv * g4.z, v[e].w * inv * g4.w);
      uint2 packed;
      packed.x = *reinterpret_cast<const unsigned*>(&lo);
      packed.y = *reinterpret_cast<const unsigned*>(&hi);
      *reinterpret_cast<uint2*>(hrow + i) = packed;
    }
  }
}

// The norm of all rows, a warp per row (rows past M: zeros).  `x_store` (block 0 only) receives x'.
template <int MT>
__device__ __forceinline__ void lay_norm(const float* x, const void* delta, int delta_is_f32, int n_partials,
                                         long long stride, const float* gain, float eps, float* x_store,
                                         unsigned char* h_s, int h_pitch, int M, int H, int warp, int lane) {
  for (int m = warp; m < 8 * MT; m += LAY_WARPS) {
    __nv_bfloat16* hrow = reinterpret_cast<__nv_bfloat16*>(h_s + (size_t)m * h_pitch);
    if (m >= M) {
      for (int i = lane * 2; i < H; i += 64) *reinterpret_cast<unsigned*>(hrow + i) = 0u;
      continue;
    }
    const float* xr = x + (size_t)m * H;
    const void* dr = nullptr;
    if (delta)
      dr = delta_is_f32 ? (const void*)(reinterpret_cast<const float*>(delta) + (size_t)m * H)
                        : (const void*)(reinterpret_cast<const __nv_bfloat16*>(delta) + (size_t)m * H);
    float* xs = x_store ? x_store + (size_t)m * H : nullptr;
    if (H <= 1024) lay_norm_row<8>(xr, dr, delta_is_f32, n_partials, stride, gain, eps, xs, hrow, H, lane);
    else if (H <= 2048) lay_norm_row<16>(xr, dr, delta_is_f32, n_partials, stride, gain, eps, xs, hrow, H, lane);
    else lay_norm_row<32>(xr, dr, delta_is_f32, n_partials, stride, gain, eps, xs, hrow, H, lane);
  }
}

// How the tiles of a product are dealt to the blocks: tile i of the product goes to block
// (first + i) mod G, so that the products with fewer tiles than blocks (q/k/v, output, down)
// start at different blocks and no block carries a share of all of them.
struct Deal {
  int n_tiles, first;
  __device__ __forceinline__ int mine(int cta, int G) const {        // tiles of this block
    const int offset = (cta - first % G + G) % G;
    return offset < n_tiles ? (n_tiles - offset + G - 1) / G : 0;
  }
  __device__ __forceinline__ int tile(int cta, int G, int i) const { // its i-th tile
    return (cta - first % G + G) % G + i * G;
  }
};

template <int MT>
__global__ void __launch_bounds__(LAY_THREADS, 1)
layer_small_m_kernel(const LayerParams p) {
  extern __shared__ __align__(128) unsigned char lay_raw[];
  const int group = p.nh / p.nkv;
  unsigned char* ring = lay_raw;
  unsigned char* work = ring + (size_t)p.n_stages * LAY_STAGE_BYTES;
  // the work area: h (later the attention's output, later a piece of the activation) and the
  // warps' partial sums; during the attention phase the same bytes stage values and hold the merge
  unsigned char* h_s = work;
  float* part = reinterpret_cast<float*>(h_s + (size_t)8 * MT * p.h_pitch);     // [warps][16][8 MT + 1]
  constexpr int kPart = LAY_WARPS * 16 * (8 * MT + 1);
  size_t work_bytes = (size_t)8 * MT * p.h_pitch + (size_t)kPart * 4;
  {
    const size_t stage = (size_t)LAY_WARPS * LAY_TILE * kVStride * 2;
    const size_t merge = (size_t)LAY_WARPS * group * kPieceRow * 4;
    const size_t att = stage > merge ? stage : merge;
    if (att > work_bytes) work_bytes = att;
    work_bytes = (work_bytes + 127) / 128 * 128;
  }
  unsigned long long* full = reinterpret_cast<unsigned long long*>(work + work_bytes);
  unsigned long long* empty = full + p.n_stages;
  int* table_s = reinterpret_cast<int*>(empty + p.n_stages);      // [LAY_TABLE_ENTRIES]: the first unit's pages
  __shared__ int grid_ok;
  __shared__ int is_last;
  __shared__ int req_s[32], pos_s[32], slot_s[32];                // the rows' requests, positions, cache slots

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int d = HEAD_DIM, half = HEAD_DIM / 2;
  const int q_width = p.nh * d;
  // stages a tile takes: its 16 rows in pieces of LAY_KC along k
  const int spt_h = (p.H + LAY_KC - 1) / LAY_KC, spt_o = (q_width + LAY_KC - 1) / LAY_KC;
  const int spt_d = (p.k_per_split_d + LAY_KC - 1) / LAY_KC;
  const int n_row_tiles = p.H / 16;
  const Deal qkv = {(p.nh + 2 * p.nkv) * (d / 16), 0};
  const Deal opr = {n_row_tiles, qkv.n_tiles};
  const Deal gup = {p.I / 8, 0};
  const Deal dwn = {n_row_tiles * p.s_down, qkv.n_tiles + opr.n_tiles};
  const int n_qkv = qkv.mine(cta, G), n_opr = opr.mine(cta, G), n_gup = gup.mine(cta, G), n_dwn = dwn.mine(cta, G);
  // the sequence numbers of the stages each product starts at, in this block
  const int c_opr = n_qkv * spt_h, c_gup = c_opr + n_opr * spt_o, c_dwn = c_gup + n_gup * spt_h;

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.n_stages; ++i) {
      lay_mbar_init(&full[i], 1);
      lay_mbar_init(&empty[i], 1);               // one warp consumes a stage
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    grid_ok = 1;
  }
  __syncthreads();

  if (warp == LAY_WARPS) {
    // ------------------------------ producer ------------------------------
    // Once the ring is full for the first time (the first stages are on their way: what the
    // first phases need must not queue behind anything), the rest of this block's share of the
    // layer's weights is asked into L2 (cp.async.bulk.prefetch: no registers, no shared memory,
    // returns at once): DRAM then streams at full rate from the kernel's first microseconds, and
    // the ring, which is only a few stages deep, has to hide the latency of L2, not that of DRAM.
    auto ahead = [&](const __nv_bfloat16* rows_lo, const __nv_bfloat16* rows_hi, int K, int k0, int kn) {
      if (lane < 16) {
        const __nv_bfloat16* src = (lane < 8 ? rows_lo + (size_t)lane * K : rows_hi + (size_t)(lane - 8) * K) + k0;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"((unsigned)kn * 2u) : "memory");
      }
    };
    bool asked = false;
    auto ask_rest = [&]() {
    asked = true;
    for (int i = 0; i < n_opr; ++i) {
      const __nv_bfloat16* rows = p.w_o + (size_t)opr.tile(cta, G, i) * 16 * q_width;
      ahead(rows, rows + (size_t)8 * q_width, q_width, 0, q_width);
    }
    for (int i = 0; i < n_gup; ++i) {
      const int out0 = gup.tile(cta, G, i) * 8;
      const __nv_bfloat16* gate = p.w_gu + (size_t)((out0 / 128) * 256 + out0 % 128) * p.H;
      ahead(gate, gate + (size_t)128 * p.H, p.H, 0, p.H);
    }
    for (int i = 0; i < n_dwn; ++i) {
      const int unit = dwn.tile(cta, G, i), split = unit / n_row_tiles, rt = unit % n_row_tiles;
      const int k_begin = split * p.k_per_split_d, k_end = min(p.I, k_begin + p.k_per_split_d);
      const __nv_bfloat16* rows = p.w_d + (size_t)rt * 16 * p.I;
      ahead(rows, rows + (size_t)8 * p.I, p.I, k_begin, k_end - k_begin);
    }
    // the small vectors: this layer's (a first layer has nobody to ask for them ahead) and those
    // the layer that runs next starts with
    if (cta < 5 && lane == 0) {
      const unsigned h_bytes = (unsigned)p.H * 4u, b_bytes = (unsigned)(p.nh + 2 * p.nkv) * d * 4u;
      const void* what = cta == 0 ? (const void*)p.gain1 : cta == 1 ? (const void*)p.gain2 :
                         cta == 2 ? (const void*)p.b_qkv : cta == 3 ? (const void*)p.next_gain : (const void*)p.next_bias;
      const unsigned bytes = (cta == 2 || cta == 4) ? b_bytes : h_bytes;
      if (what && (bytes & ~15u))
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(what), "r"(bytes & ~15u) : "memory");
    }
    // and the q/k/v share of the layer that runs next (its kernel starts with those)
    if (p.next_w) {
      for (int i = 0; i < n_qkv; ++i) {
        const int tile = qkv.tile(cta, G, i);
        const int head = tile / (d / 16), j0 = (tile % (d / 16)) * 8;
        const __nv_bfloat16* lo = p.next_w + (size_t)(head * d + j0) * p.H;
        ahead(lo, lo + (size_t)half * p.H, p.H, 0, p.H);
      }
    }
    };
    int c = 0;                                   // stages filled so far
    bool ok = true;
    auto fill = [&](const __nv_bfloat16* rows_lo, const __nv_bfloat16* rows_hi, int K, int k0, int kn) {
      // rows_lo: 8 consecutive rows of K elements (stage rows 0..7), rows_hi: stage rows 8..15
      const int stage = c % p.n_stages, use = c / p.n_stages;
      if (use > 0 && !asked) ask_rest();           // the ring is full: before the first wait
      if (use > 0) ok = ok && __all_sync(0xffffffffu, lay_mbar_wait(&empty[stage], (use - 1) & 1));
      if (ok) {
        const unsigned bytes = (unsigned)kn * 2u;
        if (lane == 0) lay_mbar_expect(&full[stage], 16u * bytes);
        __syncwarp();
        if (lane < 16) {
          const __nv_bfloat16* src = (lane < 8 ? rows_lo + (size_t)lane * K : rows_hi + (size_t)(lane - 8) * K) + k0;
          lay_bulk_copy(ring + (size_t)stage * LAY_STAGE_BYTES + lane * LAY_ROW_PITCH, src, bytes, &full[stage]);
        }
      }
      ++c;
    };
    for (int rep = 0; rep < p.repeat; ++rep) {
    // q/k/v: a tile is 8 lanes of a head and their rotation partners
    for (int i = 0; i < n_qkv && ok; ++i) {
      const int tile = qkv.tile(cta, G, i);
      const int head = tile / (d / 16), j0 = (tile % (d / 16)) * 8;
      const __nv_bfloat16* lo = p.w_qkv + (size_t)(head * d + j0) * p.H;
      for (int k0 = 0; k0 < p.H && ok; k0 += LAY_KC) fill(lo, lo + (size_t)half * p.H, p.H, k0, min(LAY_KC, p.H - k0));
    }
    // the output projection
    for (int i = 0; i < n_opr && ok; ++i) {
      const __nv_bfloat16* rows = p.w_o + (size_t)opr.tile(cta, G, i) * 16 * q_width;
      for (int k0 = 0; k0 < q_width && ok; k0 += LAY_KC)
        fill(rows, rows + (size_t)8 * q_width, q_width, k0, min(LAY_KC, q_width - k0));
    }
    // gate and up: 8 gate rows and the 8 up rows of the same outputs
    for (int i = 0; i < n_gup && ok; ++i) {
      const int out0 = gup.tile(cta, G, i) * 8;
      const __nv_bfloat16* gate = p.w_gu + (size_t)((out0 / 128) * 256 + out0 % 128) * p.H;
      for (int k0 = 0; k0 < p.H && ok; k0 += LAY_KC) fill(gate, gate + (size_t)128 * p.H, p.H, k0, min(LAY_KC, p.H - k0));
    }
    // down: a unit is (piece of k, row tile), pieces slowest
    for (int i = 0; i < n_dwn && ok; ++i) {
      const int unit = dwn.tile(cta, G, i), split = unit / n_row_tiles, rt = unit % n_row_tiles;
      const int k_begin = split * p.k_per_split_d, k_end = min(p.I, k_begin + p.k_per_split_d);
      const __nv_bfloat16* rows = p.w_d + (size_t)rt * 16 * p.I;
      for (int s = 0; s < spt_d && ok; ++s) {
        const int k0 = k_begin + s * LAY_KC;
        const int kn = k0 < k_end ? min(LAY_KC, k_end - k0) : 0;
        // a piece that ends early still takes its stages (32 elements of padding: nothing adds up)
        fill(rows, rows + (size_t)8 * p.I, p.I, kn ? k0 : k_begin, kn ? kn : 32);
      }
    }
    if (!asked) ask_rest();
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  const int tid = threadIdx.x;                   // 0 .. 255
  const int g = lane >> 2, t = lane & 3;
  bool ok = true;
  int barriers = 0;
  float acc[MT][4];
  // One stage, consumed by this warp alone: 16 weight rows x kn elements of k against the rows of
  // the activation tile in shared memory, from its column k_local0 on.
  int c_rep = 0;                                 // stages of the repetitions before this one
  // Four independent chains of mma (k steps 0, 1, 2, 3 mod 4) so that a warp working through a
  // tile alone is not one long chain of dependent instructions; they are added at the tile's end.
  float acc4[4][MT][4];
  auto multiply = [&](int c_in, int k_local0, int kn) {
    const int c = c_rep + c_in;
    const int stage = c % p.n_stages, use = c / p.n_stages;
    ok = ok && __all_sync(0xffffffffu, lay_mbar_wait(&full[stage], use & 1));
    if (ok) {
      const unsigned char* st = ring + (size_t)stage * LAY_STAGE_BYTES;
      const unsigned char* a_row = st + g * LAY_ROW_PITCH + 8 * t * 2;
      const unsigned char* b_row = st + (g + 8) * LAY_ROW_PITCH + 8 * t * 2;
      const unsigned char* x_row = h_s + (size_t)g * p.h_pitch + (k_local0 + 8 * t) * 2;
      int k = 0;
      for (; k + 128 <= kn; k += 128) {
        uint4 a[4], b[4], xv[4][MT];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          a[u] = *reinterpret_cast<const uint4*>(a_row + (k + 32 * u) * 2);
          b[u] = *reinterpret_cast<const uint4*>(b_row + (k + 32 * u) * 2);
#pragma unroll
          for (int j = 0; j < MT; ++j)
            xv[u][j] = *reinterpret_cast<const uint4*>(x_row + (size_t)8 * j * p.h_pitch + (k + 32 * u) * 2);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            lay_mma(acc4[u][j], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][j].x, xv[u][j].y);
            lay_mma(acc4[u][j], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][j].z, xv[u][j].w);
          }
        }
      }
      for (; k < kn; k += 32) {
        const uint4 a = *reinterpret_cast<const uint4*>(a_row + k * 2);
        const uint4 b = *reinterpret_cast<const uint4*>(b_row + k * 2);
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const uint4 xv = *reinterpret_cast<const uint4*>(x_row + (size_t)8 * j * p.h_pitch + k * 2);
          lay_mma(acc4[(k >> 5) & 3][j], a.x, b.x, a.y, b.y, xv.x, xv.y);
          lay_mma(acc4[(k >> 5) & 3][j], a.z, b.z, a.w, b.w, xv.z, xv.w);
        }
      }
      __syncwarp();
      if (lane == 0) lay_mbar_arrive(&empty[stage]);
    }
  };
  // acc = the sum of the four chains (after a tile's last stage)
  auto gather = [&]() {
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][e] = (acc4[0][j][e] + acc4[1][j][e]) + (acc4[2][j][e] + acc4[3][j][e]);
    }
  };
  auto clear = [&]() {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int j = 0; j < MT; ++j) acc4[u][j][0] = acc4[u][j][1] = acc4[u][j][2] = acc4[u][j][3] = 0.f;
    }
  };
  // All blocks meet: every consumer's writes are ordered before its block's arrival (block
  // barrier, then one thread's fence and atomic), and the waiters' reads after it.  A wait that
  // ran out once makes the block skip all later waits (it still arrives, for the others).
  auto grid_barrier = [&]() {
    ++barriers;
    lay_consumer_sync();
    if (tid == 0) {
      __threadfence();
      asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.sync) : "memory");
      if (grid_ok) {
        bool met = false;
        const int target = barriers * G;
        for (unsigned spin = 0; spin < LAY_GRID_WAIT_LIMIT; ++spin) {
          int seen;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.sync) : "memory");
          if (seen >= target) { met = true; break; }
        }
        if (!met) {
          atomicExch(&lay_error_flag, 2);
          tokb200_report_error(TOKB200_LIB_LAYER_SMALL_M, 2);
          grid_ok = 0;
        }
      }
      __threadfence();
    }
    lay_consumer_sync();
    ok = ok && grid_ok;
  };
  int stamp_at = 0;
  auto stamp = [&]() {
    if (p.stamps && tid == 0) {
      long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      p.stamps[(size_t)cta * 32 + stamp_at] = now;
    }
    ++stamp_at;
  };
  auto stamp_to = [&](int slot) {          // finer marks inside a phase (slots 16..31)
    if (p.stamps && tid == 0) {
      long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      p.stamps[(size_t)cta * 32 + slot] = now;
    }
  };
  stamp();             // 0: consumers start

  // ---- what the later phases need of the step's description, asked for now: the rows'
  // requests, positions, slots and block tables were written before the predecessor started ----
  if (tid < 32) {
    req_s[tid] = tid < p.M ? p.row_req[tid] : -1;
    pos_s[tid] = tid < p.M ? p.pos[tid] : 0;
    slot_s[tid] = (tid < p.M && p.slot) ? p.slot[tid] : -1;
  }
  const int n_units = p.M * p.nkv * p.att_splits;
  int u_first = 0, u_last = -1, u_splits = 0, u_req = -1, u_cached = 0;
  const int unit0 = cta;
  if (unit0 < n_units) {
    const int split = unit0 % p.att_splits, row = unit0 / (p.att_splits * p.nkv);
    u_req = p.row_req[row];
    if (u_req >= 0) {
      const int at = p.pos[row];      // (its own loads: the shared copies are not written yet)
      const int lo = (p.window >= 0 && at - p.window > 0) ? at - p.window : 0;
      const int n_keys = at - lo + 1;
      const int chunk = ((n_keys + p.att_splits - 1) / p.att_splits + LAY_TILE - 1) / LAY_TILE * LAY_TILE;
      u_splits = (n_keys + chunk - 1) / chunk;
      u_first = lo + split * chunk;
      u_last = min(at, u_first + chunk - 1);
      if (split < u_splits) {
        const int page0 = u_first / p.page, pages = u_last / p.page - page0 + 1;
        if (pages <= LAY_TABLE_ENTRIES) {
          u_cached = 1;
          for (int e = tid; e < pages; e += LAY_CONSUMERS)
            table_s[e] = p.block_table[(size_t)u_req * p.table_stride + page0 + e];
        }
      }
    }
  }
  lay_consumer_sync();
  if (u_cached) {
    // the unit's keys and values into L2 (all but the newest were written by earlier steps)
    const int kvh = (unit0 / p.att_splits) % p.nkv, page0 = u_first / p.page;
    for (int key = u_first + tid; key <= u_last; key += LAY_CONSUMERS) {
      const size_t at = ((size_t)(table_s[key / p.page - page0] * p.page + key % p.page) * p.nkv + kvh) * d;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.k_read + at));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.v_read + at));
      if (HEAD_DIM > 64) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.k_read + at + 64));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.v_read + at + 64));
      }
    }
  }
  // the gains are constants: in registers before the wait (a warp per row reads the same pieces)
  pdl_wait();          // x and the pending sums come from the predecessor; the weights do not
  pdl_launch();
  stamp();             // 1: the predecessor is done

  for (int rep = 0; rep < p.repeat; ++rep) {
  if (rep > 0) {
    grid_barrier();
    stamp_at = 2;
    c_rep += c_dwn + n_dwn * spt_d;
  }
  // ======================= phase 0: the first norm =======================
  lay_norm<MT>(p.x_in, p.delta, p.delta_is_f32, p.n_partials, p.partial_stride, p.gain1, p.eps1,
               cta == 0 ? p.x_mid : nullptr, h_s, p.h_pitch, p.M, p.H, warp, lane);
  lay_consumer_sync();
  stamp();             // 2: first norm done

  // ======================= phase 1: q, k, v with bias, rotation, cache write =======================
  // a warp per tile; a thread's accumulators hold both halves of a rotation pair: c0,c1 are lane
  // j0 + g of the head for rows 2t, 2t+1 (of each 8), c2,c3 its partner j0 + g + d/2
  for (int i = warp; i < n_qkv; i += LAY_WARPS) {
    const int tile = qkv.tile(cta, G, i);
    const int head = tile / (d / 16), ej = (tile % (d / 16)) * 8 + g;
    float bias_a = 0.f, bias_b = 0.f;
    if (p.b_qkv) {
      bias_a = p.b_qkv[head * d + ej];
      bias_b = p.b_qkv[head * d + ej + half];
    }
    float e_cos[MT][2], e_sin[MT][2];
    int e_slot[MT][2];
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = 8 * j + 2 * t + e;
        e_cos[j][e] = 1.f; e_sin[j][e] = 0.f; e_slot[j][e] = -1;
        if (m < p.M) {
          if (head >= p.nh) e_slot[j][e] = slot_s[m];
          if (head < p.nh + p.nkv) {
            const int at = pos_s[m];
            e_cos[j][e] = p.cos_t[(size_t)at * half + ej];
            e_sin[j][e] = p.sin_t[(size_t)at * half + ej];
          }
        }
      }
    }
    clear();
    stamp_to(23);              // (warp 0's tile) before the product
    for (int s = 0; s < spt_h; ++s) multiply(i * spt_h + s, s * LAY_KC, min(LAY_KC, p.H - s * LAY_KC));
    if (!ok) break;
    gather();
    stamp_to(24);              // the product is done
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = 8 * j + 2 * t + e;
        if (m >= p.M) continue;
        float a = acc[j][e] + bias_a, b = acc[j][2 + e] + bias_b;
        __nv_bfloat16* dst = nullptr;
        if (head < p.nh) {
          dst = p.q_buf + ((size_t)m * p.nh + head) * d;
        } else if (e_slot[j][e] >= 0) {
          const bool is_key = head < p.nh + p.nkv;
          __nv_bfloat16* pool = is_key ? p.k_pool : p.v_pool;
          if (pool) dst = pool + ((size_t)e_slot[j][e] * p.nkv + (head - p.nh - (is_key ? 0 : p.nkv))) * d;
        }
        if (head < p.nh + p.nkv) {                            // values are not rotated
          const float ra = a * e_cos[j][e] - b * e_sin[j][e], rb = b * e_cos[j][e] + a * e_sin[j][e];
          a = ra;
          b = rb;
        }
        if (dst) {
          dst[ej] = __float2bfloat16_rn(a);
          dst[ej + half] = __float2bfloat16_rn(b);
        }
      }
    }
  }
  stamp_to(25);          // warp 0 is through its tiles
  stamp();             // 3: q/k/v done
  grid_barrier();
  stamp();             // 4: barrier 1 passed

  // ======================= phase 2: attention =======================
  // a unit is (row, kv head, piece of the row's keys); the group's query heads are the M side of
  // the mma, so keys and values are read once per group
  {
    const float scale_log2 = p.scale * 1.4426950408889634f;
    __nv_bfloat16* v_s = reinterpret_cast<__nv_bfloat16*>(work) + (size_t)warp * LAY_TILE * kVStride;
    float* acc_s = reinterpret_cast<float*>(work);            // [warp][head][kPieceRow], after the passes
    for (int unit = cta; unit < n_units && ok; unit += G) {
      const int split = unit % p.att_splits, kvh = (unit / p.att_splits) % p.nkv, row = unit / (p.att_splits * p.nkv);
      int r, first, last, n_splits;
      const bool cached = unit == unit0 && u_cached;
      if (unit == unit0) {
        r = u_req; first = u_first; last = u_last; n_splits = u_splits;
      } else {
        r = req_s[row];
        const int at = r < 0 ? 0 : pos_s[row];
        const int lo = (p.window >= 0 && at - p.window > 0) ? at - p.window : 0;
        const int n_keys = at - lo + 1;
        const int chunk = ((n_keys + p.att_splits - 1) / p.att_splits + LAY_TILE - 1) / LAY_TILE * LAY_TILE;
        n_splits = (n_keys + chunk - 1) / chunk;
        first = lo + split * chunk;
        last = min(at, first + chunk - 1);
      }
      if (r < 0 || split >= n_splits) continue;               // uniform over the block
      const int* table = p.block_table + (size_t)r * p.table_stride;
      const int page0 = first / p.page;
      auto slot_of = [&](int key) {
        const int pg = cached ? table_s[key / p.page - page0] : table[key / p.page];
        return pg * p.page + key % p.page;
      };

      // ---- q fragments: heads g and g + 8 of the group, lanes in the permuted order ----
      unsigned qa[HEAD_DIM / 32][2][4];
      {
        const bool ok_a = g < group, ok_b = g + 8 < group;
        const __nv_bfloat16* qa_row = p.q_buf + ((size_t)row * p.nh + kvh * group + g) * d;
        const __nv_bfloat16* qb_row = qa_row + (size_t)8 * d;
#pragma unroll
        for (int st = 0; st < HEAD_DIM / 32; ++st) {
          const uint4 a = lay_load16_cg(qa_row + st * 32 + 8 * t, ok_a);
          const uint4 b = lay_load16_cg(qb_row + st * 32 + 8 * t, ok_b);
          qa[st][0][0] = a.x; qa[st][0][1] = b.x; qa[st][0][2] = a.y; qa[st][0][3] = b.y;
          qa[st][1][0] = a.z; qa[st][1][1] = b.z; qa[st][1][2] = a.w; qa[st][1][3] = b.w;
        }
      }
      stamp_to(20);            // q is here
      float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
      float o[HEAD_DIM / 8][4];
#pragma unroll
      for (int i = 0; i < HEAD_DIM / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

      for (int k0 = first + warp * LAY_TILE; k0 <= last; k0 += LAY_WARPS * LAY_TILE) {
        {
          // the tile's values go straight to their staging rows (a lane per key)
          const int key = k0 + lane;
          const bool in = key <= last;
          const __nv_bfloat16* vrow = p.v_read + ((size_t)slot_of(in ? key : k0) * p.nkv + kvh) * d;
          const unsigned dst = lay_smem(v_s + lane * kVStride);
          const int bytes = in ? 16 : 0;
#pragma unroll
          for (int cc = 0; cc < HEAD_DIM / 8; ++cc)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst + cc * 16), "l"(vrow + cc * 8), "r"(bytes));
          asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        float s[LAY_TILE / 8][4];
        uint4 kf[LAY_TILE / 8][HEAD_DIM / 32];
#pragma unroll
        for (int nt = 0; nt < LAY_TILE / 8; ++nt) {            // all of the tile's keys asked for at once
          const int key = k0 + nt * 8 + g;
          const bool in = key <= last;
          const __nv_bfloat16* krow = p.k_read + ((size_t)slot_of(in ? key : k0) * p.nkv + kvh) * d;
#pragma unroll
          for (int st = 0; st < HEAD_DIM / 32; ++st) kf[nt][st] = lay_load16_cg(krow + st * 32 + 8 * t, in);
        }
#pragma unroll
        for (int nt = 0; nt < LAY_TILE / 8; ++nt) {
          s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
          for (int st = 0; st < HEAD_DIM / 32; ++st) {
            lay_mma(s[nt], qa[st][0][0], qa[st][0][1], qa[st][0][2], qa[st][0][3], kf[nt][st].x, kf[nt][st].y);
            lay_mma(s[nt], qa[st][1][0], qa[st][1][1], qa[st][1][2], qa[st][1][3], kf[nt][st].z, kf[nt][st].w);
          }
        }
        // ---- scale, mask, running softmax: rows g (heads 0..7) and g + 8 (heads 8..15) ----
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nt = 0; nt < LAY_TILE / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = k0 + nt * 8 + 2 * t + (e & 1);
            s[nt][e] = key <= last ? s[nt][e] * scale_log2 : -INFINITY;
            m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nt][e]);
          }
        }
        float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
          m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));   // finite: key k0 is live
          corr[i] = exp2f(m_run[i] - m_new[i]);                                      // 0 on the first pass
          m_run[i] = m_new[i];
        }
#pragma unroll
        for (int nt = 0; nt < LAY_TILE / 8; ++nt) {
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
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");   // the tile's values have landed
        __syncwarp();
#pragma unroll
        for (int ks = 0; ks < LAY_TILE / 16; ++ks) {
          const unsigned p0 = lay_pack(s[2 * ks][0], s[2 * ks][1]), p1 = lay_pack(s[2 * ks][2], s[2 * ks][3]);
          const unsigned p2 = lay_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), p3 = lay_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
          for (int dp = 0; dp < HEAD_DIM / 16; ++dp) {
            unsigned vf[4];
            lay_ldmatrix_x4_trans(vf, v_s + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kVStride +
                                          dp * 16 + (lane >> 4) * 8);
            lay_mma(o[2 * dp], p0, p1, p2, p3, vf[0], vf[1]);
            lay_mma(o[2 * dp + 1], p0, p1, p2, p3, vf[2], vf[3]);
          }
        }
        __syncwarp();   // the staged values are overwritten by the next tile
      }

      // ---- merge the warps of the block (the merge buffer takes the place of the staging area) ----
      lay_consumer_sync();
      stamp_to(16);            // the passes over the keys are done
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int head = g + 8 * i;
        if (head < group) {
          float* dst = acc_s + ((size_t)warp * group + head) * kPieceRow;
#pragma unroll
          for (int nt = 0; nt < HEAD_DIM / 8; ++nt) {
            dst[nt * 8 + 2 * t] = o[nt][2 * i];
            dst[nt * 8 + 2 * t + 1] = o[nt][2 * i + 1];
          }
          if (t == 0) { dst[HEAD_DIM] = m_run[i]; dst[HEAD_DIM + 1] = l_run[i]; }
        }
      }
      lay_consumer_sync();
      const size_t per_head = (size_t)LAY_MAX_SPLITS * kPieceRow;
      float* base = p.att_part + ((size_t)row * p.nh + kvh * group) * per_head;
      for (int i = tid; i < group * HEAD_DIM; i += LAY_CONSUMERS) {
        const int head = i / HEAD_DIM, cc = i % HEAD_DIM;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < LAY_WARPS; ++w) m = fmaxf(m, acc_s[((size_t)w * group + head) * kPieceRow + HEAD_DIM]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < LAY_WARPS; ++w) {
          const float* src = acc_s + ((size_t)w * group + head) * kPieceRow;
          const float f = exp2f(src[HEAD_DIM] - m);          // a warp without keys has max -inf: weight 0
          num += f * src[cc];
          den += f * src[HEAD_DIM + 1];
        }
        if (n_splits == 1) {
          p.att_out[((size_t)row * p.nh + kvh * group + head) * d + cc] = __float2bfloat16_rn(num / den);
        } else {
          float* piece = base + head * per_head + (size_t)split * kPieceRow;
          piece[cc] = num;
          if (cc == 0) { piece[HEAD_DIM] = m; piece[HEAD_DIM + 1] = den; }
        }
      }
      if (n_splits > 1) {
        // ---- the last block to finish a (row, kv head) merges its pieces, in index order ----
        stamp_to(17);          // the piece is written
        __threadfence();
        lay_consumer_sync();
        stamp_to(18);          // fenced
        if (tid == 0) {
          const int done = atomicAdd(&p.att_count[row * p.nkv + kvh], 1);
          is_last = done == n_splits - 1;
          if (is_last) p.att_count[row * p.nkv + kvh] = 0;   // ready for the next launch
        }
        lay_consumer_sync();
        stamp_to(19);          // counted
        if (is_last) {
          __threadfence();
          for (int head = warp; head < group; head += LAY_WARPS) {
            const float* pieces = base + head * per_head;
            const bool on = lane < n_splits;
            const float m_s = on ? __ldcg(&pieces[(size_t)lane * kPieceRow + HEAD_DIM]) : -INFINITY;
            const float l_s = on ? __ldcg(&pieces[(size_t)lane * kPieceRow + HEAD_DIM + 1]) : 0.f;
            const float m_all = warp_max(m_s);
            const float f = exp2f(m_s - m_all);                 // 0 for lanes without a piece
            const float den = warp_sum(f * l_s);
            float num[HEAD_DIM / 32];
#pragma unroll
            for (int c0 = 0; c0 < HEAD_DIM / 32; ++c0) num[c0] = 0.f;
            for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {     // eight pieces' values asked for at once
              float v[8][HEAD_DIM / 32];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
#pragma unroll
                for (int c0 = 0; c0 < HEAD_DIM / 32; ++c0)
                  v[k][c0] = sp0 + k < n_splits ? __ldcg(&pieces[(size_t)(sp0 + k) * kPieceRow + c0 * 32 + lane]) : 0.f;
              }
#pragma unroll
              for (int k = 0; k < 8; ++k) {                   // in index order
                const float fk = __shfl_sync(0xffffffffu, f, (sp0 + k) & 31);
#pragma unroll
                for (int c0 = 0; c0 < HEAD_DIM / 32; ++c0) num[c0] += fk * v[k][c0];
              }
            }
#pragma unroll
            for (int c0 = 0; c0 < HEAD_DIM / 32; ++c0)
              p.att_out[((size_t)row * p.nh + kvh * group + head) * d + c0 * 32 + lane] =
                  __float2bfloat16_rn(num[c0] / den);
          }
        }
      }
      lay_consumer_sync();       // the work area is reused by the block's next unit
    }
  }
  stamp();             // 5: attention done
  grid_barrier();
  stamp();             // 6: barrier 2 passed

  // ======================= phase 3: the output projection =======================
  if (n_opr > 0) {
    // the attention's output, all rows, into shared memory (idle rows and rows past M: zeros)
    const int pieces = q_width / 8;
    for (int i0 = tid; i0 < 8 * MT * pieces; i0 += 4 * LAY_CONSUMERS) {      // four loads in flight a thread
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * LAY_CONSUMERS, m = i / pieces, piece = i % pieces;
        v[u] = lay_load16_cg(p.att_out + (size_t)m * q_width + piece * 8,
                             i < 8 * MT * pieces && m < p.M && req_s[m < 32 ? m : 0] >= 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * LAY_CONSUMERS, m = i / pieces, piece = i % pieces;
        if (i < 8 * MT * pieces) *reinterpret_cast<uint4*>(h_s + (size_t)m * p.h_pitch + piece * 16) = v[u];
      }
    }
  }
  lay_consumer_sync();
  for (int i = warp; i < n_opr; i += LAY_WARPS) {
    const int rt = opr.tile(cta, G, i);
    clear();
    for (int s = 0; s < spt_o; ++s) multiply(c_opr + i * spt_o + s, s * LAY_KC, min(LAY_KC, q_width - s * LAY_KC));
    if (!ok) break;
    gather();
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = 8 * j + 2 * t + e;
        if (m < p.M) {
          p.o_part[(size_t)m * p.H + rt * 16 + g] = acc[j][e];
          p.o_part[(size_t)m * p.H + rt * 16 + g + 8] = acc[j][2 + e];
        }
      }
    }
  }
  stamp();             // 7: output projection done
  grid_barrier();
  stamp();             // 8: barrier 3 passed

  // ======================= phase 4: the second norm =======================
  lay_norm<MT>(p.x_mid, p.o_part, 1, 1, (long long)p.M * p.H, p.gain2, p.eps2,
               cta == 0 ? p.x_out : nullptr, h_s, p.h_pitch, p.M, p.H, warp, lane);
  lay_consumer_sync();
  stamp();             // 9: second norm done

  // ======================= phase 5: gate and up, activation =======================
  for (int i = warp; i < n_gup; i += LAY_WARPS) {
    const int tile = gup.tile(cta, G, i);
    clear();
    for (int s = 0; s < spt_h; ++s) multiply(c_gup + i * spt_h + s, s * LAY_KC, min(LAY_KC, p.H - s * LAY_KC));
    if (!ok) break;
    gather();
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = 8 * j + 2 * t + e;                      // c0,c1: gate of output g; c2,c3: its up
        if (m < p.M)
          p.act[(size_t)m * p.I + tile * 8 + g] =
              __float2bfloat16_rn(gate_activation(p.activation, acc[j][e]) * acc[j][2 + e]);
      }
    }
  }
  stamp();             // 10: gate/up done
  grid_barrier();
  stamp();             // 11: barrier 4 passed

  // ======================= phase 6: down, cut along k =======================
  // a unit is (piece of k, row tile); its stages go to the warps in turn, which meet once
  for (int i = 0; i < n_dwn; ++i) {
    const int unit = dwn.tile(cta, G, i), split = unit / n_row_tiles, rt = unit % n_row_tiles;
    const int k_begin = split * p.k_per_split_d, k_end = min(p.I, k_begin + p.k_per_split_d);
    if (i == 0 || split != dwn.tile(cta, G, i - 1) / n_row_tiles) {
      // this piece's columns of the activation, all rows, into shared memory (rows past M: zeros)
      lay_consumer_sync();
      const int pieces = p.k_per_split_d / 8;
      for (int e0 = tid; e0 < 8 * MT * pieces; e0 += 8 * LAY_CONSUMERS) {    // eight loads in flight a thread
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int e = e0 + u * LAY_CONSUMERS, m = e / pieces, piece = e % pieces;
          v[u] = lay_load16_cg(p.act + (size_t)m * p.I + k_begin + piece * 8,
                               e < 8 * MT * pieces && m < p.M && k_begin + piece * 8 < k_end);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int e = e0 + u * LAY_CONSUMERS, m = e / pieces, piece = e % pieces;
          if (e < 8 * MT * pieces) *reinterpret_cast<uint4*>(h_s + (size_t)m * p.h_pitch + piece * 16) = v[u];
        }
      }
      lay_consumer_sync();
      stamp_to(21);            // the activation's piece is in shared memory
    }
    clear();
    for (int s = warp; s < spt_d; s += LAY_WARPS) {
      const int k0 = k_begin + s * LAY_KC;
      const int kn = k0 < k_end ? min(LAY_KC, k_end - k0) : 0;
      multiply(c_dwn + i * spt_d + s, kn ? s * LAY_KC : 0, kn);   // kn 0: the stage is only given back
    }
    gather();
    {
      float* mine = part + (size_t)warp * 16 * (8 * MT + 1);
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        mine[g * (8 * MT + 1) + 8 * j + 2 * t] = acc[j][0];
        mine[g * (8 * MT + 1) + 8 * j + 2 * t + 1] = acc[j][1];
        mine[(g + 8) * (8 * MT + 1) + 8 * j + 2 * t] = acc[j][2];
        mine[(g + 8) * (8 * MT + 1) + 8 * j + 2 * t + 1] = acc[j][3];
      }
    }
    lay_consumer_sync();
    stamp_to(22);              // the warps' products are done
    for (int e = tid; e < 16 * p.M && ok; e += LAY_CONSUMERS) {
      const int m = e / 16, rr = e % 16;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < LAY_WARPS; ++w) v += part[((size_t)w * 16 + rr) * (8 * MT + 1) + m];
      p.out[((size_t)split * p.M + m) * p.H + rt * 16 + rr] = v;
    }
    if (i + 1 < n_dwn) lay_consumer_sync();      // the partial sums are read before the next unit's
  }
  stamp();             // 12: down done
  }

  // ---- the last block to leave makes the barrier ready for the next launch ----
  if (tid == 0) {
    const int left = atomicAdd(&p.sync[1], 1);
    if (left == G - 1) {
      p.sync[0] = 0;
      p.sync[1] = 0;
      __threadfence();
    }
  }
}

TOKB200_API int tokb200_layer_small_m_error(void) {
  int flag = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&flag, lay_error_flag, sizeof(int)) != cudaSuccess) return -1;
  if (flag) cudaMemcpyToSymbol(lay_error_flag, &zero, sizeof(int));
  return flag;
}

TOKB200_API int tokb200_layer_small_m_head_dim(void) { return HEAD_DIM; }

// The plan for sizes on this device; blocks == 0: the kernel does not take them.
struct LayerPlan {
  int blocks, n_stages, h_pitch, s_down, k_per_split_d, smem_max;
  size_t smem;
};

static LayerPlan lay_plan(int M, int H, int I, int nh, int nkv) {
  LayerPlan plan = {};
  if (M <= 0 || M > 32 || H <= 0 || H > 4096 || I <= 0 || H % 32 || I % 128 || nh <= 0 || nkv <= 0 || nh % nkv ||
      nh / nkv > LAY_MAX_GROUP || (nh * HEAD_DIM) % 32)
    return plan;
  int device = 0, sms = 0, smem_max = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return plan;
  const int MT = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  const int row_tiles = H / 16;
  // down is cut along k so that a piece of the activation (all rows) fits the work area, and
  // further while its units (piece, row tile) still number no more than the blocks
  const int longest = MT == 4 ? 2048 : 4096;
  int s = (I + longest - 1) / longest;
  if (sms / row_tiles > s) s = sms / row_tiles;
  if (s > 16) s = 16;
  int kps = ((I + s - 1) / s + 31) / 32 * 32;
  s = (I + kps - 1) / kps;
  plan.s_down = s;
  plan.k_per_split_d = kps;
  int widest = H;
  if (nh * HEAD_DIM > widest) widest = nh * HEAD_DIM;
  if (kps > widest) widest = kps;
  plan.h_pitch = (2 * widest + 127) / 128 * 128 + 64;
  const int group = nh / nkv;
  size_t work = (size_t)8 * MT * plan.h_pitch + (size_t)LAY_WARPS * 16 * (8 * MT + 1) * 4;
  const size_t stage = (size_t)LAY_WARPS * LAY_TILE * kVStride * 2;
  const size_t merge = (size_t)LAY_WARPS * group * kPieceRow * 4;
  const size_t att = stage > merge ? stage : merge;
  if (att > work) work = att;
  work = (work + 127) / 128 * 128;
  const size_t tail = 2048;                         // the ring's barriers and the cached table entries
  const long long room = (long long)smem_max - 2048 - (long long)work - (long long)tail;
  int stages = (int)(room / LAY_STAGE_BYTES);
  if (stages > 8) stages = 8;
  if (stages < 3) return plan;
  plan.blocks = sms;
  plan.n_stages = stages;
  plan.smem_max = smem_max;
  plan.smem = work + (size_t)stages * LAY_STAGE_BYTES + tail;
  return plan;
}

// Partial sums of the feed-forward that `out` holds for these sizes (0: sizes not taken); the
// output projection's result is one plane (`o_splits` = 1).
TOKB200_API int tokb200_layer_small_m_splits(int M, int H, int I, int nh, int nkv, int* o_splits) {
  const LayerPlan plan = lay_plan(M, H, I, nh, nkv);
  if (o_splits) *o_splits = plan.blocks ? 1 : 0;
  return plan.blocks ? plan.s_down : 0;
}

struct LayerArgs {            // what the launcher takes, as plain C
  const void* w_qkv; const float* b_qkv; const void* w_o; const float* gain1; const float* gain2;
  const void* w_gu; const void* w_d; void* k_pool; void* v_pool; const void* k_read; const void* v_read;
  const float* cos_t; const float* sin_t;
  float eps1, eps2, scale; int window, activation;
  const float* x_in; const void* delta; int delta_is_f32, n_partials; long long partial_stride;
  float* x_mid; float* x_out; float* out;
  const int* pos; const int* slot; const int* row_req; const int* block_table; int table_stride, page;
  void* q_buf; float* att_part; int* att_count; void* att_out; float* o_part; void* act; int* sync;
  int M, H, I, nh, nkv, d;
  long long* stamps;          // null, or [blocks, 32] for the phases' times (profiling)
  const void* next_w_qkv;     // null, or the next layer's q/k/v weight, to be brought into L2
  const float* next_gain1;    // ... and its first gain and q/k/v bias
  const float* next_b_qkv;
  int repeat;                 // 0 or 1: once; more (profiling only): the same layer again and again in one launch
};

TOKB200_API int tokb200_layer_small_m(const LayerArgs* a, cudaStream_t stream) {
  if (a->d != HEAD_DIM) return TOKB200_BAD_SIZE;
  const LayerPlan plan = lay_plan(a->M, a->H, a->I, a->nh, a->nkv);
  if (plan.blocks == 0 || a->page <= 0 || a->activation < 0 || a->activation >= TOKB200_ACT_COUNT)
    return TOKB200_BAD_SIZE;
  if (((uintptr_t)a->w_qkv | (uintptr_t)a->w_o | (uintptr_t)a->w_gu | (uintptr_t)a->w_d | (uintptr_t)a->act |
       (uintptr_t)a->q_buf | (uintptr_t)a->att_out | (uintptr_t)a->k_read | (uintptr_t)a->v_read |
       (uintptr_t)a->x_in | (uintptr_t)a->x_mid | (uintptr_t)a->x_out | (uintptr_t)a->o_part |
       (uintptr_t)a->delta | (uintptr_t)a->gain1 | (uintptr_t)a->gain2) & 15)
    return TOKB200_BAD_ALIGNMENT;
  LayerParams p;
  p.w_qkv = (const __nv_bfloat16*)a->w_qkv; p.b_qkv = a->b_qkv; p.w_o = (const __nv_bfloat16*)a->w_o;
  p.gain1 = a->gain1; p.gain2 = a->gain2; p.w_gu = (const __nv_bfloat16*)a->w_gu; p.w_d = (const __nv_bfloat16*)a->w_d;
  p.k_pool = (__nv_bfloat16*)a->k_pool; p.v_pool = (__nv_bfloat16*)a->v_pool;
  p.k_read = (const __nv_bfloat16*)a->k_read; p.v_read = (const __nv_bfloat16*)a->v_read;
  p.cos_t = a->cos_t; p.sin_t = a->sin_t; p.eps1 = a->eps1; p.eps2 = a->eps2; p.scale = a->scale;
  p.window = a->window; p.activation = a->activation;
  p.x_in = a->x_in; p.delta = a->delta; p.delta_is_f32 = a->delta_is_f32; p.n_partials = a->n_partials;
  p.partial_stride = a->partial_stride; p.x_mid = a->x_mid; p.x_out = a->x_out; p.out = a->out;
  p.pos = a->pos; p.slot = a->slot; p.row_req = a->row_req; p.block_table = a->block_table;
  p.table_stride = a->table_stride; p.page = a->page;
  p.q_buf = (__nv_bfloat16*)a->q_buf; p.att_part = a->att_part; p.att_count = a->att_count;
  p.att_out = (__nv_bfloat16*)a->att_out; p.o_part = a->o_part; p.act = (__nv_bfloat16*)a->act; p.sync = a->sync;
  p.M = a->M; p.H = a->H; p.I = a->I; p.nh = a->nh; p.nkv = a->nkv; p.stamps = a->stamps;
  p.next_w = (const __nv_bfloat16*)a->next_w_qkv; p.next_gain = a->next_gain1; p.next_bias = a->next_b_qkv;
  p.repeat = a->repeat > 1 ? a->repeat : 1;
  p.n_stages = plan.n_stages; p.h_pitch = plan.h_pitch;
  p.s_down = plan.s_down; p.k_per_split_d = plan.k_per_split_d;
  // pieces of a row's keys: enough units for the device, none shorter than one pass of a block's
  // warps (256 keys) as far as the table reaches
  long long reach = (long long)a->table_stride * a->page;
  if (a->window >= 0 && a->window + 1 < reach) reach = a->window + 1;
  int splits = (plan.blocks + a->M * a->nkv - 1) / (a->M * a->nkv);
  const int longest = (int)((reach + LAY_WARPS * LAY_TILE - 1) / (LAY_WARPS * LAY_TILE));
  if (splits > longest) splits = longest;
  if (splits > LAY_MAX_SPLITS) splits = LAY_MAX_SPLITS;
  if (splits < 1) splits = 1;
  p.att_splits = splits;
  const int form = a->M <= 8 ? 0 : (a->M <= 16 ? 1 : 2);
  void (*kernel)(const LayerParams) = form == 0 ? layer_small_m_kernel<1> :
                                      form == 1 ? layer_small_m_kernel<2> : layer_small_m_kernel<4>;
  static bool configured[64][3] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!configured[device][form]) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_max - 1024);
    if (err != cudaSuccess) return (int)err;
    configured[device][form] = true;
  }
  // One block per SM, each with most of an SM's shared memory: all blocks become resident as the
  // predecessor's blocks leave (they wait for nothing of ours), so the barriers are met; their
  // waits are bounded all the same.
  return launch_dependent(kernel, dim3(plan.blocks), dim3(LAY_THREADS), plan.smem, stream, p);
}
