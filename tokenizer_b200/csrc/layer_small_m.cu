// A whole decoder layer of a decoding step in ONE kernel, for few rows (M <= 16, bfloat16
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
  float* o_part;                // [s_o, M, H]
  __nv_bfloat16* act;           // [M, I]
  int* sync;                    // [2] zero between launches
  // ---- sizes and the plan ----
  int M, H, I, nh, nkv;
  int n_stages, h_pitch;        // h_pitch: bytes between rows of the activation tile in shared memory
  int s_o, k_per_split_o;       // the output projection's cut along k
  int s_down, k_per_split_d;    // the down projection's cut along k
  int att_splits;               // pieces a row's keys are cut into at most
  long long* stamps;            // null, or [blocks, 16]: the time (ns) at which a block's consumers pass each phase
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
  float4 v[KVEC];
#pragma unroll
  for (int grp = 0; grp < KVEC / 4; ++grp) {
    float4 a[3][4];
    uint2 raw[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = (lane + 32 * (grp * 4 + e)) * 4;
      const bool in = i < H;
      v[grp * 4 + e] = in ? __ldcg(reinterpret_cast<const float4*>(xr + i)) : zero4;
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
      const float4 gn = *reinterpret_cast<const float4*>(gain + i);
      const __nv_bfloat162 lo = __floats2bfloat162_rn(v[e].x * inv * gn.x, v[e].y * inv * gn.y);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(v[e].z * inv * gn.z, v[e].w * inv * gn.w);
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

template <int MT>
__global__ void __launch_bounds__(LAY_THREADS, 1)
layer_small_m_kernel(const LayerParams p) {
  extern __shared__ __align__(128) unsigned char lay_raw[];
  const int group = p.nh / p.nkv;
  unsigned char* ring = lay_raw;
  unsigned char* work = ring + (size_t)p.n_stages * LAY_STAGE_BYTES;
  // the work area: h (later the attention's output, later pieces of the activation) and the
  // warps' partial sums; during the attention phase the same bytes stage values and hold the merge
  unsigned char* h_s = work;
  float* part = reinterpret_cast<float*>(h_s + (size_t)8 * MT * p.h_pitch);     // [2][warps][16][8 MT + 1]
  constexpr int kPart = LAY_WARPS * 16 * (8 * MT + 1);
  size_t work_bytes = (size_t)8 * MT * p.h_pitch + (size_t)2 * kPart * 4;
  {
    const size_t stage = (size_t)LAY_WARPS * LAY_TILE * kVStride * 2;
    const size_t merge = (size_t)LAY_WARPS * group * kPieceRow * 4;
    const size_t att = stage > merge ? stage : merge;
    if (att > work_bytes) work_bytes = att;
    work_bytes = (work_bytes + 127) / 128 * 128;
  }
  unsigned long long* full = reinterpret_cast<unsigned long long*>(work + work_bytes);
  unsigned long long* empty = full + p.n_stages;
  __shared__ int grid_ok;
  __shared__ int is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int d = HEAD_DIM, half = HEAD_DIM / 2;
  const int q_width = p.nh * d;
  const int n_tiles_qkv = (p.nh + 2 * p.nkv) * (d / 16);
  const int n_tiles_gu = p.I / 8;
  const int n_row_tiles = p.H / 16;
  // products cut along k: a block owns ONE k range (split = block mod S) and walks the row tiles
  // of that range with the other blocks of the same split, so it stages its columns once
  const int o_split = cta % p.s_o, o_first = cta / p.s_o, o_step = (G - o_split + p.s_o - 1) / p.s_o;
  const int o_k0 = o_split * p.k_per_split_o, o_k1 = min(q_width, o_k0 + p.k_per_split_o);
  const int d_split = cta % p.s_down, d_first = cta / p.s_down, d_step = (G - d_split + p.s_down - 1) / p.s_down;
  const int d_k0 = d_split * p.k_per_split_d, d_k1 = min(p.I, d_k0 + p.k_per_split_d);

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.n_stages; ++i) {
      lay_mbar_init(&full[i], 1);
      lay_mbar_init(&empty[i], LAY_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    grid_ok = 1;
  }
  __syncthreads();

  if (warp == LAY_WARPS) {
    // ------------------------------ producer ------------------------------
    int c = 0;                                   // stages filled so far
    bool ok = true;
    auto fill = [&](const __nv_bfloat16* rows_lo, const __nv_bfloat16* rows_hi, int K, int k0, int kn) {
      // rows_lo: 8 consecutive rows of K elements (stage rows 0..7), rows_hi: stage rows 8..15
      const int stage = c % p.n_stages, use = c / p.n_stages;
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
    // q/k/v: a tile is 8 lanes of a head and their rotation partners
    for (int tile = cta; tile < n_tiles_qkv && ok; tile += G) {
      const int head = tile / (d / 16), j0 = (tile % (d / 16)) * 8;
      const __nv_bfloat16* lo = p.w_qkv + (size_t)(head * d + j0) * p.H;
      for (int k0 = 0; k0 < p.H && ok; k0 += LAY_KC) fill(lo, lo + (size_t)half * p.H, p.H, k0, min(LAY_KC, p.H - k0));
    }
    // the output projection
    for (int rt = o_first; rt < n_row_tiles && ok; rt += o_step) {
      const __nv_bfloat16* rows = p.w_o + (size_t)rt * 16 * q_width;
      for (int k0 = o_k0; k0 < o_k1 && ok; k0 += LAY_KC)
        fill(rows, rows + (size_t)8 * q_width, q_width, k0, min(LAY_KC, o_k1 - k0));
    }
    // gate and up
    for (int tile = cta; tile < n_tiles_gu && ok; tile += G) {
      const int out0 = tile * 8;
      const __nv_bfloat16* gate = p.w_gu + (size_t)((out0 / 128) * 256 + out0 % 128) * p.H;
      for (int k0 = 0; k0 < p.H && ok; k0 += LAY_KC) fill(gate, gate + (size_t)128 * p.H, p.H, k0, min(LAY_KC, p.H - k0));
    }
    // down
    for (int rt = d_first; rt < n_row_tiles && ok; rt += d_step) {
      const __nv_bfloat16* rows = p.w_d + (size_t)rt * 16 * p.I;
      for (int k0 = d_k0; k0 < d_k1 && ok; k0 += LAY_KC)
        fill(rows, rows + (size_t)8 * p.I, p.I, k0, min(LAY_KC, d_k1 - k0));
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  const int tid = threadIdx.x;                   // 0 .. 255
  const int g = lane >> 2, t = lane & 3;
  int c = 0;                                     // stages consumed so far
  bool ok = true;
  int barriers = 0;
  float acc[MT][4];
  // one stage: the warp takes the steps of 32 k that are its own (warp, warp + 8, ...)
  auto multiply = [&](int k_local0, int kn) {
    const int stage = c % p.n_stages, use = c / p.n_stages;
    ok = ok && __all_sync(0xffffffffu, lay_mbar_wait(&full[stage], use & 1));
    if (ok) {
      const unsigned char* st = ring + (size_t)stage * LAY_STAGE_BYTES;
      for (int s = warp; s * 32 < kn; s += LAY_WARPS) {
        const uint4 a = *reinterpret_cast<const uint4*>(st + g * LAY_ROW_PITCH + (s * 32 + 8 * t) * 2);
        const uint4 b = *reinterpret_cast<const uint4*>(st + (g + 8) * LAY_ROW_PITCH + (s * 32 + 8 * t) * 2);
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const uint4 xv = *reinterpret_cast<const uint4*>(
              h_s + (size_t)(8 * j + g) * p.h_pitch + (k_local0 + s * 32 + 8 * t) * 2);
          lay_mma(acc[j], a.x, b.x, a.y, b.y, xv.x, xv.y);
          lay_mma(acc[j], a.z, b.z, a.w, b.w, xv.z, xv.w);
        }
      }
      __syncwarp();
      if (lane == 0) lay_mbar_arrive(&empty[stage]);
    }
    ++c;
  };
  auto clear = [&]() {
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  };
  // The warps' sums of a tile meet in one of two buffers, in turn: a thread that reads buffer
  // b for tile i has, by the barrier of tile i + 1, finished reading it, so tile i + 2 may
  // write it again, and one barrier a tile is enough.
  int turn = 0;
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
    for (int w = 0; w < LAY_WARPS; ++w) v += part[(size_t)turn * kPart + ((size_t)w * 16 + row) * (8 * MT + 1) + m];
    return v;
  };
  // All blocks meet: every consumer's writes are ordered before its block's arrival (block
  // barrier, then one thread's fence and atomic), and the waiters' reads after it.  A wait that
  // ran out once makes the block skip all later waits (it still arrives, for the others).
  auto grid_barrier = [&]() {
    ++barriers;
    lay_consumer_sync();
    if (tid == 0) {
      __threadfence();
      atomicAdd(&p.sync[0], 1);
      if (grid_ok) {
        bool met = false;
        const int target = barriers * G;
        for (unsigned spin = 0; spin < LAY_GRID_WAIT_LIMIT; ++spin) {
          int seen;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.sync) : "memory");
          if (seen >= target) { met = true; break; }
          __nanosleep(32);
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
      p.stamps[(size_t)cta * 16 + stamp_at] = now;
    }
    ++stamp_at;
  };
  stamp();             // 0: consumers start
  pdl_wait();          // x and the pending sums come from the predecessor; the weights do not
  pdl_launch();
  stamp();             // 1: the predecessor is done

  // ======================= phase 0: the first norm =======================
  lay_norm<MT>(p.x_in, p.delta, p.delta_is_f32, p.n_partials, p.partial_stride, p.gain1, p.eps1,
               cta == 0 ? p.x_mid : nullptr, h_s, p.h_pitch, p.M, p.H, warp, lane);
  lay_consumer_sync();
  stamp();             // 2: first norm done

  // ======================= phase 1: q, k, v with bias, rotation, cache write =======================
  for (int tile = cta; tile < n_tiles_qkv; tile += G) {
    const int head = tile / (d / 16), j0 = (tile % (d / 16)) * 8;
    // what the epilogue needs from memory is asked for before the product
    const int em = tid / 8, ej = j0 + tid % 8;
    float e_bias_a = 0.f, e_bias_b = 0.f, e_cos = 1.f, e_sin = 0.f;
    int e_slot = -1;
    if (tid < 8 * p.M) {
      if (p.b_qkv) {
        e_bias_a = p.b_qkv[head * d + ej];
        e_bias_b = p.b_qkv[head * d + ej + half];
      }
      if (head >= p.nh && p.slot) e_slot = p.slot[em];
      if (head < p.nh + p.nkv) {
        const int at = p.pos[em];
        e_cos = p.cos_t[(size_t)at * half + ej];
        e_sin = p.sin_t[(size_t)at * half + ej];
      }
    }
    clear();
    for (int k0 = 0; k0 < p.H; k0 += LAY_KC) multiply(k0, min(LAY_KC, p.H - k0));
    spill();
    lay_consumer_sync();
    if (tid < 8 * p.M && ok) {
      const int rr = tid % 8;
      float a = summed(rr, em) + e_bias_a, b = summed(rr + 8, em) + e_bias_b;
      __nv_bfloat16* dst = nullptr;
      if (head < p.nh) {
        dst = p.q_buf + ((size_t)em * p.nh + head) * d;
      } else if (e_slot >= 0) {
        const bool is_key = head < p.nh + p.nkv;
        __nv_bfloat16* pool = is_key ? p.k_pool : p.v_pool;
        if (pool) dst = pool + ((size_t)e_slot * p.nkv + (head - p.nh - (is_key ? 0 : p.nkv))) * d;
      }
      if (head < p.nh + p.nkv) {                              // values are not rotated
        const float ra = a * e_cos - b * e_sin, rb = b * e_cos + a * e_sin;
        a = ra;
        b = rb;
      }
      if (dst) {
        dst[ej] = __float2bfloat16_rn(a);
        dst[ej + half] = __float2bfloat16_rn(b);
      }
    }
    turn ^= 1;
  }
  stamp();             // 3: q/k/v done
  grid_barrier();
  stamp();             // 4: barrier 1 passed

  // ======================= phase 2: attention =======================
  // a unit is (row, kv head, piece of the row's keys); the group's query heads are the M side of
  // the mma, so keys and values are read once per group
  {
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int n_units = p.M * p.nkv * p.att_splits;
    __nv_bfloat16* v_s = reinterpret_cast<__nv_bfloat16*>(work) + (size_t)warp * LAY_TILE * kVStride;
    float* acc_s = reinterpret_cast<float*>(work);            // [warp][head][kPieceRow], after the passes
    for (int unit = cta; unit < n_units && ok; unit += G) {
      const int split = unit % p.att_splits, kvh = (unit / p.att_splits) % p.nkv, row = unit / (p.att_splits * p.nkv);
      const int r = p.row_req[row];
      if (r < 0) continue;                                    // uniform over the block
      const int at = p.pos[row];
      const int lo = (p.window >= 0 && at - p.window > 0) ? at - p.window : 0;
      const int n_keys = at - lo + 1;
      const int chunk = ((n_keys + p.att_splits - 1) / p.att_splits + LAY_TILE - 1) / LAY_TILE * LAY_TILE;
      const int n_splits = (n_keys + chunk - 1) / chunk;
      if (split >= n_splits) continue;
      const int first = lo + split * chunk;
      const int last = min(at, first + chunk - 1);
      const int* table = p.block_table + (size_t)r * p.table_stride;

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
      float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
      float o[HEAD_DIM / 8][4];
#pragma unroll
      for (int i = 0; i < HEAD_DIM / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

      for (int k0 = first + warp * LAY_TILE; k0 <= last; k0 += LAY_WARPS * LAY_TILE) {
        {
          // the tile's values go straight to their staging rows (a lane per key)
          const int key = k0 + lane;
          const bool in = key <= last;
          const int key_ok = in ? key : k0;
          const int s = table[key_ok / p.page] * p.page + key_ok % p.page;
          const __nv_bfloat16* vrow = p.v_read + ((size_t)s * p.nkv + kvh) * d;
          const unsigned dst = lay_smem(v_s + lane * kVStride);
          const int bytes = in ? 16 : 0;
#pragma unroll
          for (int cc = 0; cc < HEAD_DIM / 8; ++cc)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst + cc * 16), "l"(vrow + cc * 8), "r"(bytes));
          asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        float s[LAY_TILE / 8][4];
#pragma unroll
        for (int nt = 0; nt < LAY_TILE / 8; ++nt) {
          s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
          const int key = k0 + nt * 8 + g;
          const bool in = key <= last;
          const int key_ok = in ? key : k0;
          const int sl = table[key_ok / p.page] * p.page + key_ok % p.page;
          const __nv_bfloat16* krow = p.k_read + ((size_t)sl * p.nkv + kvh) * d;
#pragma unroll
          for (int st = 0; st < HEAD_DIM / 32; ++st) {
            const uint4 kv = lay_load16_cg(krow + st * 32 + 8 * t, in);
            lay_mma(s[nt], qa[st][0][0], qa[st][0][1], qa[st][0][2], qa[st][0][3], kv.x, kv.y);
            lay_mma(s[nt], qa[st][1][0], qa[st][1][1], qa[st][1][2], qa[st][1][3], kv.z, kv.w);
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
        __threadfence();
        lay_consumer_sync();
        if (tid == 0) {
          const int done = atomicAdd(&p.att_count[row * p.nkv + kvh], 1);
          is_last = done == n_splits - 1;
          if (is_last) p.att_count[row * p.nkv + kvh] = 0;   // ready for the next launch
        }
        lay_consumer_sync();
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
            for (int c0 = 0; c0 < HEAD_DIM; c0 += 32) {
              const int cc = c0 + lane;
              float num = 0.f;
              for (int sp = 0; sp < n_splits; ++sp)
                num += __shfl_sync(0xffffffffu, f, sp) * __ldcg(&pieces[(size_t)sp * kPieceRow + cc]);
              p.att_out[((size_t)row * p.nh + kvh * group + head) * d + cc] = __float2bfloat16_rn(num / den);
            }
          }
        }
      }
      lay_consumer_sync();       // the work area is reused by the block's next unit
    }
  }
  stamp();             // 5: attention done
  grid_barrier();
  stamp();             // 6: barrier 2 passed

  // ======================= phase 3: the output projection, cut along k =======================
  if (o_first < n_row_tiles) {
    // this block's k range of the attention's output, all rows, into shared memory (idle rows and
    // rows past M: zeros, so that they add nothing)
    const int pieces = p.k_per_split_o / 8;
    for (int i = tid; i < 8 * MT * pieces; i += LAY_CONSUMERS) {
      const int m = i / pieces, piece = i % pieces;
      const bool live = m < p.M && o_k0 + piece * 8 < o_k1 && p.row_req[m] >= 0;
      const uint4 v = lay_load16_cg(p.att_out + (size_t)m * q_width + o_k0 + piece * 8, live);
      *reinterpret_cast<uint4*>(h_s + (size_t)m * p.h_pitch + piece * 16) = v;
    }
  }
  lay_consumer_sync();
  for (int rt = o_first; rt < n_row_tiles; rt += o_step) {
    clear();
    for (int k0 = o_k0; k0 < o_k1; k0 += LAY_KC) multiply(k0 - o_k0, min(LAY_KC, o_k1 - k0));
    spill();
    lay_consumer_sync();
    for (int i = tid; i < 16 * p.M; i += LAY_CONSUMERS) {
      const int m = i / 16, rr = i % 16;
      p.o_part[((size_t)o_split * p.M + m) * p.H + rt * 16 + rr] = summed(rr, m);
    }
    turn ^= 1;
  }
  stamp();             // 7: output projection done
  grid_barrier();
  stamp();             // 8: barrier 3 passed

  // ======================= phase 4: the second norm =======================
  lay_norm<MT>(p.x_mid, p.o_part, 1, p.s_o, (long long)p.M * p.H, p.gain2, p.eps2,
               cta == 0 ? p.x_out : nullptr, h_s, p.h_pitch, p.M, p.H, warp, lane);
  lay_consumer_sync();
  stamp();             // 9: second norm done

  // ======================= phase 5: gate and up, activation =======================
  for (int tile = cta; tile < n_tiles_gu; tile += G) {
    clear();
    for (int k0 = 0; k0 < p.H; k0 += LAY_KC) multiply(k0, min(LAY_KC, p.H - k0));
    spill();
    lay_consumer_sync();
    for (int i = tid; i < 8 * p.M; i += LAY_CONSUMERS) {
      const int m = i / 8, rr = i % 8;
      const float gate = summed(rr, m), up = summed(rr + 8, m);
      p.act[(size_t)m * p.I + tile * 8 + rr] = __float2bfloat16_rn(gate_activation(p.activation, gate) * up);
    }
    turn ^= 1;
  }
  stamp();             // 10: gate/up done
  grid_barrier();
  stamp();             // 11: barrier 4 passed

  // ======================= phase 6: down, cut along k =======================
  if (d_first < n_row_tiles) {
    const int pieces = p.k_per_split_d / 8;
    for (int i = tid; i < 8 * MT * pieces; i += LAY_CONSUMERS) {
      const int m = i / pieces, piece = i % pieces;
      const uint4 v = lay_load16_cg(p.act + (size_t)m * p.I + d_k0 + piece * 8, m < p.M && d_k0 + piece * 8 < d_k1);
      *reinterpret_cast<uint4*>(h_s + (size_t)m * p.h_pitch + piece * 16) = v;
    }
  }
  lay_consumer_sync();
  for (int rt = d_first; rt < n_row_tiles; rt += d_step) {
    clear();
    for (int k0 = d_k0; k0 < d_k1; k0 += LAY_KC) multiply(k0 - d_k0, min(LAY_KC, d_k1 - k0));
    spill();
    lay_consumer_sync();
    for (int i = tid; i < 16 * p.M; i += LAY_CONSUMERS) {
      const int m = i / 16, rr = i % 16;
      p.out[((size_t)d_split * p.M + m) * p.H + rt * 16 + rr] = summed(rr, m);
    }
    turn ^= 1;
  }
  stamp();             // 12: down done

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
  int blocks, n_stages, h_pitch, s_o, k_per_split_o, s_down, k_per_split_d, smem_max;
  size_t smem;
};

static int lay_cut(int sms, int row_tiles, int K, int* k_per_split) {
  // about two units (row tile, piece of k) a block; pieces of whole 32s
  int s = (2 * sms + row_tiles / 2) / row_tiles;
  if (s < 1) s = 1;
  if (s > 16) s = 16;
  int kps = ((K + s - 1) / s + 31) / 32 * 32;
  s = (K + kps - 1) / kps;
  *k_per_split = kps;
  return s;
}

static LayerPlan lay_plan(int M, int H, int I, int nh, int nkv) {
  LayerPlan plan = {};
  if (M <= 0 || M > 16 || H <= 0 || H > 4096 || I <= 0 || H % 32 || I % 128 || nh <= 0 || nkv <= 0 || nh % nkv ||
      nh / nkv > LAY_MAX_GROUP || (nh * HEAD_DIM) % 32)
    return plan;
  int device = 0, sms = 0, smem_max = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return plan;
  const int MT = M <= 8 ? 1 : 2;
  const int row_tiles = H / 16;
  plan.s_o = lay_cut(sms, row_tiles, nh * HEAD_DIM, &plan.k_per_split_o);
  plan.s_down = lay_cut(sms, row_tiles, I, &plan.k_per_split_d);
  int widest = H;
  if (plan.k_per_split_o > widest) widest = plan.k_per_split_o;
  if (plan.k_per_split_d > widest) widest = plan.k_per_split_d;
  plan.h_pitch = (2 * widest + 127) / 128 * 128 + 64;
  const int group = nh / nkv;
  size_t work = (size_t)8 * MT * plan.h_pitch + (size_t)2 * LAY_WARPS * 16 * (8 * MT + 1) * 4;
  const size_t stage = (size_t)LAY_WARPS * LAY_TILE * kVStride * 2;
  const size_t merge = (size_t)LAY_WARPS * group * kPieceRow * 4;
  const size_t att = stage > merge ? stage : merge;
  if (att > work) work = att;
  work = (work + 127) / 128 * 128;
  const long long room = (long long)smem_max - 2048 - (long long)work - 1024;
  int stages = (int)(room / LAY_STAGE_BYTES);
  if (stages > 8) stages = 8;
  if (stages < 3) return plan;
  plan.blocks = sms;
  plan.n_stages = stages;
  plan.smem_max = smem_max;
  plan.smem = work + (size_t)stages * LAY_STAGE_BYTES + 1024;
  return plan;
}

// Partial sums of the feed-forward that `out` holds for these sizes (0: sizes not taken), and
// those of the output projection that `o_part` must hold.
TOKB200_API int tokb200_layer_small_m_splits(int M, int H, int I, int nh, int nkv, int* o_splits) {
  const LayerPlan plan = lay_plan(M, H, I, nh, nkv);
  if (o_splits) *o_splits = plan.blocks ? plan.s_o : 0;
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
  long long* stamps;          // null, or [blocks, 16] for the phases' times (profiling)
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
  p.n_stages = plan.n_stages; p.h_pitch = plan.h_pitch; p.s_o = plan.s_o; p.k_per_split_o = plan.k_per_split_o;
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
  void (*kernel)(const LayerParams) = a->M <= 8 ? layer_small_m_kernel<1> : layer_small_m_kernel<2>;
  static bool configured[64][2] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!configured[device][a->M <= 8 ? 0 : 1]) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_max - 1024);
    if (err != cudaSuccess) return (int)err;
    configured[device][a->M <= 8 ? 0 : 1] = true;
  }
  // One block per SM, each with most of an SM's shared memory: all blocks become resident as the
  // predecessor's blocks leave (they wait for nothing of ours), so the barriers are met; their
  // waits are bounded all the same.
  return launch_dependent(kernel, dim3(plan.blocks), dim3(LAY_THREADS), plan.smem, stream, p);
}
