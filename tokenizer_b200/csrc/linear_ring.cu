// y[M,N] = x[M,K] W[N,K]^T for few rows (M <= 32) and a LARGE weight (the matrices of a wide
// model's decoding step: tens to hundreds of MB each), bfloat16 operands, 32-bit accumulation.
// The product is bound by reading W once, and this kernel is built to keep that stream at the
// device's rate from the first cycle to the last:
//
//   * one block per multiprocessor stays for the whole product (no block starts or ends while
//     the stream runs) and takes row tiles of 16 weight rows in turn;
//   * the weights pass through shared memory: every warp owns a ring of stages of 16 rows x 128
//     bytes (a step of 64 k of the tile's rows) that it fills itself with 16-byte asynchronous
//     copies (cp.async), 8 lanes on a row's 128-byte line, always LR_DEPTH - 1 steps ahead and
//     straight on into the block's next tile.  The bytes in flight cost no registers; a stream
//     of such copies reads 6.1 to 6.5 TB/s from one block a multiprocessor, where plain loads
//     into registers need four to eight resident blocks (`bench.py --stream-probe`);
//   * the rows of x the block needs (its piece of k) are staged in shared memory once, so the
//     steps read nothing from global memory but the weights;
//   * the 8 warps of a block share a tile by interleaved steps of k (mma.sync m16n8k16 with the
//     weight rows as the M side and a permuted k, as in linear_small_m.cu) and add up through
//     shared memory in warp order; K may also be cut over the blocks into `k_splits` pieces whose
//     32-bit partial results [k_splits, M, N] the consumer adds in index order.  Every sum has a
//     fixed order: results are reproducible.
//
// GATED: w [N, K] holds, for every 128 outputs, their 128 "gate" rows followed by their 128 "up"
// rows; a row tile is then 8 gate rows and the 8 up rows of the same outputs, and the result is
// act(gate) * up, [M, N / 2].
#include "common.cuh"

#define LR_WARPS 8
#define LR_THREADS (LR_WARPS * 32)
#define LR_PITCH 144                        // bytes between a stage's rows: the 8 lanes of a quarter warp cover all banks
#define LR_STAGE (16 * LR_PITCH)

__device__ __forceinline__ void lr_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct LrParams {
  const __nv_bfloat16* x;       // [M, K]
  const __nv_bfloat16* w;       // [N, K]
  const float* bias;            // [N] or null (k_splits == 1 only)
  void* out;                    // [M, N] bfloat16 / float32, or float32 [k_splits, M, N]; GATED: [M, N / 2] bfloat16
  int out_is_f32;
  int M, N, K;
  int k_splits, k_per_split;    // k_per_split a multiple of 64
  int depth;                    // stages of a warp's ring
  int x_pitch;                  // bytes between rows of x in shared memory (16 mod 128)
  int act;
};

template <int MT, bool GATED>
__global__ void __launch_bounds__(LR_THREADS, 1)
linear_ring_kernel(const LrParams p) {
  extern __shared__ __align__(128) unsigned char lr_raw[];
  unsigned char* ring = lr_raw;                                                     // [warps][depth][LR_STAGE]
  unsigned char* x_s = ring + (size_t)LR_WARPS * p.depth * LR_STAGE;               // [8 MT][x_pitch]
  float* part = reinterpret_cast<float*>(x_s + (size_t)8 * MT * p.x_pitch);        // [2][warps][16][8 MT + 1]
  constexpr int kPart = LR_WARPS * 16 * (8 * MT + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = gridDim.x, cta = blockIdx.x;
  // a block owns one piece of k (split = block mod S) and walks the row tiles with the other blocks of its piece
  const int split = cta % p.k_splits, rank = cta / p.k_splits;
  const int peers = (G - split + p.k_splits - 1) / p.k_splits;
  const int k_begin = split * p.k_per_split, k_end = min(p.K, k_begin + p.k_per_split);
  const int n_tiles = GATED ? (p.N / 2 + 7) / 8 : (p.N + 15) / 16;
  const int my_tiles = rank < n_tiles ? (n_tiles - rank + peers - 1) / peers : 0;
  const int steps = (k_end - k_begin + 63) / 64;                 // steps of 64 k in the piece
  const int my_steps = steps > warp ? (steps - warp + LR_WARPS - 1) / LR_WARPS : 0;
  const int total = my_tiles * my_steps;                         // this warp's steps over all of the block's tiles
  unsigned char* mine = ring + (size_t)warp * p.depth * LR_STAGE;

  // this lane's four 16-byte pieces of a stage: piece c * 32 + lane -> row of the tile and place in its line
  int piece_row[4], piece_at[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int piece = c * 32 + lane;
    piece_row[c] = piece >> 3;
    piece_at[c] = (piece & 7) * 8;                               // elements
  }
  // The fill cursor walks the warp's steps in order (tile by tile, step by step) without divisions:
  // where the next step's rows start, its k, and the stage it goes to.
  int fill_tile = rank, fill_step = 0, fill_stage = 0, filled = 0;
  const __nv_bfloat16* fill_src[4];
  bool fill_row_ok[4];
  auto fill_rows = [&]() {                                       // the tile's rows behind this lane's four pieces
    int first_row = fill_tile * 16, second_half = first_row + 8;
    if (GATED) {
      const int out0 = fill_tile * 8;
      first_row = (out0 / 128) * 256 + out0 % 128;
      second_half = first_row + 128;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = piece_row[c];
      const int row = r < 8 ? first_row + r : second_half + (r - 8);
      fill_row_ok[c] = row < p.N;
      fill_src[c] = p.w + (size_t)(fill_row_ok[c] ? row : 0) * p.K + k_begin + warp * 64 + piece_at[c];
    }
  };
  fill_rows();
  auto fill = [&]() {                                            // the warp's next step into the next stage
    if (filled < total) {
      const int k_off = LR_WARPS * 64 * fill_step;               // from the warp's first step of the piece
      const int k = k_begin + warp * 64 + k_off;
      const unsigned base = (unsigned)__cvta_generic_to_shared(mine + fill_stage * LR_STAGE);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const bool ok = fill_row_ok[c] && k + piece_at[c] + 8 <= k_end;     // past the matrix or the piece: zeros
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                     ::"r"(base + (unsigned)(piece_row[c] * LR_PITCH + piece_at[c] * 2)),
                       "l"(ok ? fill_src[c] + k_off : p.w), "r"(ok ? 16 : 0));
      }
      ++filled;
      if (++fill_step == my_steps) {
        fill_step = 0;
        fill_tile += peers;
        fill_rows();
      }
      if (++fill_stage == p.depth) fill_stage = 0;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // weights are written by no kernel of the step: the ring fills before the wait on the predecessor
  for (int f = 0; f < p.depth - 1; ++f) fill();
  pdl_wait();          // x comes from the predecessor
  pdl_launch();

  // ---- the block's piece of x into shared memory (asynchronous copies, all in flight at once),
  // rows past M and pieces past the end of k as zeros ----
  {
    const int pieces = p.k_per_split / 8;                        // 16-byte pieces a row: the whole piece of k
    for (int i = threadIdx.x; i < 8 * MT * pieces; i += LR_THREADS) {
      const int m = i / pieces, at = (i % pieces) * 8;
      const bool ok = m < p.M && k_begin + at + 8 <= k_end;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(x_s + (size_t)m * p.x_pitch + at * 2);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                   ::"r"(dst), "l"(ok ? p.x + (size_t)m * p.K + k_begin + at : p.x), "r"(ok ? 16 : 0));
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");         // x (and the ring's first stages, asked for long before)
  }
  __syncthreads();

  int f = 0, turn = 0, read_stage = 0;
  for (int ti = 0; ti < my_tiles; ++ti) {
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    for (int i = 0; i < my_steps; ++i, ++f) {
      fill();                                     // step f + depth - 1, into the stage that step f - 1 has finished reading
      // all but the newest depth - 1 groups have landed: step f is among them
      switch (p.depth) {
        case 4: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 6: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
      }
      __syncwarp();
      const unsigned char* st = mine + read_stage * LR_STAGE;
      if (++read_stage == p.depth) read_stage = 0;
      const int kl = (warp + LR_WARPS * i) * 64;                 // the step's place in the block's piece of k
      uint4 a[2], b[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {               // lane t: k = 16t .. 16t+15 of rows g and g + 8
        a[h] = *reinterpret_cast<const uint4*>(st + g * LR_PITCH + t * 32 + 16 * h);
        b[h] = *reinterpret_cast<const uint4*>(st + (g + 8) * LR_PITCH + t * 32 + 16 * h);
      }
#pragma unroll
      for (int j = 0; j < MT; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          // (pieces of x past the piece of k are zeros, as the weights' are)
          const uint4 xv = *reinterpret_cast<const uint4*>(x_s + (size_t)(8 * j + g) * p.x_pitch + (kl + 16 * t + 8 * h) * 2);
          lr_mma(acc[j], a[h].x, b[h].x, a[h].y, b[h].y, xv.x, xv.y);
          lr_mma(acc[j], a[h].z, b[h].z, a[h].w, b[h].w, xv.z, xv.w);
        }
      }
      __syncwarp();                               // all lanes have read the stage before it is filled again
    }
    // ---- the warps' sums of the tile meet in one of two buffers, in turn: a thread that reads
    // buffer b for tile i has finished by the barrier of tile i + 1, so tile i + 2 may write it ----
    float* mine_part = part + (size_t)turn * kPart + (size_t)warp * 16 * (8 * MT + 1);
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      mine_part[g * (8 * MT + 1) + 8 * j + 2 * t] = acc[j][0];
      mine_part[g * (8 * MT + 1) + 8 * j + 2 * t + 1] = acc[j][1];
      mine_part[(g + 8) * (8 * MT + 1) + 8 * j + 2 * t] = acc[j][2];
      mine_part[(g + 8) * (8 * MT + 1) + 8 * j + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    const int tile = rank + ti * peers;
    const float* all = part + (size_t)turn * kPart;
    if (GATED) {
      const int half = p.N / 2;
      for (int i = threadIdx.x; i < 8 * p.M; i += LR_THREADS) {
        const int m = i / 8, rr = i % 8;
        const int n = tile * 8 + rr;
        if (n >= half) continue;
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int s = 0; s < LR_WARPS; ++s) {
          gate += all[((size_t)s * 16 + rr) * (8 * MT + 1) + m];
          up += all[((size_t)s * 16 + rr + 8) * (8 * MT + 1) + m];
        }
        reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * half + n] =
            __float2bfloat16_rn(gate_activation(p.act, gate) * up);
      }
    } else {
      for (int i = threadIdx.x; i < 16 * p.M; i += LR_THREADS) {
        const int m = i / 16, rr = i % 16;
        const int n = tile * 16 + rr;
        if (n >= p.N) continue;
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < LR_WARPS; ++s) v += all[((size_t)s * 16 + rr) * (8 * MT + 1) + m];
        if (p.k_splits > 1) {
          reinterpret_cast<float*>(p.out)[((size_t)split * p.M + m) * p.N + n] = v;
        } else {
          if (p.bias) v += p.bias[n];
          if (p.out_is_f32) reinterpret_cast<float*>(p.out)[(size_t)m * p.N + n] = v;
          else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
        }
      }
    }
    turn ^= 1;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// The plan for sizes (M, N, K, k_splits) on this device: blocks, the piece of k, the ring's depth and
// shared memory; 0 blocks if the kernel does not take the sizes.
struct LrPlan {
  int blocks, k_per_split, depth, x_pitch;
  size_t smem;
};

static LrPlan lr_plan(int M, int N, int K, int k_splits, bool gated) {
  LrPlan plan = {};
  if (M <= 0 || M > 32 || N <= 0 || K <= 0 || K % 8 || k_splits < 1 || k_splits > 16) return plan;
  if (gated && (N % 256 || k_splits != 1)) return plan;
  int device = 0, sms = 0, smem_max = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return plan;
  if (cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return plan;
  const int MT = M <= 8 ? 1 : M <= 16 ? 2 : 4;
  int kps = ((K + k_splits - 1) / k_splits + 63) / 64 * 64;
  if ((long long)(k_splits - 1) * kps >= K) return plan;               // an empty piece
  if (kps < 64 * LR_WARPS) return plan;                                 // every warp has a step to take
  const int x_pitch = kps * 2 + 16;                                     // 16 mod 128: fragment reads miss each other's banks
  const size_t fixed = (size_t)8 * MT * x_pitch + (size_t)2 * LR_WARPS * 16 * (8 * MT + 1) * 4;
  int depth = 0;
  const int depths[3] = {8, 6, 4};
  for (int i = 0; i < 3 && !depth; ++i)
    if (fixed + (size_t)LR_WARPS * depths[i] * LR_STAGE + 1024 <= (size_t)smem_max) depth = depths[i];
  if (!depth) return plan;
  const int tiles = gated ? (N / 2 + 7) / 8 : (N + 15) / 16;
  const long long units = (long long)tiles * k_splits;
  plan.blocks = (int)(units < sms ? units : sms);
  if (plan.blocks < k_splits) return plan;
  plan.k_per_split = kps;
  plan.depth = depth;
  plan.x_pitch = x_pitch;
  plan.smem = fixed + (size_t)LR_WARPS * depth * LR_STAGE;
  return plan;
}

// 1 when the kernel takes the sizes on this device
TOKB200_API int tokb200_linear_ring_supported(int M, int N, int K, int k_splits, int gated) {
  return lr_plan(M, N, K, k_splits, gated != 0).blocks > 0;
}

template <int MT, bool GATED>
static int lr_launch(const LrParams& p, const LrPlan& plan, cudaStream_t stream) {
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return TOKB200_BAD_SIZE;
  if (!configured[device]) {
    int smem_max = 0;
    if (cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess)
      return TOKB200_BAD_SIZE;
    cudaError_t err = cudaFuncSetAttribute(linear_ring_kernel<MT, GATED>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
    if (err != cudaSuccess) return (int)err;
    configured[device] = true;
  }
  return launch_dependent(linear_ring_kernel<MT, GATED>, dim3(plan.blocks), dim3(LR_THREADS), plan.smem, stream, p);
}

// out: [M, N] bfloat16 or float32 when k_splits == 1 (bias added); float32 partial sums
// [k_splits, M, N] otherwise (no bias: the consumer adds them up).
TOKB200_API int tokb200_linear_ring(const void* x, const void* w, const float* bias, void* out, int out_is_f32,
                                    int M, int N, int K, int k_splits, cudaStream_t stream) {
  const LrPlan plan = lr_plan(M, N, K, k_splits, false);
  if (plan.blocks == 0) return TOKB200_BAD_SIZE;
  if (k_splits > 1 && (bias || !out_is_f32)) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TOKB200_BAD_ALIGNMENT;
  LrParams p;
  p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = bias; p.out = out; p.out_is_f32 = out_is_f32;
  p.M = M; p.N = N; p.K = K; p.k_splits = k_splits; p.k_per_split = plan.k_per_split; p.depth = plan.depth;
  p.x_pitch = plan.x_pitch; p.act = 0;
  return M <= 8 ? lr_launch<1, false>(p, plan, stream)
                : M <= 16 ? lr_launch<2, false>(p, plan, stream) : lr_launch<4, false>(p, plan, stream);
}

// out[M, N/2] (bfloat16) = act(x Wg^T) * (x Wu^T), w in the 128-gate / 128-up row blocks (N a multiple of 256)
TOKB200_API int tokb200_linear_ring_gated(const void* x, const void* w, void* out, int M, int N, int K, int act,
                                          cudaStream_t stream) {
  const LrPlan plan = lr_plan(M, N, K, 1, true);
  if (plan.blocks == 0 || act < 0 || act >= TOKB200_ACT_COUNT) return TOKB200_BAD_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TOKB200_BAD_ALIGNMENT;
  LrParams p;
  p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = nullptr; p.out = out; p.out_is_f32 = 0;
  p.M = M; p.N = N; p.K = K; p.k_splits = 1; p.k_per_split = plan.k_per_split; p.depth = plan.depth;
  p.x_pitch = plan.x_pitch; p.act = act;
  return M <= 8 ? lr_launch<1, true>(p, plan, stream)
                : M <= 16 ? lr_launch<2, true>(p, plan, stream) : lr_launch<4, true>(p, plan, stream);
}
