// Read-only streams over a [N, K] bfloat16 matrix in the access patterns the decoding kernels
// choose between, with nothing but the loads: what each pattern can reach on this device.
// `bench.py --stream-probe` times them.
//
//   coalesced       a warp reads 512 contiguous bytes per instruction
//   fragment        the mma operand pattern of a product of few rows: a block of 8 warps on a tile
//                   of 16 weight rows, lane (g, t) reads 16 bytes of rows g and g + 8 at k + 8t, the
//                   warps take steps of 32 k in turn (a quad asks for half a 128-byte line, another
//                   warp for the other half)
//   fragment, wide  the same with 32 bytes a lane at k + 16t as two loads next to each other, steps
//                   of 64 k (a quad asks for a whole line)
//   async ring      the fragment pattern's rows through a ring of shared-memory stages a warp, filled by
//                   16-byte cp.async copies: the bytes in flight cost no registers
//   bulk            one block per multiprocessor, a producer warp copies row pieces into a ring of
//                   shared-memory stages with cp.async.bulk, a consumer warp frees them
#include "common.cuh"

__device__ __forceinline__ uint4 probe_load16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ unsigned probe_fold(const uint4& v) { return v.x ^ v.y ^ v.z ^ v.w; }

template <int PRE>
__global__ void __launch_bounds__(256) probe_coalesced_kernel(const char* w, size_t bytes, unsigned* sink) {
  const size_t stride = (size_t)gridDim.x * blockDim.x * 16;
  size_t at = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 16;
  unsigned acc = 0;
  for (; at + (PRE - 1) * stride < bytes; at += PRE * stride) {
    uint4 v[PRE];
#pragma unroll
    for (int i = 0; i < PRE; ++i) v[i] = probe_load16(w + at + i * stride);
#pragma unroll
    for (int i = 0; i < PRE; ++i) acc ^= probe_fold(v[i]);
  }
  if (acc == 0x12345678u) sink[0] = acc;      // keeps the loads alive
}

// WIDE = 0: 16 bytes a lane, steps of 32 k; 1: 32 bytes a lane, steps of 64 k.  PRE steps in flight.
template <int PRE, int WIDE>
__global__ void __launch_bounds__(256) probe_fragment_kernel(const char* w, int N, int K, unsigned* sink) {
  constexpr int kStep = WIDE ? 64 : 32, kLane = WIDE ? 16 : 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  unsigned acc = 0;
  for (int tile = blockIdx.x; tile < N / 16; tile += gridDim.x) {
    const char* wa = w + ((size_t)(tile * 16 + g) * K + kLane * t) * 2;
    const char* wb = wa + (size_t)8 * K * 2;
    for (int k = warp * kStep; k < K; k += PRE * 8 * kStep) {
      uint4 a[PRE][1 + WIDE], b[PRE][1 + WIDE];
#pragma unroll
      for (int i = 0; i < PRE; ++i) {
        const int kk = k + i * 8 * kStep;
#pragma unroll
        for (int h = 0; h <= WIDE; ++h) {
          const bool in = kk + kLane * t + 8 * h + 8 <= K;
          a[i][h] = in ? probe_load16(wa + kk * 2 + 16 * h) : make_uint4(0, 0, 0, 0);
          b[i][h] = in ? probe_load16(wb + kk * 2 + 16 * h) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int i = 0; i < PRE; ++i)
#pragma unroll
        for (int h = 0; h <= WIDE; ++h) acc ^= probe_fold(a[i][h]) ^ probe_fold(b[i][h]);
    }
  }
  if (acc == 0x12345678u) sink[0] = acc;
}

// The fragment pattern's rows through shared memory instead of registers: every warp owns a ring of
// DEPTH stages of 16 rows x 128 bytes (steps of 64 k) that it fills with 16-byte asynchronous copies
// (cp.async), 8 lanes on a row's line, and reads a word of when a stage has landed.
template <int DEPTH>
__global__ void __launch_bounds__(256) probe_async_ring_kernel(const char* w, int N, int K, unsigned* sink) {
  extern __shared__ __align__(128) unsigned char probe_ring[];
  constexpr int kPitch = 144, kStage = 16 * kPitch;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* mine = probe_ring + (size_t)warp * DEPTH * kStage;
  unsigned acc = 0;
  const int steps = K / 64;                       // steps of 64 k in a tile; warps take them in turn
  const int my_steps = (steps - warp + 7) / 8;
  for (int tile = blockIdx.x; tile < N / 16; tile += gridDim.x) {
    const char* rows = w + (size_t)tile * 16 * K * 2;
    auto fill = [&](int i) {                      // the warp's i-th step of this tile into stage i % DEPTH
      if (i < my_steps) {
        const int k = (warp + 8 * i) * 64;
        unsigned char* st = mine + (i % DEPTH) * kStage;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int piece = c * 32 + lane, row = piece >> 3, at = (piece & 7) * 16;
          const unsigned dst = (unsigned)__cvta_generic_to_shared(st + row * kPitch + at);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(rows + ((size_t)row * K + k) * 2 + at));
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int i = 0; i < DEPTH - 1; ++i) fill(i);
    for (int i = 0; i < my_steps; ++i) {
      fill(i + DEPTH - 1);
      asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
      __syncwarp();
      acc ^= *reinterpret_cast<const unsigned*>(mine + (i % DEPTH) * kStage + (lane >> 1) * kPitch + (lane & 1) * 64);
      __syncwarp();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
  if (acc == 0x12345678u) sink[0] = acc;
}

__device__ __forceinline__ unsigned probe_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool probe_wait(unsigned long long* bar, unsigned parity) {
  for (unsigned spin = 0; spin < (1u << 18); ++spin) {      // bounded: gives up after some seconds at most
    unsigned done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(probe_smem(bar)), "r"(parity), "r"(20000u) : "memory");
    if (done) return true;
  }
  return false;
}

// rows_per_stage row pieces of `piece` bytes a stage, `stages` stages (at most 16)
__global__ void __launch_bounds__(64, 1) probe_bulk_kernel(const char* w, int N, int K, int piece, int rows_per_stage,
                                                           int stages, unsigned* sink) {
  extern __shared__ __align__(128) unsigned char probe_raw[];
  unsigned long long* full = reinterpret_cast<unsigned long long*>(probe_raw);
  unsigned long long* empty = full + 16;
  unsigned char* ring = probe_raw + 256;
  const int stage_bytes = rows_per_stage * piece;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(probe_smem(&full[i])), "r"(1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(probe_smem(&empty[i])), "r"(1));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int tiles = N / rows_per_stage, per = (tiles + gridDim.x - 1) / gridDim.x;
  const int t0 = blockIdx.x * per, t1 = min(tiles, t0 + per);
  const int slabs = K * 2 / piece;
  if (warp == 0) {
    int c = 0;
    for (int tile = t0; tile < t1; ++tile)
      for (int sl = 0; sl < slabs; ++sl, ++c) {
        const int stage = c % stages, use = c / stages;
        if (use > 0 && !__all_sync(0xffffffffu, probe_wait(&empty[stage], (use - 1) & 1))) return;
        if (lane == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(probe_smem(&full[stage])),
                       "r"(stage_bytes) : "memory");
        __syncwarp();
        for (int r = lane; r < rows_per_stage; r += 32)
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(probe_smem(ring + (size_t)stage * stage_bytes + r * piece)),
                         "l"(w + ((size_t)(tile * rows_per_stage + r) * K) * 2 + (size_t)sl * piece), "r"(piece),
                         "r"(probe_smem(&full[stage])) : "memory");
      }
  } else {
    unsigned acc = 0;
    int c = 0;
    for (int tile = t0; tile < t1; ++tile)
      for (int sl = 0; sl < slabs; ++sl, ++c) {
        const int stage = c % stages, use = c / stages;
        if (!__all_sync(0xffffffffu, probe_wait(&full[stage], use & 1))) return;
        acc ^= *reinterpret_cast<unsigned*>(ring + (size_t)stage * stage_bytes + lane * 16);
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(probe_smem(&empty[stage])) : "memory");
      }
    if (acc == 0x12345678u) sink[0] = acc;
  }
}

// pattern 0: coalesced, 1: fragment, 2: fragment wide (pre = 2, 4 or 8 steps in flight)
TOKB200_API int tokb200_stream_probe_loads(const void* w, int N, int K, int pattern, int pre, int blocks,
                                           unsigned* sink, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || N % 16 || K % 64 || blocks <= 0 || ((uintptr_t)w & 15)) return TOKB200_BAD_SIZE;
  const char* p = (const char*)w;
  const size_t bytes = (size_t)N * K * 2;
#define PROBE_PRE(kernel_of, ...)                                                                  \
  switch (pre) {                                                                                   \
    case 2: kernel_of(2)<<<blocks, 256, 0, stream>>>(__VA_ARGS__); break;                          \
    case 4: kernel_of(4)<<<blocks, 256, 0, stream>>>(__VA_ARGS__); break;                          \
    case 8: kernel_of(8)<<<blocks, 256, 0, stream>>>(__VA_ARGS__); break;                          \
    default: return TOKB200_BAD_SIZE;                                                              \
  }
#define PROBE_COALESCED(n) probe_coalesced_kernel<n>
#define PROBE_NARROW(n) probe_fragment_kernel<n, 0>
#define PROBE_WIDE(n) probe_fragment_kernel<n, 1>
  if (pattern == 0) { PROBE_PRE(PROBE_COALESCED, p, bytes, sink) }
  else if (pattern == 1) { PROBE_PRE(PROBE_NARROW, p, N, K, sink) }
  else if (pattern == 2) { PROBE_PRE(PROBE_WIDE, p, N, K, sink) }
  else return TOKB200_BAD_SIZE;
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? TOKB200_OK : (int)err;
}

// the fragment pattern through a ring of `depth` (4, 6 or 8) stages a warp in shared memory
TOKB200_API int tokb200_stream_probe_async_ring(const void* w, int N, int K, int depth, int blocks, unsigned* sink,
                                                cudaStream_t stream) {
  if (N <= 0 || K <= 0 || N % 16 || K % 64 || blocks <= 0 || ((uintptr_t)w & 15)) return TOKB200_BAD_SIZE;
  const size_t smem = (size_t)8 * depth * 16 * 144;
  cudaError_t err = cudaSuccess;
#define PROBE_RING(n)                                                                                            \
  err = cudaFuncSetAttribute(probe_async_ring_kernel<n>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
  if (err == cudaSuccess) probe_async_ring_kernel<n><<<blocks, 256, smem, stream>>>((const char*)w, N, K, sink);
  if (depth == 4) { PROBE_RING(4) }
  else if (depth == 6) { PROBE_RING(6) }
  else if (depth == 8) { PROBE_RING(8) }
  else return TOKB200_BAD_SIZE;
  if (err == cudaSuccess) err = cudaGetLastError();
  return err == cudaSuccess ? TOKB200_OK : (int)err;
}

TOKB200_API int tokb200_stream_probe_bulk(const void* w, int N, int K, int piece, int rows_per_stage, int stages,
                                          int blocks, unsigned* sink, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || piece <= 0 || piece % 16 || (K * 2) % piece || rows_per_stage <= 0 || N % rows_per_stage ||
      stages < 2 || stages > 16 || blocks <= 0 || ((uintptr_t)w & 15))
    return TOKB200_BAD_SIZE;
  const size_t smem = 256 + (size_t)stages * rows_per_stage * piece;
  if (smem > 220 * 1024) return TOKB200_BAD_SIZE;
  cudaError_t err = cudaFuncSetAttribute(probe_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  if (err != cudaSuccess) return (int)err;
  probe_bulk_kernel<<<blocks, 64, smem, stream>>>((const char*)w, N, K, piece, rows_per_stage, stages, sink);
  err = cudaGetLastError();
  return err == cudaSuccess ? TOKB200_OK : (int)err;
}
