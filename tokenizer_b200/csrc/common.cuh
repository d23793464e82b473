// Shared helpers of the sm_100a kernels: the export macro, status codes,
// element conversions and block reductions.  Launchers are `extern "C"`, take
// raw device pointers and a stream, allocate nothing and return a status:
// 0, a cudaError_t (> 0), or one of the negative codes below.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TOKB200_API extern "C" __attribute__((visibility("default")))

enum : int {
  TOKB200_OK = 0,
  TOKB200_BAD_SIZE = -1,      // a size this kernel refuses (message in Python)
  TOKB200_BAD_DTYPE = -2,
  TOKB200_BAD_ALIGNMENT = -3,
  TOKB200_TIMEOUT = -4,       // a bounded device wait gave up
};

// dtype tags shared with Python
enum : int { TOKB200_F32 = 0, TOKB200_BF16 = 1 };

static inline int tokb200_launch_status() {
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? TOKB200_OK : (int)err;
}

// ---- one error word for all libraries ------------------------------------------
// Every wait on the device is bounded.  A wait that gives up sets its library's own flag
// (read and cleared by that library's `..._error()` function) AND stores a non-zero code in
// one word of mapped pinned host memory that all libraries of a process share: the host
// hands each library the word's device address once, after loading it
// (`tokb200_set_error_word`), and reads the word without any CUDA call wherever it has
// just synchronised with the device (after it read a step's ids or logits).  The code is
// library * 16 + reason; a later code may overwrite an earlier one, the flags keep both.
enum : int {
  TOKB200_LIB_GEMM_TCGEN05 = 1,
  TOKB200_LIB_ATTENTION_TCGEN05 = 2,
  TOKB200_LIB_FFN_SMALL_M = 3,
  TOKB200_LIB_LINEAR_STREAM = 4,
  TOKB200_LIB_LAYER_SMALL_M = 5,
};
__device__ int* tokb200_error_word = nullptr;

__device__ __forceinline__ void tokb200_report_error(int library, int reason) {
  int* word = tokb200_error_word;
  if (word != nullptr) {
    *reinterpret_cast<volatile int*>(word) = library * 16 + reason;
    __threadfence_system();
  }
}

// `device_pointer`: the device-side address of the shared word (or null to detach).  A
// synchronous copy: call it outside stream capture.
TOKB200_API int tokb200_set_error_word(int* device_pointer) {
  cudaError_t err = cudaMemcpyToSymbol(tokb200_error_word, &device_pointer, sizeof(int*));
  return err == cudaSuccess ? TOKB200_OK : (int)err;
}

// One int of mapped pinned host memory, zeroed: its host and device addresses.
TOKB200_API int tokb200_error_word_alloc(int** host_pointer, int** device_pointer) {
  int* host = nullptr;
  cudaError_t err = cudaHostAlloc((void**)&host, 64, cudaHostAllocMapped | cudaHostAllocPortable);
  if (err != cudaSuccess) return (int)err;
  *host = 0;
  err = cudaHostGetDevicePointer((void**)device_pointer, host, 0);
  if (err != cudaSuccess) return (int)err;
  *host_pointer = host;
  return TOKB200_OK;
}

// ---- programmatic dependent launch -------------------------------------------
// The step's kernels are launched with the attribute below: a kernel may start
// while its predecessor in the stream still runs, so that its launch and its
// reads of weights (which no kernel of the step writes) overlap the
// predecessor's tail.  `pdl_wait()` returns once the predecessor has completed
// and its writes are visible; every kernel calls it before it touches anything
// a predecessor wrote and before it writes anything a predecessor may read, and
// every block calls it before it exits, so completion stays transitive along the
// stream.  `pdl_launch()` lets the successor start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;"); }

// `early`: whether this launch may start before its predecessor has completed (false: the
// kernel still takes part in the chain, its own successor may start early, but it starts
// strictly after its predecessor).
template <typename... KArgs, typename... Args>
static inline int launch_ordered(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args);

template <typename... KArgs, typename... Args>
static inline int launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                   cudaStream_t stream, Args... args) {
  return launch_ordered(true, kernel, grid, block, smem, stream, args...);
}

template <typename... KArgs, typename... Args>
static inline int launch_ordered(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  // TOKB200_PDL=0 in the environment launches every kernel strictly after its predecessor;
  // TOKB200_PDL_OFF=name[,name...] does so for the kernels of the libraries whose file names
  // contain one of the names (to find which early start a fault depends on)
  static const int overlap = [] {
    const char* v = getenv("TOKB200_PDL");
    if (v && v[0] == '0') return 0;
    const char* off = getenv("TOKB200_PDL_OFF");
    Dl_info here;
    if (off && off[0] && dladdr((const void*)&tokb200_set_error_word, &here) && here.dli_fname) {
      const char* at = off;
      while (*at) {
        const char* end = strchr(at, ',');
        const size_t n = end ? (size_t)(end - at) : strlen(at);
        char name[128];
        if (n > 0 && n < sizeof(name)) {
          memcpy(name, at, n);
          name[n] = 0;
          if (strstr(here.dli_fname, name)) return 0;
        }
        at = end ? end + 1 : at + n;
      }
    }
    return 1;
  }();
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = early ? overlap : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  cudaError_t err = cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
  return err == cudaSuccess ? TOKB200_OK : (int)err;
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// ---- the activation of a gated feed-forward -------------------------------------------
// out = act(gate) * up.  Which activation is a PARAMETER of every kernel that applies one
// (the separate gate kernels, the epilogues of the gated products, the fused feed-forward),
// computed in 32-bit; the tags are shared with Python.
enum : int { TOKB200_ACT_SILU = 0, TOKB200_ACT_GELU_TANH = 1, TOKB200_ACT_RELU = 2, TOKB200_ACT_COUNT = 3 };

__device__ __forceinline__ float gate_activation(int kind, float g) {
  if (kind == TOKB200_ACT_SILU) return g / (1.0f + expf(-g));            // z * sigmoid(z)
  if (kind == TOKB200_ACT_GELU_TANH) {
    const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(inner));
  }
  return fmaxf(g, 0.f);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions for blocks of up to 1024 threads (a multiple of 32).
// `scratch` holds 33 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < warps ? scratch[lane] : 0.f;
    w = warp_sum(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < warps ? scratch[lane] : -INFINITY;
    w = warp_max(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
