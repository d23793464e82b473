/* An entry point that allocates nothing.  It has no counterpart in the reference
 * (MahadRana/tokenizer has no GPU code at all); it exists for callers of this
 * library that cannot allocate device memory themselves.
 *
 * Who cannot allocate: code that runs while a CUDA stream is being captured into
 * a graph (cudaMalloc is not allowed there), a host that was handed a fixed
 * memory budget and must not grow it (a plug-in inside another process's memory
 * pool, a real-time loop that may not call into the allocator because the call
 * can block or fail), and C callers without torch, which is where the Python
 * side of this package keeps its scratch tensors.
 *
 * tokb200_argmax_no_alloc is the greedy choice of the next token: for each of
 * n_rows rows of `vocab` float32 logits it writes the index of the largest one
 * (equal values: the lower index) to out[row].  It is the same kernel as
 * tokb200_argmax; the difference is where the kernel's scratch lives.  The
 * vocabulary of a row is cut over 32 blocks that leave their candidates in
 * scratch memory and count themselves off; here that scratch is a file-scope
 * __device__ array inside the library (about 65 KB, held by every GPU that loads
 * the library until the process exits) instead of memory the caller provides.
 *
 * Limits and rules:
 *  - n_rows <= tokb200_argmax_no_alloc_max_rows() (256).  More rows are refused
 *    with TOKB200_BAD_SIZE (-1) and nothing is launched; so are vocab <= 0 and
 *    null pointers.  tokb200_no_alloc_error(status) gives the reason as text.
 *  - The first call on each device looks up the array's device address (with that
 *    device current) and keeps it.  Make that first call outside any stream
 *    capture; later calls only enqueue a small memset and the kernel on `stream`.
 *  - All calls share the one array, and it keeps what the last call left there.
 *    The counters that must start at zero are cleared on `stream` before every
 *    launch.  Two calls that can run at the same time on one GPU (different
 *    streams, or different host threads) race on the array: keep calls on one
 *    GPU in one stream order.
 *  - logits and out are device pointers owned by the caller; nothing is
 *    allocated or freed, by this function or by anything it calls.
 *
 * Returns 0, a cudaError_t (> 0), or a negative status of this library. */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int tokb200_argmax_no_alloc(const float* logits, int n_rows, int vocab, int* out,
                            cudaStream_t stream);
int tokb200_argmax_no_alloc_max_rows(void);
const char* tokb200_no_alloc_error(int status);

#ifdef __cplusplus
}
#endif
