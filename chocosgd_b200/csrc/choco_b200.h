/* C API of libchoco_b200.so: entry points meant to be called from outside Python.
 * All functions return 0 on success, a cudaError_t value, or one of the codes below. */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Sign + L1-norm compression of one fp32 tensor of n elements on the current device:
 *   words[(n + 31) / 32]  bit b of word w = (x[32 w + b] < 0)
 *   norm_out[0]           sum of |x|
 * `scratch` is device memory of at least sign_l1_scratch_bytes(n) bytes. */
long long sign_l1_scratch_bytes(long long n);
int sign_l1_compress(const void* x, long long n, void* words, void* norm_out, void* scratch, cudaStream_t stream);

/* Same operation for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference implementation.  It exists for
 * code that runs where cudaMalloc is off limits: inside a communication progress thread or
 * a callback of another runtime, in a process whose memory pool is owned and fully
 * pre-reserved by someone else (an inference server, a framework allocator that has taken
 * the whole device), or in a latency-critical path where an allocation could stall behind
 * other work on the device.  Such callers own x, words and norm_out already; what they
 * cannot provide is the small work area for the two-level norm reduction.
 *
 * - The work area is a fixed array inside the library (64 KiB + 128 B per GPU, resident from
 *   library load until process exit).  Nothing is allocated or freed by this call, neither
 *   with cudaMalloc / cudaFree nor through any allocating library routine.
 * - n must satisfy 1 <= n <= SIGN_L1_NOALLOC_MAX_ELEMS (134,217,728 elements); otherwise
 *   the call does nothing and returns SIGN_L1_NOALLOC_TOO_LARGE.
 * - The first call on each device looks up the device address of the work area
 *   (cudaGetSymbolAddress).  Make that first call with the device current and before any
 *   stream capture begins; later calls only enqueue a 4-byte memset and the kernel.
 * - Every call on a device uses the same work area, and the area keeps the contents of the
 *   previous call (the call clears the one word that must start at zero).  Two calls
 *   whose kernels can overlap on the GPU (different streams, no ordering between them) race
 *   on it and produce wrong norms: order them on one stream or with events. */
#define SIGN_L1_NOALLOC_MAX_BLOCKS 16384
#define SIGN_L1_NOALLOC_MAX_ELEMS (16384LL * 8192LL)
#define SIGN_L1_NOALLOC_TOO_LARGE (-2)
int sign_l1_compress_noalloc(const void* x, long long n, void* words, void* norm_out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
