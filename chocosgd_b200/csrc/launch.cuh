// Kernel launch with programmatic dependent launch (PDL), and the two device-side calls.
//
// A kernel launched through launch_k() may start while the previous kernel of the same stream is
// still draining: its CTAs are scheduled as soon as every CTA of the previous kernel has called
// pdl_trigger() (or exited), run their prologue (shared-memory and barrier set-up, TMEM
// allocation), and block in pdl_wait() until the previous kernel has completed and its writes
// are visible.  Rules followed by every kernel in this library that is launched this way:
//   * pdl_wait() is executed unconditionally by every CTA before its first access to global
//     memory (so completion stays transitive along the stream);
//   * nothing is written to global memory before pdl_wait().
// Inside a captured CUDA graph the attribute becomes a programmatic dependency edge.  Without the
// attribute (the default, or a launch by plain <<<>>>) both calls are no-ops.
//
// Switched by CHOCO_PDL (read at the first launch), which ops/_lib.py: configure_pdl() sets from --pdl: on for
// bf16-autocast training, off otherwise.  Measured on B200: inside the captured fp32 ResNet-20 step (about 140
// kernels of 3 - 10 us) programmatic edges made the step slower, 1.30 ms against 1.25 ms with plain edges (1.34 ms
// when the trigger precedes the wait and several kernels of the chain become resident at once): a graph's
// kernel-to-kernel hand-over is already cheaper than the bookkeeping of the early launch at that kernel size.
// The bf16 ResNet-50 step (kernels of 10 - 200 us, each with a ring of bulk copies or an operand tile to set up
// before its first load) gains: 12.45 - 12.65 ms against 12.76 - 12.78 ms.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>
#include <utility>

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// SMs of the current device (148 on B200), queried once per process
static inline int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  }
  return sms;
}

static inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("CHOCO_PDL");
    v = (e != nullptr && atoi(e) != 0) ? 1 : 0;
  }
  return v != 0;
}

template <typename... P, typename... A>
static inline cudaError_t launch_k(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                   A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);
}
