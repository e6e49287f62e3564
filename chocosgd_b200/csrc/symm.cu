// Peer-mapped ("symmetric") device allocations for the in-kernel NVLink transport.
//
// Each rank cudaMallocs its mailbox region, exports a CUDA IPC handle, and opens the
// handles of its graph neighbours (exchanged once through the bootstrap process group).
// Opening a handle with cudaIpcMemLazyEnablePeerAccess maps the peer's memory into this
// process, so kernels reach it with ordinary loads and stores that travel over
// NVLink / NVSwitch.  No NVLink multicast object is created: a rank that exits leaves no
// multicast binding behind.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" int symm_alloc(void** ptr, long long bytes) {
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*ptr, 0, (size_t)bytes);
}

extern "C" int symm_free(void* ptr) { return (int)cudaFree(ptr); }

extern "C" int symm_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

extern "C" int symm_get_handle(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

extern "C" int symm_open_handle(const void* handle, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
}

extern "C" int symm_close_handle(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

extern "C" int symm_can_access_peer(int dev, int peer) {
  int ok = 0;
  cudaDeviceCanAccessPeer(&ok, dev, peer);
  return ok;
}

extern "C" const char* choco_cuda_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }
