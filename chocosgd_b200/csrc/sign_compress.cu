// Stand-alone sign + L1-norm compression of one fp32 tensor (the "sign" operator of
// dl_code/pcode/optim/parallel_choco_v.py:476-499 / ef_sign_sgd.py:149-153 for a single
// tensor):  words[w] bit b = (x[32 w + b] < 0),  norm = sum |x|.
//
// The norm is reduced in two deterministic levels: every block writes the partial sum of its
// tile to SCRATCH memory, the last block to arrive (a counter, also in scratch) adds the
// partials in a fixed order.  Two entry points share the kernel:
//   sign_l1_compress          scratch supplied by the caller (normally a torch allocation)
//   sign_l1_compress_noalloc  scratch in a file-scope device array; see choco_b200.h
#include "choco_b200.h"
#include "common.cuh"

#define SLC_TILE 8192  // elements per block

__global__ void __launch_bounds__(CHOCO_THREADS) sign_l1_kernel(const float* __restrict__ x, long long n,
                                                               uint32_t* __restrict__ words,
                                                               float* __restrict__ norm_out,
                                                               float* __restrict__ partial, uint32_t* counter) {
  __shared__ float red[32];
  __shared__ int last;
  const long long t0 = (long long)blockIdx.x * SLC_TILE;
  float acc = 0.f;
  for (int i = threadIdx.x; i < SLC_TILE; i += CHOCO_THREADS) {  // warp-uniform trip count
    const long long pos = t0 + i;
    const bool in = pos < n;
    const float v = in ? x[pos] : 0.f;
    acc += fabsf(v);
    const uint32_t w = __ballot_sync(0xffffffffu, in && v < 0.f);
    if ((threadIdx.x & 31) == 0 && (pos - (pos & 31)) < n) words[pos >> 5] = w;
  }
  const float tot = block_sum(acc, red);
  if (threadIdx.x == 0) {
    partial[blockIdx.x] = tot;
    __threadfence();
    last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    if (last) __threadfence();
  }
  __syncthreads();
  if (last) {
    float a = 0.f;
    for (int c = threadIdx.x; c < (int)gridDim.x; c += CHOCO_THREADS) a += __ldcg(partial + c);
    const float s = block_sum(a, red);
    if (threadIdx.x == 0) {
      *norm_out = s;
      *counter = 0;
    }
  }
}

static int launch_sign_l1(const void* x, long long n, void* words, void* norm_out, float* partial, uint32_t* counter,
                          cudaStream_t stream) {
  const long long blocks = (n + SLC_TILE - 1) / SLC_TILE;
  sign_l1_kernel<<<(unsigned)blocks, CHOCO_THREADS, 0, stream>>>(
      reinterpret_cast<const float*>(x), n, reinterpret_cast<uint32_t*>(words), reinterpret_cast<float*>(norm_out),
      partial, counter);
  return (int)cudaGetLastError();
}

extern "C" long long sign_l1_scratch_bytes(long long n) {
  const long long blocks = (n + SLC_TILE - 1) / SLC_TILE;
  return (blocks + 32) * 4;  // partials + one counter word (on its own 128-byte line)
}

extern "C" int sign_l1_compress(const void* x, long long n, void* words, void* norm_out, void* scratch,
                                cudaStream_t stream) {
  if (n <= 0) return (int)cudaErrorInvalidValue;
  const long long blocks = (n + SLC_TILE - 1) / SLC_TILE;
  float* partial = reinterpret_cast<float*>(scratch);
  uint32_t* counter = reinterpret_cast<uint32_t*>(partial + blocks);
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return (int)e;
  return launch_sign_l1(x, n, words, norm_out, partial, counter, stream);
}

// ---- entry point that allocates nothing -----------------------------------------------------
// Scratch of the no-alloc variant: SIGN_L1_NOALLOC_MAX_BLOCKS partial sums + the arrival
// counter.  64 KiB + 128 B of device memory per GPU that loads this library, held until exit.
__device__ __align__(256) static float g_noalloc_scratch[SIGN_L1_NOALLOC_MAX_BLOCKS + 32];

#define NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES];  // device address of the array, per device

extern "C" int sign_l1_compress_noalloc(const void* x, long long n, void* words, void* norm_out,
                                        cudaStream_t stream) {
  if (n <= 0 || n > SIGN_L1_NOALLOC_MAX_ELEMS) return SIGN_L1_NOALLOC_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
  if (g_noalloc_ptr[dev] == nullptr) {
    // first call on this device: resolve the device address of the array (the name itself is
    // only a host-side handle).  Do this first call outside of any stream capture.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev] = reinterpret_cast<float*>(p);
  }
  float* partial = g_noalloc_ptr[dev];
  uint32_t* counter = reinterpret_cast<uint32_t*>(partial + SIGN_L1_NOALLOC_MAX_BLOCKS);
  // the array keeps whatever the previous call left: the counter must start at zero
  e = cudaMemsetAsync(counter, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return (int)e;
  return launch_sign_l1(x, n, words, norm_out, partial, counter, stream);
}
