// Stand-alone sign bit packing / unpacking: the native replacement of the external
// "bit2byte" torch extension the reference imports (dl_code/pcode/utils/sparsification.py:7,
// :129-163).  One warp ballot produces one 32-bit word: bit b of word w = (x[32 w + b] < 0).
// Unpacking writes +1 / -1 (zero decodes to +1, like the reference's -(v - 1) mapping).
#include "common.cuh"
#include "launch.cuh"

__global__ void sign_pack_kernel(const float* __restrict__ x, long long n, uint32_t* __restrict__ words) {
  const long long n_pad = (n + 31) & ~31ll;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_pad;
       i += (long long)gridDim.x * blockDim.x) {
    const bool neg = (i < n) && (x[i] < 0.f);
    const uint32_t w = __ballot_sync(0xffffffffu, neg);
    if ((threadIdx.x & 31) == 0) words[i >> 5] = w;
  }
}

__global__ void sign_unpack_kernel(const uint32_t* __restrict__ words, long long n, float* __restrict__ out,
                                   float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const uint32_t w = words[i >> 5];
    out[i] = ((w >> (i & 31)) & 1u) ? -scale : scale;
  }
}

extern "C" int sign_pack(const void* x, long long n, void* words, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long n_pad = (n + 31) & ~31ll;
  long long blocks = (n_pad + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  sign_pack_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(x), n,
                                                   reinterpret_cast<uint32_t*>(words));
  return (int)cudaGetLastError();
}

extern "C" int sign_unpack(const void* words, long long n, void* out, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  sign_unpack_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(words), n,
                                                     reinterpret_cast<float*>(out), scale);
  return (int)cudaGetLastError();
}
