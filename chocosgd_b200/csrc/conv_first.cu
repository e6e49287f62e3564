// First layer of the CIFAR networks: 3x3 / stride 1 / pad 1 convolution with 3 input channels
// (NHWC fp32 images, 12 bytes per pixel) and C_out in {16, 32, 64}.  K = 27 is far too small for a
// tensor-core tile and a 12-byte pixel cannot be a TMA row, so both directions are plain fp32 FMA
// kernels that read the image once:
//   forward   thread = (pixel, 4 output channels); its 108 filter values stay in registers while it
//             walks over pixels; optional per-CTA (sum, sum of squares) rows for the batch-norm
//             that follows (same contract as the tcgen05 convolution's epilogue)
//   wgrad     thread = (pixel, 2 output channels) with 54 accumulators; fixed-order reduction inside
//             the CTA, one slice per CTA, slices added in index order by a second kernel
// The input gradient is not needed (the input is the image).
// Replaces the library's direct-convolution and wgrad kernels for this layer
// (dl_code/pcode/models/resnet.py:189, the first convolution of the CIFAR ResNet).
#include <cuda_runtime.h>
#include "launch.cuh"
#include <stdint.h>

#define CF_THREADS 256

struct ConvFirstArgs {
  const float* x;    // [N, H, W, 3]
  const float* w;    // [C_out, 3, 3, 3]
  float* y;          // forward: [N, H, W, C_out]
  const float* dy;   // wgrad
  float* stats;      // forward, optional: [gridDim.x][2 C_out]
  float* partial;    // wgrad: [gridDim.x][C_out * 27]
  int N, H, W;
};

// the 27 input values around pixel (n, h, w): v[(r * 3 + s) * 3 + ci], zero outside the image
__device__ __forceinline__ void cf_load_patch(const ConvFirstArgs& a, int n, int h, int w, float* v) {
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    const int hh = h + r - 1;
    const bool hin = hh >= 0 && hh < a.H;
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const int ww = w + s - 1;
      const bool in = hin && ww >= 0 && ww < a.W;
      const float* p = a.x + (((size_t)n * a.H + (in ? hh : 0)) * a.W + (in ? ww : 0)) * 3;
#pragma unroll
      for (int c = 0; c < 3; ++c) v[(r * 3 + s) * 3 + c] = in ? __ldg(p + c) : 0.f;
    }
  }
}

template <int COUT>
__global__ void __launch_bounds__(CF_THREADS) conv_first_fwd_kernel(ConvFirstArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int Q = COUT / 4;                 // channel quads per pixel
  constexpr int PPB = CF_THREADS / Q;         // pixels per CTA per trip
  __shared__ float red[CF_THREADS * 8];
  const int q = threadIdx.x % Q, pl = threadIdx.x / Q;
  float wr[4][27];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int k = 0; k < 27; ++k) wr[j][k] = __ldg(a.w + (size_t)(q * 4 + j) * 27 + k);
  const long long P = (long long)a.N * a.H * a.W;
  float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
  for (long long p = (long long)blockIdx.x * PPB + pl; p < P; p += (long long)gridDim.x * PPB) {
    const int w = (int)(p % a.W), h = (int)((p / a.W) % a.H), n = (int)(p / ((long long)a.W * a.H));
    float v[27];
    cf_load_patch(a, n, h, w, v);
    float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < 27; ++k)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = fmaf(v[k], wr[j][k], o[j]);
    *reinterpret_cast<float4*>(a.y + p * COUT + q * 4) = make_float4(o[0], o[1], o[2], o[3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s0[j] += o[j];
      s1[j] = fmaf(o[j], o[j], s1[j]);
    }
  }
  if (a.stats == nullptr) return;
  // fixed-order tree over the PPB pixel lanes of each channel quad
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    red[threadIdx.x * 8 + j] = s0[j];
    red[threadIdx.x * 8 + 4 + j] = s1[j];
  }
  __syncthreads();
  for (int stride = PPB >> 1; stride > 0; stride >>= 1) {
    if (pl < stride) {
      float* mine = red + threadIdx.x * 8;
      const float* other = red + (threadIdx.x + stride * Q) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) mine[e] += other[e];
    }
    __syncthreads();
  }
  if (threadIdx.x < Q) {
    float* dst = a.stats + (size_t)blockIdx.x * 2 * COUT;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      dst[q * 4 + j] = red[threadIdx.x * 8 + j];
      dst[COUT + q * 4 + j] = red[threadIdx.x * 8 + 4 + j];
    }
  }
}

template <int COUT>
__global__ void __launch_bounds__(CF_THREADS) conv_first_wgrad_kernel(ConvFirstArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int Q = COUT / 2;                 // channel pairs per pixel
  constexpr int PPB = CF_THREADS / Q;
  extern __shared__ float cf_red[];           // [CF_THREADS][54]
  const int q = threadIdx.x % Q, pl = threadIdx.x / Q;
  float acc[2][27];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int k = 0; k < 27; ++k) acc[j][k] = 0.f;
  const long long P = (long long)a.N * a.H * a.W;
  for (long long p = (long long)blockIdx.x * PPB + pl; p < P; p += (long long)gridDim.x * PPB) {
    const int w = (int)(p % a.W), h = (int)((p / a.W) % a.H), n = (int)(p / ((long long)a.W * a.H));
    float v[27];
    cf_load_patch(a, n, h, w, v);
    const float2 g = *reinterpret_cast<const float2*>(a.dy + p * COUT + q * 2);
#pragma unroll
    for (int k = 0; k < 27; ++k) {
      acc[0][k] = fmaf(g.x, v[k], acc[0][k]);
      acc[1][k] = fmaf(g.y, v[k], acc[1][k]);
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int k = 0; k < 27; ++k) cf_red[threadIdx.x * 54 + j * 27 + k] = acc[j][k];
  __syncthreads();
  // output o = co * 27 + k; the PPB pixel lanes of its channel pair are added in index order
  float* out = a.partial + (size_t)blockIdx.x * COUT * 27;
  for (int o = threadIdx.x; o < COUT * 27; o += CF_THREADS) {
    const int co = o / 27, k = o % 27;
    const int qq = co >> 1, j = co & 1;
    float t = 0.f;
    for (int l = 0; l < PPB; ++l) t += cf_red[(l * Q + qq) * 54 + j * 27 + k];
    out[o] = t;
  }
}

// dw[i] = sum over slices of partial[slice][i]: 16 outputs per CTA, 16 threads per output (slices q, q + 16, ...
// in order, eight loads in flight per trip; then the sixteen sub-sums in order).  The first layer's weight
// gradient is the last thing a backward pass computes, so this kernel's latency is not hidden by anything.
__global__ void __launch_bounds__(256) conv_first_reduce_kernel(const float* __restrict__ partial, int n_parts, int n,
                                                                float* __restrict__ dw) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sub[16][16];
  const int il = threadIdx.x & 15, q = threadIdx.x >> 4;
  const int i = blockIdx.x * 16 + il;
  float acc = 0.f;
  if (i < n) {
    for (int s0 = q; s0 < n_parts; s0 += 16 * 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int sl = s0 + 16 * u;
        v[u] = sl < n_parts ? __ldcg(partial + (size_t)sl * n + i) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) acc += v[u];
    }
  }
  sub[q][il] = acc;
  __syncthreads();
  if (q == 0 && i < n) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) t += sub[j][il];
    dw[i] = t;
  }
}

extern "C" int conv_first_supported(int Cin, int Cout) { return Cin == 3 && (Cout == 16 || Cout == 32 || Cout == 64); }

// CTAs of the forward kernel (= rows of statistics partials): one per SM, at most 8192 / (2 C_out)
extern "C" int conv_first_grid(int N, int H, int W, int Cout) {
  const long long P = (long long)N * H * W;
  const int ppb = CF_THREADS / (Cout / 4);
  long long g = (P + ppb - 1) / ppb;
  long long cap = 8192 / (2 * Cout);
  if (cap > 148) cap = 148;   // 166 registers per thread: one CTA per SM
  if (g > cap) g = cap;
  return (int)(g < 1 ? 1 : g);
}

extern "C" int conv_first_wgrad_parts(int N, int H, int W, int Cout) {
  const long long P = (long long)N * H * W;
  const int ppb = CF_THREADS / (Cout / 2);
  long long g = (P + ppb - 1) / ppb;
  if (g > sm_count() * 2) g = sm_count() * 2;
  return (int)(g < 1 ? 1 : g);
}

extern "C" int conv_first_forward(const void* x, const void* w, void* y, void* stats, int N, int H, int W, int Cout,
                                  cudaStream_t st) {
  if (!conv_first_supported(3, Cout)) return -1;
  ConvFirstArgs a = {};
  a.x = reinterpret_cast<const float*>(x);
  a.w = reinterpret_cast<const float*>(w);
  a.y = reinterpret_cast<float*>(y);
  a.stats = reinterpret_cast<float*>(stats);
  a.N = N; a.H = H; a.W = W;
  const int grid = conv_first_grid(N, H, W, Cout);
  if (Cout == 16) launch_k(conv_first_fwd_kernel<16>, dim3(grid), dim3(CF_THREADS), 0, st, a);
  else if (Cout == 32) launch_k(conv_first_fwd_kernel<32>, dim3(grid), dim3(CF_THREADS), 0, st, a);
  else launch_k(conv_first_fwd_kernel<64>, dim3(grid), dim3(CF_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}

// scratch: conv_first_wgrad_parts() * C_out * 27 floats; dw: [C_out, 3, 3, 3]
extern "C" int conv_first_wgrad(const void* x, const void* dy, void* dw, void* scratch, int N, int H, int W, int Cout,
                                cudaStream_t st) {
  if (!conv_first_supported(3, Cout)) return -1;
  ConvFirstArgs a = {};
  a.x = reinterpret_cast<const float*>(x);
  a.dy = reinterpret_cast<const float*>(dy);
  a.partial = reinterpret_cast<float*>(scratch);
  a.N = N; a.H = H; a.W = W;
  const int grid = conv_first_wgrad_parts(N, H, W, Cout);
  const int smem = CF_THREADS * 54 * 4;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(conv_first_wgrad_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(conv_first_wgrad_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(conv_first_wgrad_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  if (Cout == 16) launch_k(conv_first_wgrad_kernel<16>, dim3(grid), dim3(CF_THREADS), smem, st, a);
  else if (Cout == 32) launch_k(conv_first_wgrad_kernel<32>, dim3(grid), dim3(CF_THREADS), smem, st, a);
  else launch_k(conv_first_wgrad_kernel<64>, dim3(grid), dim3(CF_THREADS), smem, st, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const int n = Cout * 27;
  launch_k(conv_first_reduce_kernel, dim3((n + 15) / 16), dim3(256), 0, st, reinterpret_cast<const float*>(scratch), grid, n,
                                                           reinterpret_cast<float*>(dw));
  return (int)cudaGetLastError();
}
