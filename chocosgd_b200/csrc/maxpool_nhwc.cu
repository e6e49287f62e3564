// 3x3 / stride 2 / pad 1 max pooling on NHWC tensors (bf16 or fp32), forward and backward: the pooling
// layer behind the stem of the ImageNet ResNets (dl_code/pcode/models/resnet.py:196, 223).
//
// forward : y[n, ho, wo, c] = max over the 3x3 window of x; the position of the maximum inside the
//           window (0 .. 8, first maximum in row-major order, as the library breaks ties) goes into a
//           byte per output element instead of a 64-bit flat index.
// backward: gather form, no atomics and no zero-fill pass: an input pixel (h, w) lies in the windows of
//           at most four output pixels; it sums the gradients of those whose recorded position points at
//           it.  Every dx element is written exactly once, in a fixed order (reproducible).
//
// A thread moves VEC channels (16 bytes) of one pixel; C must be a multiple of VEC.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>
#include "launch.cuh"

#define MP_THREADS 256

template <typename T> struct MpVec;
template <> struct MpVec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* v) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  __device__ static void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct MpVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* v) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  __device__ static void store(__nv_bfloat16* p, const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 q = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&q);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// x [N, H, W, C] -> y [N, HO, WO, C], idx [N, HO, WO, C] bytes; HO = (H + 1) / 2, WO = (W + 1) / 2
template <typename T>
__global__ void __launch_bounds__(MP_THREADS) maxpool3x3s2_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                     uint8_t* __restrict__ idx, int N, int H, int W, int C,
                                                                     int HO, int WO) {
  pdl_wait();
  pdl_trigger();
  constexpr int V = MpVec<T>::N;
  const int cv = C / V;
  const long long total = (long long)N * HO * WO * cv;
  for (long long i = (long long)blockIdx.x * MP_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * MP_THREADS) {
    const int c = (int)(i % cv) * V;
    long long p = i / cv;
    const int wo = (int)(p % WO); p /= WO;
    const int ho = (int)(p % HO);
    const int n = (int)(p / HO);
    float best[V];
    uint8_t pos[V];
#pragma unroll
    for (int e = 0; e < V; ++e) { best[e] = -INFINITY; pos[e] = 0; }
    bool first = true;
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int h = 2 * ho - 1 + r;
      if (h < 0 || h >= H) continue;
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        const int w = 2 * wo - 1 + s;
        if (w < 0 || w >= W) continue;
        float v[V];
        MpVec<T>::load(x + (((long long)n * H + h) * W + w) * C + c, v);
#pragma unroll
        for (int e = 0; e < V; ++e)
          if (first || v[e] > best[e] || v[e] != v[e]) {   // first maximum wins; NaN propagates like the library
            best[e] = v[e];
            pos[e] = (uint8_t)(3 * r + s);
          }
        first = false;
      }
    }
    const long long o = (((long long)n * HO + ho) * WO + wo) * C + c;
    MpVec<T>::store(y + o, best);
    if (V == 8) {
      uint2 pk;
      pk.x = pos[0] | (pos[1] << 8) | (pos[2] << 16) | (pos[3] << 24);
      pk.y = pos[4] | (pos[5] << 8) | (pos[6] << 16) | (pos[7] << 24);
      *reinterpret_cast<uint2*>(idx + o) = pk;
    } else {
      *reinterpret_cast<uint32_t*>(idx + o) = pos[0] | (pos[1] << 8) | (pos[2] << 16) | (pos[3] << 24);
    }
  }
}

// dy [N, HO, WO, C], idx -> dx [N, H, W, C]
template <typename T>
__global__ void __launch_bounds__(MP_THREADS) maxpool3x3s2_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ idx,
                                                                     T* __restrict__ dx, int N, int H, int W, int C, int HO,
                                                                     int WO) {
  pdl_wait();
  pdl_trigger();
  constexpr int V = MpVec<T>::N;
  const int cv = C / V;
  const long long total = (long long)N * H * W * cv;
  for (long long i = (long long)blockIdx.x * MP_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * MP_THREADS) {
    const int c = (int)(i % cv) * V;
    long long p = i / cv;
    const int w = (int)(p % W); p /= W;
    const int h = (int)(p % H);
    const int n = (int)(p / H);
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.f;
    // windows that contain (h, w): ho with 2 ho - 1 <= h <= 2 ho + 1, i.e. ho in {h / 2, (h + 1) / 2}
    const int ho0 = h >> 1, ho1 = (h + 1) >> 1, wo0 = w >> 1, wo1 = (w + 1) >> 1;
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int ho = a ? ho1 : ho0;
      if ((a && ho1 == ho0) || ho >= HO) continue;
      const int r = h - (2 * ho - 1);            // row of (h, w) inside that window
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int wo = b ? wo1 : wo0;
        if ((b && wo1 == wo0) || wo >= WO) continue;
        const int s = w - (2 * wo - 1);
        const uint8_t want = (uint8_t)(3 * r + s);
        const long long o = (((long long)n * HO + ho) * WO + wo) * C + c;
        uint8_t pos[V];
        if (V == 8) {
          const uint2 pk = *reinterpret_cast<const uint2*>(idx + o);
#pragma unroll
          for (int e = 0; e < 4; ++e) { pos[e] = (pk.x >> (8 * e)) & 0xFF; pos[4 + e] = (pk.y >> (8 * e)) & 0xFF; }
        } else {
          const uint32_t pk = *reinterpret_cast<const uint32_t*>(idx + o);
#pragma unroll
          for (int e = 0; e < 4; ++e) pos[e] = (pk >> (8 * e)) & 0xFF;
        }
        bool any = false;
#pragma unroll
        for (int e = 0; e < V; ++e) any |= pos[e] == want;
        if (!any) continue;
        float g[V];
        MpVec<T>::load(dy + o, g);
#pragma unroll
        for (int e = 0; e < V; ++e)
          if (pos[e] == want) acc[e] += g[e];
      }
    }
    MpVec<T>::store(dx + (((long long)n * H + h) * W + w) * C + c, acc);
  }
}

static int mp_grid(long long work) {
  long long b = (work + MP_THREADS - 1) / MP_THREADS;
  const long long cap = 8LL * sm_count();
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

// dtype: 0 = fp32 (C a multiple of 4), 1 = bf16 (C a multiple of 8)
extern "C" int maxpool3x3s2_supported(int N, int H, int W, int C, int dtype) {
  if (N < 1 || H < 2 || W < 2 || C < 1) return 0;
  return dtype == 1 ? (C % 8 == 0) : (dtype == 0 ? (C % 4 == 0) : 0);
}

extern "C" int maxpool3x3s2_forward(const void* x, void* y, void* idx, int N, int H, int W, int C, int dtype,
                                    cudaStream_t st) {
  if (!maxpool3x3s2_supported(N, H, W, C, dtype)) return -1;
  const int HO = (H + 1) / 2, WO = (W + 1) / 2;
  const long long work = (long long)N * HO * WO * (C / (dtype ? 8 : 4));
  if (dtype)
    launch_k(maxpool3x3s2_fwd_kernel<__nv_bfloat16>, dim3(mp_grid(work)), dim3(MP_THREADS), 0, st,
             reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(y),
             reinterpret_cast<uint8_t*>(idx), N, H, W, C, HO, WO);
  else
    launch_k(maxpool3x3s2_fwd_kernel<float>, dim3(mp_grid(work)), dim3(MP_THREADS), 0, st,
             reinterpret_cast<const float*>(x), reinterpret_cast<float*>(y), reinterpret_cast<uint8_t*>(idx), N, H, W, C,
             HO, WO);
  return (int)cudaGetLastError();
}

extern "C" int maxpool3x3s2_backward(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int dtype,
                                     cudaStream_t st) {
  if (!maxpool3x3s2_supported(N, H, W, C, dtype)) return -1;
  const int HO = (H + 1) / 2, WO = (W + 1) / 2;
  const long long work = (long long)N * H * W * (C / (dtype ? 8 : 4));
  if (dtype)
    launch_k(maxpool3x3s2_bwd_kernel<__nv_bfloat16>, dim3(mp_grid(work)), dim3(MP_THREADS), 0, st,
             reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const uint8_t*>(idx),
             reinterpret_cast<__nv_bfloat16*>(dx), N, H, W, C, HO, WO);
  else
    launch_k(maxpool3x3s2_bwd_kernel<float>, dim3(mp_grid(work)), dim3(MP_THREADS), 0, st,
             reinterpret_cast<const float*>(dy), reinterpret_cast<const uint8_t*>(idx), reinterpret_cast<float*>(dx), N, H,
             W, C, HO, WO);
  return (int)cudaGetLastError();
}
