// Classifier head of the CIFAR ResNets in one kernel per direction:
//
//   forward :  pooled[b,c] = mean_p feat[b,p,c]            (global average pooling, NHWC feature map)
//              z[b,j]      = sum_c W[j,c] pooled[b,c] + bias[j]
//              loss        = mean_b ( log sum_j exp z[b,j] - z[b,t_b] ),  top-1 / top-5 of the same logits
//              dz[b,j]     = ( softmax(z[b])_j - [j == t_b] ) / B      kept for the backward kernel
//   backward:  dW[j,c] = g sum_b dz[b,j] pooled[b,c] ;  dbias[j] = g sum_b dz[b,j]
//              dfeat[b,p,c] = g / P sum_j dz[b,j] W[j,c]     (g = gradient of the loss, a device scalar)
//
// It replaces avg_pool2d + addmm + log_softmax + nll_loss + topk (metrics) and their five backward
// kernels (dl_code/pcode/models/resnet.py:286-294 and the criterion / metric calls of
// dl_code/pcode/distributed_running_cv.py:52-56).  One CTA per sample; per-sample results are added by
// the last CTA in a fixed order (reproducible loss).  C in {16, 32, 64, 128}, K <= 128 classes.
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch.cuh"

#define HEAD_THREADS 128

struct HeadArgs {
  const float* feat;       // [B, P, C]
  const float* w;          // [K, C]
  const float* bias;       // [K] or null
  const long long* tgt;    // [B]
  float* pooled;           // [B, C]
  float* dz;               // [B, K]
  float* row_loss;         // [B]
  int* row_rank;           // [B]
  unsigned* counter;       // arrival counter (zero before the first call, self-resetting)
  float* out;              // [4] loss, top-1 %, top-5 %, counted rows
  float* loss_out;         // [1]
  const float* g;          // backward: gradient of the loss (null = 1)
  float* dfeat;            // backward: [B, P, C]
  float* dw;               // backward: [K, C]
  float* dbias;            // backward: [K] or null
  int B, P, C, K;
};

__device__ __forceinline__ float head_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(HEAD_THREADS) head_forward_kernel(HeadArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float part[HEAD_THREADS];
  __shared__ float pooled[128];
  __shared__ float z[128];
  __shared__ int last;
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = a.C, K = a.K, groups = HEAD_THREADS / C;
  const int c = tid % C, grp = tid / C;
  // pooling: group grp adds the pixels p = grp, grp + groups, ... of channel c (coalesced over c)
  float s = 0.f;
  const float* fb = a.feat + (size_t)b * a.P * C;
  for (int p = grp; p < a.P; p += groups) s += fb[(size_t)p * C + c];
  part[tid] = s;
  __syncthreads();
  if (tid < C) {
    float t = 0.f;
    for (int gi = 0; gi < groups; ++gi) t += part[gi * C + tid];   // fixed order
    t *= 1.f / (float)a.P;
    pooled[tid] = t;
    a.pooled[(size_t)b * C + tid] = t;
  }
  __syncthreads();
  // logits: one warp per class, lanes stride over the channels
  for (int j = warp; j < K; j += HEAD_THREADS / 32) {
    float d = 0.f;
    for (int cc = lane; cc < C; cc += 32) d = fmaf(a.w[(size_t)j * C + cc], pooled[cc], d);
    d = head_warp_sum(d);
    if (lane == 0) z[j] = d + (a.bias != nullptr ? a.bias[j] : 0.f);
  }
  __syncthreads();
  if (warp == 0) {
    const long long t = a.tgt[b];
    const bool valid = t >= 0 && t < K;
    float m = -INFINITY;
    for (int j = lane; j < K; j += 32) m = fmaxf(m, z[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float zt = valid ? z[t] : 0.f;
    float se = 0.f;
    int rank = 0;
    for (int j = lane; j < K; j += 32) {
      se += __expf(z[j] - m);
      rank += z[j] > zt;
    }
    se = head_warp_sum(se);
    for (int o = 16; o > 0; o >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
    const float inv = 1.f / se, scale = valid ? 1.f / (float)a.B : 0.f;
    for (int j = lane; j < K; j += 32) {
      float p = __expf(z[j] - m) * inv;
      if (j == t) p -= 1.f;
      a.dz[(size_t)b * K + j] = p * scale;
    }
    if (lane == 0) {
      a.row_loss[b] = valid ? (logf(se) + m - zt) : 0.f;
      a.row_rank[b] = valid ? rank : -1;
      __threadfence();
      last = (atomicAdd(a.counter, 1u) == (unsigned)a.B - 1);
      if (last) __threadfence();
    }
  }
  __syncthreads();
  if (!last) return;
  // the last sample's CTA adds the per-sample results in a fixed order
  float ls = 0.f;
  int n1 = 0, n5 = 0, nv = 0;
  for (int i = tid; i < a.B; i += HEAD_THREADS) {
    const int r = __ldcg(a.row_rank + i);
    if (r >= 0) {
      ls += __ldcg(a.row_loss + i);
      n1 += r < 1;
      n5 += r < 5;
      nv += 1;
    }
  }
  __shared__ float fl[HEAD_THREADS];
  __shared__ int i1[HEAD_THREADS], i5[HEAD_THREADS], iv[HEAD_THREADS];
  fl[tid] = ls; i1[tid] = n1; i5[tid] = n5; iv[tid] = nv;
  __syncthreads();
  for (int o = HEAD_THREADS / 2; o > 0; o >>= 1) {
    if (tid < o) {
      fl[tid] += fl[tid + o];
      i1[tid] += i1[tid + o];
      i5[tid] += i5[tid + o];
      iv[tid] += iv[tid + o];
    }
    __syncthreads();
  }
  if (tid == 0) {
    const float n = iv[0] > 0 ? (float)iv[0] : 1.f;
    a.out[0] = fl[0] / n;
    *a.loss_out = fl[0] / n;
    a.out[1] = 100.f * (float)i1[0] / n;
    a.out[2] = 100.f * (float)i5[0] / n;
    a.out[3] = (float)iv[0];
    *a.counter = 0;
  }
}

// CTAs [0, B): gradient of the feature map of one sample.  CTAs [B, B + K): one row of dW (and dbias).
__global__ void __launch_bounds__(HEAD_THREADS) head_backward_kernel(HeadArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float dzs[128];
  __shared__ float dpool[128];
  const int tid = threadIdx.x, C = a.C, K = a.K;
  const float g = a.g != nullptr ? *a.g : 1.f;
  if ((int)blockIdx.x < a.B) {
    const int b = blockIdx.x;
    for (int j = tid; j < K; j += HEAD_THREADS) dzs[j] = a.dz[(size_t)b * K + j];
    __syncthreads();
    if (tid < C) {
      float d = 0.f;
      for (int j = 0; j < K; ++j) d = fmaf(dzs[j], a.w[(size_t)j * C + tid], d);
      dpool[tid] = d * g / (float)a.P;
    }
    __syncthreads();
    float* ob = a.dfeat + (size_t)b * a.P * C;
    const int n4 = a.P * C / 4;
    for (int i = tid; i < n4; i += HEAD_THREADS) {
      const int cc = (i * 4) % C;
      *reinterpret_cast<float4*>(ob + (size_t)i * 4) = make_float4(dpool[cc], dpool[cc + 1], dpool[cc + 2], dpool[cc + 3]);
    }
    return;
  }
  const int j = blockIdx.x - a.B;
  // dW[j, c] = g sum_b dz[b, j] pooled[b, c]: thread = channel (two halves of the batch when C = 64, ...)
  const int groups = HEAD_THREADS / C, c = tid % C, grp = tid / C;
  __shared__ float part[HEAD_THREADS];
  float s = 0.f, sb = 0.f;
  for (int b = grp; b < a.B; b += groups) {
    const float d = a.dz[(size_t)b * K + j];
    s = fmaf(d, a.pooled[(size_t)b * C + c], s);
    sb += d;
  }
  part[tid] = s;
  __syncthreads();
  if (tid < C) {
    float t = 0.f;
    for (int gi = 0; gi < groups; ++gi) t += part[gi * C + tid];
    a.dw[(size_t)j * C + tid] = t * g;
  }
  if (a.dbias != nullptr) {
    __syncthreads();
    part[tid] = (c == 0) ? sb : 0.f;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int gi = 0; gi < groups; ++gi) t += part[gi * C];
      a.dbias[j] = t * g;
    }
  }
}

extern "C" int head_supported(int P, int C, int K) {
  return (C == 16 || C == 32 || C == 64 || C == 128) && K >= 1 && K <= 128 && P >= 1 && (P * C) % 4 == 0;
}

// scratch: B floats + B ints + 1 unsigned (zeroed once by the caller)
extern "C" int head_forward(const void* feat, const void* w, const void* bias, const void* tgt, void* pooled, void* dz,
                            void* scratch, void* out, void* loss_out, int B, int P, int C, int K, cudaStream_t st) {
  if (!head_supported(P, C, K) || B < 1) return -1;
  HeadArgs a = {};
  a.feat = reinterpret_cast<const float*>(feat);
  a.w = reinterpret_cast<const float*>(w);
  a.bias = reinterpret_cast<const float*>(bias);
  a.tgt = reinterpret_cast<const long long*>(tgt);
  a.pooled = reinterpret_cast<float*>(pooled);
  a.dz = reinterpret_cast<float*>(dz);
  a.row_loss = reinterpret_cast<float*>(scratch);
  a.row_rank = reinterpret_cast<int*>(a.row_loss + B);
  a.counter = reinterpret_cast<unsigned*>(a.row_rank + B);
  a.out = reinterpret_cast<float*>(out);
  a.loss_out = reinterpret_cast<float*>(loss_out);
  a.B = B; a.P = P; a.C = C; a.K = K;
  launch_k(head_forward_kernel, dim3(B), dim3(HEAD_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}

extern "C" int head_backward(const void* w, const void* pooled, const void* dz, const void* g, void* dfeat, void* dw,
                             void* dbias, int B, int P, int C, int K, cudaStream_t st) {
  if (!head_supported(P, C, K) || B < 1) return -1;
  HeadArgs a = {};
  a.w = reinterpret_cast<const float*>(w);
  a.pooled = reinterpret_cast<float*>(const_cast<void*>(pooled));
  a.dz = reinterpret_cast<float*>(const_cast<void*>(dz));
  a.g = reinterpret_cast<const float*>(g);
  a.dfeat = reinterpret_cast<float*>(dfeat);
  a.dw = reinterpret_cast<float*>(dw);
  a.dbias = reinterpret_cast<float*>(dbias);
  a.B = B; a.P = P; a.C = C; a.K = K;
  launch_k(head_backward_kernel, dim3(B + K), dim3(HEAD_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}
