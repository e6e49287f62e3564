// Training-mode BatchNorm fused with the residual add and ReLU around it, NHWC bf16 activations
// (fp32 statistics, gamma / beta and their gradients): the form a bf16-autocast ImageNet ResNet needs.
//
//   forward :  y = relu( (x - mean_c) * invstd_c * gamma_c + beta_c  [+ residual] )
//   backward:  g = dy * [y > 0] ;  dbeta = sum g ;  dgamma = sum g * xhat ;
//              dx = gamma invstd (g - dbeta / P - xhat dgamma / P) ;  dresidual = g
//
// Three kernels per direction: per-channel partial sums per CTA (one pass over the activation), a
// small finalize (partials added per channel in a fixed order, in double precision: reproducible),
// and one elementwise pass.  Replaces, per layer, the library's statistics + transform kernels and the
// separate add / ReLU kernels forward, and ReLU-backward + reduce + elementwise kernels backward
// (dl_code/pcode/models/resnet.py:86-127: conv -> bn -> relu ... conv -> bn -> += residual -> relu).
//
// Layout: [P, C] with C contiguous, C a multiple of 8, C / 8 a power of two <= 256 (C = 8 ... 2048);
// a thread moves 8 channels (16 bytes) at a time.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "bn_args.h"
#include "launch.cuh"

#define BN16_THREADS 256

struct F8 {
  float v[8];
};

__device__ __forceinline__ F8 bn16_ld8(const void* base, size_t elem_off) {
  const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem_off);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  F8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    r.v[2 * i] = __uint_as_float(w[i] << 16);            // bf16 = the upper half of an fp32
    r.v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
  return r;
}

__device__ __forceinline__ void bn16_st8(void* base, size_t elem_off, const F8& f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f.v[2 * i], f.v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + elem_off) = make_uint4(w[0], w[1], w[2], w[3]);
}

// per-channel sums over this CTA's rows -> partial[blockIdx.x][2 C]
//   forward : (sum x, sum x^2)        backward: (sum g, sum g * xhat), g = dy * [y > 0]
// (two CTAs per SM also in the backward form, whose three operand streams need the registers)
template <bool BACKWARD>
__global__ void __launch_bounds__(BN16_THREADS, 2) bn16_reduce_kernel(BnArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sh[BN16_THREADS * 16];
  const int C = a.C, tpr = C >> 3;             // threads per row
  const int rpb = BN16_THREADS / tpr;           // rows per pass
  const int col = (threadIdx.x % tpr) * 8, rsub = threadIdx.x / tpr;
  const int rows_per_cta = (a.P + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(a.P, r0 + rows_per_cta);
  float s0[8], s1[8], mu[8], is[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    s0[e] = 0.f; s1[e] = 0.f;
    mu[e] = BACKWARD ? a.mean[col + e] : 0.f;
    is[e] = BACKWARD ? a.invstd[col + e] : 1.f;
  }
  // UN rows per trip: all their loads are issued before the first accumulate
  constexpr int UN = BACKWARD ? 2 : 4;
  for (int r = r0 + rsub; r < r1; r += UN * rpb) {
    F8 xv[UN], gv[UN], yv[UN];
    bool in[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int rr = r + u * rpb;
      in[u] = rr < r1;
      const size_t off = (size_t)(in[u] ? rr : r) * C + col;
      xv[u] = bn16_ld8(a.x, off);
      if (BACKWARD) {
        gv[u] = bn16_ld8(a.dy, off);
        if (a.relu) yv[u] = bn16_ld8(a.y, off);
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      if (!in[u]) continue;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x = xv[u].v[e];
        if (!BACKWARD) {
          s0[e] += x;
          s1[e] = fmaf(x, x, s1[e]);
        } else {
          float g = gv[u].v[e];
          if (a.relu) g = yv[u].v[e] > 0.f ? g : 0.f;
          s0[e] += g;
          s1[e] = fmaf(g, (x - mu[e]) * is[e], s1[e]);
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    sh[threadIdx.x * 16 + e] = s0[e];
    sh[threadIdx.x * 16 + 8 + e] = s1[e];
  }
  __syncthreads();
  // fixed-shape tree over the rows held by this CTA (rpb is a power of two): reproducible
  for (int stride = rpb >> 1; stride > 0; stride >>= 1) {
    if (rsub < stride) {
      float* mine = sh + threadIdx.x * 16;
      const float* other = sh + (threadIdx.x + stride * tpr) * 16;
#pragma unroll
      for (int e = 0; e < 16; ++e) mine[e] += other[e];
    }
    __syncthreads();
  }
  if (threadIdx.x < tpr) {
    float* dst = a.partial + (size_t)blockIdx.x * 2 * C;
    const float* p = sh + threadIdx.x * 16;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dst[col + e] = p[e];
      dst[C + col + e] = p[8 + e];
    }
  }
}

// A CTA finalizes 16 channels: 16 threads per channel add strided subsets of the G partial rows (four
// independent loads per trip), then the 16 sub-sums are added in order (double accumulation, a fixed
// order: reproducible).
#define BN16_FIN_CH 16
#define BN16_FIN_SUB (BN16_THREADS / BN16_FIN_CH)
template <bool BACKWARD>
__global__ void __launch_bounds__(BN16_THREADS) bn16_finalize_kernel(BnArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ double sh0[BN16_FIN_SUB][BN16_FIN_CH], sh1[BN16_FIN_SUB][BN16_FIN_CH];
  const int cl = threadIdx.x % BN16_FIN_CH, sub = threadIdx.x / BN16_FIN_CH;
  const int c = blockIdx.x * BN16_FIN_CH + cl;
  const int C2 = 2 * a.C, G = a.n_partials;
  double t0 = 0.0, t1 = 0.0;
  if (c < a.C) {
    int b = sub;
    for (; b + 3 * BN16_FIN_SUB < G; b += 4 * BN16_FIN_SUB) {
      float u0[4], u1[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        u0[q] = __ldcg(a.partial + (size_t)(b + q * BN16_FIN_SUB) * C2 + c);
        u1[q] = __ldcg(a.partial + (size_t)(b + q * BN16_FIN_SUB) * C2 + a.C + c);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        t0 += (double)u0[q];
        t1 += (double)u1[q];
      }
    }
    for (; b < G; b += BN16_FIN_SUB) {
      t0 += (double)__ldcg(a.partial + (size_t)b * C2 + c);
      t1 += (double)__ldcg(a.partial + (size_t)b * C2 + a.C + c);
    }
  }
  sh0[sub][cl] = t0;
  sh1[sub][cl] = t1;
  __syncthreads();
  if (sub != 0 || c >= a.C) return;
  t0 = 0.0; t1 = 0.0;
  for (int j = 0; j < BN16_FIN_SUB; ++j) {
    t0 += sh0[j][cl];
    t1 += sh1[j][cl];
  }
  if (!BACKWARD) {
    const double mean = t0 / a.P;
    double var = t1 / a.P - mean * mean;
    if (var < 0.0) var = 0.0;
    a.mean[c] = (float)mean;
    a.invstd[c] = (float)(1.0 / sqrt(var + (double)a.eps));
    if (a.running_mean != nullptr) {
      const double unbiased = a.P > 1 ? var * a.P / (a.P - 1) : var;
      a.running_mean[c] = (1.f - a.momentum) * a.running_mean[c] + a.momentum * (float)mean;
      a.running_var[c] = (1.f - a.momentum) * a.running_var[c] + a.momentum * (float)unbiased;
    }
  } else {
    a.dbeta[c] = (float)t0;
    a.dgamma[c] = (float)t1;
  }
}

// Elementwise passes.  Per-channel constants are folded into (scale, shift) pairs in shared memory first:
//   forward : y = x * A + B,               A = gamma invstd,  B = beta - mean A
//   backward: dx = g * A - x * Bx - K,     A = gamma invstd,  Bx = A invstd dgamma / P,
//                                          K = A (dbeta / P - mean invstd dgamma / P)
#define BN16_MAX_C 2048

__global__ void __launch_bounds__(BN16_THREADS) bn16_fwd_apply_kernel(BnArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float cA[BN16_MAX_C], cB[BN16_MAX_C];
  for (int c = threadIdx.x; c < a.C; c += BN16_THREADS) {
    const float A = a.gamma[c] * a.invstd[c];
    cA[c] = A;
    cB[c] = a.beta[c] - a.mean[c] * A;
  }
  __syncthreads();
  const size_t n8 = (size_t)a.P * a.C / 8;
  const int c8 = a.C >> 3;
  const size_t stride = (size_t)gridDim.x * BN16_THREADS;
  // two 16-byte loads (four with a residual) in flight per thread
  for (size_t i0 = (size_t)blockIdx.x * BN16_THREADS + threadIdx.x; i0 < n8; i0 += 2 * stride) {
    F8 xv[2], rv[2];
    bool in[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const size_t i = i0 + u * stride;
      in[u] = i < n8;
      if (in[u]) {
        xv[u] = bn16_ld8(a.x, i * 8);
        if (a.residual != nullptr) rv[u] = bn16_ld8(a.residual, i * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (!in[u]) continue;
      const size_t i = i0 + u * stride;
      const int col = (int)(i & (size_t)(c8 - 1)) * 8;   // C / 8 is a power of two
      F8 y;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float v = fmaf(xv[u].v[e], cA[col + e], cB[col + e]);
        if (a.residual != nullptr) v += rv[u].v[e];
        if (a.relu) v = fmaxf(v, 0.f);
        y.v[e] = v;
      }
      bn16_st8(a.out, i * 8, y);
    }
  }
}

__global__ void __launch_bounds__(BN16_THREADS) bn16_bwd_apply_kernel(BnArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float cA[BN16_MAX_C], cBx[BN16_MAX_C], cK[BN16_MAX_C];
  const float inv_p = 1.f / (float)a.P;
  for (int c = threadIdx.x; c < a.C; c += BN16_THREADS) {
    const float is = a.invstd[c], A = a.gamma[c] * is;
    const float dg = a.dgamma[c] * inv_p, db = a.dbeta[c] * inv_p;
    cA[c] = A;
    cBx[c] = A * is * dg;
    cK[c] = A * (db - a.mean[c] * is * dg);
  }
  __syncthreads();
  const size_t n8 = (size_t)a.P * a.C / 8;
  const int c8 = a.C >> 3;
  const size_t stride = (size_t)gridDim.x * BN16_THREADS;
  for (size_t i0 = (size_t)blockIdx.x * BN16_THREADS + threadIdx.x; i0 < n8; i0 += 2 * stride) {
    F8 xv[2], gv[2], yv[2];
    bool in[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const size_t i = i0 + u * stride;
      in[u] = i < n8;
      if (in[u]) {
        xv[u] = bn16_ld8(a.x, i * 8);
        gv[u] = bn16_ld8(a.dy, i * 8);
        if (a.relu) yv[u] = bn16_ld8(a.y, i * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (!in[u]) continue;
      const size_t i = i0 + u * stride;
      const int col = (int)(i & (size_t)(c8 - 1)) * 8;   // C / 8 is a power of two
      F8 dx, g;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float gg = gv[u].v[e];
        if (a.relu) gg = yv[u].v[e] > 0.f ? gg : 0.f;
        g.v[e] = gg;
        dx.v[e] = gg * cA[col + e] - xv[u].v[e] * cBx[col + e] - cK[col + e];
      }
      bn16_st8(a.out, i * 8, dx);
      if (a.out2 != nullptr) bn16_st8(a.out2, i * 8, g);
    }
  }
}

// ---------------------------------- host side ----------------------------------------------
static int bn16_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  }
  return sms;
}

extern "C" int bn16_supported(int P, int C) {
  if (P < 1 || C < 8 || C % 8 != 0 || C > BN16_MAX_C) return 0;
  const int tpr = C / 8;
  return tpr <= BN16_THREADS && BN16_THREADS % tpr == 0;
}

// CTAs of the reduction kernel = rows of partials ([grid][2 C] floats of scratch)
extern "C" int bn16_reduce_grid(int P, int C) {
  if (!bn16_supported(P, C)) return 0;
  const int rpb = BN16_THREADS / (C / 8);
  const long long trips = ((long long)P + rpb * 4 - 1) / (rpb * 4);
  long long g = (trips + 1) / 2;               // at least two trips per CTA
  const long long cap = 2LL * bn16_sm_count();
  if (g > cap) g = cap;
  return (int)(g < 1 ? 1 : g);
}

// CTAs of an elementwise kernel: exactly one resident wave (every CTA walks the tensor with a grid stride),
// so that no partial last wave leaves SMs idle
template <typename K>
static int bn16_apply_grid(K kernel, long long n8) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, BN16_THREADS, 0) != cudaSuccess || per_sm < 1)
    per_sm = 2;
  long long b = (n8 + 2 * BN16_THREADS - 1) / (2 * BN16_THREADS);
  const long long cap = (long long)per_sm * bn16_sm_count();
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

// x, residual, out: bf16 [P, C]; partial: bn16_reduce_grid() * 2 C floats
extern "C" int bn16_forward(const BnArgs* args, cudaStream_t st) {
  BnArgs a = *args;
  if (!bn16_supported(a.P, a.C) || a.partial == nullptr) return -1;
  a.n_partials = bn16_reduce_grid(a.P, a.C);
  launch_k(bn16_reduce_kernel<false>, dim3(a.n_partials), dim3(BN16_THREADS), 0, st, a);
  launch_k(bn16_finalize_kernel<false>, dim3((a.C + BN16_FIN_CH - 1) / BN16_FIN_CH), dim3(BN16_THREADS), 0, st, a);
  launch_k(bn16_fwd_apply_kernel, dim3(bn16_apply_grid(bn16_fwd_apply_kernel, (long long)a.P * a.C / 8)), dim3(BN16_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}

// x, dy, y, out (dx), out2 (dresidual, optional): bf16 [P, C]
extern "C" int bn16_backward(const BnArgs* args, cudaStream_t st) {
  BnArgs a = *args;
  if (!bn16_supported(a.P, a.C) || a.partial == nullptr) return -1;
  a.n_partials = bn16_reduce_grid(a.P, a.C);
  launch_k(bn16_reduce_kernel<true>, dim3(a.n_partials), dim3(BN16_THREADS), 0, st, a);
  launch_k(bn16_finalize_kernel<true>, dim3((a.C + BN16_FIN_CH - 1) / BN16_FIN_CH), dim3(BN16_THREADS), 0, st, a);
  launch_k(bn16_bwd_apply_kernel, dim3(bn16_apply_grid(bn16_bwd_apply_kernel, (long long)a.P * a.C / 8)), dim3(BN16_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}
