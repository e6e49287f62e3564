// Training-mode BatchNorm fused with the residual add and ReLU around it, NHWC fp32.
//
//   forward :  y = relu( (x - mean_c) * invstd_c * gamma_c + beta_c  [+ residual] )
//   backward:  g = dy * [y > 0] ;  dbeta = sum g ;  dgamma = sum g * xhat ;
//              dx = gamma invstd (g - dbeta / P - xhat dgamma / P) ;  dresidual = g
//
// Each direction is two kernels: a per-channel reduction over all P = N*H*W pixels into per-CTA
// partials, and one elementwise pass.  When the partials are few (G * 2C <= 8192 floats) every
// CTA of the elementwise kernel adds them itself, in a fixed order in double precision, before it
// starts (CTA 0 also stores the statistics and updates the running ones): the reduction kernel
// then has no serial tail.  Otherwise the last CTA of the reduction kernel adds the partials.  That replaces the
// library batch-norm kernel plus separate add / ReLU / ReLU-backward / add-backward kernels
// (dl_code/pcode/models/resnet.py:37-56: conv -> bn -> relu, conv -> bn -> += residual -> relu).
//
// Layout: x is [P, C] with C contiguous, C a multiple of 4, C/4 a power of two <= 256.
#include <cuda_runtime.h>
#include "launch.cuh"
#include <stdint.h>
#include <stdlib.h>

#define BN_THREADS 256

#include "bn_args.h"

// per-channel sums of (a, b) over this CTA's rows -> partial; last CTA finalises
template <bool BACKWARD>
__global__ void __launch_bounds__(BN_THREADS) bn_reduce_kernel(BnArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sh[BN_THREADS * 8];
  __shared__ int last;
  const int C = a.C, tpr = C >> 2;            // threads per row
  const int rpb = BN_THREADS / tpr;            // rows per pass
  const int col = (threadIdx.x % tpr) * 4, rsub = threadIdx.x / tpr;
  const int rows_per_cta = (a.P + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(a.P, r0 + rows_per_cta);
  float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
  float mu[4] = {0.f, 0.f, 0.f, 0.f}, is[4] = {1.f, 1.f, 1.f, 1.f};
  if (BACKWARD) {
    const float4 m = *reinterpret_cast<const float4*>(a.mean + col);
    const float4 v = *reinterpret_cast<const float4*>(a.invstd + col);
    mu[0] = m.x; mu[1] = m.y; mu[2] = m.z; mu[3] = m.w;
    is[0] = v.x; is[1] = v.y; is[2] = v.z; is[3] = v.w;
  }
  // four rows per trip: all their loads are issued before the first accumulate
  for (int r = r0 + rsub; r < r1; r += 4 * rpb) {
    float4 xv[4], gv[4], yv[4];
    bool in[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int rr = r + u * rpb;
      in[u] = rr < r1;
      const size_t off = (size_t)(in[u] ? rr : r) * C + col;
      xv[u] = *reinterpret_cast<const float4*>(a.x + off);
      if (BACKWARD) {
        gv[u] = *reinterpret_cast<const float4*>(a.dy + off);
        if (a.relu) yv[u] = *reinterpret_cast<const float4*>(a.y + off);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!in[u]) continue;
      const float xa[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
      if (!BACKWARD) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s0[e] += xa[e];
          s1[e] = fmaf(xa[e], xa[e], s1[e]);
        }
      } else {
        float ga[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w};
        if (a.relu) {
          const float ya[4] = {yv[u].x, yv[u].y, yv[u].z, yv[u].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) ga[e] = ya[e] > 0.f ? ga[e] : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s0[e] += ga[e];
          s1[e] = fmaf(ga[e], (xa[e] - mu[e]) * is[e], s1[e]);
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    sh[threadIdx.x * 8 + e] = s0[e];
    sh[threadIdx.x * 8 + 4 + e] = s1[e];
  }
  __syncthreads();
  // fixed-shape tree over the rows held by this CTA (rpb is a power of two): reproducible
  for (int stride = rpb >> 1; stride > 0; stride >>= 1) {
    if (rsub < stride) {
      float* mine = sh + threadIdx.x * 8;
      const float* other = sh + (threadIdx.x + stride * tpr) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) mine[e] += other[e];
    }
    __syncthreads();
  }
  if (threadIdx.x < tpr) {
    float* dst = a.partial + (size_t)blockIdx.x * 2 * C;
    const float* p = sh + threadIdx.x * 8;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      dst[col + e] = p[e];
      dst[C + col + e] = p[4 + e];
    }
  }
  if (a.fused_finalize) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    last = (atomicAdd(a.counter, 1u) == gridDim.x - 1);
    if (last) __threadfence();
  }
  __syncthreads();
  if (!last) return;
  // final reduction over the CTAs' partials: BN_THREADS / C threads per channel, each adds a
  // strided subset in a fixed order, then the subsets are added in a fixed order (reproducible)
  double* shd = reinterpret_cast<double*>(sh);  // 2 * BN_THREADS doubles = 4 KiB
  for (int cbase = 0; cbase < C; cbase += BN_THREADS) {
    const int cw = min(C - cbase, BN_THREADS);   // channels in this pass
    const int nsub = BN_THREADS / cw;
    const int c = cbase + threadIdx.x % cw, sub = threadIdx.x / cw;
    double t0 = 0.0, t1 = 0.0;
    if (sub < nsub) {
      // four independent loads per trip (the adds stay in a fixed order)
      unsigned b = sub;
      for (; b + 3 * nsub < gridDim.x; b += 4 * nsub) {
        float u0[4], u1[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          u0[q] = __ldcg(a.partial + (size_t)(b + q * nsub) * 2 * C + c);
          u1[q] = __ldcg(a.partial + (size_t)(b + q * nsub) * 2 * C + C + c);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          t0 += (double)u0[q];
          t1 += (double)u1[q];
        }
      }
      for (; b < gridDim.x; b += nsub) {
        t0 += (double)__ldcg(a.partial + (size_t)b * 2 * C + c);
        t1 += (double)__ldcg(a.partial + (size_t)b * 2 * C + C + c);
      }
    }
    __syncthreads();
    shd[threadIdx.x * 2] = t0;
    shd[threadIdx.x * 2 + 1] = t1;
    __syncthreads();
    if (threadIdx.x < cw) {
      t0 = 0.0; t1 = 0.0;
      for (int j = 0; j < nsub; ++j) {
        t0 += shd[(j * cw + threadIdx.x) * 2];
        t1 += shd[(j * cw + threadIdx.x) * 2 + 1];
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
  }
  if (threadIdx.x == 0) *a.counter = 0;
}

#define BN_MAX_C 1024
#define BN_FUSED_LIMIT 8192   // floats of partials a CTA of the elementwise kernel may add itself

// Statistics of the elementwise kernels in shared memory: st0 / st1 = mean / invstd (forward) or
// dbeta / dgamma (backward).  fused_finalize: derived here from the partials [G][2C] with a fixed
// summation order (sub-sums of strided subsets, then the subsets in order), so that every CTA
// obtains bit-identical values; CTA 0 publishes them.  Otherwise they are read from global memory.
template <bool BACKWARD>
__device__ void bn_stats_to_smem(const BnArgs& a, float* st0, float* st1, double* tot, double* shd) {
  const int C = a.C;
  if (!a.fused_finalize) {
    for (int c = threadIdx.x; c < C; c += BN_THREADS) {
      st0[c] = BACKWARD ? a.dbeta[c] : a.mean[c];
      st1[c] = BACKWARD ? a.dgamma[c] : a.invstd[c];
    }
    __syncthreads();
    return;
  }
  const int C2 = 2 * C, G = a.n_partials;
  const int cw = C2 < BN_THREADS ? C2 : BN_THREADS, nsub = BN_THREADS / cw;
  for (int cbase = 0; cbase < C2; cbase += BN_THREADS) {
    const int col = cbase + threadIdx.x % cw, sub = threadIdx.x / cw;
    double t = 0.0;
    if (sub < nsub) {
      // eight independent loads per trip; the adds keep a fixed order
      int b = sub;
      for (; b + 7 * nsub < G; b += 8 * nsub) {
        float u[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) u[q] = __ldcg(a.partial + (size_t)(b + q * nsub) * C2 + col);
#pragma unroll
        for (int q = 0; q < 8; ++q) t += (double)u[q];
      }
      for (; b < G; b += nsub) t += (double)__ldcg(a.partial + (size_t)b * C2 + col);
    }
    shd[threadIdx.x] = t;
    __syncthreads();
    if (threadIdx.x < cw) {
      double acc = 0.0;
      for (int j = 0; j < nsub; ++j) acc += shd[j * cw + threadIdx.x];
      tot[col] = acc;
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < C; c += BN_THREADS) {
    const double t0 = tot[c], t1 = tot[C + c];
    if (!BACKWARD) {
      const double mean = t0 / a.P;
      double var = t1 / a.P - mean * mean;
      if (var < 0.0) var = 0.0;
      const float mf = (float)mean, isf = (float)(1.0 / sqrt(var + (double)a.eps));
      st0[c] = mf;
      st1[c] = isf;
      if (blockIdx.x == 0) {
        a.mean[c] = mf;
        a.invstd[c] = isf;
        if (a.running_mean != nullptr) {
          const double unbiased = a.P > 1 ? var * a.P / (a.P - 1) : var;
          a.running_mean[c] = (1.f - a.momentum) * a.running_mean[c] + a.momentum * mf;
          a.running_var[c] = (1.f - a.momentum) * a.running_var[c] + a.momentum * (float)unbiased;
        }
      }
    } else {
      st0[c] = (float)t0;
      st1[c] = (float)t1;
      if (blockIdx.x == 0) {
        a.dbeta[c] = (float)t0;
        a.dgamma[c] = (float)t1;
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(BN_THREADS) bn_fwd_apply_kernel(BnArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float st0[BN_MAX_C], st1[BN_MAX_C];
  __shared__ double tot[2 * BN_MAX_C], shd[BN_THREADS];
  bn_stats_to_smem<false>(a, st0, st1, tot, shd);
  const size_t n4 = (size_t)a.P * a.C / 4;
  const int c4 = a.C >> 2;
  for (size_t i = (size_t)blockIdx.x * BN_THREADS + threadIdx.x; i < n4; i += (size_t)gridDim.x * BN_THREADS) {
    const int col = (int)(i % c4) * 4;
    const float4 xv = reinterpret_cast<const float4*>(a.x)[i];
    const float4 m = *reinterpret_cast<const float4*>(st0 + col);
    const float4 s = *reinterpret_cast<const float4*>(st1 + col);
    const float4 g = *reinterpret_cast<const float4*>(a.gamma + col);
    const float4 b = *reinterpret_cast<const float4*>(a.beta + col);
    float4 y;
    y.x = fmaf((xv.x - m.x) * s.x, g.x, b.x);
    y.y = fmaf((xv.y - m.y) * s.y, g.y, b.y);
    y.z = fmaf((xv.z - m.z) * s.z, g.z, b.z);
    y.w = fmaf((xv.w - m.w) * s.w, g.w, b.w);
    if (a.residual != nullptr) {
      const float4 r = reinterpret_cast<const float4*>(a.residual)[i];
      y.x += r.x; y.y += r.y; y.z += r.z; y.w += r.w;
    }
    if (a.relu) {
      y.x = fmaxf(y.x, 0.f); y.y = fmaxf(y.y, 0.f); y.z = fmaxf(y.z, 0.f); y.w = fmaxf(y.w, 0.f);
    }
    reinterpret_cast<float4*>(a.out)[i] = y;
  }
}

__global__ void __launch_bounds__(BN_THREADS) bn_bwd_apply_kernel(BnArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float st0[BN_MAX_C], st1[BN_MAX_C];
  __shared__ double tot[2 * BN_MAX_C], shd[BN_THREADS];
  bn_stats_to_smem<true>(a, st0, st1, tot, shd);
  const size_t n4 = (size_t)a.P * a.C / 4;
  const int c4 = a.C >> 2;
  const float inv_p = 1.f / (float)a.P;
  for (size_t i = (size_t)blockIdx.x * BN_THREADS + threadIdx.x; i < n4; i += (size_t)gridDim.x * BN_THREADS) {
    const int col = (int)(i % c4) * 4;
    const float4 xv = reinterpret_cast<const float4*>(a.x)[i];
    float4 gv = reinterpret_cast<const float4*>(a.dy)[i];
    if (a.relu) {
      const float4 yv = reinterpret_cast<const float4*>(a.y)[i];
      gv.x = yv.x > 0.f ? gv.x : 0.f; gv.y = yv.y > 0.f ? gv.y : 0.f;
      gv.z = yv.z > 0.f ? gv.z : 0.f; gv.w = yv.w > 0.f ? gv.w : 0.f;
    }
    if (a.out2 != nullptr) reinterpret_cast<float4*>(a.out2)[i] = gv;
    const float4 m = *reinterpret_cast<const float4*>(a.mean + col);
    const float4 s = *reinterpret_cast<const float4*>(a.invstd + col);
    const float4 g = *reinterpret_cast<const float4*>(a.gamma + col);
    const float4 db = *reinterpret_cast<const float4*>(st0 + col);
    const float4 dg = *reinterpret_cast<const float4*>(st1 + col);
    float4 dx;
    dx.x = g.x * s.x * (gv.x - db.x * inv_p - (xv.x - m.x) * s.x * dg.x * inv_p);
    dx.y = g.y * s.y * (gv.y - db.y * inv_p - (xv.y - m.y) * s.y * dg.y * inv_p);
    dx.z = g.z * s.z * (gv.z - db.z * inv_p - (xv.z - m.z) * s.z * dg.z * inv_p);
    dx.w = g.w * s.w * (gv.w - db.w * inv_p - (xv.w - m.w) * s.w * dg.w * inv_p);
    reinterpret_cast<float4*>(a.out)[i] = dx;
  }
}

// ---- backward in ONE kernel ---------------------------------------------------------------------
// One CTA per SM keeps its rows of x and of the masked gradient g in shared memory: phase 1 reads
// x, dy, y once and leaves per-CTA partial sums, a grid-wide barrier follows (all CTAs are
// co-resident: at most one per SM; bounded wait), then every CTA adds the partials in the same
// fixed order and writes dx (and dresidual) from shared memory.  Half the global traffic and one
// launch instead of two.  barrier[0] = arrivals, barrier[1] = generation, barrier[2] = error flag.
__device__ __forceinline__ unsigned bn_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(BN_THREADS, 1) bn_bwd_fused_kernel(BnArgs a, unsigned* barrier, int rows_per_cta) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float bn_dyn[];
  __shared__ float st0[BN_MAX_C], st1[BN_MAX_C];
  __shared__ double tot[2 * BN_MAX_C], shd[BN_THREADS];
  __shared__ float sh[BN_THREADS * 8];
  __shared__ int ok_flag;
  const int C = a.C, tpr = C >> 2, rpb = BN_THREADS / tpr;
  const int col = (threadIdx.x % tpr) * 4, rsub = threadIdx.x / tpr;
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(a.P, r0 + rows_per_cta);
  float* xs = bn_dyn;                                   // [rows_per_cta][C]
  float* gs = bn_dyn + (size_t)rows_per_cta * C;
  const unsigned my_gen = (threadIdx.x == 0) ? bn_ld_acquire(barrier + 1) : 0u;

  const float4 m4 = *reinterpret_cast<const float4*>(a.mean + col);
  const float4 i4 = *reinterpret_cast<const float4*>(a.invstd + col);
  const float mu[4] = {m4.x, m4.y, m4.z, m4.w}, is[4] = {i4.x, i4.y, i4.z, i4.w};
  float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
  for (int r = r0 + rsub; r < r1; r += 4 * rpb) {
    float4 xv[4], gv[4], yv[4];
    bool in[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int rr = r + u * rpb;
      in[u] = rr < r1;
      const size_t off = (size_t)(in[u] ? rr : r) * C + col;
      xv[u] = *reinterpret_cast<const float4*>(a.x + off);
      gv[u] = *reinterpret_cast<const float4*>(a.dy + off);
      if (a.relu) yv[u] = *reinterpret_cast<const float4*>(a.y + off);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!in[u]) continue;
      const float xa[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
      float ga[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w};
      if (a.relu) {
        const float ya[4] = {yv[u].x, yv[u].y, yv[u].z, yv[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) ga[e] = ya[e] > 0.f ? ga[e] : 0.f;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s0[e] += ga[e];
        s1[e] = fmaf(ga[e], (xa[e] - mu[e]) * is[e], s1[e]);
      }
      const size_t lo = (size_t)(r + u * rpb - r0) * C + col;
      *reinterpret_cast<float4*>(xs + lo) = xv[u];
      *reinterpret_cast<float4*>(gs + lo) = make_float4(ga[0], ga[1], ga[2], ga[3]);
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    sh[threadIdx.x * 8 + e] = s0[e];
    sh[threadIdx.x * 8 + 4 + e] = s1[e];
  }
  __syncthreads();
  for (int stride = rpb >> 1; stride > 0; stride >>= 1) {
    if (rsub < stride) {
      float* mine = sh + threadIdx.x * 8;
      const float* other = sh + (threadIdx.x + stride * tpr) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) mine[e] += other[e];
    }
    __syncthreads();
  }
  if (threadIdx.x < tpr) {
    float* dst = a.partial + (size_t)blockIdx.x * 2 * C;
    const float* p = sh + threadIdx.x * 8;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      dst[col + e] = p[e];
      dst[C + col + e] = p[4 + e];
    }
  }
  __syncthreads();
  // ---- grid barrier (bounded) ---------------------------------------------------------------
  if (threadIdx.x == 0) {
    int ok = 1;
    __threadfence();
    if (atomicAdd(barrier, 1u) == gridDim.x - 1) {
      *barrier = 0;
      __threadfence();
      atomicAdd(barrier + 1, 1u);
    } else {
      unsigned spins = 0;
      while (bn_ld_acquire(barrier + 1) == my_gen) {
        __nanosleep(32);
        if (++spins > (1u << 24)) { ok = 0; atomicExch(barrier + 2, 1u); break; }
      }
    }
    ok_flag = ok;
  }
  __syncthreads();
  if (!ok_flag) return;
  // ---- statistics from the partials, then dx from shared memory -------------------------------------
  bn_stats_to_smem<true>(a, st0, st1, tot, shd);
  const float4 g4 = *reinterpret_cast<const float4*>(a.gamma + col);
  const float ga4[4] = {g4.x, g4.y, g4.z, g4.w};
  const float inv_p = 1.f / (float)a.P;
  float cb[4], cg[4], sc[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    cb[e] = st0[col + e] * inv_p;
    cg[e] = st1[col + e] * inv_p;
    sc[e] = ga4[e] * is[e];
  }
  for (int r = r0 + rsub; r < r1; r += rpb) {
    const size_t lo = (size_t)(r - r0) * C + col, off = (size_t)r * C + col;
    const float4 xv = *reinterpret_cast<const float4*>(xs + lo);
    const float4 gv = *reinterpret_cast<const float4*>(gs + lo);
    const float xa[4] = {xv.x, xv.y, xv.z, xv.w}, gg[4] = {gv.x, gv.y, gv.z, gv.w};
    float dx[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) dx[e] = sc[e] * (gg[e] - cb[e] - (xa[e] - mu[e]) * is[e] * cg[e]);
    *reinterpret_cast<float4*>(a.out + off) = make_float4(dx[0], dx[1], dx[2], dx[3]);
    if (a.out2 != nullptr) *reinterpret_cast<float4*>(a.out2 + off) = gv;
  }
}

// CTAs of the elementwise kernels.  Every CTA first reads the rows of partials (fused finalize),
// so their number is kept lower when there are partials to read: 4 per SM instead of 8.
static int grid_for(long long n4, int fused = 0) {
  static int cap_fused = 0;
  if (cap_fused == 0) {
    const char* e = getenv("CHOCO_BN_APPLY_CTAS");
    cap_fused = e != nullptr && atoi(e) > 0 ? atoi(e) : sm_count() * 4;
  }
  const long long cap = fused ? cap_fused : sm_count() * 8;
  long long b = (n4 + BN_THREADS - 1) / BN_THREADS;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

// CTAs of the reduction kernel: four 4-row trips per thread, at most one CTA per SM.  Few enough
// partials -> the elementwise kernel adds them (fused finalize); otherwise the last CTA of the
// reduction kernel does, and the grid is capped lower to keep that serial pass short.
extern "C" int bn_reduce_grid(int P, int C) {
  const int rpb = BN_THREADS / (C / 4);
  const int trips = (P + rpb * 4 - 1) / (rpb * 4);
  static int cap = 0, cap_last = 0;
  if (cap == 0) {
    const char* e = getenv("CHOCO_BN_GRID_CAP");
    cap = e != nullptr && atoi(e) > 0 ? atoi(e) : sm_count();
    cap_last = cap < 74 ? cap : 74;
  }
  int g = (trips + 3) / 4;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  if ((long long)g * 2 * C > BN_FUSED_LIMIT && g > cap_last) g = cap_last;
  return g;
}

static int bn_prepare(BnArgs& a) {
  if (a.C % 4 != 0 || BN_THREADS % (a.C / 4) != 0 || a.C / 4 > BN_THREADS || a.C > BN_MAX_C) return -1;
  a.n_partials = bn_reduce_grid(a.P, a.C);
  static int allow = -1;
  if (allow < 0) {
    const char* e = getenv("CHOCO_BN_FUSED_FINALIZE");
    allow = e == nullptr || atoi(e) != 0;
  }
  a.fused_finalize = allow && (long long)a.n_partials * 2 * a.C <= BN_FUSED_LIMIT;
  return 0;
}

extern "C" int bn_forward(const BnArgs* args, cudaStream_t st) {
  BnArgs a = *args;
  if (bn_prepare(a) != 0) return -1;
  launch_k(bn_reduce_kernel<false>, dim3(a.n_partials), dim3(BN_THREADS), 0, st, a);
  launch_k(bn_fwd_apply_kernel, dim3(grid_for((long long)a.P * a.C / 4, a.fused_finalize)), dim3(BN_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}

// Forward when the producer of x already left per-CTA (sum, sum of squares) rows in args->partial
// ([n_partials][2C], e.g. the convolution epilogue): no reduction pass over x at all.
extern "C" int bn_forward_partials(const BnArgs* args, int n_partials, cudaStream_t st) {
  BnArgs a = *args;
  if (a.C % 4 != 0 || BN_THREADS % (a.C / 4) != 0 || a.C / 4 > BN_THREADS || a.C > BN_MAX_C) return -1;
  if (n_partials < 1 || (long long)n_partials * 2 * a.C > BN_FUSED_LIMIT || a.partial == nullptr) return -2;
  a.n_partials = n_partials;
  a.fused_finalize = 1;
  launch_k(bn_fwd_apply_kernel, dim3(grid_for((long long)a.P * a.C / 4, a.fused_finalize)), dim3(BN_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}

// Backward when the producer of dy already masked it with the ReLU and left per-CTA rows of
// (sum dy, sum dy * xhat) in args->partial (the input-gradient convolution's epilogue): one
// elementwise kernel, no reduction pass; dgamma / dbeta are published by its first CTA.
extern "C" int bn_backward_partials(const BnArgs* args, int n_partials, cudaStream_t st) {
  BnArgs a = *args;
  if (a.C % 4 != 0 || BN_THREADS % (a.C / 4) != 0 || a.C / 4 > BN_THREADS || a.C > BN_MAX_C) return -1;
  if (n_partials < 1 || (long long)n_partials * 2 * a.C > BN_FUSED_LIMIT || a.partial == nullptr) return -2;
  a.n_partials = n_partials;
  a.fused_finalize = 1;
  a.relu = 0;
  a.out2 = nullptr;
  launch_k(bn_bwd_apply_kernel, dim3(grid_for((long long)a.P * a.C / 4, a.fused_finalize)), dim3(BN_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}

static unsigned* g_bn_barrier[64];

static unsigned* bn_barrier_words() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (g_bn_barrier[dev] == nullptr) {
    if (cudaMalloc(&g_bn_barrier[dev], 4 * sizeof(unsigned)) != cudaSuccess) return nullptr;
    cudaMemset(g_bn_barrier[dev], 0, 4 * sizeof(unsigned));
  }
  return g_bn_barrier[dev];
}

// 1 when a grid barrier of the one-kernel backward gave up (reads the flag; synchronises)
extern "C" int bn_last_error() {
  unsigned* w = bn_barrier_words();
  unsigned v[4] = {0, 0, 0, 0};
  if (w == nullptr || cudaMemcpy(v, w, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)v[2];
}

extern "C" int bn_backward(const BnArgs* args, cudaStream_t st) {
  BnArgs a = *args;
  if (bn_prepare(a) != 0) return -1;
  static int fused_ok = -1, sms = 0;
  if (fused_ok < 0) {
    // opt-in: with the weight-gradient kernels of the same step running on a second stream the
    // barrier has to wait until every SM is free, which measured slower (1.39 against 1.31 ms per
    // ResNet-20 step) than the two-kernel form; alone on the GPU it halves the traffic
    const char* e = getenv("CHOCO_BN_BWD_FUSED");
    fused_ok = e != nullptr && atoi(e) != 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  }
  // one CTA per SM; its rows of x and g must fit in shared memory, its partial rows in the finalize
  int G = sms;
  while ((long long)G * 2 * a.C > BN_FUSED_LIMIT && G > 1) G >>= 1;
  const int rows = (a.P + G - 1) / G;
  G = (a.P + rows - 1) / rows;
  const size_t dyn = (size_t)rows * a.C * 2 * sizeof(float);
  if (fused_ok && a.fused_finalize && dyn <= 150 * 1024) {
    unsigned* bar = bn_barrier_words();
    if (bar == nullptr) return -13;
    static size_t configured = 0;
    if (dyn > configured) {
      cudaError_t e = cudaFuncSetAttribute(bn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(150 * 1024));
      if (e != cudaSuccess) return (int)e;
      configured = 150 * 1024;
    }
    a.n_partials = G;
    a.fused_finalize = 1;
    launch_k(bn_bwd_fused_kernel, dim3(G), dim3(BN_THREADS), dyn, st, a, bar, rows);
    return (int)cudaGetLastError();
  }
  launch_k(bn_reduce_kernel<true>, dim3(a.n_partials), dim3(BN_THREADS), 0, st, a);
  launch_k(bn_bwd_apply_kernel, dim3(grid_for((long long)a.P * a.C / 4, a.fused_finalize)), dim3(BN_THREADS), 0, st, a);
  return (int)cudaGetLastError();
}

extern "C" int bn_args_size() { return (int)sizeof(BnArgs); }
