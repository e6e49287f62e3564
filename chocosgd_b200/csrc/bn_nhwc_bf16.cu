// Training-mode BatchNorm fused with the residual add and ReLU around it, NHWC bf16 activations
// (fp32 statistics, gamma / beta and their gradients): the form a bf16-autocast ImageNet ResNet needs.
//
//   forward :  y = relu( (x - mean_c) * invstd_c * gamma_c + beta_c  [+ residual] )
//   backward:  g = dy * [y > 0] ;  dbeta = sum g ;  dgamma = sum g * xhat ;
//              dx = gamma invstd (g - dbeta / P - xhat dgamma / P) ;  dresidual = g
//
// Three kernels per direction: per-channel partial sums per CTA (one pass over the activation), a
// small finalize (partials added per channel in a fixed order, in double precision: reproducible),
// and one elementwise pass.  (Folding the finalize into the last CTAs of the first kernel was measured
// slower on the ResNet-50 step, 13.2 ms against 12.9 ms: its two serial levels cost more than a launch.)  Replaces, per layer, the library's statistics + transform kernels and the
// separate add / ReLU kernels forward, and ReLU-backward + reduce + elementwise kernels backward
// (dl_code/pcode/models/resnet.py:86-127: conv -> bn -> relu ... conv -> bn -> += residual -> relu).
//
// The four passes over activations are pure streams, so their operands come in through the bulk-copy
// engine: the flat [P C] arrays are cut into chunks of 4 - 16 KB, a CTA owns every gridDim.x-th chunk and
// keeps a ring of 2 - 4 chunks per operand in flight (cp.async.bulk global -> shared, completion on an
// mbarrier).  The bytes in flight per SM (about 150 KB) no longer depend on registers or occupancy, which
// is what limited the version with plain loads to half of the copy rate.  Results leave through ordinary
// coalesced 16-byte stores.
//
// Layout: [P, C] with C contiguous, C a multiple of 8, C / 8 a power of two <= 256 (C = 8 ... 2048).
// A chunk is a whole number of rows and thread t takes 16-byte pieces t, t + 256, ... of it, so a thread
// always meets the same 8 channels: their constants and running sums live in registers.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "bn_args.h"
#include "launch.cuh"
#include "tc_common.cuh"

#define BN16_THREADS 256
#define BN16_STAGE 16384                              // bytes of a ring slot (chunks are 4, 8 or 16 KB)
#define BN16_PPT (BN16_STAGE / 16 / BN16_THREADS)     // 16-byte pieces per thread and slot: 4

struct F8 {
  float v[8];
};

__device__ __forceinline__ F8 bn16_unpack(const uint4 raw) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  F8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    r.v[2 * i] = __uint_as_float(w[i] << 16);            // bf16 = the upper half of an fp32
    r.v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
  return r;
}

__device__ __forceinline__ uint4 bn16_pack(const F8& f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f.v[2 * i], f.v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void bn16_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ int* bn16_error_word_dev;   // set by the host before the first launch

// ring slots per operand count: 64 KB (one operand) or 96 KB of shared memory per CTA, two CTAs per SM
template <int T> struct Bn16Ring { static constexpr int S = T == 1 ? 4 : (T == 2 ? 3 : 2); };
template <int T> constexpr int bn16_smem_bytes() { return Bn16Ring<T>::S * T * BN16_STAGE + 128; }

// Streams T operands ([total] bytes each, the same cut into chunks of `ch` bytes) through the ring and calls
// body(slot, byte offset of the chunk, bytes of the chunk) for every chunk of this CTA; slot + t * BN16_STAGE
// is operand t.  Returns false when a wait ran out (the error word is set and the copies in flight are
// waited for once more before the CTA goes on to exit).
// REVERSE: the chunks are taken from the end of the arrays backwards.  The reductions run that way and the
// elementwise kernels forwards, so each kernel starts on the part of the tensor that its predecessor touched
// last and that is still in L2 (a producer leaves the tail of what it wrote, a backward reader the head).
template <int T, bool REVERSE, typename Body>
__device__ __forceinline__ bool bn16_stream(const void* s0, const void* s1, const void* s2, size_t total, int ch,
                                            uint8_t* smem, int* error, Body&& body) {
  constexpr int S = Bn16Ring<T>::S;
  const uint8_t* src[3] = {reinterpret_cast<const uint8_t*>(s0), reinterpret_cast<const uint8_t*>(s1),
                           reinterpret_cast<const uint8_t*>(s2)};
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * T * BN16_STAGE);
  const size_t n_chunks = (total + ch - 1) / ch;
  const int n_mine = blockIdx.x < n_chunks ? (int)((n_chunks - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
  auto chunk_off = [&](int it) {
    const size_t k = (size_t)blockIdx.x + (size_t)it * gridDim.x;
    return (REVERSE ? n_chunks - 1 - k : k) * (size_t)ch;
  };
  auto issue = [&](int it) {
    const size_t off = chunk_off(it);
    const uint32_t bytes = (uint32_t)(total - off < (size_t)ch ? total - off : (size_t)ch);
    const int s = it % S;
    mbar_expect_tx(full + s, T * bytes);
#pragma unroll
    for (int t = 0; t < T; ++t) bn16_bulk_load(smem + (s * T + t) * BN16_STAGE, src[t] + off, bytes, full + s);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) mbar_init(full + s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int it = 0; it < S && it < n_mine; ++it) issue(it);
  }
  __syncthreads();
  for (int it = 0; it < n_mine; ++it) {
    const int s = it % S;
    const bool bad = !mbar_wait(full + s, (it / S) & 1);
    if (__syncthreads_or(bad)) {
      if (threadIdx.x == 0) {
        atomicExch(error, 1);
        const int issued = it - 1 + S < n_mine ? it - 1 + S : n_mine;   // chunks it .. issued - 1 may still be landing
        for (int j = it; j < issued; ++j) mbar_wait(full + (j % S), (j / S) & 1);
      }
      __syncthreads();
      return false;
    }
    // (the barrier above also tells that every thread is done with the slot of the previous chunk)
    if (threadIdx.x == 0 && it >= 1 && it - 1 + S < n_mine) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue(it - 1 + S);
    }
    const size_t off = chunk_off(it);
    const uint32_t bytes = (uint32_t)(total - off < (size_t)ch ? total - off : (size_t)ch);
    body(smem + s * T * BN16_STAGE, off, bytes);
  }
  return true;
}

// channel c from its two sums: forward (sum x, sum x^2) -> mean, invstd, running statistics;
// backward (sum g, sum g xhat) -> dbeta, dgamma
template <bool BACKWARD>
__device__ __forceinline__ void bn16_finish(const BnArgs& a, int c, double t0, double t1) {
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

// per-channel sums over this CTA's chunks -> partial[blockIdx.x][2 C]
//   forward : (sum x, sum x^2)        backward: (sum g, sum g * xhat), g = dy * [y > 0]
// T: operands streamed: 1 forward (x), 2 backward without the output (x, dy), 3 backward with ReLU (x, dy, y)
// XMASK (T = 2): ReLU without a residual: the mask [y > 0] is recomputed from x with the forward's own
// arithmetic (y = max(fma(x, A, B), 0) is positive exactly when the fma is) instead of reading y
template <bool BACKWARD, int T, bool XMASK = false>
__global__ void __launch_bounds__(BN16_THREADS, T == 1 ? 3 : 2) bn16_reduce_kernel(BnArgs a, int ch) {
  extern __shared__ __align__(128) uint8_t bn16_smem[];
  const int C = a.C, tpr = C >> 3;             // threads per row
  const int rpb = BN16_THREADS / tpr;           // rows per sweep of the CTA
  const int col = (threadIdx.x % tpr) * 8, rsub = threadIdx.x / tpr;
  pdl_wait();
  pdl_trigger();
  float s0[8], s1[8], mu[8], is[8], fA[8], fB[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    s0[e] = 0.f; s1[e] = 0.f;
    mu[e] = BACKWARD ? a.mean[col + e] : 0.f;
    is[e] = BACKWARD ? a.invstd[col + e] : 1.f;
    if (XMASK) {
      fA[e] = a.gamma[col + e] * is[e];
      fB[e] = a.beta[col + e] - mu[e] * fA[e];
    }
  }
  const bool ok = bn16_stream<T, true>(a.x, a.dy, a.y, (size_t)a.P * C * 2, ch, bn16_smem, bn16_error_word_dev,
                                 [&](const uint8_t* slot, size_t, uint32_t bytes) {
    uint4 xr[BN16_PPT], gr[BN16_PPT], yr[BN16_PPT];
#pragma unroll
    for (int m = 0; m < BN16_PPT; ++m) {
      const uint32_t o = (m * BN16_THREADS + threadIdx.x) * 16;
      if (o < bytes) {
        xr[m] = *reinterpret_cast<const uint4*>(slot + o);
        if (T >= 2) gr[m] = *reinterpret_cast<const uint4*>(slot + BN16_STAGE + o);
        if (T >= 3) yr[m] = *reinterpret_cast<const uint4*>(slot + 2 * BN16_STAGE + o);
      }
    }
#pragma unroll
    for (int m = 0; m < BN16_PPT; ++m) {
      const uint32_t o = (m * BN16_THREADS + threadIdx.x) * 16;
      if (o >= bytes) continue;
      const F8 xv = bn16_unpack(xr[m]);
      if (!BACKWARD) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          s0[e] += xv.v[e];
          s1[e] = fmaf(xv.v[e], xv.v[e], s1[e]);
        }
      } else {
        const F8 gv = bn16_unpack(gr[m]);
        F8 yv;
        if (T >= 3) yv = bn16_unpack(yr[m]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float g = gv.v[e];
          if (T >= 3) g = yv.v[e] > 0.f ? g : 0.f;
          if (XMASK) g = fmaf(xv.v[e], fA[e], fB[e]) > 0.f ? g : 0.f;
          s0[e] += g;
          s1[e] = fmaf(g, (xv.v[e] - mu[e]) * is[e], s1[e]);
        }
      }
    }
  });
  if (!ok) return;
  __syncthreads();                              // the ring is free: its memory holds the tree below
  float* sh = reinterpret_cast<float*>(bn16_smem);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    sh[threadIdx.x * 16 + e] = s0[e];
    sh[threadIdx.x * 16 + 8 + e] = s1[e];
  }
  __syncthreads();
  // fixed-shape tree over the threads that hold the same channels (rpb is a power of two): reproducible
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

// A CTA finalizes 4 channels: 64 threads per channel, each with at most 8 of the G <= 4 * SMs partial rows per
// trip and all their loads issued before the first add (the kernel is a chain of L2 round trips and nothing
// else: one trip instead of seven), then the 64 sub-sums are added in order (double accumulation, a fixed
// order: reproducible).
#define BN16_FIN_CH 4
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
    for (int b = sub; b < G; b += 8 * BN16_FIN_SUB) {
      float u0[8], u1[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int r = b + q * BN16_FIN_SUB;
        u0[q] = r < G ? __ldcg(a.partial + (size_t)r * C2 + c) : 0.f;
        u1[q] = r < G ? __ldcg(a.partial + (size_t)r * C2 + a.C + c) : 0.f;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        t0 += (double)u0[q];
        t1 += (double)u1[q];
      }
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
  bn16_finish<BACKWARD>(a, c, t0, t1);
}

// Elementwise passes.  Per-channel constants are folded into (scale, shift) pairs, in registers:
//   forward : y = x * A + B,               A = gamma invstd,  B = beta - mean A
//   backward: dx = g * A - x * Bx - K,     A = gamma invstd,  Bx = A invstd dgamma / P,
//                                          K = A (dbeta / P - mean invstd dgamma / P)
#define BN16_MAX_C 2048

// T: 1 = x, 2 = x and residual
template <int T>
__global__ void __launch_bounds__(BN16_THREADS, 2) bn16_fwd_apply_kernel(BnArgs a, int ch) {
  extern __shared__ __align__(128) uint8_t bn16_smem[];
  const int col = (threadIdx.x % (a.C >> 3)) * 8;
  pdl_wait();
  pdl_trigger();
  float cA[8], cB[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    cA[e] = a.gamma[col + e] * a.invstd[col + e];
    cB[e] = a.beta[col + e] - a.mean[col + e] * cA[e];
  }
  uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
  const bool relu = a.relu != 0;
  bn16_stream<T, false>(a.x, a.residual, nullptr, (size_t)a.P * a.C * 2, ch, bn16_smem, bn16_error_word_dev,
                 [&](const uint8_t* slot, size_t off, uint32_t bytes) {
    uint4 xr[BN16_PPT], rr[BN16_PPT];
#pragma unroll
    for (int m = 0; m < BN16_PPT; ++m) {
      const uint32_t o = (m * BN16_THREADS + threadIdx.x) * 16;
      if (o < bytes) {
        xr[m] = *reinterpret_cast<const uint4*>(slot + o);
        if (T >= 2) rr[m] = *reinterpret_cast<const uint4*>(slot + BN16_STAGE + o);
      }
    }
#pragma unroll
    for (int m = 0; m < BN16_PPT; ++m) {
      const uint32_t o = (m * BN16_THREADS + threadIdx.x) * 16;
      if (o >= bytes) continue;
      const F8 xv = bn16_unpack(xr[m]);
      F8 rv, y;
      if (T >= 2) rv = bn16_unpack(rr[m]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float v = fmaf(xv.v[e], cA[e], cB[e]);
        if (T >= 2) v += rv.v[e];
        if (relu) v = fmaxf(v, 0.f);
        y.v[e] = v;
      }
      *reinterpret_cast<uint4*>(out + off + o) = bn16_pack(y);
    }
  });
}

// T: 2 = x and dy (no ReLU, or XMASK: the ReLU mask recomputed from x), 3 = x, dy and y
template <int T, bool XMASK = false>
__global__ void __launch_bounds__(BN16_THREADS, 2) bn16_bwd_apply_kernel(BnArgs a, int ch) {
  extern __shared__ __align__(128) uint8_t bn16_smem[];
  const int col = (threadIdx.x % (a.C >> 3)) * 8;
  pdl_wait();
  pdl_trigger();
  const float inv_p = 1.f / (float)a.P;
  float cA[8], cBx[8], cK[8], fB[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float is = a.invstd[col + e], A = a.gamma[col + e] * is;
    const float dg = a.dgamma[col + e] * inv_p, db = a.dbeta[col + e] * inv_p;
    cA[e] = A;
    cBx[e] = A * is * dg;
    cK[e] = A * (db - a.mean[col + e] * is * dg);
    if (XMASK) fB[e] = a.beta[col + e] - a.mean[col + e] * A;
  }
  uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
  uint8_t* out2 = reinterpret_cast<uint8_t*>(a.out2);
  bn16_stream<T, false>(a.x, a.dy, a.y, (size_t)a.P * a.C * 2, ch, bn16_smem, bn16_error_word_dev,
                 [&](const uint8_t* slot, size_t off, uint32_t bytes) {
    uint4 xr[BN16_PPT], gr[BN16_PPT], yr[BN16_PPT];
#pragma unroll
    for (int m = 0; m < BN16_PPT; ++m) {
      const uint32_t o = (m * BN16_THREADS + threadIdx.x) * 16;
      if (o < bytes) {
        xr[m] = *reinterpret_cast<const uint4*>(slot + o);
        gr[m] = *reinterpret_cast<const uint4*>(slot + BN16_STAGE + o);
        if (T >= 3) yr[m] = *reinterpret_cast<const uint4*>(slot + 2 * BN16_STAGE + o);
      }
    }
#pragma unroll
    for (int m = 0; m < BN16_PPT; ++m) {
      const uint32_t o = (m * BN16_THREADS + threadIdx.x) * 16;
      if (o >= bytes) continue;
      const F8 xv = bn16_unpack(xr[m]), gv = bn16_unpack(gr[m]);
      F8 yv, dx, g;
      if (T >= 3) yv = bn16_unpack(yr[m]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float gg = gv.v[e];
        if (T >= 3) gg = yv.v[e] > 0.f ? gg : 0.f;
        if (XMASK) gg = fmaf(xv.v[e], cA[e], fB[e]) > 0.f ? gg : 0.f;
        g.v[e] = gg;
        dx.v[e] = gg * cA[e] - xv.v[e] * cBx[e] - cK[e];
      }
      *reinterpret_cast<uint4*>(out + off + o) = bn16_pack(dx);
      if (out2 != nullptr) *reinterpret_cast<uint4*>(out2 + off + o) = bn16_pack(g);
    }
  });
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

static int* bn16_error_word() {
  static int* err = nullptr;
  if (err == nullptr) {
    if (cudaMalloc(&err, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(err, 0, sizeof(int));
    if (cudaMemcpyToSymbol(bn16_error_word_dev, &err, sizeof(err)) != cudaSuccess) return nullptr;
  }
  return err;
}

// 1 when a bounded wait on the copy ring ran out since the last call (the word is cleared)
extern "C" int bn16_last_error() {
  int* err = bn16_error_word();
  if (err == nullptr) return -1;
  int h = 0;
  if (cudaMemcpy(&h, err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (h != 0) cudaMemset(err, 0, sizeof(int));
  return h;
}

// CTAs per SM of a streaming kernel with its ring (asked once per kernel), at most 4: the partial-sum scratch
// is sized for 4 rows per SM
template <typename K>
static int bn16_per_sm(K kernel, int smem) {
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -1;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, BN16_THREADS, smem) != cudaSuccess || per_sm < 1)
    return -1;
  return per_sm > 4 ? 4 : per_sm;
}

struct Bn16Plan {
  int grid, ch;
};
// chunk size and CTAs for `total` bytes per operand: one resident wave, and at least four chunks per CTA where
// the tensor allows it (chunks of 16, 8 or 4 KB; a chunk is a whole number of rows: rows are at most 4 KB)
static Bn16Plan bn16_plan(long long total, int per_sm) {
  const long long cap = (long long)per_sm * bn16_sm_count();
  int ch = BN16_STAGE;
  while (ch > 4096 && (total + ch - 1) / ch < 4 * cap) ch >>= 1;
  long long g = (total + ch - 1) / ch;
  if (g > cap) g = cap;
  return {(int)(g < 1 ? 1 : g), ch};
}

template <typename K>
static int bn16_launch(K kernel, int smem, int& per_sm_cache, const BnArgs& a, bool is_reduce, int* n_partials, cudaStream_t st) {
  if (per_sm_cache == 0) per_sm_cache = bn16_per_sm(kernel, smem);
  if (per_sm_cache < 1) return -3;
  const Bn16Plan p = bn16_plan((long long)a.P * a.C * 2, per_sm_cache);
  if (is_reduce) *n_partials = p.grid;
  launch_k(kernel, dim3(p.grid), dim3(BN16_THREADS), (size_t)smem, st, a, p.ch);
  return 0;
}

// CTAs of the reduction kernel = rows of partials ([grid][2 C] floats of scratch), at most 4 per SM
extern "C" int bn16_reduce_grid(int P, int C) {
  if (!bn16_supported(P, C)) return 0;
  return 4 * bn16_sm_count();
}

// a bulk copy wants 16-byte aligned addresses (null: operand not used)
static bool bn16_aligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// x, residual, out: bf16 [P, C]; partial: 4 * SMs * 2 C floats
extern "C" int bn16_forward(const BnArgs* args, cudaStream_t st) {
  BnArgs a = *args;
  if (!bn16_supported(a.P, a.C) || a.partial == nullptr || bn16_error_word() == nullptr) return -1;
  if (!bn16_aligned(a.x) || !bn16_aligned(a.residual) || !bn16_aligned(a.out)) return -4;
  static int occ_red = 0, occ_a1 = 0, occ_a2 = 0;
  int rc = bn16_launch(bn16_reduce_kernel<false, 1>, bn16_smem_bytes<1>(), occ_red, a, true, &a.n_partials, st);
  if (rc) return rc;
  launch_k(bn16_finalize_kernel<false>, dim3((a.C + BN16_FIN_CH - 1) / BN16_FIN_CH), dim3(BN16_THREADS), 0, st, a);
  if (a.residual != nullptr)
    rc = bn16_launch(bn16_fwd_apply_kernel<2>, bn16_smem_bytes<2>(), occ_a2, a, false, nullptr, st);
  else
    rc = bn16_launch(bn16_fwd_apply_kernel<1>, bn16_smem_bytes<1>(), occ_a1, a, false, nullptr, st);
  return rc ? rc : (int)cudaGetLastError();
}

// x, dy, y, out (dx), out2 (dresidual, optional): bf16 [P, C]; relu: 0 none, 1 mask from y, 2 mask from x
extern "C" int bn16_backward(const BnArgs* args, cudaStream_t st) {
  BnArgs a = *args;
  if (!bn16_supported(a.P, a.C) || a.partial == nullptr || bn16_error_word() == nullptr) return -1;
  if (!bn16_aligned(a.x) || !bn16_aligned(a.dy) || !bn16_aligned(a.y) || !bn16_aligned(a.out) || !bn16_aligned(a.out2)) return -4;
  static int occ_r2 = 0, occ_r3 = 0, occ_a2 = 0, occ_a3 = 0, occ_rx = 0, occ_ax = 0;
  const bool xmask = a.relu == 2;      // ReLU without a residual: the mask comes from x (beta must be given)
  if (xmask && (a.beta == nullptr || a.out2 != nullptr)) return -1;
  int rc;
  if (xmask)
    rc = bn16_launch(bn16_reduce_kernel<true, 2, true>, bn16_smem_bytes<2>(), occ_rx, a, true, &a.n_partials, st);
  else if (a.relu)
    rc = bn16_launch(bn16_reduce_kernel<true, 3>, bn16_smem_bytes<3>(), occ_r3, a, true, &a.n_partials, st);
  else
    rc = bn16_launch(bn16_reduce_kernel<true, 2>, bn16_smem_bytes<2>(), occ_r2, a, true, &a.n_partials, st);
  if (rc) return rc;
  launch_k(bn16_finalize_kernel<true>, dim3((a.C + BN16_FIN_CH - 1) / BN16_FIN_CH), dim3(BN16_THREADS), 0, st, a);
  if (xmask)
    rc = bn16_launch(bn16_bwd_apply_kernel<2, true>, bn16_smem_bytes<2>(), occ_ax, a, false, nullptr, st);
  else if (a.relu)
    rc = bn16_launch(bn16_bwd_apply_kernel<3>, bn16_smem_bytes<3>(), occ_a3, a, false, nullptr, st);
  else
    rc = bn16_launch(bn16_bwd_apply_kernel<2>, bn16_smem_bytes<2>(), occ_a2, a, false, nullptr, st);
  return rc ? rc : (int)cudaGetLastError();
}
