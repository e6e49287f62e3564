// Regularised logistic loss of the node-averaged iterate on the full data set:
//   f(x) = 1/N sum_i log(1 + exp(-y_i a_i . x)) + lambda/2 ||x||^2
// (convex_code/base_logistic.py:25-32), the expensive part of the convex simulator's logging
// (a 40 000 x 2000 GEMV ten times per epoch).  One warp per data row: fp32 features, fp64 dot product
// and accumulation, a numerically stable softplus, deterministic two-level reduction.
#include <cuda_runtime.h>
#include "launch.cuh"
#include <stdint.h>

#define LR_THREADS 256

__global__ void __launch_bounds__(LR_THREADS) logreg_loss_kernel(const float* __restrict__ A, const float* __restrict__ y,
                                                                const double* __restrict__ x, long long N, int d,
                                                                double* partial, unsigned* counter, double lambda,
                                                                double* out) {
  __shared__ double red[LR_THREADS / 32];
  __shared__ int last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warps_total = (long long)gridDim.x * (LR_THREADS / 32);
  double acc = 0.0;
  for (long long row = (long long)blockIdx.x * (LR_THREADS / 32) + warp; row < N; row += warps_total) {
    const float* a = A + row * d;
    double dot = 0.0;
    for (int j = lane * 4; j + 3 < d; j += 128) {
      const float4 v = *reinterpret_cast<const float4*>(a + j);
      dot += (double)v.x * x[j] + (double)v.y * x[j + 1] + (double)v.z * x[j + 2] + (double)v.w * x[j + 3];
    }
    for (int j = (d & ~3) + lane; j < d; j += 32) dot += (double)a[j] * x[j];
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) {
      const double z = -(double)y[row] * dot;
      acc += z > 0.0 ? z + log1p(exp(-z)) : log1p(exp(z));
    }
  }
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < LR_THREADS / 32; ++w) t += red[w];
    partial[blockIdx.x] = t;
    __threadfence();
    last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    if (last) __threadfence();
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    double t = 0.0;
    for (unsigned b = 0; b < gridDim.x; ++b) t += partial[b];
    double reg = 0.0;
    for (int j = 0; j < d; ++j) reg += x[j] * x[j];
    *out = t / (double)N + 0.5 * lambda * reg;
    *counter = 0;
  }
}

extern "C" int logreg_loss_blocks() { return sm_count() * 4; }

// A [N, d] fp32 row-major (d % 4 == 0 and 16-byte aligned rows), y [N] fp32 (+1 / -1), x [d] fp64.
// scratch: (blocks + 1) doubles.  out: 1 double.
extern "C" int logreg_loss(const void* A, const void* y, const void* x, long long N, int d, double lambda, void* scratch,
                           void* out, cudaStream_t st) {
  if (d % 4 != 0) return -1;
  const int blocks = logreg_loss_blocks();
  double* partial = reinterpret_cast<double*>(scratch);
  unsigned* counter = reinterpret_cast<unsigned*>(partial + blocks);
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(unsigned), st);
  if (e != cudaSuccess) return (int)e;
  logreg_loss_kernel<<<blocks, LR_THREADS, 0, st>>>(reinterpret_cast<const float*>(A), reinterpret_cast<const float*>(y),
                                                    reinterpret_cast<const double*>(x), N, d, partial, counter, lambda,
                                                    reinterpret_cast<double*>(out));
  return (int)cudaGetLastError();
}

// ---- one iteration of the decentralized simulator, all nodes, in ONE kernel -------------------------
//
// State x, x_hat in R^{n x d} (node-major: the d coordinates of a node are contiguous), fp64 like the
// numpy simulator (convex_code/logistic.py:152-199).  CTA m is node m: it takes the stochastic
// gradient step on its sampled row, the communication step of the chosen method in matrix form and
// the column compressor, entirely on chip:
//
//   delta_m = lr ( y a sigma(-y a.x_m) - lambda x_m )                                (:167-178)
//   plain     x_m <- sum_i W[i,m] (x_i + delta_i)                                    (:181-182)
//   choco     x_m <- x_m + delta_m + gamma sum_i xh_i (W - I)[i,m];  xh_m += Q(x_m - xh_m)   (:183-187)
//   dcd-psgd  x_m <- x_m + Q( sum_i W[i,m] x_i + delta_m - x_m )                     (:188-191)
//   ecd-psgd  x_new = sum_i W[i,m] xh_i + delta_m;  z = (1 - (t+1)/2) x_m + (t+1)/2 x_new;
//             xh_m <- (1 - 2/(t+1)) xh_m + 2/(t+1) Q(z);  x_m <- x_new               (:192-197)
//
// Q: none, top-k of |.| (exact k, a 64-bit radix select in shared memory, ties to the lower index),
// random-k (keyed Feistel permutation of [0, d): a different random stream than numpy's), QSGD with s
// levels (counter-hash uniforms).  Inputs are read from (x_in, xh_in) and written to (x_out, xh_out):
// neighbours read the old state while a node writes its new one, so the kernel needs no grid barrier.
#include "common.cuh"

#define LRI_THREADS 256
#define LRI_MAX_NODES 64

struct LogregIterArgs {
  const float* A;          // [N, d]
  const float* y;          // [N]
  const long long* rows;   // [n] sampled row of every node for this iteration
  const double* x_in;      // [n, d]
  const double* xh_in;     // [n, d]
  double* x_out;           // [n, d]
  double* xh_out;          // [n, d]
  const double* W;         // [n, n]
  double lr, lambda, gamma;
  long long t;             // iteration index (0-based)
  int n, d;
  int method;              // 0 plain, 1 choco, 2 dcd-psgd, 3 ecd-psgd
  int quant;               // 0 full, 1 top-k, 2 random-k (biased), 3 random-k (unbiased), 4 qsgd (biased), 5 qsgd (unbiased)
  int k, levels;
  uint32_t seed;
};

__device__ __forceinline__ double lri_block_sum(double v, double* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = 0.0;
  for (int w = 0; w < LRI_THREADS / 32; ++w) t += red[w];
  return t;
}

// -y a sigma(...) coefficient of node i's sampled row against its own iterate
__device__ double lri_coef(const LogregIterArgs& a, int i, double* red) {
  const float* row = a.A + a.rows[i] * (long long)a.d;
  const double* xi = a.x_in + (size_t)i * a.d;
  double dot = 0.0;
  for (int j = threadIdx.x; j < a.d; j += LRI_THREADS) dot += (double)row[j] * xi[j];
  dot = lri_block_sum(dot, red);
  const double yy = (double)a.y[a.rows[i]];
  return yy / (1.0 + exp(yy * dot));   // y sigma(-y a.x)
}

__global__ void __launch_bounds__(LRI_THREADS) logreg_iter_kernel(LogregIterArgs a) {
  extern __shared__ double lri_v[];          // [d] the vector handed to the compressor
  __shared__ double red[LRI_THREADS / 32];
  __shared__ unsigned hist[256];
  __shared__ unsigned long long sel_prefix;
  __shared__ unsigned sel_need, sel_equal;
  const int m = blockIdx.x, d = a.d, n = a.n;
  const double* xm = a.x_in + (size_t)m * d;
  const double* xhm = a.xh_in + (size_t)m * d;
  double* xo = a.x_out + (size_t)m * d;
  double* xho = a.xh_out + (size_t)m * d;
  const float* arow = a.A + a.rows[m] * (long long)d;
  const double tt = (double)(a.t + 1);

  if (a.method == 0) {
    // plain: needs the gradient steps of the neighbours too (recomputed here: a few dot products)
    for (int j = threadIdx.x; j < d; j += LRI_THREADS) lri_v[j] = 0.0;
    __syncthreads();
    for (int i = 0; i < n; ++i) {
      const double w = a.W[(size_t)i * n + m];
      if (w == 0.0) continue;                                  // uniform over the CTA
      const double coef = lri_coef(a, i, red);
      const float* ri = a.A + a.rows[i] * (long long)d;
      const double* xi = a.x_in + (size_t)i * d;
      for (int j = threadIdx.x; j < d; j += LRI_THREADS)
        lri_v[j] += w * (xi[j] + a.lr * (coef * (double)ri[j] - a.lambda * xi[j]));
      __syncthreads();
    }
    for (int j = threadIdx.x; j < d; j += LRI_THREADS) {
      xo[j] = lri_v[j];
      xho[j] = xhm[j];
    }
    return;
  }

  const double coef = lri_coef(a, m, red);
  // the vector to compress (lri_v) and what is kept besides it
  for (int j = threadIdx.x; j < d; j += LRI_THREADS) {
    const double delta = a.lr * (coef * (double)arow[j] - a.lambda * xm[j]);
    double mix = 0.0;
    const double* src = a.method == 2 ? a.x_in : a.xh_in;     // dcd mixes x, choco / ecd mix x_hat
    for (int i = 0; i < n; ++i) {
      const double w = a.W[(size_t)i * n + m];
      if (w != 0.0) mix += w * src[(size_t)i * d + j];
    }
    if (a.method == 1) {
      const double xn = xm[j] + delta + a.gamma * (mix - xhm[j]);   // x_hat (W - I)
      xo[j] = xn;
      lri_v[j] = xn - xhm[j];
    } else if (a.method == 2) {
      lri_v[j] = mix + delta - xm[j];
    } else {
      const double xn = mix + delta;
      xo[j] = xn;
      lri_v[j] = (1.0 - 0.5 * tt) * xm[j] + 0.5 * tt * xn;
    }
  }
  __syncthreads();

  // ---- compressor on lri_v (in place: entries that are not sent become zero) ----
  if (a.quant == 1) {
    // exact top-k of |v|: 8-bit radix select on the 63 magnitude bits, then a pass that keeps keys
    // above the threshold and the first `need` keys equal to it in index order
    unsigned long long prefix = 0, mask = 0;
    unsigned need = (unsigned)a.k;
    for (int shift = 56; shift >= 0; shift -= 8) {
      for (int b = threadIdx.x; b < 256; b += LRI_THREADS) hist[b] = 0;
      __syncthreads();
      for (int j = threadIdx.x; j < d; j += LRI_THREADS) {
        const unsigned long long key = (unsigned long long)__double_as_longlong(fabs(lri_v[j]));
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (threadIdx.x < 32) {
        // lane l owns the bins 255 - 8 l ... 248 - 8 l (descending); the digit is the first bin, from
        // the top, at which the running count reaches `need`
        const int top = 255 - 8 * (int)threadIdx.x;
        unsigned mine = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) mine += hist[top - q];
        unsigned incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const unsigned v = __shfl_up_sync(0xffffffffu, incl, o);
          if ((int)threadIdx.x >= o) incl += v;
        }
        const unsigned excl = incl - mine;
        const unsigned hit = __ballot_sync(0xffffffffu, incl >= need);
        const int owner = hit ? __ffs(hit) - 1 : 31;
        if ((int)threadIdx.x == owner) {
          unsigned above = excl;
          int b = top;
          for (int q = 0; q < 7; ++q, --b) {
            if (above + hist[b] >= need) break;
            above += hist[b];
          }
          sel_prefix = prefix | ((unsigned long long)b << shift);
          sel_need = need - above;
          sel_equal = hist[b];
        }
      }
      __syncthreads();
      prefix = sel_prefix;
      need = sel_need;
      mask |= 0xFFull << shift;
      __syncthreads();
    }
    // prefix = k-th largest key; `need` of the keys equal to it are kept (lowest indices first)
    for (int j = threadIdx.x; j < d; j += LRI_THREADS) {
      const unsigned long long key = (unsigned long long)__double_as_longlong(fabs(lri_v[j]));
      if (key < prefix) lri_v[j] = 0.0;
    }
    if (need < sel_equal) {   // more entries tie with the threshold than may be kept (uniform over the CTA)
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned taken = 0;
        for (int j = 0; j < d; ++j) {
          const unsigned long long key = (unsigned long long)__double_as_longlong(fabs(lri_v[j]));
          if (key == prefix && lri_v[j] != 0.0) {
            if (taken < need) ++taken;
            else lri_v[j] = 0.0;
          }
        }
      }
    }
    __syncthreads();
  } else if (a.quant == 2 || a.quant == 3) {
    // random-k: keep the first k images of a keyed permutation of [0, d); mark them in shared memory
    uint32_t keys[4];
    for (uint32_t r = 0; r < 4; ++r) keys[r] = feistel_key(a.seed, (uint32_t)a.t, (uint32_t)m, r);
    const int hb = feistel_half_bits((uint32_t)d);
    // flags live in the low bit of a side array: reuse hist when d is small, else mark by sign trick
    // (simple and exact: a second buffer of flags in global memory is avoided by scanning k images)
    const double scale = a.quant == 3 ? (double)d / (double)a.k : 1.0;
    // pass 1: copy kept values into x_out's slot of the payload (xho is free to use as scratch here)
    for (int j = threadIdx.x; j < d; j += LRI_THREADS) xho[j] = 0.0;
    __syncthreads();
    for (int e = threadIdx.x; e < a.k; e += LRI_THREADS) {
      const uint32_t idx = feistel_perm((uint32_t)e, (uint32_t)d, hb, keys);
      xho[idx] = scale * lri_v[idx];
    }
    __syncthreads();
    for (int j = threadIdx.x; j < d; j += LRI_THREADS) lri_v[j] = xho[j];
    __syncthreads();
  } else if (a.quant == 4 || a.quant == 5) {
    double sq = 0.0;
    for (int j = threadIdx.x; j < d; j += LRI_THREADS) sq += lri_v[j] * lri_v[j];
    const double norm = sqrt(lri_block_sum(sq, red));
    const double s = (double)a.levels;
    double scale = 1.0;
    if (a.quant == 4) scale = 1.0 / (fmin((double)d / (s * s), sqrt((double)d) / s) + 1.0);
    const uint32_t ubase = uniform_base(a.seed + 7919u * (uint32_t)m, (uint32_t)a.t);
    for (int j = threadIdx.x; j < d; j += LRI_THREADS) {
      const double v = lri_v[j];
      double q = 0.0;
      if (norm > 0.0) {
        const double level = s * fabs(v) / norm, low = floor(level);
        const double up = (double)counter_uniform(ubase, (uint32_t)j) < (level - low) ? 1.0 : 0.0;
        q = scale * (v > 0.0 ? 1.0 : (v < 0.0 ? -1.0 : 0.0)) * norm * (low + up) / s;
      }
      lri_v[j] = q;
    }
    __syncthreads();
  }

  // ---- apply the compressed vector ----
  for (int j = threadIdx.x; j < d; j += LRI_THREADS) {
    const double q = lri_v[j];
    if (a.method == 1) {
      xho[j] = xhm[j] + q;
    } else if (a.method == 2) {
      xo[j] = xm[j] + q;
      xho[j] = xhm[j];
    } else {
      xho[j] = (1.0 - 2.0 / tt) * xhm[j] + (2.0 / tt) * q;
    }
  }
}

extern "C" int logreg_iter_args_size() { return (int)sizeof(LogregIterArgs); }

extern "C" int logreg_iter(const LogregIterArgs* args, cudaStream_t st) {
  const LogregIterArgs& a = *args;
  if (a.n < 1 || a.n > LRI_MAX_NODES || a.d < 1 || a.d * 8 > 96 * 1024) return -1;
  if (a.method < 0 || a.method > 3 || a.quant < 0 || a.quant > 5) return -1;
  if ((a.quant >= 1 && a.quant <= 3) && (a.k < 1 || a.k > a.d)) return -1;
  if (a.quant >= 4 && a.levels < 1) return -1;
  const size_t smem = (size_t)a.d * sizeof(double);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(logreg_iter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = 96 * 1024;
  }
  logreg_iter_kernel<<<a.n, LRI_THREADS, smem, st>>>(a);
  return (int)cudaGetLastError();
}
