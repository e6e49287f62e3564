// Regularised logistic loss of the node-averaged iterate on the full data set:
//   f(x) = 1/N sum_i log(1 + exp(-y_i a_i . x)) + lambda/2 ||x||^2
// (convex_code/base_logistic.py:25-32), the expensive part of the convex simulator's logging
// (a 40 000 x 2000 GEMV ten times per epoch).  One warp per data row: fp32 features, fp64 dot product
// and accumulation, a numerically stable softplus, deterministic two-level reduction.
#include <cuda_runtime.h>
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

extern "C" int logreg_loss_blocks() { return 148 * 4; }

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
