// Softmax cross-entropy (mean over the batch) fused with its gradient and the top-1 / top-5
// accuracy of the same logits: one kernel instead of log_softmax + nll_loss + topk + eq + sums
// + their backward kernels (dl_code/pcode/create_metrics.py:31-48 and the criterion call of
// dl_code/pcode/distributed_running_cv.py:52-56, each with its own .item() synchronisation).
//
//   loss   = mean_i ( log sum_j exp(z_ij) - z_i,t_i )
//   dz_ij  = ( softmax(z_i)_j - [j == t_i] ) / B               written in the same pass
//   top-k  = 100 / B * #{ i : #{ j : z_ij > z_i,t_i } < k }     (rank of the label's score)
//
// One CTA per row (three passes over the row, which stays in L1/L2 for classifier-sized rows
// and is 133 KB for a 33 278-word vocabulary); the last CTA to arrive adds the per-row results
// in a fixed order, so the loss is reproducible run to run.  Rows whose label lies outside
// [0, C) contribute neither loss nor gradient and are not counted in the mean.
#include <cuda_runtime.h>
#include "launch.cuh"
#include <stdint.h>

#define CE_THREADS 128

__device__ __forceinline__ float ce_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float ce_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// out[0] = loss, out[1] = top-1 %, out[2] = top-5 %, out[3] = number of counted rows
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(const float* __restrict__ z, const long long* __restrict__ tgt,
                                                                  float* __restrict__ dz, float* row_loss, int* row_rank,
                                                                  unsigned* counter, float* out, float* loss_out, int B, int C,
                                                                  long long ld) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[CE_THREADS / 32];
  __shared__ int redi[CE_THREADS / 32];
  __shared__ int last;
  const int row = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const float* zr = z + (size_t)row * ld;    // ld >= C floats per row (padded rows of a GEMM output)
  float* dr = dz + (size_t)row * ld;
  const long long t = tgt[row];
  const bool valid = t >= 0 && t < C;
  // pass 1: row maximum
  float m = -INFINITY;
  for (int j = threadIdx.x; j < C; j += CE_THREADS) m = fmaxf(m, zr[j]);
  m = ce_warp_max(m);
  if (lane == 0) red[wid] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int w = 1; w < CE_THREADS / 32; ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  // pass 2: sum of exponentials, rank of the label's score
  const float zt = valid ? zr[t] : 0.f;
  float s = 0.f;
  int rank = 0;
  for (int j = threadIdx.x; j < C; j += CE_THREADS) {
    const float v = zr[j];
    s += __expf(v - m);
    rank += v > zt;
  }
  s = ce_warp_sum(s);
  for (int o = 16; o > 0; o >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
  if (lane == 0) { red[wid] = s; redi[wid] = rank; }
  __syncthreads();
  s = 0.f; rank = 0;
#pragma unroll
  for (int w = 0; w < CE_THREADS / 32; ++w) { s += red[w]; rank += redi[w]; }
  // pass 3: gradient
  const float inv_s = 1.f / s, scale = valid ? 1.f / (float)B : 0.f;
  for (int j = threadIdx.x; j < C; j += CE_THREADS) {
    float p = __expf(zr[j] - m) * inv_s;
    if (j == t) p -= 1.f;
    dr[j] = p * scale;
  }
  if (threadIdx.x == 0) {
    row_loss[row] = valid ? (logf(s) + m - zt) : 0.f;
    row_rank[row] = valid ? rank : -1;
    __threadfence();
    last = (atomicAdd(counter, 1u) == (unsigned)B - 1);
    if (last) __threadfence();
  }
  __syncthreads();
  if (!last) return;
  // fixed-order reduction over the rows
  float ls = 0.f;
  int n1 = 0, n5 = 0, nv = 0;
  for (int i = threadIdx.x; i < B; i += CE_THREADS) {
    const int r = __ldcg(row_rank + i);
    if (r >= 0) {
      ls += __ldcg(row_loss + i);
      n1 += r < 1;
      n5 += r < 5;
      nv += 1;
    }
  }
  __shared__ float fl[CE_THREADS];
  __shared__ int i1[CE_THREADS], i5[CE_THREADS], iv[CE_THREADS];
  fl[threadIdx.x] = ls; i1[threadIdx.x] = n1; i5[threadIdx.x] = n5; iv[threadIdx.x] = nv;
  __syncthreads();
  for (int o = CE_THREADS / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      fl[threadIdx.x] += fl[threadIdx.x + o];
      i1[threadIdx.x] += i1[threadIdx.x + o];
      i5[threadIdx.x] += i5[threadIdx.x + o];
      iv[threadIdx.x] += iv[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float n = iv[0] > 0 ? (float)iv[0] : 1.f;
    out[0] = fl[0] / n;
    *loss_out = fl[0] / n;
    out[1] = 100.f * (float)i1[0] / n;
    out[2] = 100.f * (float)i5[0] / n;
    out[3] = (float)iv[0];
    *counter = 0;
  }
}

// With ignored rows the mean runs over the counted rows only: rescale the gradient (B / n_valid).
__global__ void ce_rescale_kernel(float* dz, const float* out, long long n, int B) {
  pdl_wait();
  pdl_trigger();
  const float nv = out[3];
  if (nv == (float)B || nv <= 0.f) return;
  const float f = (float)B / nv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dz[i] *= f;
}

// scratch: B floats + B ints + 1 unsigned (counter: zero before the first call, self-resetting);
// out: 4 floats; loss_out: 1 float
extern "C" int cross_entropy_fused_ld(const void* logits, const void* target, void* dlogits, void* scratch, void* out,
                                      void* loss_out, int B, int C, long long ld, int may_ignore, cudaStream_t st);

extern "C" int cross_entropy_fused(const void* logits, const void* target, void* dlogits, void* scratch, void* out,
                                   void* loss_out, int B, int C, int may_ignore, cudaStream_t st) {
  return cross_entropy_fused_ld(logits, target, dlogits, scratch, out, loss_out, B, C, C, may_ignore, st);
}

// same with `ld` floats between consecutive rows of logits and of dlogits (ld >= C)
extern "C" int cross_entropy_fused_ld(const void* logits, const void* target, void* dlogits, void* scratch, void* out,
                                      void* loss_out, int B, int C, long long ld, int may_ignore, cudaStream_t st) {
  if (B < 1 || C < 1 || ld < C) return -1;
  float* row_loss = reinterpret_cast<float*>(scratch);
  int* row_rank = reinterpret_cast<int*>(row_loss + B);
  unsigned* counter = reinterpret_cast<unsigned*>(row_rank + B);
  launch_k(cross_entropy_kernel, dim3(B), dim3(CE_THREADS), 0, st, reinterpret_cast<const float*>(logits),
                                                 reinterpret_cast<const long long*>(target),
                                                 reinterpret_cast<float*>(dlogits), row_loss, row_rank, counter,
                                                 reinterpret_cast<float*>(out), reinterpret_cast<float*>(loss_out), B, C, ld);
  if (may_ignore) {
    const long long n = (long long)B * ld;   // padding columns included: scaling them is harmless
    long long blocks = (n + 255) / 256;
    if (blocks > 8 * sm_count()) blocks = 8 * sm_count();
    launch_k(ce_rescale_kernel, dim3((int)blocks), dim3(256), 0, st, reinterpret_cast<float*>(dlogits), reinterpret_cast<const float*>(out), n, B);
  }
  return (int)cudaGetLastError();
}
