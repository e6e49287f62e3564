// Embedding lookup and its gradient (fp32): the input layer of the language model
// (dl_code/pcode/models/rnn_lm.py:29, 53).
//
//   forward : out[i, :] = weight[idx[i], :]
//   backward: grad[v, :] += sum over positions i with idx[i] == v of dy[i, :]
//
// The gradient is accumulated IN PLACE into an existing [V, D] tensor (with tied weights: the decoder's weight
// gradient), so no [V, D] tensor of zeros is built and added.  It is reproducible without a sort: CTA i owns
// position i; it does nothing unless i is the FIRST position of its token (a scan of the preceding indices); the
// owner adds the rows of all later positions with the same token in position order and then updates the token's
// gradient row, which no other CTA touches.  The positions of a token are marked in a shared-memory bit mask by
// one parallel scan of the indices, so the owner's loop visits only them.
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch.cuh"

#define EMB_THREADS 256

__global__ void __launch_bounds__(EMB_THREADS) embedding_fwd_kernel(const long long* __restrict__ idx,
                                                                  const float* __restrict__ weight, float* __restrict__ out,
                                                                  int N, int D, int V, int* __restrict__ error) {
  pdl_wait();
  pdl_trigger();
  for (int i = blockIdx.x; i < N; i += gridDim.x) {
    const long long v = idx[i];
    if (v < 0 || v >= V) {                       // recorded, row left zero (the host raises)
      if (threadIdx.x == 0) atomicExch(error, 1);
      for (int c = threadIdx.x; c < D; c += EMB_THREADS) out[(size_t)i * D + c] = 0.f;
      continue;
    }
    for (int c = threadIdx.x; c < D; c += EMB_THREADS) out[(size_t)i * D + c] = weight[(size_t)v * D + c];
  }
}

#define EMB_MAX_POS 65536   // positions per call covered by the shared-memory bit mask

__global__ void __launch_bounds__(EMB_THREADS) embedding_bwd_kernel(const long long* __restrict__ idx,
                                                                  const float* __restrict__ dy, float* __restrict__ grad,
                                                                  int N, int D, int V) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t mask[EMB_MAX_POS / 32];    // bit k: position k holds this CTA's token
  __shared__ int dup;
  const int i = blockIdx.x;
  const long long v = idx[i];
  if (v < 0 || v >= V) return;                   // uniform over the CTA
  const int nwords = (N + 31) >> 5;
  for (int w = threadIdx.x; w < nwords; w += EMB_THREADS) mask[w] = 0;
  if (threadIdx.x == 0) dup = 0;
  __syncthreads();
  for (int j = threadIdx.x; j < N; j += EMB_THREADS)
    if (idx[j] == v) atomicOr(&mask[j >> 5], 1u << (j & 31));
  __syncthreads();
  // an earlier position with the same token owns it
  for (int w = threadIdx.x; w <= (i >> 5); w += EMB_THREADS) {
    uint32_t bits = mask[w];
    if (w == (i >> 5)) bits &= (1u << (i & 31)) - 1u;
    if (bits) dup = 1;                           // benign race: every writer stores 1
  }
  __syncthreads();
  if (dup) return;
  // the owner adds the rows of all positions of its token in position order, then updates the gradient row
  for (int c = threadIdx.x; c < D; c += EMB_THREADS) {
    float acc = 0.f;
    for (int w = i >> 5; w < nwords; ++w) {
      uint32_t bits = mask[w];
      while (bits) {
        const int k = (w << 5) + __ffs(bits) - 1;
        bits &= bits - 1;
        acc += dy[(size_t)k * D + c];
      }
    }
    grad[(size_t)v * D + c] += acc;
  }
}

static int* g_emb_error[64];
static int* emb_error_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (g_emb_error[dev] == nullptr) {
    if (cudaMalloc(&g_emb_error[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(g_emb_error[dev], 0, sizeof(int));
  }
  return g_emb_error[dev];
}

// 1 when a lookup met an index outside [0, V) since the last call (synchronises; clears the flag)
extern "C" int embedding_last_error() {
  int* w = emb_error_word();
  int v = -1;
  if (w == nullptr || cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) cudaMemset(w, 0, sizeof(int));
  return v;
}

// idx: int64 [N]; weight: [V, D]; out: [N, D]
extern "C" int embedding_forward(const void* idx, const void* weight, void* out, int N, int D, int V, cudaStream_t st) {
  if (N < 1 || D < 1 || V < 1) return -1;
  int* err = emb_error_word();
  if (err == nullptr) return -13;
  const int grid = N < 8 * sm_count() ? N : 8 * sm_count();
  launch_k(embedding_fwd_kernel, dim3(grid), dim3(EMB_THREADS), 0, st, reinterpret_cast<const long long*>(idx),
           reinterpret_cast<const float*>(weight), reinterpret_cast<float*>(out), N, D, V, err);
  return (int)cudaGetLastError();
}

// grad [V, D] += scatter of dy [N, D] by idx [N]
extern "C" int embedding_backward_accumulate(const void* idx, const void* dy, void* grad, int N, int D, int V,
                                             cudaStream_t st) {
  if (N < 1 || N > EMB_MAX_POS || D < 1 || V < 1) return -1;
  launch_k(embedding_bwd_kernel, dim3(N), dim3(EMB_THREADS), 0, st, reinterpret_cast<const long long*>(idx),
           reinterpret_cast<const float*>(dy), reinterpret_cast<float*>(grad), N, D, V);
  return (int)cudaGetLastError();
}
