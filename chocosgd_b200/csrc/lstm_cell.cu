// Fused LSTM cell pointwise kernels (gate order i, f, g, o as in torch.nn.LSTM):
//   forward :  i,f,o = sigmoid(.), g = tanh(.);  c = f c_prev + i g;  h = o tanh(c)
//              (the activated gates overwrite the pre-activations: they are what backward needs)
//   backward:  given dh, dc_next -> d(pre-activations) in place of the gates, dc_prev
// The gate GEMMs around them ([T B, in] x W_ih^T once per layer, [B, H] x W_hh^T per step) are issued
// by the Python layer (ops/lstm.py); these kernels replace the ~12 elementwise launches per time step.
#include <cuda_runtime.h>

__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + __expf(-x)); }

// gates: [B, 4H] (pre-activations in, activations out); c_prev, c, h: [B, H]
__global__ void lstm_cell_fwd_kernel(float* __restrict__ gates, const float* __restrict__ c_prev, float* __restrict__ c,
                                     float* __restrict__ h, int B, int H) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  float* g = gates + (size_t)b * 4 * H;
  const float i = sigm(g[j]), f = sigm(g[H + j]), gg = tanhf(g[2 * H + j]), o = sigm(g[3 * H + j]);
  const float cn = fmaf(f, c_prev[idx], i * gg);
  g[j] = i; g[H + j] = f; g[2 * H + j] = gg; g[3 * H + j] = o;
  c[idx] = cn;
  h[idx] = o * tanhf(cn);
}

// gates hold the activations; on exit they hold d(pre-activations).  dc_io: dc_next in, dc_prev out.
__global__ void lstm_cell_bwd_kernel(float* __restrict__ gates, const float* __restrict__ c_prev,
                                     const float* __restrict__ c, const float* __restrict__ dh, float* __restrict__ dc_io,
                                     int B, int H) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  float* g = gates + (size_t)b * 4 * H;
  const float i = g[j], f = g[H + j], gg = g[2 * H + j], o = g[3 * H + j];
  const float tc = tanhf(c[idx]);
  const float dhv = dh[idx];
  const float dc = fmaf(dhv * o, 1.f - tc * tc, dc_io[idx]);
  g[j] = dc * gg * i * (1.f - i);
  g[H + j] = dc * c_prev[idx] * f * (1.f - f);
  g[2 * H + j] = dc * i * (1.f - gg * gg);
  g[3 * H + j] = dhv * tc * o * (1.f - o);
  dc_io[idx] = dc * f;
}

extern "C" int lstm_cell_fwd(void* gates, const void* c_prev, void* c, void* h, int B, int H, cudaStream_t st) {
  const int n = B * H;
  lstm_cell_fwd_kernel<<<(n + 255) / 256, 256, 0, st>>>(reinterpret_cast<float*>(gates), reinterpret_cast<const float*>(c_prev),
                                                       reinterpret_cast<float*>(c), reinterpret_cast<float*>(h), B, H);
  return (int)cudaGetLastError();
}

extern "C" int lstm_cell_bwd(void* gates, const void* c_prev, const void* c, const void* dh, void* dc_io, int B, int H,
                             cudaStream_t st) {
  const int n = B * H;
  lstm_cell_bwd_kernel<<<(n + 255) / 256, 256, 0, st>>>(reinterpret_cast<float*>(gates), reinterpret_cast<const float*>(c_prev),
                                                       reinterpret_cast<const float*>(c), reinterpret_cast<const float*>(dh),
                                                       reinterpret_cast<float*>(dc_io), B, H);
  return (int)cudaGetLastError();
}
