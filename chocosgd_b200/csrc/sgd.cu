// Fused multi-segment momentum-SGD update and global gradient-norm clipping.
//
// fused_sgd: one launch updates every parameter tensor of the flat arena
//   d = g + wd_seg x;  m = d (first step) | mu m + d;  d' = d + mu m (Nesterov) | m;  x -= lr d'
// (dl_code/pcode/optim/utils.py:13-47, which issues 4-6 elementwise launches per tensor),
// and clears the gradient in the same pass.  With apply == 0 it writes d' into g instead
// (the "apply_grad_to_model=False" variant used by DCD/ECD-PSGD).
//
// grad_clip_coef: deterministic two-level sum of squares of the flat gradient; the last
// CTA stores min(1, max_norm / (norm + 1e-6)) into hyper[HYP_GSCALE], which the update
// kernels multiply into the gradient (torch.nn.utils.clip_grad_norm_ semantics,
// dl_code/pcode/distributed_running_nlp.py:94-97).
#include "common.cuh"
#include "launch.cuh"

__global__ void __launch_bounds__(CHOCO_THREADS) fused_sgd_kernel(const ChocoParams* __restrict__ params, int apply) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = blockIdx.x;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const float lr = p.hyper[HYP_LR], mu = p.hyper[HYP_MOMENTUM], gscale = p.hyper[HYP_GSCALE];
  const bool nesterov = p.hyper[HYP_NESTEROV] != 0.f;
  const bool mom_init = p.step[1] != 0;
  const float wd = tb.seg_wd[seg];
  const int span = (valid + 3) & ~3;
  for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 4) {
    const int pos = start + base;
    const float4 xv = *reinterpret_cast<const float4*>(p.x + pos);
    const float4 gv = load_grad4(p, seg, pos, base, valid);
    float x_a[4] = {xv.x, xv.y, xv.z, xv.w}, g_a[4] = {gv.x, gv.y, gv.z, gv.w};
    float m_a[4] = {0.f, 0.f, 0.f, 0.f}, d_a[4] = {0.f, 0.f, 0.f, 0.f};
    if (mu != 0.f && mom_init) {
      const float4 mv = *reinterpret_cast<const float4*>(p.m + pos);
      m_a[0] = mv.x; m_a[1] = mv.y; m_a[2] = mv.z; m_a[3] = mv.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (base + e < valid) {
        d_a[e] = sgd_direction(x_a[e], g_a[e] * gscale, m_a[e], wd, mu, nesterov, mom_init);
        x_a[e] = fmaf(-lr, d_a[e], x_a[e]);
      }
    }
    if (mu != 0.f) *reinterpret_cast<float4*>(p.m + pos) = make_float4(m_a[0], m_a[1], m_a[2], m_a[3]);
    if (apply) {
      *reinterpret_cast<float4*>(p.x + pos) = make_float4(x_a[0], x_a[1], x_a[2], x_a[3]);
      clear_grad4(p, pos);
    } else {
      *reinterpret_cast<float4*>(p.g + pos) = make_float4(d_a[0], d_a[1], d_a[2], d_a[3]);  // flat gradients only
    }
  }
  // last CTA marks the momentum buffer as initialised
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.done_count + 2, 1u) == (uint32_t)tb.n_chunks - 1) {
      p.done_count[2] = 0;
      p.step[1] = 1;
    }
  }
}

extern "C" int fused_sgd_step(const void* params_dev, int n_chunks, int n_ranks, int apply, cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  launch_k(fused_sgd_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev), apply);
  return (int)cudaGetLastError();
}

// ---- global gradient-norm clipping --------------------------------------------------------
__global__ void __launch_bounds__(CHOCO_THREADS) grad_clip_kernel(const ChocoParams* __restrict__ params,
                                                                 float max_norm, float* norm_out) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = blockIdx.x;
  __shared__ float red[32];
  __shared__ int last;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int span = (valid + 3) & ~3;
  float acc = 0.f;
  // fixed element -> thread mapping: the sum is reproducible run to run
  for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 4) {
    const float4 v = load_grad4(p, seg, start + base, base, valid);
    if (base + 0 < valid) acc = fmaf(v.x, v.x, acc);
    if (base + 1 < valid) acc = fmaf(v.y, v.y, acc);
    if (base + 2 < valid) acc = fmaf(v.z, v.z, acc);
    if (base + 3 < valid) acc = fmaf(v.w, v.w, acc);
  }
  const float tot = block_sum(acc, red);
  if (threadIdx.x == 0) {
    p.partial[chunk] = tot;
    __threadfence();
    last = (atomicAdd(p.done_count + 3, 1u) == (uint32_t)tb.n_chunks - 1);
    if (last) __threadfence();
  }
  __syncthreads();
  if (last) {
    float a = 0.f;
    for (int c = threadIdx.x; c < tb.n_chunks; c += CHOCO_THREADS) a += __ldcg(p.partial + c);
    const float sq = block_sum(a, red);
    if (threadIdx.x == 0) {
      const float norm = sqrtf(sq);
      const float coef = max_norm / (norm + 1e-6f);
      const_cast<float*>(p.hyper)[HYP_GSCALE] = coef < 1.f ? coef : 1.f;
      if (norm_out) norm_out[blockIdx.y] = norm;
      p.done_count[3] = 0;
    }
  }
}

extern "C" int grad_clip_coef(const void* params_dev, int n_chunks, int n_ranks, float max_norm, void* norm_out,
                              cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  launch_k(grad_clip_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev), max_norm,
                                                      reinterpret_cast<float*>(norm_out));
  return (int)cudaGetLastError();
}
