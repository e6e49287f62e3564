// Argument block shared by the fp32 (bn_nhwc.cu) and bf16 (bn_nhwc_bf16.cu) batch-norm kernels; mirrored by a
// ctypes.Structure (ops/bn.py).  In the bf16 kernels x, dy, y, residual, out and out2 point to bf16 data;
// statistics, gamma / beta and their gradients are fp32 in both.
#pragma once

struct BnArgs {
  const float* x;        // [P, C]
  const float* dy;       // backward: upstream gradient
  const float* y;        // backward: forward output (ReLU mask)
  const float* residual; // forward: optional
  const float* gamma;
  const float* beta;
  float* out;            // forward: y ; backward: dx
  float* out2;           // backward: dresidual (optional)
  float* mean;           // [C] batch mean (saved)
  float* invstd;         // [C] 1/sqrt(var + eps) (saved)
  float* running_mean;   // optional
  float* running_var;    // optional
  float* dgamma;         // [C]
  float* dbeta;          // [C]
  float* partial;        // [grid][2 C] scratch
  unsigned* counter;     // arrival counter (self-resetting)
  int P, C, relu;
  float eps, momentum;
  int n_partials;        // G: CTAs of the reduction kernel (set by the launcher)
  int fused_finalize;    // 1: the elementwise kernel adds the partials (set by the launcher)
};

