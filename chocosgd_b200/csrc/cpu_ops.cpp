// CPU twins of the packing / compression kernels: used on CPU (Gloo) ranks and as an
// independent oracle for the CUDA kernels.  Plain C ABI, OpenMP over words / segments.
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <numeric>
#include <vector>

#include "common.cuh"

extern "C" void cpu_sign_pack(const float* x, long long n, uint32_t* words) {
  const long long nw = (n + 31) / 32;
#pragma omp parallel for schedule(static)
  for (long long w = 0; w < nw; ++w) {
    uint32_t v = 0;
    const long long lim = std::min<long long>(32, n - w * 32);
    for (long long b = 0; b < lim; ++b) v |= (x[w * 32 + b] < 0.f ? 1u : 0u) << b;
    words[w] = v;
  }
}

extern "C" void cpu_sign_unpack(const uint32_t* words, long long n, float* out, float scale) {
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < n; ++i) out[i] = ((words[i >> 5] >> (i & 31)) & 1u) ? -scale : scale;
}

// k largest |x| of one tensor, ties to the lowest index, output ordered by index.
extern "C" void cpu_top_k(const float* x, int n, int k, int* idx_out, float* val_out) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  auto cmp = [&](int a, int b) {
    const float fa = fabsf(x[a]), fb = fabsf(x[b]);
    return fa > fb || (fa == fb && a < b);
  };
  if (k < n) std::nth_element(order.begin(), order.begin() + k, order.end(), cmp);
  std::sort(order.begin(), order.begin() + k);
  for (int i = 0; i < k; ++i) {
    idx_out[i] = order[i];
    val_out[i] = x[order[i]];
  }
}

extern "C" void cpu_random_k_indices(int n, int k, uint32_t seed, uint32_t step, uint32_t seg, int* idx_out) {
  uint32_t keys[4];
  for (uint32_t r = 0; r < 4; ++r) keys[r] = feistel_key(seed, step, seg, r);
  const int hb = feistel_half_bits((uint32_t)n);
  for (int j = 0; j < k; ++j) idx_out[j] = (int)feistel_perm((uint32_t)j, (uint32_t)n, hb, keys);
}

extern "C" void cpu_counter_uniform(uint32_t seed, uint32_t step, long long n, float* out) {
  const uint32_t base = uniform_base(seed, step);
  for (long long i = 0; i < n; ++i) out[i] = counter_uniform(base, (uint32_t)i);
}
