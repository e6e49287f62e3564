// Device-side decoders of the dense wire formats, shared by the CHOCO kernels and the kernels
// of the other algorithms.
//   QSGD   per 32-position group: nbits level planes + one sign plane (bit-sliced words)
//   sign   one bit per position (set = negative), magnitude ||v_seg||_1 / n_seg from the header
#pragma once
#include "common.cuh"

__device__ __forceinline__ float qsgd_scale_of(int n, int s, int biased) {
  if (!biased) return 1.f;
  const float a = (float)n / ((float)s * (float)s), b = sqrtf((float)n) / (float)s;
  return 1.f / (fminf(a, b) + 1.f);
}

// value of element `bit` of a 32-position group given its plane words
__device__ __forceinline__ float qsgd_value(const uint32_t* planes, int nbits, int bit, float unit) {
  uint32_t lv = 0;
  for (int b = 0; b < nbits; ++b) lv |= ((planes[b] >> bit) & 1u) << b;
  const float mag = unit * (float)lv;
  return ((planes[nbits] >> bit) & 1u) ? -mag : mag;
}

// Decode 4 consecutive positions of one group and accumulate  acc[e] += unit * level * sign.
// Up to 8 plane words (nbits <= 7) stay in registers (fully unrolled, predicated loads).
__device__ __forceinline__ void qsgd_accumulate4(const uint32_t* __restrict__ src, int nbits, int bit0, int n_valid,
                                                 float unit, float* acc, float* acc2, float w2) {
  if (nbits <= 7) {
    // The four positions' bits of one plane are a nibble; multiplying it by 0x00204081 and masking
    // with 0x01010101 drops bit e into byte e, so the four levels are assembled side by side in
    // one register with a handful of operations per plane (not per plane and position).
    uint32_t levels = 0, sgn = 0;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (b <= nbits) {
        const uint32_t nib = (__ldcg(src + b) >> bit0) & 0xFu;
        if (b < nbits) levels |= ((nib * 0x00204081u) & 0x01010101u) << b;
        else sgn = nib;
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (e < n_valid) {
        float q = unit * (float)((levels >> (8 * e)) & 0xFFu);
        q = ((sgn >> e) & 1u) ? -q : q;
        acc[e] += q;
        if (acc2 != nullptr) acc2[e] += w2 * q;
      }
    }
  } else {
    uint32_t planes[33];
    for (int b = 0; b <= nbits; ++b) planes[b] = __ldcg(src + b);
    for (int e = 0; e < 4; ++e)
      if (e < n_valid) {
        const float q = qsgd_value(planes, nbits, bit0 + e, unit);
        acc[e] += q;
        if (acc2 != nullptr) acc2[e] += w2 * q;
      }
  }
}


// sign codec: accumulate the 4 positions starting at bit `bit0` of `word`
__device__ __forceinline__ void sign_accumulate4(uint32_t word, int bit0, int n_valid, float mag, float* acc) {
#pragma unroll
  for (int e = 0; e < 4; ++e)
    if (e < n_valid) acc[e] += ((word >> (bit0 + e)) & 1u) ? -mag : mag;
}
