// Stem of the ImageNet ResNets: 7x7 / stride 2 / pad 3 convolution of a 3-channel image into 64 channels
// (dl_code/pcode/models/resnet.py:214-222), bf16 operands, fp32 accumulation in TMEM, tcgen05.mma kind::f16.
//
// A 6- or 12-byte pixel cannot be a TMA row, so the im2col tile is built by ordinary threads straight into
// the 128-byte-swizzled K-major layout that the tensor core reads:
//
//   K index   k = 24 r + 3 i + c,  r = 0..6 filter row, i = 0..7 window pixel, c = 0..2 channel.
//             The window of output pixel (ho, wo) starts at input pixel 2 wo - 4 (one pixel left of the
//             7-wide filter): it then starts on an even pixel, 24 floats = 12 aligned float2 loads, and
//             fills exactly three 16-byte chunks of bf16.  Window pixel i = 0 has zero weight.
//             K = 168, padded with one zero chunk to 176 = 11 MMAs of K = 16.
//   forward   D[pixel, co] = A[pixel, k] B[co, k]: M = 128 output pixels per tile, N = 64.  Persistent CTAs;
//             sixteen producer warps build tile t+1 while the tensor core works on tile t and four epilogue
//             warps write tile t-1 (TMEM -> bf16 -> shared staging -> one contiguous 16 KB block of y).
//             Optional per-CTA (sum, sum of squares) rows for the batch-norm that follows (the bf16
//             batch-norm does not take them yet: the Python side passes no buffer).
//   wgrad     D[co, k] = dy^T[co, pixel] P^T[k, pixel]: the pixel is the contraction index, so producers
//             write both operands TRANSPOSED (2-byte stores, consecutive lanes = consecutive pixels of one
//             row: conflict-free).  M = 128 (rows 64..127 stay zero), N = 176, one accumulator per CTA over
//             all its tiles, per-CTA slices added in index order by a second kernel (reproducible).
// The image is read as fp32 and rounded to bf16 on the way into the tile (what autocast's cast does); the
// input gradient is not needed.  Every mbarrier wait is bounded; a wait that runs out sets the error word
// and the CTA drains and frees its TMEM.
#include <cuda_bf16.h>
#include "launch.cuh"
#include "tc_common.cuh"

#define ST_THREADS 672        // warps 0-3 epilogue, 4-19 producers, 20 MMA issue
#define ST_PROD 512
#define ST_MMA_WARP (4 + ST_PROD / 32)
#define ST_K 176
#define ST_COUT 64

struct StemArgs {
  const float* x;              // [N, H, W, 3]
  const float* w;              // [64, 7, 7, 3]
  __nv_bfloat16* y;            // forward: [N, HO, WO, 64]
  const __nv_bfloat16* dy;     // wgrad:   [N, HO, WO, 64]
  float* stats;                // forward, optional: [grid][128]
  float* partial;              // wgrad: [grid][64][176]
  int* error;
  int N, H, W, HO, WO, n_tiles;
  long long P;                 // N HO WO
};

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 q = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&q);
}
__device__ __forceinline__ void st_epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool st_epi_bar_or(bool flag) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "r"((uint32_t)flag) : "memory");
  return r != 0;
}

// the 24 window floats of output pixel p under filter row r (zero outside the image)
struct StemPix {
  const float* base;   // address of window float 0 of filter row 0 (may lie outside the image: never dereferenced there)
  int h0, lo, hi;      // first input row; valid window floats are [lo, hi)
  bool valid;
};
__device__ __forceinline__ StemPix stem_pixel(const StemArgs& a, long long p) {
  StemPix s;
  s.valid = p < a.P;
  const long long pp = s.valid ? p : 0;
  const int wo = (int)(pp % a.WO);
  const int ho = (int)((pp / a.WO) % a.HO);
  const int n = (int)(pp / ((long long)a.WO * a.HO));
  const int w_start = 2 * wo - 4;
  s.h0 = 2 * ho - 3;
  s.lo = w_start < 0 ? -3 * w_start : 0;
  const int room = a.W - w_start;
  s.hi = 3 * (room < 8 ? room : 8);
  s.base = a.x + (((long long)n * a.H + s.h0) * a.W + w_start) * 3;
  return s;
}
__device__ __forceinline__ void stem_load_row(const StemArgs& a, const StemPix& s, int r, float2* v) {
  const int h = s.h0 + r;
  const bool hv = s.valid && h >= 0 && h < a.H;
  const float* src = s.base + (long long)r * a.W * 3;
#pragma unroll
  for (int i = 0; i < 12; ++i) {
    const bool in = hv && 2 * i >= s.lo && 2 * i < s.hi;
    v[i] = in ? __ldg(reinterpret_cast<const float2*>(src + 2 * i)) : make_float2(0.f, 0.f);
  }
}

struct StemSmem {
  static constexpr int A_SLAB = 128 * 128;            // forward: 128 pixel rows x 64 k
  static constexpr int A_BYTES = 3 * A_SLAB;
  static constexpr int B_SLAB = ST_COUT * 128;
  static constexpr int B_BYTES = 3 * B_SLAB;
  static constexpr int STAGE_ROW = 144;
  static constexpr int STAGE_BYTES = 128 * STAGE_ROW;
  static constexpr int FWD_BYTES = 2 * A_BYTES + B_BYTES + STAGE_BYTES + 256 + 1024;
  // wgrad: A = dy^T [128 rows (64 used)][128 pixels], B = patches^T [176 rows][128 pixels]
  static constexpr int WA_SLAB = 128 * 128;
  static constexpr int WA_BYTES = 2 * WA_SLAB;
  static constexpr int WB_SLAB = ST_K * 128;
  static constexpr int WB_BYTES = 2 * WB_SLAB;
  static constexpr int WG_BYTES = 2 * (WA_BYTES + WB_BYTES) + 256 + 1024;
};

__global__ void __launch_bounds__(ST_THREADS, 1) stem7_fwd_kernel(StemArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = StemSmem;
  uint8_t* sA = smem;                               // [2][A_BYTES]
  uint8_t* sB = sA + 2 * L::A_BYTES;                // [B_BYTES]
  uint8_t* sT = sB + L::B_BYTES;                    // [128][STAGE_ROW]
  uint64_t* full = reinterpret_cast<uint64_t*>(sT + L::STAGE_BYTES);   // [2]
  uint64_t* empty = full + 2;                       // [2]
  uint64_t* acc_full = empty + 2;                   // [2]
  uint64_t* acc_empty = acc_full + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(full + b, ST_PROD / 32);      // one arrival per producer warp
      mbar_init(empty + b, 1);
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  constexpr uint32_t TMEM_COLS = 128;         // two accumulators of 64 columns
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();
  pdl_trigger();
  // the filter as the B operand: row co, k = 24 r + 3 (s + 1) + c; everything else zero
  for (int i = threadIdx.x; i < L::B_BYTES / 16; i += ST_THREADS) reinterpret_cast<uint4*>(sB)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  for (int i = threadIdx.x; i < ST_COUT * 147; i += ST_THREADS) {
    const int co = i / 147, e = i % 147, r = e / 21, sc = e % 21;
    const int k = 24 * r + 3 + sc, q = k >> 3;
    const uint32_t off = (uint32_t)(q >> 3) * L::B_SLAB + co * 128 + (((q & 7) ^ (co & 7)) << 4) + (k & 7) * 2;
    *reinterpret_cast<__nv_bfloat16*>(sB + off) = __float2bfloat16(__ldg(a.w + i));
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 4 && warp < ST_MMA_WARP) {
    // ---- producers: thread = (pixel row of the tile, quarter: filter rows 2 q and 2 q + 1) ----------
    // both rows' 24 loads are issued before the first use: a producer's time per tile is one round trip
    const int pt = threadIdx.x - 128, row = pt & 127, quarter = pt >> 7;
    uint32_t lt = 0;
    int ok = 1;
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      // the loads do not depend on the slot: they are issued before the wait for it, so their latency runs
      // under the tensor core's and the epilogue's work on the two tiles before
      const StemPix s = stem_pixel(a, (long long)tile * 128 + row);
      float2 v[2][12];
      stem_load_row(a, s, 2 * quarter, v[0]);
      if (quarter < 3) stem_load_row(a, s, 2 * quarter + 1, v[1]);
      if (lane == 0) {
        if (lt >= 2 && !mbar_wait(empty + buf, ((lt >> 1) - 1) & 1)) ok = 0;
        if (*abort_flag) ok = 0;
        if (!ok) *abort_flag = 1;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      uint8_t* A = sA + buf * L::A_BYTES;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u == 1 && quarter == 3) break;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const int q = 3 * (2 * quarter + u) + j;
          const uint4 c = make_uint4(pack_bf16(v[u][4 * j].x, v[u][4 * j].y), pack_bf16(v[u][4 * j + 1].x, v[u][4 * j + 1].y),
                                     pack_bf16(v[u][4 * j + 2].x, v[u][4 * j + 2].y),
                                     pack_bf16(v[u][4 * j + 3].x, v[u][4 * j + 3].y));
          *reinterpret_cast<uint4*>(A + (q >> 3) * L::A_SLAB + row * 128 + (((q & 7) ^ (row & 7)) << 4)) = c;
        }
      }
      if (quarter == 3)   // chunk 21: the zero padding of K
        *reinterpret_cast<uint4*>(A + 2 * L::A_SLAB + row * 128 + ((5 ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full + buf);
    }
  } else if (warp == ST_MMA_WARP && lane == 0) {
    // ---- MMA issue ------------------------------------------------------------------------------------
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ST_COUT >> 3) << 17) | ((128u >> 4) << 24);
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      if (lt >= 2 && !mbar_wait(acc_empty + buf, ((lt >> 1) - 1) & 1)) { *abort_flag = 1; break; }
      if (!mbar_wait(full + buf, (lt >> 1) & 1)) { *abort_flag = 1; break; }
      tc_fence_after();
      const uint32_t d = tmem_base + buf * ST_COUT;
      const uint32_t a_addr = smem_u32(sA + buf * L::A_BYTES), b_addr = smem_u32(sB);
#pragma unroll
      for (int ks = 0; ks < ST_K / 16; ++ks)
        umma_bf16(d, make_desc(a_addr + (ks >> 2) * L::A_SLAB + (ks & 3) * 32, 16, 1024),
                  make_desc(b_addr + (ks >> 2) * L::B_SLAB + (ks & 3) * 32, 16, 1024), idesc, ks > 0 ? 1u : 0u);
      tc_commit(empty + buf);
      tc_commit(acc_full + buf);
    }
  } else if (warp < 4) {
    // ---- epilogue ---------------------------------------------------------------------------------------
    const int t128 = threadIdx.x;
    float s0[8], s1[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s0[e] = s1[e] = 0.f;
    uint32_t lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      const bool bad = !mbar_wait(acc_full + buf, (lt >> 1) & 1) || *abort_flag != 0;
      if (st_epi_bar_or(bad)) {
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      uint8_t* trow = sT + t128 * L::STAGE_ROW;
#pragma unroll
      for (int c = 0; c < ST_COUT; c += 16) {
        uint32_t v[16];
        tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * ST_COUT + (uint32_t)c, v);
        uint32_t h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = pack_bf16(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        *reinterpret_cast<uint4*>(trow + c * 2) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(trow + c * 2 + 16) = make_uint4(h[4], h[5], h[6], h[7]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buf);
      st_epi_bar();
      // the tile's 128 pixels are one contiguous 16 KB block of y: a linear, fully coalesced pass
      const long long p0 = (long long)tile * 128;
      const int rows = a.P - p0 < 128 ? (int)(a.P - p0) : 128;
      uint4* dst = reinterpret_cast<uint4*>(a.y + p0 * ST_COUT);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int q = t128 + 128 * j, row = q >> 3;
        if (row < rows) {
          const uint4 c = *reinterpret_cast<const uint4*>(sT + row * L::STAGE_ROW + (q & 7) * 16);
          dst[q] = c;
          if (a.stats != nullptr) {
            const uint32_t wv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float f0 = __uint_as_float(wv[e] << 16), f1 = __uint_as_float(wv[e] & 0xFFFF0000u);
              s0[2 * e] += f0; s0[2 * e + 1] += f1;
              s1[2 * e] = fmaf(f0, f0, s1[2 * e]); s1[2 * e + 1] = fmaf(f1, f1, s1[2 * e + 1]);
            }
          }
        }
      }
      // (the barrier at the top of the next iteration keeps the next tile's staging writes behind this pass)
    }
    if (a.stats != nullptr && ok) {
      // threads with the same t & 7 hold sums of the same eight channels: add the 16 of them in a fixed order
      st_epi_bar();
      float* red = reinterpret_cast<float*>(sT);     // [128][16]
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        red[t128 * 16 + e] = s0[e];
        red[t128 * 16 + 8 + e] = s1[e];
      }
      st_epi_bar();
      if (t128 < ST_COUT) {
        const int cg = t128 >> 3, e = t128 & 7;
        float a0 = 0.f, a1 = 0.f;
        for (int g = 0; g < 16; ++g) {
          a0 += red[(g * 8 + cg) * 16 + e];
          a1 += red[(g * 8 + cg) * 16 + 8 + e];
        }
        a.stats[(size_t)blockIdx.x * 2 * ST_COUT + t128] = a0;
        a.stats[(size_t)blockIdx.x * 2 * ST_COUT + ST_COUT + t128] = a1;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(a.error, 1);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

__global__ void __launch_bounds__(ST_THREADS, 1) stem7_wgrad_kernel(StemArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = StemSmem;
  uint8_t* sA = smem;                               // [2][WA_BYTES]
  uint8_t* sB = sA + 2 * L::WA_BYTES;               // [2][WB_BYTES]
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + 2 * L::WB_BYTES);   // [2]
  uint64_t* empty = full + 2;                       // [2]
  uint64_t* acc_full = empty + 2;                   // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(full + b, ST_PROD / 32);
      mbar_init(empty + b, 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  constexpr uint32_t TMEM_COLS = 256;         // 176 used
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // rows 64..127 of A and rows 168..175 of B are never written again: they stay zero
  for (int i = threadIdx.x; i < 2 * (L::WA_BYTES + L::WB_BYTES) / 16; i += ST_THREADS)
    reinterpret_cast<uint4*>(sA)[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_trigger();

  if (warp >= 4 && warp < ST_MMA_WARP) {
    // ---- producers: thread = (pixel column of the tile, quarter: 16 rows of dy^T, filter rows 2 q and 2 q + 1) ----
    const int pt = threadIdx.x - 128, col = pt & 127, quarter = pt >> 7;
    const uint32_t col_slab = col >> 6, col_chunk = (col & 63) >> 3, col_byte = (col & 7) * 2;
    uint32_t lt = 0;
    int ok = 1;
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      const long long p = (long long)tile * 128 + col;
      const StemPix s = stem_pixel(a, p);
      // every global load of the tile is issued before the wait for the slot and before the first store
      uint4 d[2];
#pragma unroll
      for (int j = 0; j < 2; ++j)
        d[j] = s.valid ? __ldg(reinterpret_cast<const uint4*>(a.dy + p * ST_COUT + quarter * 16 + j * 8)) : make_uint4(0, 0, 0, 0);
      float2 v[2][12];
      stem_load_row(a, s, 2 * quarter, v[0]);
      if (quarter < 3) stem_load_row(a, s, 2 * quarter + 1, v[1]);
      if (lane == 0) {
        if (lt >= 2 && !mbar_wait(empty + buf, ((lt >> 1) - 1) & 1)) ok = 0;
        if (*abort_flag) ok = 0;
        if (!ok) *abort_flag = 1;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      uint8_t* A = sA + buf * L::WA_BYTES + col_slab * L::WA_SLAB + col_byte;
      uint8_t* B = sB + buf * L::WB_BYTES + col_slab * L::WB_SLAB + col_byte;
      // dy^T: rows co = 16 q .. 16 q + 15
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t wv[4] = {d[j].x, d[j].y, d[j].z, d[j].w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t row = quarter * 16 + j * 8 + e;
          const uint16_t hv = (uint16_t)((e & 1) ? (wv[e >> 1] >> 16) : (wv[e >> 1] & 0xFFFFu));
          *reinterpret_cast<uint16_t*>(A + row * 128 + ((col_chunk ^ (row & 7)) << 4)) = hv;
        }
      }
      // patches^T: rows 24 r + e
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u == 1 && quarter == 3) break;
        const int r = 2 * quarter + u;
#pragma unroll
        for (int i = 0; i < 12; ++i) {
          const uint32_t w2 = pack_bf16(v[u][i].x, v[u][i].y);
          const uint32_t row0 = 24 * r + 2 * i, row1 = row0 + 1;
          *reinterpret_cast<uint16_t*>(B + row0 * 128 + ((col_chunk ^ (row0 & 7)) << 4)) = (uint16_t)(w2 & 0xFFFFu);
          *reinterpret_cast<uint16_t*>(B + row1 * 128 + ((col_chunk ^ (row1 & 7)) << 4)) = (uint16_t)(w2 >> 16);
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full + buf);
    }
  } else if (warp == ST_MMA_WARP && lane == 0) {
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ST_K >> 3) << 17) | ((128u >> 4) << 24);
    uint32_t lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      if (!mbar_wait(full + buf, (lt >> 1) & 1)) { *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      const uint32_t a_addr = smem_u32(sA + buf * L::WA_BYTES), b_addr = smem_u32(sB + buf * L::WB_BYTES);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16(tmem_base, make_desc(a_addr + (ks >> 2) * L::WA_SLAB + (ks & 3) * 32, 16, 1024),
                  make_desc(b_addr + (ks >> 2) * L::WB_SLAB + (ks & 3) * 32, 16, 1024), idesc, (lt > 0 || ks > 0) ? 1u : 0u);
      tc_commit(empty + buf);
    }
    if (ok) tc_commit(acc_full);
  } else if (warp < 2 && blockIdx.x < a.n_tiles) {
    // ---- epilogue: rows co = 0..63 of the accumulator -> this CTA's slice ----------------------------------
    if (!mbar_wait(acc_full, 0) || *abort_flag != 0) {
      *abort_flag = 1;
    } else {
      tc_fence_after();
      float* dst = a.partial + ((size_t)blockIdx.x * ST_COUT + threadIdx.x) * ST_K;
#pragma unroll 1
      for (int c = 0; c < ST_K; c += 16) {
        uint32_t v[16];
        tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c, v);
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4*>(dst + c + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(a.error, 1);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// dw[co][r][s][c] = sum over slices, in index order, of slice[co][24 r + 3 (s + 1) + c]
__global__ void __launch_bounds__(256) stem7_wgrad_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                                                 int parts) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= ST_COUT * 147) return;
  const int co = i / 147, e = i % 147, r = e / 21, sc = e % 21;
  const float* src = partial + (size_t)co * ST_K + 24 * r + 3 + sc;
  // eight independent loads per trip, added in slice order
  float acc = 0.f;
  int g = 0;
  for (; g + 7 < parts; g += 8) {
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = __ldcg(src + (size_t)(g + q) * ST_COUT * ST_K);
#pragma unroll
    for (int q = 0; q < 8; ++q) acc += v[q];
  }
  for (; g < parts; ++g) acc += __ldcg(src + (size_t)g * ST_COUT * ST_K);
  dw[i] = acc;
}

static int* stem_error_word() {
  static int* err = nullptr;
  if (err == nullptr) {
    if (cudaMalloc(&err, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(err, 0, sizeof(int));
  }
  return err;
}

extern "C" int conv_stem_supported(int N, int H, int W, int Cin, int Cout) {
  return Cin == 3 && Cout == ST_COUT && N >= 1 && H >= 8 && W >= 8 && W % 2 == 0 && H % 2 == 0;
}

// CTAs of both kernels (rows of the statistics partials, slices of the weight gradient)
extern "C" int conv_stem_grid(int N, int H, int W) {
  const long long P = (long long)N * (H / 2) * (W / 2);
  const long long tiles = (P + 127) / 128;
  return (int)(tiles < sm_count() ? tiles : sm_count());
}

// 1 when a bounded wait of one of the kernels ran out since the last call (the word is cleared)
extern "C" int conv_stem_last_error() {
  int* err = stem_error_word();
  if (err == nullptr) return -1;
  int h = 0;
  if (cudaMemcpy(&h, err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (h != 0) cudaMemset(err, 0, sizeof(int));
  return h;
}

static int stem_fill(StemArgs& a, int N, int H, int W) {
  a.N = N; a.H = H; a.W = W; a.HO = H / 2; a.WO = W / 2;
  a.P = (long long)N * a.HO * a.WO;
  a.n_tiles = (int)((a.P + 127) / 128);
  a.error = stem_error_word();
  return a.error == nullptr ? -2 : 0;
}

extern "C" int conv_stem_forward(const void* x, const void* w, void* y, void* stats, int N, int H, int W, cudaStream_t st) {
  if (!conv_stem_supported(N, H, W, 3, ST_COUT)) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 7) != 0 || (reinterpret_cast<uintptr_t>(y) & 15) != 0) return -1;
  StemArgs a = {};
  a.x = reinterpret_cast<const float*>(x);
  a.w = reinterpret_cast<const float*>(w);
  a.y = reinterpret_cast<__nv_bfloat16*>(y);
  a.stats = reinterpret_cast<float*>(stats);
  if (int rc = stem_fill(a, N, H, W)) return rc;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(stem7_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, StemSmem::FWD_BYTES) != cudaSuccess)
      return -3;
    attr = true;
  }
  launch_k(stem7_fwd_kernel, dim3(conv_stem_grid(N, H, W)), dim3(ST_THREADS), StemSmem::FWD_BYTES, st, a);
  return (int)cudaGetLastError();
}

// scratch: conv_stem_grid() * 64 * 176 floats
extern "C" int conv_stem_wgrad(const void* x, const void* dy, void* dw, void* scratch, int N, int H, int W, cudaStream_t st) {
  if (!conv_stem_supported(N, H, W, 3, ST_COUT)) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 7) != 0 || (reinterpret_cast<uintptr_t>(dy) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(scratch) & 15) != 0)
    return -1;
  StemArgs a = {};
  a.x = reinterpret_cast<const float*>(x);
  a.dy = reinterpret_cast<const __nv_bfloat16*>(dy);
  a.partial = reinterpret_cast<float*>(scratch);
  if (int rc = stem_fill(a, N, H, W)) return rc;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(stem7_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, StemSmem::WG_BYTES) != cudaSuccess)
      return -3;
    attr = true;
  }
  const int grid = conv_stem_grid(N, H, W);
  launch_k(stem7_wgrad_kernel, dim3(grid), dim3(ST_THREADS), StemSmem::WG_BYTES, st, a);
  launch_k(stem7_wgrad_reduce_kernel, dim3((ST_COUT * 147 + 255) / 256), dim3(256), 0, st,
           reinterpret_cast<const float*>(scratch), reinterpret_cast<float*>(dw), grid);
  return (int)cudaGetLastError();
}
