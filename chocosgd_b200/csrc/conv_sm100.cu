// 3x3 / stride 1 / pad 1 convolution as an implicit GEMM on tcgen05 tensor cores, NHWC fp32 (TF32).
//
//   y[n,h,w,:] = sum_{r,s} x[n, h+r-1, w+s-1, :] . W[:, r, s, :]^T        M = N H W, N = C_out, K = 9 C_in
//
// The im2col matrix is never built.  A CTA owns 128 consecutive output pixels (TW x TH x TN
// box of the image tensor); for each of the 9 filter taps and each block of KC <= 32 input
// channels ONE 4-d TMA load fetches the shifted activation tile straight from the NHWC tensor
// (coordinates may run outside the image: TMA fills zeros, which is exactly the padding) and
// one 2-d TMA load fetches the matching [C_out, KC] slice of the KRSC weight tensor.  Both
// land K-major with a 64- or 128-byte swizzle, a single thread issues tcgen05.mma
// (M = 128, N = C_out, K = 8 per instruction), the accumulator stays in TMEM across all
// 9 C_in / KC blocks, and the epilogue writes 128 NHWC output rows.
//
// The input gradient of such a convolution is the same operation applied to dy with the
// filter flipped and its channel roles exchanged (conv_flip_weights), so one kernel serves
// forward and dgrad.  Bounded mbarrier waits as in the GEMM kernel; no cluster multicast.
// Two kernels follow: the one-tile-per-CTA form and the persistent form (default) further down.
#include "tc_common.cuh"
#include "launch.cuh"
#include <stdlib.h>

#define CONV_THREADS 192
#define CONV_STAGES 6

struct ConvArgs {
  float* y;        // [N*H*W, C_out]
  int* error;
  int H, W, Cin;
  int TH, TN;      // tile: W x TH x TN = 128 pixels
  int tiles_h;     // H / TH
  int relu;
};

template <int COUT, int KC>
__global__ void __launch_bounds__(CONV_THREADS, 1)
conv3x3_tf32_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, ConvArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int ROW = KC * 4;                  // bytes per K-major row: 64 or 128
  constexpr int A_BYTES = 128 * ROW;
  constexpr int B_BYTES = COUT * ROW;
  constexpr uint32_t LAYOUT = ROW == 128 ? 2u : 4u;   // 128-byte / 64-byte swizzle
  constexpr uint32_t SBO = 8 * ROW;                   // 8 rows
  uint8_t* sA = smem;
  uint8_t* sB = smem + CONV_STAGES * A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + CONV_STAGES * B_BYTES);
  uint64_t* empty = full + CONV_STAGES;
  uint64_t* acc_ready = empty + CONV_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x;
  const int n0 = (tile / g.tiles_h) * g.TN, h0 = (tile % g.tiles_h) * g.TH;
  const int cblocks = g.Cin / KC;
  const int n_kb = 9 * cblocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < CONV_STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_ready, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  constexpr uint32_t TMEM_COLS = COUT < 32 ? 32 : COUT;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // set-up above touched shared memory and TMEM only
  pdl_trigger();

  if (warp == 4 && lane == 0) {
    for (int i = 0; i < n_kb; ++i) {
      const int s = i % CONV_STAGES;
      if (i >= CONV_STAGES && !mbar_wait(empty + s, ((i / CONV_STAGES) - 1) & 1)) { *abort_flag = 1; break; }
      if (*abort_flag) break;
      const int tap = i / cblocks, c0 = (i % cblocks) * KC;
      const int r = tap / 3, t = tap % 3;
      mbar_expect_tx(full + s, A_BYTES + B_BYTES);
      // the channel coordinate is a multiple of 16 elements: 16-byte aligned as TMA requires
      tma_load_4d(sA + s * A_BYTES, &map_x, full + s, c0, t - 1, h0 + r - 1, n0);
      tma_load_2d(sB + s * B_BYTES, &map_w, full + s, tap * g.Cin + c0, 0);
    }
  } else if (warp == 5 && lane == 0) {
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(COUT >> 3) << 17) | ((128u >> 4) << 24);
    bool ok = true;
    for (int i = 0; i < n_kb && ok; ++i) {
      const int s = i % CONV_STAGES;
      if (!mbar_wait(full + s, (i / CONV_STAGES) & 1)) { *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      const uint32_t a_addr = smem_u32(sA + s * A_BYTES), b_addr = smem_u32(sB + s * B_BYTES);
#pragma unroll
      for (int k = 0; k < KC / 8; ++k)
        umma_tf32(tmem_base, make_desc(a_addr + k * 32, 16, SBO, LAYOUT), make_desc(b_addr + k * 32, 16, SBO, LAYOUT),
                  idesc, (i > 0 || k > 0) ? 1u : 0u);
      tc_commit(empty + s);
    }
    if (ok) tc_commit(acc_ready);
  } else if (warp < 4) {
    bool ok = mbar_wait(acc_ready, 0);
    if (!ok) *abort_flag = 1;
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      // the tile's 128 pixels are consecutive rows of the [N*H*W, C_out] output
      const size_t pix = ((size_t)n0 * g.H + h0) * g.W + warp * 32 + lane;
      float* out = g.y + pix * COUT;
#pragma unroll 1
      for (int c = 0; c < COUT; c += 16) {
        uint32_t v[16];
        tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c, v);
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                 __uint_as_float(v[j + 3]));
          if (g.relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
          *reinterpret_cast<float4*>(out + c + j) = o;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(g.error, 1);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- persistent variant ---------------------------------------------------------------------------
// One CTA per SM walks over several 128-pixel tiles.  The TMA producer keeps running ahead across
// tile boundaries, the accumulator is double-buffered in TMEM (tile t+1 is multiplied while the
// epilogue warps drain tile t), and the epilogue can also produce the per-channel sum and sum of
// squares of everything the CTA wrote - the batch-norm statistics of the layer that follows - as
// ONE row [2 C_out] of partials per CTA, added in a fixed order (reproducible).  The batch-norm
// forward then needs no reduction pass over the activation tensor.
struct ConvPArgs {
  float* y;        // [N*H*W, C_out]
  float* stats;    // optional [gridDim.x][2 C_out]: sum, sum of squares per channel
  // backward epilogue (BWD kernels): result = (acc + add) * [mask > 0]; with bnx the two statistics
  // become sum(result) and sum(result * (bnx - bn_mean) * bn_invstd), the batch-norm backward sums
  const float* add;        // optional [N*H*W, C_out]
  const float* mask;       // optional [N*H*W, C_out]
  const float* bnx;        // optional [N*H*W, C_out]
  const float* bn_mean;    // [C_out]
  const float* bn_invstd;  // [C_out]
  int* error;
  int H, W, Cin;    // H, W: OUTPUT height and width (the tiles are tiles of the output)
  int TH, TN;
  int tiles_h;
  int n_tiles;
  int relu;
  int taps;         // 9 (3x3, pad 1) or 1 (1x1, pad 0)
  int stride;       // 1 or 2: the input tensor map then loads every second pixel of a twice as large box
  // mode 1: input gradient of a 3x3 / stride 2 / pad 1 convolution (plus, optionally, of the 1x1 / stride 2
  // shortcut that reads the same tensor).  The result [N, 2H, 2W, C_out] is produced as four parity
  // classes (row parity, column parity) of H x W pixels each; H, W, TH, TN, tiles_h describe ONE class,
  // which has the geometry of dy.  A result pixel (2a + ph, 2b + pw) receives the filter taps (r, s) with
  // r = 1 for ph = 0 and r in {0, 2} for ph = 1 (same for s / pw), each reading dy at (a + (ph + 1 - r) / 2,
  // b + (pw + 1 - s) / 2): unit-stride boxes of dy, 1 / 2 / 2 / 4 taps for the four classes.
  int mode;
  int cb2;              // k-blocks of the shortcut's dy (class 0 only); 0 = no shortcut
  int tiles_per_class;
};

// k-blocks (filter tap x KC-channel block) of a tile of parity class cls in mode 1
__device__ __forceinline__ int s2_n_kb(int cls, int cblocks, int cb2) {
  const int nt = ((cls >> 1) ? 2 : 1) * ((cls & 1) ? 2 : 1);
  return nt * cblocks + (cls == 0 ? cb2 : 0);
}

// One CTA per SM has a single MMA-issuing thread and a single barrier round trip per pipeline
// slot, so a slot holds GK k-blocks (all 9 filter taps for 16 channels, 3 otherwise): one wait,
// 2 GK .. 4 GK tensor-core instructions, one commit.  GK lanes of the producer warp issue the
// loads of a slot in parallel.  As many slots as fit beside the epilogue tile in ~200 KB.
template <int COUT, int KC, bool BWD = false>
struct ConvPCfg {
  static constexpr int TSTRIDE = COUT + 4;  // floats per row of the epilogue tile (bank-conflict free)
  static constexpr int KB_BYTES = 128 * KC * 4 + COUT * KC * 4;
  static constexpr int TILES = 1;            // one shared tile for the epilogue (forward and backward form)
  static constexpr int ROOM = 200 * 1024 - TILES * 128 * TSTRIDE * 4;
#ifndef CONV_GK_MAX
#define CONV_GK_MAX 9
#endif
  static constexpr int GK = (CONV_GK_MAX >= 9 && 2 * 9 * KB_BYTES <= ROOM) ? 9 : (2 * 3 * KB_BYTES <= ROOM ? 3 : 1);
  static constexpr int FIT = ROOM / (GK * KB_BYTES);
  static constexpr int STAGES = FIT > 8 ? 8 : (FIT < 2 ? 2 : FIT);
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// barrier of the 128 epilogue threads that also ORs a flag: every thread gets the same answer
__device__ __forceinline__ bool epi_bar_or(bool flag) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "r"((uint32_t)flag) : "memory");
  return r != 0;
}

template <int COUT, int KC, bool BWD>
__global__ void __launch_bounds__(CONV_THREADS, 1)
conv3x3_persist_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ CUtensorMap map_x2, const __grid_constant__ CUtensorMap map_w2, ConvPArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using Cfg = ConvPCfg<COUT, KC, BWD>;
  constexpr int S = Cfg::STAGES, TS = Cfg::TSTRIDE, GK = Cfg::GK;
  constexpr int ROW = KC * 4;
  constexpr int A_BYTES = 128 * ROW;
  constexpr int B_BYTES = COUT * ROW;
  constexpr uint32_t LAYOUT = ROW == 128 ? 2u : 4u;
  constexpr uint32_t SBO = 8 * ROW;
  uint8_t* sA = smem;                          // [S][GK][A_BYTES]
  uint8_t* sB = smem + S * GK * A_BYTES;        // [S][GK][B_BYTES]
  float* sT = reinterpret_cast<float*>(sB + S * GK * B_BYTES);     // [128][TS] epilogue tile
  uint64_t* full = reinterpret_cast<uint64_t*>(sT + Cfg::TILES * 128 * TS);
  uint64_t* empty = full + S;
  uint64_t* acc_full = empty + S;    // [2]
  uint64_t* acc_empty = acc_full + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cblocks = g.Cin / KC;
  const int n_kb0 = g.taps * cblocks;           // k-blocks per tile (mode 0); a pipeline slot holds up to GK of them
  const int pad = g.taps == 9 ? 1 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, 4);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  constexpr uint32_t TMEM_COLS = 2 * COUT < 32 ? 32 : 2 * COUT;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // set-up above touched shared memory and TMEM only
  pdl_trigger();

  if (warp == 4) {
    uint32_t it = 0;
    int ok = 1;
    for (int tile = blockIdx.x; tile < g.n_tiles && ok; tile += gridDim.x) {
      const int cls = g.mode ? tile / g.tiles_per_class : 0;
      const int sub = g.mode ? tile % g.tiles_per_class : tile;
      const int n0 = (sub / g.tiles_h) * g.TN, h0 = (sub % g.tiles_h) * g.TH;
      const int n_kb = g.mode ? s2_n_kb(cls, cblocks, g.cb2) : n_kb0;
      for (int g0 = 0; g0 < n_kb; g0 += GK, ++it) {
        const uint32_t s = it % S;
        const int cnt = n_kb - g0 < GK ? n_kb - g0 : GK;
        if (lane == 0) {
          if (it >= (uint32_t)S && !mbar_wait(empty + s, ((it / S) - 1) & 1)) ok = 0;
          if (*abort_flag) ok = 0;
          if (ok) mbar_expect_tx(full + s, cnt * (A_BYTES + B_BYTES));
          else *abort_flag = 1;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (lane < cnt) {
          const int i = g0 + lane;
          uint8_t* dA = sA + (s * GK + lane) * A_BYTES;
          uint8_t* dB = sB + (s * GK + lane) * B_BYTES;
          if (!g.mode) {
            const int tap = i / cblocks, c0 = (i % cblocks) * KC;
            const int r = g.taps == 9 ? tap / 3 : 0, t = g.taps == 9 ? tap % 3 : 0;
            // input coordinates of the tile's first output pixel under filter tap (r, t); with stride 2
            // the box covers 2 W x 2 TH input pixels of which the map's element strides keep every second
            tma_load_4d(dA, &map_x, full + s, c0, t - pad, g.stride * h0 + r - pad, n0);
            tma_load_2d(dB, &map_w, full + s, tap * g.Cin + c0, 0);
          } else {
            const int ph = cls >> 1, pw = cls & 1;
            const int nts = pw ? 2 : 1, n_main = (ph ? 2 : 1) * nts * cblocks;
            if (i < n_main) {
              const int ti = i / cblocks, c0 = (i % cblocks) * KC;
              const int r = ph ? ((ti / nts) ? 2 : 0) : 1, t = pw ? ((ti % nts) ? 2 : 0) : 1;
              tma_load_4d(dA, &map_x, full + s, c0, (pw + 1 - t) >> 1, h0 + ((ph + 1 - r) >> 1), n0);
              // the flipped filter holds forward tap (r, t) at index 8 - (3 r + t)
              tma_load_2d(dB, &map_w, full + s, (8 - (3 * r + t)) * g.Cin + c0, 0);
            } else {
              const int c0 = (i - n_main) * KC;      // the shortcut: a 1x1 filter, class (0, 0) only
              tma_load_4d(dA, &map_x2, full + s, c0, 0, h0, n0);
              tma_load_2d(dB, &map_w2, full + s, c0, 0);
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 5 && lane == 0) {
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(COUT >> 3) << 17) | ((128u >> 4) << 24);
    uint32_t it = 0, lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < g.n_tiles && ok; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      if (lt >= 2 && !mbar_wait(acc_empty + buf, ((lt >> 1) - 1) & 1)) { *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      const uint32_t d = tmem_base + buf * COUT;
      const int n_kb = g.mode ? s2_n_kb(tile / g.tiles_per_class, cblocks, g.cb2) : n_kb0;
      for (int g0 = 0; g0 < n_kb; g0 += GK, ++it) {
        const uint32_t s = it % S;
        const int cnt = n_kb - g0 < GK ? n_kb - g0 : GK;
        if (!mbar_wait(full + s, (it / S) & 1)) { *abort_flag = 1; ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < GK; ++j) {
          if (j >= cnt) break;
          const uint32_t a_addr = smem_u32(sA + (s * GK + j) * A_BYTES), b_addr = smem_u32(sB + (s * GK + j) * B_BYTES);
#pragma unroll
          for (int k = 0; k < KC / 8; ++k)
            umma_tf32(d, make_desc(a_addr + k * 32, 16, SBO, LAYOUT), make_desc(b_addr + k * 32, 16, SBO, LAYOUT), idesc,
                      (g0 > 0 || j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(empty + s);
      }
      if (ok) tc_commit(acc_full + buf);
    }
  } else if (warp < 4) {
    const int t128 = threadIdx.x;                 // 0..127
    // Epilogue in two steps.  (1) The accumulator goes TMEM -> registers -> shared tile, one pixel row
    // per thread (padded rows: conflict-free).  (2) The 128 threads walk the tile linearly: a tile's 128
    // pixels are consecutive rows of the [N H W, C_out] tensors, i.e. ONE contiguous block of memory, so
    // every global load (skip gradient, ReLU mask, batch-norm input) and the store of the result is
    // fully coalesced.  In that pass a thread always meets the same four channels, so the two
    // per-channel statistics accumulate in registers across rows and tiles.
    constexpr int C4 = COUT / 4;           // float4 columns of a row
    constexpr int RSTEP = 128 / C4;        // rows covered by one sweep of the 128 threads
    const int c4 = t128 % C4, r0 = t128 / C4;
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    float mu[4] = {0.f, 0.f, 0.f, 0.f}, is[4] = {0.f, 0.f, 0.f, 0.f};
    if (BWD && g.bnx != nullptr) {
      const float4 m4 = *reinterpret_cast<const float4*>(g.bn_mean + c4 * 4);
      const float4 i4 = *reinterpret_cast<const float4*>(g.bn_invstd + c4 * 4);
      mu[0] = m4.x; mu[1] = m4.y; mu[2] = m4.z; mu[3] = m4.w;
      is[0] = i4.x; is[1] = i4.y; is[2] = i4.z; is[3] = i4.w;
    }
    uint32_t lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < g.n_tiles; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      const bool bad = !mbar_wait(acc_full + buf, (lt >> 1) & 1) || *abort_flag != 0;
      if (epi_bar_or(bad)) {                       // the same decision in all 128 epilogue threads
        *abort_flag = 1;                           // (also orders the previous tile's linear pass before this write)
        ok = false;
        break;
      }
      tc_fence_after();
      const int cls = g.mode ? tile / g.tiles_per_class : 0;
      const int sub = g.mode ? tile % g.tiles_per_class : tile;
      const int n0 = (sub / g.tiles_h) * g.TN, h0 = (sub % g.tiles_h) * g.TH;
      const size_t tile_off = (((size_t)n0 * g.H + h0) * g.W) * COUT;   // first float of the tile (mode 0)
      float* trow = sT + t128 * TS;
#pragma unroll 1
      for (int c = 0; c < COUT; c += 16) {
        uint32_t v[16];
        tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * COUT + (uint32_t)c, v);
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4*>(trow + c + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                 __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
      // the accumulator buffer may be overwritten by the tile after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buf);
      epi_bar();
      const bool want_stats = g.stats != nullptr;
      // four rows per trip: all their global loads are issued before the first use (the 128 epilogue
      // threads of an SM are few, so the pass lives on memory-level parallelism)
      constexpr int UN = (128 / RSTEP) >= 4 ? 4 : (128 / RSTEP);
#pragma unroll 1
      for (int rb = r0; rb < 128; rb += UN * RSTEP) {
        float4 o[UN], ra[UN], rm[UN], rx[UN];
        size_t off[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int row = rb + u * RSTEP;
          if (!g.mode) {
            off[u] = tile_off + (size_t)row * COUT + c4 * 4;
          } else {
            // row -> pixel (n, a, b) of the class image -> pixel (2a + ph, 2b + pw) of the result
            const int b = row % g.W, a = (row / g.W) % g.TH, nn = row / (g.W * g.TH);
            off[u] = ((((size_t)(n0 + nn) * (2 * g.H) + 2 * (h0 + a) + (cls >> 1)) * (2 * g.W)) + 2 * b + (cls & 1)) * COUT +
                     c4 * 4;
          }
          if (BWD) {
            if (g.add != nullptr) ra[u] = __ldg(reinterpret_cast<const float4*>(g.add + off[u]));
            if (g.mask != nullptr) rm[u] = __ldg(reinterpret_cast<const float4*>(g.mask + off[u]));
            if (want_stats) rx[u] = __ldg(reinterpret_cast<const float4*>(g.bnx + off[u]));
          }
          o[u] = *reinterpret_cast<const float4*>(sT + row * TS + c4 * 4);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          float4 v = o[u];
          if (BWD) {
            if (g.add != nullptr) { v.x += ra[u].x; v.y += ra[u].y; v.z += ra[u].z; v.w += ra[u].w; }
            if (g.mask != nullptr) {
              v.x = rm[u].x > 0.f ? v.x : 0.f; v.y = rm[u].y > 0.f ? v.y : 0.f;
              v.z = rm[u].z > 0.f ? v.z : 0.f; v.w = rm[u].w > 0.f ? v.w : 0.f;
            }
            if (want_stats) {
              s0[0] += v.x; s0[1] += v.y; s0[2] += v.z; s0[3] += v.w;
              s1[0] = fmaf(v.x, (rx[u].x - mu[0]) * is[0], s1[0]);
              s1[1] = fmaf(v.y, (rx[u].y - mu[1]) * is[1], s1[1]);
              s1[2] = fmaf(v.z, (rx[u].z - mu[2]) * is[2], s1[2]);
              s1[3] = fmaf(v.w, (rx[u].w - mu[3]) * is[3], s1[3]);
            }
          } else {
            if (g.relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
            if (want_stats) {
              s0[0] += v.x; s0[1] += v.y; s0[2] += v.z; s0[3] += v.w;
              s1[0] = fmaf(v.x, v.x, s1[0]); s1[1] = fmaf(v.y, v.y, s1[1]);
              s1[2] = fmaf(v.z, v.z, s1[2]); s1[3] = fmaf(v.w, v.w, s1[3]);
            }
          }
          *reinterpret_cast<float4*>(g.y + off[u]) = v;
        }
      }
      // (the barrier at the top of the next iteration keeps the next tile's writes to the shared tile
      // behind this pass)
    }
    if (g.stats != nullptr && ok) {
      // threads r0 = 0 .. RSTEP-1 hold partial sums of the same four channels: add them in a fixed order
      epi_bar();
      float* red = sT;                               // [RSTEP][C4][8]
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        red[(r0 * C4 + c4) * 8 + e] = s0[e];
        red[(r0 * C4 + c4) * 8 + 4 + e] = s1[e];
      }
      epi_bar();
      if (t128 < COUT) {
        const int cc4 = t128 / 4, e = t128 % 4;
        float a0 = 0.f, a1 = 0.f;
        for (int r = 0; r < RSTEP; ++r) {
          a0 += red[(r * C4 + cc4) * 8 + e];
          a1 += red[(r * C4 + cc4) * 8 + 4 + e];
        }
        g.stats[(size_t)blockIdx.x * 2 * COUT + t128] = a0;
        g.stats[(size_t)blockIdx.x * 2 * COUT + COUT + t128] = a1;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(g.error, 1);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// W'[ci, r, s, co] = W[co, 2 - r, 2 - s, ci]   (both KRSC): the filter of the input-gradient convolution
__global__ void conv_flip_weights_kernel(const float* __restrict__ w, float* __restrict__ out, int cout, int cin) {
  pdl_wait();
  pdl_trigger();
  const int total = cout * 9 * cin;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int co = i % cout, tap = (i / cout) % 9, ci = i / (9 * cout);
    out[i] = w[(co * 9 + (8 - tap)) * cin + ci];
  }
}

// all registered layers in one launch: table[l] = {w, out, cout, cin, taps}; gridDim.y = layer
// (taps = 9: 3x3 filters; taps = 1: a 1x1 filter, i.e. a plain transpose)
struct FlipEntry {
  const float* w;
  float* out;
  int cout, cin, taps, pad_;
};

__global__ void conv_flip_weights_multi_kernel(const FlipEntry* __restrict__ table) {
  pdl_wait();
  pdl_trigger();
  const FlipEntry e = table[blockIdx.y];
  const int total = e.cout * e.taps * e.cin;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int co = i % e.cout, tap = (i / e.cout) % e.taps, ci = i / (e.taps * e.cout);
    e.out[i] = e.w[(co * e.taps + (e.taps - 1 - tap)) * e.cin + ci];
  }
}

extern "C" int conv_flip_entry_size() { return (int)sizeof(FlipEntry); }

extern "C" int conv_flip_weights_multi(const void* table, int n_layers, int max_elems, cudaStream_t st) {
  dim3 grid((max_elems + 255) / 256 > 64 ? 64 : (max_elems + 255) / 256, n_layers);
  launch_k(conv_flip_weights_multi_kernel, dim3(grid), dim3(256), 0, st, reinterpret_cast<const FlipEntry*>(table));
  return (int)cudaGetLastError();
}

extern "C" int conv_flip_weights(const void* w, void* out, int cout, int cin, cudaStream_t st) {
  const int total = cout * 9 * cin;
  launch_k(conv_flip_weights_kernel, dim3((total + 255) / 256), dim3(256), 0, st, reinterpret_cast<const float*>(w),
                                                                 reinterpret_cast<float*>(out), cout, cin);
  return (int)cudaGetLastError();
}

// ---------------------------------- host side ----------------------------------------------
static int* g_conv_error[64];

static int* conv_error_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (g_conv_error[dev] == nullptr) {
    if (cudaMalloc(&g_conv_error[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(g_conv_error[dev], 0, sizeof(int));
  }
  return g_conv_error[dev];
}

extern "C" int conv3x3_last_error() {
  int* w = conv_error_word();
  int v = -1;
  if (w != nullptr) cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

template <int COUT, int KC>
static int launch_conv(const CUtensorMap& mx, const CUtensorMap& mw, const ConvArgs& g, int tiles, cudaStream_t st) {
  constexpr int smem = CONV_STAGES * (128 * KC * 4 + COUT * KC * 4) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv3x3_tf32_kernel<COUT, KC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_k(conv3x3_tf32_kernel<COUT, KC>, dim3(tiles), dim3(CONV_THREADS), smem, st, mx, mw, g);
  return (int)cudaGetLastError();
}

template <int COUT, int KC, bool BWD>
static int launch_conv_persist_t(const CUtensorMap& mx, const CUtensorMap& mw, const ConvPArgs& g, int grid, cudaStream_t st,
                                 const CUtensorMap* mx2 = nullptr, const CUtensorMap* mw2 = nullptr) {
  using Cfg = ConvPCfg<COUT, KC, BWD>;
  constexpr int smem = Cfg::STAGES * Cfg::GK * Cfg::KB_BYTES + Cfg::TILES * 128 * Cfg::TSTRIDE * 4 + 1024 + 512;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv3x3_persist_kernel<COUT, KC, BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // (the second pair of maps is read in mode 1 only: any valid map fills the slots otherwise)
  launch_k(conv3x3_persist_kernel<COUT, KC, BWD>, dim3(grid), dim3(CONV_THREADS), smem, st, mx, mw,
           mx2 != nullptr ? *mx2 : mx, mw2 != nullptr ? *mw2 : mw, g);
  return (int)cudaGetLastError();
}

template <int COUT, int KC>
static int launch_conv_persist(const CUtensorMap& mx, const CUtensorMap& mw, const ConvPArgs& g, int grid, cudaStream_t st) {
  const bool bwd = g.add != nullptr || g.mask != nullptr || g.bnx != nullptr;
  return bwd ? launch_conv_persist_t<COUT, KC, true>(mx, mw, g, grid, st)
             : launch_conv_persist_t<COUT, KC, false>(mx, mw, g, grid, st);
}

// 1 when conv3x3_tf32 handles this shape
extern "C" int conv3x3_supported(int N, int H, int W, int Cin, int Cout) {
  if (!(W == 8 || W == 16 || W == 32)) return 0;
  if (!(Cin == 16 || Cin == 32 || Cin == 64 || Cin == 128)) return 0;
  if (!(Cout == 16 || Cout == 32 || Cout == 64 || Cout == 128)) return 0;
  int th = 128 / W;
  if (th > H) th = H;
  const int tn = 128 / (W * th);
  if (W * th * tn != 128) return 0;
  if (H % th != 0 || N % tn != 0) return 0;
  if (tn > 1 && th != H) return 0;
  return 1;
}

static int conv_use_persistent() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("CHOCO_CONV_PERSISTENT");
    v = e == nullptr || atoi(e) != 0;
  }
  return v;
}

// CTAs of the persistent kernel: one per SM at most, and few enough that the rows of statistics
// partials (2 C_out floats per CTA) can be added by every CTA of the batch-norm kernel itself.
extern "C" int conv3x3_grid(int N, int H, int W, int Cout) {
  int th = 128 / W;
  if (th > H) th = H;
  const int tn = 128 / (W * th);
  if (tn < 1 || th < 1) return 0;
  const int tiles = (N / tn) * (H / th);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  }
  int g = tiles < sms ? tiles : sms;
  const int cap = 8192 / (2 * Cout);
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  // even out the tiles per CTA (e.g. 256 tiles on 128 CTAs rather than 148 with one or two each)
  const int per = (tiles + g - 1) / g;
  g = (tiles + per - 1) / per;
  return g;
}

struct ConvBwdEpilogue {
  const void* add;
  const void* mask;
  const void* bnx;
  const void* bn_mean;
  const void* bn_invstd;
};

static int conv3x3_run(const void* x, const void* w, void* y, void* stats, int N, int H, int W, int Cin, int Cout,
                       int relu, cudaStream_t st, const ConvBwdEpilogue* bwd = nullptr, int ks = 3, int stride = 1);

// 1 when conv_fwd_tf32 handles a ks x ks convolution (3x3 pad 1 or 1x1 pad 0) of the given stride
// whose OUTPUT is [N, HO, WO, Cout]
extern "C" int conv_fwd_supported(int N, int HO, int WO, int Cin, int Cout, int ks, int stride) {
  if (!(ks == 3 || ks == 1) || !(stride == 1 || stride == 2)) return 0;
  if (stride * WO > 256) return 0;   // a TMA box is at most 256 elements wide before the element stride
  return conv3x3_supported(N, HO, WO, Cin, Cout);
}

// General forward: x [N, stride HO, stride WO, Cin], w [Cout, ks, ks, Cin], y [N, HO, WO, Cout]; stats
// (optional) as in conv3x3_tf32_stats.  A strided convolution is the same implicit GEMM: the tensor map
// of x gets element strides (1, stride, stride, 1), so the box of a filter tap delivers exactly the
// input pixels of the tile's 128 output pixels, and nothing else changes in the kernel.
extern "C" int conv_fwd_tf32(const void* x, const void* w, void* y, void* stats, int N, int HO, int WO, int Cin, int Cout,
                             int ks, int stride, cudaStream_t st) {
  if (!conv_fwd_supported(N, HO, WO, Cin, Cout, ks, stride)) return -1;
  return conv3x3_run(x, w, y, stats, N, HO, WO, Cin, Cout, 0, st, nullptr, ks, stride);
}

// x [N,H,W,Cin], w [Cout,3,3,Cin], y [N,H,W,Cout], all fp32 NHWC / KRSC
extern "C" int conv3x3_tf32(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int relu,
                            cudaStream_t st) {
  return conv3x3_run(x, w, y, nullptr, N, H, W, Cin, Cout, relu, st);
}

// same, and stats[conv3x3_grid()][2 Cout] receives per-CTA (sum, sum of squares) of y per channel
extern "C" int conv3x3_tf32_stats(const void* x, const void* w, void* y, void* stats, int N, int H, int W, int Cin,
                                  int Cout, cudaStream_t st) {
  if (stats == nullptr) return -1;
  return conv3x3_run(x, w, y, stats, N, H, W, Cin, Cout, 0, st);
}

// Input gradient with the work that follows it folded into the epilogue:
//   result = (conv(dy, flipped filter) + add) * [mask > 0]
// and, when bnx / bn_mean / bn_invstd / stats are given, per-CTA rows [conv3x3_grid()][2 Cout] of
// (sum result, sum result * xhat): the two reductions of the batch-norm backward of the layer whose
// output fed this convolution.  add = gradient arriving over the skip connection, mask = that
// layer's ReLU output.  Any of add / mask / (bnx ...) may be null.
extern "C" int conv3x3_dgrad_fused(const void* dy, const void* w_flipped, void* out, const void* add, const void* mask,
                                   const void* bnx, const void* bn_mean, const void* bn_invstd, void* stats, int N,
                                   int H, int W, int Cin, int Cout, cudaStream_t st) {
  if ((bnx != nullptr) != (stats != nullptr)) return -1;
  if (bnx != nullptr && (bn_mean == nullptr || bn_invstd == nullptr)) return -1;
  ConvBwdEpilogue e = {add, mask, bnx, bn_mean, bn_invstd};
  return conv3x3_run(dy, w_flipped, out, stats, N, H, W, Cin, Cout, 0, st, &e);
}

static int conv3x3_run(const void* x, const void* w, void* y, void* stats, int N, int H, int W, int Cin, int Cout,
                       int relu, cudaStream_t st, const ConvBwdEpilogue* bwd, int ks, int stride) {
  if (!conv3x3_supported(N, H, W, Cin, Cout)) return -1;
  const int taps = ks * ks;
  const bool general = ks != 3 || stride != 1;
  int th = 128 / W;
  if (th > H) th = H;
  const int tn = 128 / (W * th);
  const int kc = Cin >= 32 ? 32 : 16;
  const CUtensorMapSwizzle sw = kc == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUtensorMap mx, mw;
  {
    const cuuint64_t WI = (cuuint64_t)W * stride, HI = (cuuint64_t)H * stride;   // input extent
    cuuint64_t dims[4] = {(cuuint64_t)Cin, WI, HI, (cuuint64_t)N};
    cuuint64_t str[3] = {(cuuint64_t)Cin * 4, WI * Cin * 4, HI * WI * Cin * 4};
    cuuint32_t box[4] = {(cuuint32_t)kc, (cuuint32_t)(W * stride), (cuuint32_t)(th * stride), (cuuint32_t)tn};
    cuuint32_t est[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
    int rc = tc_make_map(&mx, x, 4, dims, str, box, sw, est);
    if (rc) return rc;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)taps * Cin, (cuuint64_t)Cout};
    cuuint64_t str[1] = {(cuuint64_t)taps * Cin * 4};
    cuuint32_t box[2] = {(cuuint32_t)kc, (cuuint32_t)Cout};
    int rc = tc_make_map(&mw, w, 2, dims, str, box, sw);
    if (rc) return rc;
  }
  ConvArgs g;
  g.y = reinterpret_cast<float*>(y);
  g.error = conv_error_word();
  if (g.error == nullptr) return -13;
  g.H = H; g.W = W; g.Cin = Cin; g.TH = th; g.TN = tn; g.tiles_h = H / th; g.relu = relu;
  const int tiles = (N / tn) * (H / th);
  if (stats != nullptr || bwd != nullptr || general || conv_use_persistent()) {
    ConvPArgs pg;
    pg.taps = taps; pg.stride = stride; pg.mode = 0; pg.cb2 = 0; pg.tiles_per_class = 0;
    pg.y = g.y; pg.stats = reinterpret_cast<float*>(stats); pg.error = g.error;
    pg.add = pg.mask = pg.bnx = pg.bn_mean = pg.bn_invstd = nullptr;
    if (bwd != nullptr) {
      pg.add = reinterpret_cast<const float*>(bwd->add);
      pg.mask = reinterpret_cast<const float*>(bwd->mask);
      pg.bnx = reinterpret_cast<const float*>(bwd->bnx);
      pg.bn_mean = reinterpret_cast<const float*>(bwd->bn_mean);
      pg.bn_invstd = reinterpret_cast<const float*>(bwd->bn_invstd);
    }
    pg.H = H; pg.W = W; pg.Cin = Cin; pg.TH = th; pg.TN = tn; pg.tiles_h = H / th; pg.n_tiles = tiles; pg.relu = relu;
    const int grid = conv3x3_grid(N, H, W, Cout);
#define CONVP_CASE(CO)                                                             \
  if (Cout == CO) return kc == 32 ? launch_conv_persist<CO, 32>(mx, mw, pg, grid, st) : launch_conv_persist<CO, 16>(mx, mw, pg, grid, st);
    CONVP_CASE(16) CONVP_CASE(32) CONVP_CASE(64) CONVP_CASE(128)
#undef CONVP_CASE
    return -1;
  }
#define CONV_CASE(CO)                                                              \
  if (Cout == CO) return kc == 32 ? launch_conv<CO, 32>(mx, mw, g, tiles, st) : launch_conv<CO, 16>(mx, mw, g, tiles, st);
  CONV_CASE(16) CONV_CASE(32) CONV_CASE(64) CONV_CASE(128)
#undef CONV_CASE
  return -1;
}

// ---- input gradient of the strided layers ---------------------------------------------------------
static int conv_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  }
  return sms;
}

// dy: [N, HO, WO, Cdy].  1 when conv3x3s2_dgrad_fused covers the shape.
extern "C" int conv3x3s2_dgrad_supported(int N, int HO, int WO, int Cdy, int Cx, int Cdy2) {
  if (!(Cx == 16 || Cx == 32 || Cx == 64) || Cdy % 32 != 0 || Cdy < 32 || Cdy > 128) return 0;
  if (Cdy2 != 0 && (Cdy2 % 32 != 0 || Cdy2 > 128)) return 0;
  return conv3x3_supported(N, HO, WO, Cdy, Cx);
}

// CTAs (= rows of statistics partials) of conv3x3s2_dgrad_fused
extern "C" int conv3x3s2_dgrad_grid(int N, int HO, int WO, int Cx) {
  int th = 128 / WO;
  if (th > HO) th = HO;
  const int tn = 128 / (WO * th);
  if (tn < 1 || th < 1) return 0;
  const int tiles = 4 * (N / tn) * (HO / th);
  int g = tiles < conv_sm_count() ? tiles : conv_sm_count();
  const int cap = 8192 / (2 * Cx);
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  const int per = (tiles + g - 1) / g;
  return (tiles + per - 1) / per;
}

// Input gradient of y = conv3x3(x, w, stride 2, pad 1) and, when dy2 is given, of the shortcut
// y2 = conv1x1(x, w2, stride 2) that reads the same x, in ONE launch:
//   out[N, 2 HO, 2 WO, Cx] = dgrad(dy, w) + dgrad(dy2, w2)   then the same epilogue as conv3x3_dgrad_fused
// w_flipped: [Cx, 9, Cdy] (conv_flip_weights of w); w2_t: [Cx, Cdy2] (w2 transposed).
extern "C" int conv3x3s2_dgrad_fused(const void* dy, const void* w_flipped, const void* dy2, const void* w2_t, void* out,
                                     const void* add, const void* mask, const void* bnx, const void* bn_mean,
                                     const void* bn_invstd, void* stats, int N, int HO, int WO, int Cdy, int Cx, int Cdy2,
                                     cudaStream_t st) {
  if (dy2 == nullptr) Cdy2 = 0;
  if (!conv3x3s2_dgrad_supported(N, HO, WO, Cdy, Cx, Cdy2)) return -1;
  if ((bnx != nullptr) != (stats != nullptr)) return -1;
  if (bnx != nullptr && (bn_mean == nullptr || bn_invstd == nullptr)) return -1;
  if (Cdy2 != 0 && w2_t == nullptr) return -1;
  int th = 128 / WO;
  if (th > HO) th = HO;
  const int tn = 128 / (WO * th);
  constexpr int kc = 32;
  const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap mx, mw, mx2, mw2;
  auto act_map = [&](CUtensorMap* m, const void* p, int C) {
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)WO, (cuuint64_t)HO, (cuuint64_t)N};
    cuuint64_t str[3] = {(cuuint64_t)C * 4, (cuuint64_t)WO * C * 4, (cuuint64_t)HO * WO * C * 4};
    cuuint32_t box[4] = {(cuuint32_t)kc, (cuuint32_t)WO, (cuuint32_t)th, (cuuint32_t)tn};
    return tc_make_map(m, p, 4, dims, str, box, sw);
  };
  auto w_map = [&](CUtensorMap* m, const void* p, int K) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)Cx};
    cuuint64_t str[1] = {(cuuint64_t)K * 4};
    cuuint32_t box[2] = {(cuuint32_t)kc, (cuuint32_t)Cx};
    return tc_make_map(m, p, 2, dims, str, box, sw);
  };
  int rc = act_map(&mx, dy, Cdy);
  if (rc) return rc;
  rc = w_map(&mw, w_flipped, 9 * Cdy);
  if (rc) return rc;
  if (Cdy2 != 0) {
    rc = act_map(&mx2, dy2, Cdy2);
    if (rc) return rc;
    rc = w_map(&mw2, w2_t, Cdy2);
    if (rc) return rc;
  }
  ConvPArgs pg;
  pg.y = reinterpret_cast<float*>(out);
  pg.stats = reinterpret_cast<float*>(stats);
  pg.add = reinterpret_cast<const float*>(add);
  pg.mask = reinterpret_cast<const float*>(mask);
  pg.bnx = reinterpret_cast<const float*>(bnx);
  pg.bn_mean = reinterpret_cast<const float*>(bn_mean);
  pg.bn_invstd = reinterpret_cast<const float*>(bn_invstd);
  pg.error = conv_error_word();
  if (pg.error == nullptr) return -13;
  pg.H = HO; pg.W = WO; pg.Cin = Cdy; pg.TH = th; pg.TN = tn; pg.tiles_h = HO / th;
  pg.tiles_per_class = (N / tn) * (HO / th);
  pg.n_tiles = 4 * pg.tiles_per_class;
  pg.relu = 0; pg.taps = 9; pg.stride = 1; pg.mode = 1; pg.cb2 = Cdy2 / kc;
  const int grid = conv3x3s2_dgrad_grid(N, HO, WO, Cx);
  const CUtensorMap* p2 = Cdy2 != 0 ? &mx2 : nullptr;
  const CUtensorMap* q2 = Cdy2 != 0 ? &mw2 : nullptr;
  if (Cx == 16) return launch_conv_persist_t<16, 32, true>(mx, mw, pg, grid, st, p2, q2);
  if (Cx == 32) return launch_conv_persist_t<32, 32, true>(mx, mw, pg, grid, st, p2, q2);
  if (Cx == 64) return launch_conv_persist_t<64, 32, true>(mx, mw, pg, grid, st, p2, q2);
  return -1;
}
