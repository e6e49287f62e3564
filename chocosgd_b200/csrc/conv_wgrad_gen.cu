// Weight gradient of the small convolutions of a CIFAR ResNet that the two specialised kernels do
// not cover (NHWC fp32, TF32 products, fp32 accumulation):
//
//   dW[co, r, s, ci] = sum over output pixels (n, h, w) of  dY[n, h, w, co] * X[n, S h + r - P, S w + s - P, ci]
//
//   * 3x3 / stride 1 / pad 1 with 32 -> 32 and 64 -> 64 channels,
//   * 3x3 / stride 2 / pad 1 with 16 -> 32 and 32 -> 64 channels (first convolution of a stage),
//   * 1x1 / stride 2 / pad 0 with 16 -> 32 and 32 -> 64 channels (the down-sampling shortcut).
//
// The result is at most 64 x 576 while the reduction runs over all N H W output pixels: the
// operation is bound by reading X and dY once and by launch latency, not by arithmetic (0.6 GFLOP at
// batch 128).  The reduction dimension is the pixel index, so for tcgen05 both operands would be
// MN-major and need 128-byte rows (32 floats per pixel) and, for a stride of 2, a gather that the
// tensor-map engine cannot express for the dY-aligned pixel order; the kernel therefore uses
// warp-level m16n8k8 TF32 tensor-core instructions like the 16-channel kernel:
//   * a CTA walks over tiles of TP output pixels (TH full output rows of one image); per tile the dY
//     tile and the X tile with its halo are copied to shared memory with 16-byte asynchronous copies
//     (zero fill outside the image = the padding), double buffered across tiles;
//   * pixels lie PS floats apart in shared memory, PS chosen so that every fragment load is conflict
//     free for the layer's stride;
//   * a warp owns 16 output channels x one filter row (KS taps x C_in) of the result and every
//     KSPLIT-th 8-pixel slice of the tile; its accumulators stay in registers for the whole kernel;
//   * the KSPLIT partial results are added in a fixed order in shared memory, each CTA writes one
//     slice of partial results, and a second small kernel adds the slices in index order
//     (reproducible, no atomics).
#include <cuda_runtime.h>
#include <stdint.h>
#include "launch.cuh"

struct WgGenArgs {
  const float* x;    // [N, HI, WI, CIN]
  const float* dy;   // [N, HO, WO, COUT]
  float* partial;    // [gridDim.x][COUT * KS * KS * CIN]
  int N, HO;
  int tiles_h, n_tiles, tiles_per_cta;
};

__device__ __forceinline__ uint32_t wgg_tf32(float f) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(f));
  return r;
}
__device__ __forceinline__ void wgg_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void wgg_cp16(float* dst, const float* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

// CIN, COUT: channels; KS: 1 or 3; STRIDE: 1 or 2; WO: output width; TP: output pixels per tile;
// COB: 16-channel blocks of dY per CTA (gridDim.y = COUT / 16 / COB); KSPLIT: pixel-slice split
template <int CIN, int COUT, int KS, int STRIDE, int WO, int TP, int COB, int KSPLIT>
struct WgGenCfg {
  static constexpr int PAD = KS / 2;
  static constexpr int TH = TP / WO;                         // output rows per tile
  // a 1x1 convolution reads only every STRIDE-th pixel: the tile holds exactly those, densely
  static constexpr int SSTEP = KS == 1 ? 1 : STRIDE;         // shared-memory pixels between neighbouring outputs
  static constexpr int GSTEP = KS == 1 ? STRIDE : 1;         // image pixels between neighbouring tile pixels
  static constexpr int XR = (TH - 1) * SSTEP + KS, XC = (WO - 1) * SSTEP + KS;
  static constexpr int PS = CIN + (SSTEP == 1 ? 8 : 4);      // SSTEP * PS = 8 or 24 (mod 32): conflict-free
  static constexpr int DC = COB * 16;                        // dY channels held by a CTA
  static constexpr int DS = DC + 8;
  static constexpr int DY_FLOATS = TP * DS, X_FLOATS = XR * XC * PS;
  static constexpr int STAGE = DY_FLOATS + X_FLOATS;
  static constexpr int WARPS = COB * KS * KSPLIT;
  static constexpr int THREADS = WARPS * 32;
  static constexpr int SLICE = DC * KS * KS * CIN;           // results of one CTA
  static constexpr int RED_FLOATS = KSPLIT > 1 ? KSPLIT * SLICE : 0;
  static constexpr int SMEM_FLOATS = 2 * STAGE > RED_FLOATS ? 2 * STAGE : RED_FLOATS;
  static constexpr int OUT = COUT * KS * KS * CIN;
  static_assert(TP % WO == 0 && TP % 8 == 0 && WO % 8 == 0, "8-pixel slices lie inside one output row");
  static_assert((TP / 8) % KSPLIT == 0, "slices divide evenly");
  static_assert(COUT % (16 * COB) == 0 && CIN % 8 == 0, "channel blocks");
};

template <int CIN, int COUT, int KS, int STRIDE, int WO, int TP, int COB, int KSPLIT>
__global__ void __launch_bounds__(WgGenCfg<CIN, COUT, KS, STRIDE, WO, TP, COB, KSPLIT>::THREADS)
conv_wgrad_gen_kernel(WgGenArgs g) {
  pdl_wait();
  pdl_trigger();
  using C = WgGenCfg<CIN, COUT, KS, STRIDE, WO, TP, COB, KSPLIT>;
  constexpr int HI_PER_HO = STRIDE, WI = WO * STRIDE, NT = CIN / 8;
  extern __shared__ float wgg_smem[];
  const int HI = g.HO * HI_PER_HO;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  // warp -> (pixel-slice part, 16-channel block, filter row)
  const int kpart = warp / (COB * KS), cbl = (warp / KS) % COB, dr = warp % KS;
  const int co_base = (blockIdx.y * COB) * 16;
  const int t_begin = blockIdx.x * g.tiles_per_cta;
  int t_end = t_begin + g.tiles_per_cta;
  if (t_end > g.n_tiles) t_end = g.n_tiles;

  auto load_tile = [&](int stage, int tile) {
    float* dys = wgg_smem + stage * C::STAGE;
    float* xs = dys + C::DY_FLOATS;
    const int n = tile / g.tiles_h, h0 = (tile % g.tiles_h) * C::TH;
    const float* dy0 = g.dy + (((size_t)n * g.HO + h0) * WO) * COUT + co_base;
    constexpr int DCH = C::DC / 4;
    for (int idx = threadIdx.x; idx < TP * DCH; idx += C::THREADS) {
      const int px = idx / DCH, ch = (idx % DCH) * 4;
      wgg_cp16(dys + px * C::DS + ch, dy0 + (size_t)px * COUT + ch, true);
    }
    constexpr int XCH = CIN / 4;
    const int gh0 = h0 * STRIDE - C::PAD;
    for (int idx = threadIdx.x; idx < C::XR * C::XC * XCH; idx += C::THREADS) {
      const int hp = idx / XCH, ch = (idx % XCH) * 4;
      const int hr = hp / C::XC, hc = hp % C::XC;
      const int gh = gh0 + hr * C::GSTEP, gw = hc * C::GSTEP - C::PAD;
      const bool valid = gh >= 0 && gh < HI && gw >= 0 && gw < WI;
      const float* src = valid ? g.x + (((size_t)n * HI + gh) * WI + gw) * CIN + ch : g.x;
      wgg_cp16(xs + hp * C::PS + ch, src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[KS][NT][4];
#pragma unroll
  for (int t = 0; t < KS; ++t)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[t][n][e] = 0.f;

  if (t_begin < t_end) load_tile(0, t_begin);
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int st = (tile - t_begin) & 1;
    if (tile + 1 < t_end) {
      load_tile(st ^ 1, tile + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* dys = wgg_smem + st * C::STAGE + cbl * 16;
    const float* xs = wgg_smem + st * C::STAGE + C::DY_FLOATS;
#pragma unroll 1
    for (int ks = kpart; ks < TP / 8; ks += KSPLIT) {
      const int p0 = ks * 8, r = p0 / WO, c0 = p0 % WO;
      uint32_t a[4];
      a[0] = wgg_tf32(dys[(p0 + tq) * C::DS + gq]);
      a[1] = wgg_tf32(dys[(p0 + tq) * C::DS + gq + 8]);
      a[2] = wgg_tf32(dys[(p0 + tq + 4) * C::DS + gq]);
      a[3] = wgg_tf32(dys[(p0 + tq + 4) * C::DS + gq + 8]);
#pragma unroll
      for (int dc = 0; dc < KS; ++dc) {
        const float* row = xs + ((r * C::SSTEP + dr) * C::XC + (c0 + tq) * C::SSTEP + dc) * C::PS + gq;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t b0 = wgg_tf32(row[nt * 8]);
          const uint32_t b1 = wgg_tf32(row[4 * C::SSTEP * C::PS + nt * 8]);
          wgg_mma(acc[dc][nt], a, b0, b1);
        }
      }
    }
    __syncthreads();   // the buffer is refilled two tiles later
  }

  // element (co, tap, ci) of dW lives at (co * KS * KS + tap) * CIN + ci; a CTA owns DC consecutive co
  float* out = g.partial + (size_t)blockIdx.x * C::OUT + (size_t)co_base * KS * KS * CIN;
  auto store_acc = [&](float* dst) {
#pragma unroll
    for (int dc = 0; dc < KS; ++dc)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int tap = dr * KS + dc, ci = nt * 8 + 2 * tq;
        const int lo = ((cbl * 16 + gq) * KS * KS + tap) * CIN + ci;
        const int hi = ((cbl * 16 + gq + 8) * KS * KS + tap) * CIN + ci;
        *reinterpret_cast<float2*>(dst + lo) = make_float2(acc[dc][nt][0], acc[dc][nt][1]);
        *reinterpret_cast<float2*>(dst + hi) = make_float2(acc[dc][nt][2], acc[dc][nt][3]);
      }
  };
  if (KSPLIT == 1) {
    store_acc(out);
  } else {
    float* red = wgg_smem;   // [KSPLIT][SLICE]: the tile buffers are free after the last barrier
    store_acc(red + kpart * C::SLICE);
    __syncthreads();
    for (int i = threadIdx.x * 4; i < C::SLICE; i += C::THREADS * 4) {
      float4 s = *reinterpret_cast<const float4*>(red + i);
#pragma unroll
      for (int k = 1; k < KSPLIT; ++k) {
        const float4 v = *reinterpret_cast<const float4*>(red + k * C::SLICE + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      *reinterpret_cast<float4*>(out + i) = s;
    }
  }
}

// dw[i] = sum over slices of partial[slice][i]: 64 outputs per CTA, 4 threads per output (slices q,
// q + 4, ... in order, then the four sub-sums in order)
__global__ void __launch_bounds__(256) wgrad_gen_reduce_kernel(const float* __restrict__ partial, int n_parts, int n,
                                                               float* __restrict__ dw) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sub[4][64];
  const int il = threadIdx.x & 63, q = threadIdx.x >> 6;
  const int i = blockIdx.x * 64 + il;
  float acc = 0.f;
  if (i < n) {
#pragma unroll 8
    for (int s = q; s < n_parts; s += 4) acc += __ldcg(partial + (size_t)s * n + i);
  }
  sub[q][il] = acc;
  __syncthreads();
  if (q == 0 && i < n) dw[i] = ((sub[0][il] + sub[1][il]) + sub[2][il]) + sub[3][il];
}

// ---------------------------------- host side ----------------------------------------------
static int wgg_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  }
  return sms;
}

struct WgGenPlan {
  int tiles_h, n_tiles, tiles_per_cta, grid_x, grid_y;
};

template <int CIN, int COUT, int KS, int STRIDE, int WO, int TP, int COB, int KSPLIT>
static bool wgg_plan(int N, int HO, WgGenPlan* p) {
  using C = WgGenCfg<CIN, COUT, KS, STRIDE, WO, TP, COB, KSPLIT>;
  if (N < 1 || HO < C::TH || HO % C::TH != 0) return false;
  p->tiles_h = HO / C::TH;
  p->n_tiles = N * p->tiles_h;
  p->grid_y = COUT / 16 / COB;
  int want = wgg_sm_count() / p->grid_y;
  if (want < 1) want = 1;
  p->tiles_per_cta = (p->n_tiles + want - 1) / want;
  p->grid_x = (p->n_tiles + p->tiles_per_cta - 1) / p->tiles_per_cta;
  return true;
}

template <int CIN, int COUT, int KS, int STRIDE, int WO, int TP, int COB, int KSPLIT>
static int wgg_launch(const void* x, const void* dy, void* dw, void* scratch, int N, int HO, cudaStream_t st) {
  using C = WgGenCfg<CIN, COUT, KS, STRIDE, WO, TP, COB, KSPLIT>;
  WgGenPlan p;
  if (!wgg_plan<CIN, COUT, KS, STRIDE, WO, TP, COB, KSPLIT>(N, HO, &p)) return -1;
  WgGenArgs g;
  g.x = reinterpret_cast<const float*>(x);
  g.dy = reinterpret_cast<const float*>(dy);
  g.partial = reinterpret_cast<float*>(scratch);
  g.N = N; g.HO = HO; g.tiles_h = p.tiles_h; g.n_tiles = p.n_tiles; g.tiles_per_cta = p.tiles_per_cta;
  constexpr int smem = C::SMEM_FLOATS * 4;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv_wgrad_gen_kernel<CIN, COUT, KS, STRIDE, WO, TP, COB, KSPLIT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_k(conv_wgrad_gen_kernel<CIN, COUT, KS, STRIDE, WO, TP, COB, KSPLIT>, dim3(p.grid_x, p.grid_y), dim3(C::THREADS),
           smem, st, g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  launch_k(wgrad_gen_reduce_kernel, dim3((C::OUT + 63) / 64), dim3(256), 0, st, reinterpret_cast<const float*>(scratch),
           p.grid_x, (int)C::OUT, reinterpret_cast<float*>(dw));
  return (int)cudaGetLastError();
}

// The shapes with a kernel: (C_in, C_out, kernel size, stride, output width) -> template instance.
//                         CIN COUT KS ST  WO   TP COB KSPLIT
#define WGG_SHAPES(X)                   \
  X(32, 32, 3, 1, 16, 128, 2, 2)        \
  X(64, 64, 3, 1, 8, 64, 1, 4)          \
  X(16, 32, 3, 2, 16, 128, 2, 2)        \
  X(32, 64, 3, 2, 8, 64, 2, 2)          \
  X(16, 32, 1, 2, 16, 128, 2, 4)        \
  X(32, 64, 1, 2, 8, 64, 2, 4)

// number of partial slices (0: shape not covered).  HO, WO: OUTPUT height and width.
extern "C" int conv_wgrad_gen_parts(int N, int HO, int WO, int Cin, int Cout, int ks, int stride) {
  WgGenPlan p;
#define X(CI, CO, K, S, W, TP, COB, KSP) \
  if (Cin == CI && Cout == CO && ks == K && stride == S && WO == W) \
    return wgg_plan<CI, CO, K, S, W, TP, COB, KSP>(N, HO, &p) ? p.grid_x : 0;
  WGG_SHAPES(X)
#undef X
  return 0;
}

// x [N, stride HO, stride WO, Cin], dy [N, HO, WO, Cout], dw [Cout, ks, ks, Cin], all fp32 NHWC / KRSC;
// scratch: conv_wgrad_gen_parts() * Cout ks ks Cin floats
extern "C" int conv_wgrad_gen(const void* x, const void* dy, void* dw, void* scratch, int N, int HO, int WO, int Cin,
                              int Cout, int ks, int stride, cudaStream_t st) {
#define X(CI, CO, K, S, W, TP, COB, KSP) \
  if (Cin == CI && Cout == CO && ks == K && stride == S && WO == W) \
    return wgg_launch<CI, CO, K, S, W, TP, COB, KSP>(x, dy, dw, scratch, N, HO, st);
  WGG_SHAPES(X)
#undef X
  return -1;
}
