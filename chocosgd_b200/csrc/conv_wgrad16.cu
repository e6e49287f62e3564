// Weight gradient of a 3x3 / stride 1 / pad 1 convolution with 16 input and 16 output channels
// (NHWC fp32, TF32 products, fp32 accumulation):
//
//   dW[co, r, s, ci] = sum over pixels p of  dY[p, co] * X[p + (r-1, s-1), ci]
//
// The output is 16 x 144 and the reduction runs over all N*H*W pixels, so the operation is bound
// by reading X and dY once, not by arithmetic.  A tcgen05 instruction needs at least 64 rows and,
// for operands whose reduction dimension is the pixel index, shared-memory rows of 128 bytes;
// 16-channel pixels are 64 bytes.  This kernel therefore uses warp-level m16n8k8 tensor-core
// instructions, which match the 16 x 16 output exactly:
//   * a CTA walks over tiles of 128 pixels (TH full image rows); per tile the dY tile and the X tile
//     with a one-pixel halo are copied to shared memory with 16-byte asynchronous copies (zero fill
//     outside the image = the padding), double buffered across tiles;
//   * pixels lie 24 floats apart in shared memory, which makes every fragment load conflict free;
//   * each warp owns 8-pixel slices of the tile and accumulates all 9 taps (18 instructions per
//     slice, the dY fragment is loaded once) in 72 registers for the whole kernel;
//   * the warps' accumulators are added in a fixed order, each CTA writes one slice of partial
//     results, and a second small kernel adds the slices in index order (reproducible, no atomics).
#include <cuda_runtime.h>
#include "launch.cuh"
#include <stdint.h>

#define WG16_THREADS 256
#define WG16_PS 24            // floats between consecutive pixels in shared memory
#define WG16_OUT 2304         // 16 * 9 * 16

struct Wg16Args {
  const float* x;
  const float* dy;
  float* partial;   // [gridDim.x][WG16_OUT]
  int N, H, W;
  int TH, tiles_h, n_tiles, tiles_per_cta;
};

__device__ __forceinline__ uint32_t wg16_tf32(float f) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(f));
  return r;
}
__device__ __forceinline__ void wg16_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void wg16_cp16(float* dst, const float* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

template <int W>
__global__ void __launch_bounds__(WG16_THREADS) conv3x3_wgrad16_kernel(Wg16Args g) {
  pdl_wait();
  pdl_trigger();
  constexpr int TH = 128 / W, HW = W + 2, HH = TH + 2;
  constexpr int DY_FLOATS = 128 * WG16_PS, X_FLOATS = HH * HW * WG16_PS;
  extern __shared__ float wg16_smem[];
  float* dy_s[2] = {wg16_smem, wg16_smem + DY_FLOATS + X_FLOATS};
  float* x_s[2] = {wg16_smem + DY_FLOATS, wg16_smem + 2 * DY_FLOATS + X_FLOATS};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const int t_begin = blockIdx.x * g.tiles_per_cta;
  int t_end = t_begin + g.tiles_per_cta;
  if (t_end > g.n_tiles) t_end = g.n_tiles;

  auto load_tile = [&](int stage, int tile) {
    const int n = tile / g.tiles_h, h0 = (tile % g.tiles_h) * TH;
    const float* dy0 = g.dy + ((size_t)n * g.H + h0) * W * 16;
    for (int idx = threadIdx.x; idx < 128 * 4; idx += WG16_THREADS) {
      const int px = idx >> 2, ch = (idx & 3) * 4;
      wg16_cp16(dy_s[stage] + px * WG16_PS + ch, dy0 + px * 16 + ch, true);
    }
    for (int idx = threadIdx.x; idx < HH * HW * 4; idx += WG16_THREADS) {
      const int hp = idx >> 2, ch = (idx & 3) * 4;
      const int hr = hp / HW, hc = hp % HW;
      const int gh = h0 + hr - 1, gw = hc - 1;
      const bool valid = gh >= 0 && gh < g.H && gw >= 0 && gw < W;
      const float* src = valid ? g.x + (((size_t)n * g.H + gh) * W + gw) * 16 + ch : g.x;
      wg16_cp16(x_s[stage] + hp * WG16_PS + ch, src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[9][2][4];
#pragma unroll
  for (int t = 0; t < 9; ++t)
#pragma unroll
    for (int n = 0; n < 2; ++n)
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
    const float* dys = dy_s[st];
    const float* xs = x_s[st];
#pragma unroll 1
    for (int ks = warp; ks < 16; ks += WG16_THREADS / 32) {
      const int p0 = ks * 8, r = p0 / W, c0 = p0 % W;
      uint32_t a[4];
      a[0] = wg16_tf32(dys[(p0 + tq) * WG16_PS + gq]);
      a[1] = wg16_tf32(dys[(p0 + tq) * WG16_PS + gq + 8]);
      a[2] = wg16_tf32(dys[(p0 + tq + 4) * WG16_PS + gq]);
      a[3] = wg16_tf32(dys[(p0 + tq + 4) * WG16_PS + gq + 8]);
#pragma unroll
      for (int dr = 0; dr < 3; ++dr)
#pragma unroll
        for (int dc = 0; dc < 3; ++dc) {
          const float* row = xs + ((r + dr) * HW + c0 + dc + tq) * WG16_PS + gq;
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            const uint32_t b0 = wg16_tf32(row[nt * 8]);
            const uint32_t b1 = wg16_tf32(row[4 * WG16_PS + nt * 8]);
            wg16_mma(acc[dr * 3 + dc][nt], a, b0, b1);
          }
        }
    }
    __syncthreads();   // the buffer is refilled two tiles later
  }

  // ---- add the eight warps' accumulators in a fixed order ---------------------------------------
  // element (co, tap, ci) of dW lives at (co * 9 + tap) * 16 + ci
  float* red = wg16_smem;   // [4][WG16_OUT] floats = 36 KiB (fits in the tile buffers)
  auto store_acc = [&](float* dst) {
#pragma unroll
    for (int t = 0; t < 9; ++t)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int ci = nt * 8 + 2 * tq;
        dst[(gq * 9 + t) * 16 + ci] = acc[t][nt][0];
        dst[(gq * 9 + t) * 16 + ci + 1] = acc[t][nt][1];
        dst[((gq + 8) * 9 + t) * 16 + ci] = acc[t][nt][2];
        dst[((gq + 8) * 9 + t) * 16 + ci + 1] = acc[t][nt][3];
      }
  };
  if (warp >= 4) store_acc(red + (warp - 4) * WG16_OUT);
  __syncthreads();
  if (warp < 4) {
    const float* src = red + warp * WG16_OUT;
#pragma unroll
    for (int t = 0; t < 9; ++t)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int ci = nt * 8 + 2 * tq;
        acc[t][nt][0] += src[(gq * 9 + t) * 16 + ci];
        acc[t][nt][1] += src[(gq * 9 + t) * 16 + ci + 1];
        acc[t][nt][2] += src[((gq + 8) * 9 + t) * 16 + ci];
        acc[t][nt][3] += src[((gq + 8) * 9 + t) * 16 + ci + 1];
      }
  }
  __syncthreads();
  if (warp < 4) store_acc(red + warp * WG16_OUT);
  __syncthreads();
  float* out = g.partial + (size_t)blockIdx.x * WG16_OUT;
  for (int i = threadIdx.x; i < WG16_OUT; i += WG16_THREADS)
    out[i] = ((red[i] + red[WG16_OUT + i]) + red[2 * WG16_OUT + i]) + red[3 * WG16_OUT + i];
}

// 64 outputs per CTA, 4 threads per output (slices q, q + 4, ... in order, then the four sub-sums)
__global__ void __launch_bounds__(256) wgrad16_reduce_kernel(const float* __restrict__ partial, int n_parts,
                                                             float* __restrict__ dw) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sub[4][64];
  const int il = threadIdx.x & 63, q = threadIdx.x >> 6;
  const int i = blockIdx.x * 64 + il;
  float acc = 0.f;
#pragma unroll 8
  for (int s = q; s < n_parts; s += 4) acc += __ldcg(partial + (size_t)s * WG16_OUT + i);
  sub[q][il] = acc;
  __syncthreads();
  if (q == 0) dw[i] = ((sub[0][il] + sub[1][il]) + sub[2][il]) + sub[3][il];
}

extern "C" int conv3x3_wgrad16_supported(int N, int H, int W) {
  if (!(W == 32 || W == 16)) return 0;
  const int th = 128 / W;
  return N >= 1 && H % th == 0;
}

// number of partial slices = CTAs
extern "C" int conv3x3_wgrad16_parts(int N, int H, int W) {
  const int th = 128 / W;
  const int n_tiles = N * (H / th);
  const int per = (n_tiles + sm_count() - 1) / sm_count();
  return (n_tiles + per - 1) / per;
}

// x, dy: [N, H, W, 16] fp32 NHWC; dw: [16, 3, 3, 16]; scratch: conv3x3_wgrad16_parts() * 2304 floats
extern "C" int conv3x3_wgrad16(const void* x, const void* dy, void* dw, void* scratch, int N, int H, int W,
                               cudaStream_t st) {
  if (!conv3x3_wgrad16_supported(N, H, W)) return -1;
  Wg16Args g;
  g.x = reinterpret_cast<const float*>(x);
  g.dy = reinterpret_cast<const float*>(dy);
  g.partial = reinterpret_cast<float*>(scratch);
  g.N = N; g.H = H; g.W = W;
  g.TH = 128 / W; g.tiles_h = H / g.TH; g.n_tiles = N * g.tiles_h;
  g.tiles_per_cta = (g.n_tiles + sm_count() - 1) / sm_count();
  const int grid = (g.n_tiles + g.tiles_per_cta - 1) / g.tiles_per_cta;
  const int hh = g.TH + 2, hw = W + 2;
  const int smem = 2 * (128 * WG16_PS + hh * hw * WG16_PS) * 4;
  cudaError_t e;
  if (W == 32) {
    static bool cfg = false;
    if (!cfg) {
      e = cudaFuncSetAttribute(conv3x3_wgrad16_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return (int)e;
      cfg = true;
    }
    launch_k(conv3x3_wgrad16_kernel<32>, dim3(grid), dim3(WG16_THREADS), smem, st, g);
  } else {
    static bool cfg = false;
    if (!cfg) {
      e = cudaFuncSetAttribute(conv3x3_wgrad16_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return (int)e;
      cfg = true;
    }
    launch_k(conv3x3_wgrad16_kernel<16>, dim3(grid), dim3(WG16_THREADS), smem, st, g);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  launch_k(wgrad16_reduce_kernel, dim3(WG16_OUT / 64), dim3(256), 0, st, reinterpret_cast<const float*>(scratch), grid,
                                                               reinterpret_cast<float*>(dw));
  return (int)cudaGetLastError();
}
