// Weight gradient of a 3x3 / stride 1 / pad 1 convolution on tcgen05 tensor cores (NHWC fp32, TF32):
//
//   dW[co, r, s, ci] = sum over pixels p of  dY[p, co] * X[p + (r-1, s-1), ci]
//
// A GEMM whose reduction runs over the pixels, so both operands are "MN-major" for the tensor core:
// dY tiles ([pixels, C_out], channel contiguous) and, per filter tap, the shifted X tile fetched by a 4-d
// TMA box (zero fill = padding) are used exactly as they lie in memory; no transpose, no im2col.
// The only shared-memory layout the tensor core accepts for MN-major 32-bit operands is the 128-byte
// swizzle with 32-byte units, which TMA produces (SWIZZLE_128B_ATOM_32B) for rows of exactly 32 floats:
// the kernel therefore covers C = 32 and C = 64 (two 32-channel blocks); 16-channel layers use the
// warp-level kernel of conv_wgrad16.cu.
//
// One CTA reduces a contiguous range of 128-pixel tiles: the dY tile is loaded once per tile and
// multiplied with the 9 shifted X tiles into 9 accumulators of 32 columns in TMEM (M = 128 with the
// 32- or 64-row operand replicated, N = 32).  Each CTA stores its partial dW into its own slice of a
// scratch buffer; a second small kernel adds the slices in a fixed order (reproducible, no atomics).
#include "tc_common.cuh"
#include "launch.cuh"

#define WG_THREADS 192
#define WG_BSTAGES 9

struct WgradArgs {
  float* dw;       // partial results: [gridDim.x][C, 9, C]
  int* error;
  int H, W, C;
  int TH, TN, tiles_h, n_tiles;
  int tiles_per_cta;
};

template <int C>
__global__ void __launch_bounds__(WG_THREADS, 1)
conv3x3_wgrad_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x, WgradArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  static_assert(C == 32 || C == 64, "rows of 32 floats are required");
  constexpr int KROWS = 128;                        // reduction rows (pixels) per tile
  constexpr int TILE = KROWS * 128;                 // bytes of one 32-float-wide operand block
  constexpr int A_BLOCKS = C == 64 ? 2 : 1;         // 32-float blocks of dY channels
  constexpr int A_BYTES = A_BLOCKS * TILE;
  uint8_t* sA = smem;                               // 2 buffers
  uint8_t* sB = smem + 2 * A_BYTES;                 // WG_BSTAGES tap tiles
  uint64_t* a_full = reinterpret_cast<uint64_t*>(sB + WG_BSTAGES * TILE);
  uint64_t* a_empty = a_full + 2;
  uint64_t* b_full = a_empty + 2;
  uint64_t* b_empty = b_full + WG_BSTAGES;
  uint64_t* acc_ready = b_empty + WG_BSTAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t_begin = blockIdx.x * g.tiles_per_cta;
  int t_end = t_begin + g.tiles_per_cta;
  if (t_end > g.n_tiles) t_end = g.n_tiles;
  const int n_my = t_end - t_begin;
  const int ci0 = blockIdx.y * 32;                  // input-channel block (C = 64 has two)

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(a_full + s, 1); mbar_init(a_empty + s, 1); }
    for (int s = 0; s < WG_BSTAGES; ++s) { mbar_init(b_full + s, 1); mbar_init(b_empty + s, 1); }
    mbar_init(acc_ready, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  constexpr uint32_t TMEM_COLS = 512;               // 9 accumulators x 32 columns = 288 -> next power of two
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

  if (n_my > 0) {
    if (warp == 4) {
      // ---------------- TMA producer ----------------
      // lane 9 loads the dY tiles, lanes 0..8 one filter tap each: ten threads issue in parallel
      // (a single thread cannot issue bulk-tensor loads fast enough to keep one SM busy)
      if (lane == 9) {
        for (int i = 0; i < n_my && !*abort_flag; ++i) {
          const int tile = t_begin + i;
          const int n0 = (tile / g.tiles_h) * g.TN, h0 = (tile % g.tiles_h) * g.TH;
          const int p0 = (n0 * g.H + h0) * g.W;       // first pixel of the tile
          const int ab = i & 1;
          if (i >= 2 && !mbar_wait(a_empty + ab, ((i >> 1) - 1) & 1)) { *abort_flag = 1; break; }
          mbar_expect_tx(a_full + ab, A_BYTES);
          for (int j = 0; j < A_BLOCKS; ++j)
            tma_load_2d(sA + ab * A_BYTES + j * TILE, &map_dy, a_full + ab, 32 * j, p0);
        }
      } else if (lane < 9) {
        const int tap = lane;
        for (int i = 0; i < n_my && !*abort_flag; ++i) {
          const int tile = t_begin + i;
          const int n0 = (tile / g.tiles_h) * g.TN, h0 = (tile % g.tiles_h) * g.TH;
          const int bcount = i * 9 + tap;
          const int s = bcount % WG_BSTAGES;
          if (bcount >= WG_BSTAGES && !mbar_wait(b_empty + s, ((bcount / WG_BSTAGES) - 1) & 1)) { *abort_flag = 1; break; }
          mbar_expect_tx(b_full + s, TILE);
          tma_load_4d(sB + s * TILE, &map_x, b_full + s, ci0, tap % 3 - 1, h0 + tap / 3 - 1, n0);
        }
      }
    } else if (warp == 5 && lane == 0) {
      // ---------------- MMA issuer ----------------
      // both operands MN-major (bits 15, 16), fp32 accumulate, tf32 inputs, N = 32, M = 128
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) | ((32u >> 3) << 17) |
                             ((128u >> 4) << 24);
      // dY has 32 (or 2 x 32) real channel rows; the 128-row operand repeats them: block stride 0 for
      // one real block, TILE for two (rows 64..127 then read the buffers that follow: ignored garbage)
      constexpr uint32_t A_LBO = A_BLOCKS == 2 ? TILE : 0;
      int bcount = 0;
      bool ok = true;
      for (int i = 0; i < n_my && ok; ++i) {
        const int ab = i & 1;
        if (!mbar_wait(a_full + ab, (i >> 1) & 1)) { *abort_flag = 1; ok = false; break; }
        const uint32_t a_addr = smem_u32(sA + ab * A_BYTES);
        for (int tap = 0; tap < 9 && ok; ++tap, ++bcount) {
          const int s = bcount % WG_BSTAGES;
          if (!mbar_wait(b_full + s, (bcount / WG_BSTAGES) & 1)) { *abort_flag = 1; ok = false; break; }
          tc_fence_after();
          const uint32_t b_addr = smem_u32(sB + s * TILE);
#pragma unroll 4
          for (int k = 0; k < KROWS / 8; ++k)
            umma_tf32(tmem_base + tap * 32, make_desc(a_addr + k * 1024, A_LBO, 512, 1),
                      make_desc(b_addr + k * 1024, 0, 512, 1), idesc, (i > 0 || k > 0) ? 1u : 0u);
          tc_commit(b_empty + s);
        }
        if (ok) tc_commit(a_empty + ab);
      }
      if (ok) tc_commit(acc_ready);
    } else if (warp < 4) {
      // ---------------- epilogue: TMEM -> atomics into dW ----------------
      bool ok = mbar_wait(acc_ready, 0);
      if (!ok) *abort_flag = 1;
      ok = __all_sync(0xffffffffu, ok);
      constexpr int REAL_ROWS = C == 64 ? 64 : 32;
      if (ok && warp * 32 < REAL_ROWS) {
        tc_fence_after();
        const int co = warp * 32 + lane;                    // accumulator row = output channel
#pragma unroll 1
        for (int tap = 0; tap < 9; ++tap) {
#pragma unroll 1
          for (int c = 0; c < 32; c += 16) {
            uint32_t v[16];
            tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(tap * 32 + c), v);
            float* dst = g.dw + (size_t)blockIdx.x * (C * 9 * C) + ((size_t)co * 9 + tap) * C + ci0 + c;
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
          }
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

// ---------------------------------- host side ----------------------------------------------
static int* g_wg_error[64];

static int* wg_error_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (g_wg_error[dev] == nullptr) {
    if (cudaMalloc(&g_wg_error[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(g_wg_error[dev], 0, sizeof(int));
  }
  return g_wg_error[dev];
}

extern "C" int conv3x3_wgrad_last_error() {
  int* w = wg_error_word();
  int v = -1;
  if (w != nullptr) cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

extern "C" int conv3x3_wgrad_supported(int N, int H, int W, int Cin, int Cout) {
  if (Cin != Cout || !(Cin == 32 || Cin == 64)) return 0;
  if (!(W == 8 || W == 16 || W == 32)) return 0;
  int th = 128 / W;
  if (th > H) th = H;
  const int tn = 128 / (W * th);
  if (W * th * tn != 128 || H % th != 0 || N % tn != 0) return 0;
  if (tn > 1 && th != H) return 0;
  return 1;
}

template <int C>
static int launch_wgrad(const CUtensorMap& mdy, const CUtensorMap& mx, const WgradArgs& g, dim3 grid, cudaStream_t st) {
  constexpr int tile = 128 * 128;
  constexpr int smem = 2 * (C == 64 ? 2 : 1) * tile + WG_BSTAGES * tile + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv3x3_wgrad_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_k(conv3x3_wgrad_kernel<C>, dim3(grid), dim3(WG_THREADS), smem, st, mdy, mx, g);
  return (int)cudaGetLastError();
}

// dw[i] = sum over slices of partial[slice][i].  64 outputs per CTA, 4 threads per output: thread q
// adds the slices q, q + 4, ... in order, then the four sub-sums are added in order (reproducible).
__global__ void __launch_bounds__(256) wgrad_reduce_kernel(const float* __restrict__ partial, int n_parts, int n,
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

extern "C" int conv3x3_wgrad_parts(int N, int H, int W) {
  int th = 128 / W;
  if (th > H) th = H;
  const int tn = 128 / (W * th);
  const int n_tiles = (N / tn) * (H / th);
  const int per = (n_tiles + sm_count() - 1) / sm_count();
  return (n_tiles + per - 1) / per;
}

// x, dy: [N, H, W, C] fp32 NHWC; dw: [C, 3, 3, C]; scratch: conv3x3_wgrad_parts() * 9 C C floats.
extern "C" int conv3x3_wgrad_tf32(const void* x, const void* dy, void* dw, void* scratch, int N, int H, int W, int C,
                                  cudaStream_t st) {
  if (!conv3x3_wgrad_supported(N, H, W, C, C)) return -1;
  int th = 128 / W;
  if (th > H) th = H;
  const int tn = 128 / (W * th);
  const long long P = (long long)N * H * W;
  CUtensorMap mdy, mx;
  {
    cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)P};
    cuuint64_t str[1] = {(cuuint64_t)C * 4};
    cuuint32_t box[2] = {32, 128};
    int rc = tc_make_map(&mdy, dy, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc) return rc;
  }
  {
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    cuuint64_t str[3] = {(cuuint64_t)C * 4, (cuuint64_t)W * C * 4, (cuuint64_t)H * W * C * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)W, (cuuint32_t)th, (cuuint32_t)tn};
    int rc = tc_make_map(&mx, x, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc) return rc;
  }
  WgradArgs g;
  g.dw = reinterpret_cast<float*>(scratch);
  g.error = wg_error_word();
  if (g.error == nullptr) return -13;
  g.H = H; g.W = W; g.C = C; g.TH = th; g.TN = tn; g.tiles_h = H / th;
  g.n_tiles = (N / tn) * (H / th);
  g.tiles_per_cta = (g.n_tiles + sm_count() - 1) / sm_count();
  dim3 grid((g.n_tiles + g.tiles_per_cta - 1) / g.tiles_per_cta, C == 64 ? 2 : 1);
  const int rc = C == 32 ? launch_wgrad<32>(mdy, mx, g, grid, st) : launch_wgrad<64>(mdy, mx, g, grid, st);
  if (rc) return rc;
  const int n = C * 9 * C;
  launch_k(wgrad_reduce_kernel, dim3((n + 63) / 64), dim3(256), 0, st, reinterpret_cast<const float*>(scratch), (int)grid.x, n,
                                                       reinterpret_cast<float*>(dw));
  return (int)cudaGetLastError();
}
