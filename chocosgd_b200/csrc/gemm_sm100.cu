// TF32 GEMM on the 5th-generation tensor cores (sm_100a):  D[M,N] (+)= A . B^T (+ bias)
//
//   * operands are staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle,
//     no cluster multicast), 4-stage ring guarded by mbarriers;
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::tf32, M = 128, N = BN);
//     the fp32 accumulator lives in tensor memory (TMEM), allocated by warp 0;
//   * tcgen05.commit releases smem stages and finally signals the epilogue, which reads the
//     accumulator with tcgen05.ld (warp w owns TMEM lanes 32w .. 32w+31 = output rows);
//   * either operand may be K-major ([rows, K], K contiguous) or MN-major ([K, rows], rows
//     contiguous), so forward (x W^T), input-gradient (dY W) and weight-gradient (dY^T x)
//     GEMMs of a linear layer run without any transpose pass;
//   * split-K (gridDim.z) with fp32 atomic accumulation for reductions over a long K with a
//     small output (weight gradients).
//
// Every mbarrier wait is bounded: on expiry the CTA records an error code, skips to the
// teardown (TMEM is always freed) and returns.
#include "tc_common.cuh"
#include "launch.cuh"
#include <stdlib.h>

#define GEMM_BM 128
#define GEMM_BK 32          // tf32 elements per k-block = 128 bytes = one swizzle row
#define GEMM_STAGES 4
#define GEMM_THREADS 192    // warps 0-3: epilogue (warp 0 also owns TMEM), warp 4: TMA, warp 5: MMA

#define GEMM_ERR_TIMEOUT 1

struct GemmArgs {
  float* d;            // [M, N] row-major, ldd elements per row
  const float* bias;   // [N] or null
  int* error;          // device word, set non-zero on a timed-out wait
  int M, N, K, ldd;
  int k_blocks_per_split;
  int relu;
  int passes;          // 1: plain TF32;  3: split-operand passes (hi.hi + hi.lo + lo.hi), see gemm_tf32x3
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b_lo, GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address bits
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int A_BYTES = GEMM_BM * GEMM_BK * 4;  // 16 KiB
  constexpr int B_BYTES = BN * GEMM_BK * 4;
  uint8_t* sA = smem;
  uint8_t* sB = smem + GEMM_STAGES * A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + GEMM_STAGES * B_BYTES);
  uint64_t* empty = full + GEMM_STAGES;
  uint64_t* acc_ready = empty + GEMM_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * GEMM_BM, n0 = blockIdx.y * BN;
  const int total_kb = (g.K + GEMM_BK - 1) / GEMM_BK;
  const int kb_begin = blockIdx.z * g.k_blocks_per_split;
  int kb_end = kb_begin + g.k_blocks_per_split;
  if (kb_end > total_kb) kb_end = total_kb;
  const int n_kb1 = kb_end - kb_begin;
  // split-operand product (passes == 3): one pipeline stage holds A_hi, A_lo, B_hi, B_lo of a k-block and
  // feeds the three MMA groups hi.hi, hi.lo, lo.hi (every operand tile is fetched once)
  const bool x3 = g.passes == 3;
  const int n_kb = n_kb1;
  const int NST = x3 ? GEMM_STAGES / 2 : GEMM_STAGES;
  const int SA = x3 ? 2 * A_BYTES : A_BYTES, SB = x3 ? 2 * B_BYTES : B_BYTES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GEMM_STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_ready, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (n_kb > 0) {
    if (warp == 4 && lane == 0) {
      // ---------------- TMA producer ----------------
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % NST;
        if (i >= NST && !mbar_wait(empty + s, ((i / NST) - 1) & 1)) { *abort_flag = 1; break; }
        if (*abort_flag) break;
        const int k0 = (kb_begin + i) * GEMM_BK;
        mbar_expect_tx(full + s, SA + SB);
        for (int half = 0; half < (x3 ? 2 : 1); ++half) {
          const CUtensorMap* pa = half ? &map_a_lo : &map_a;
          const CUtensorMap* pb = half ? &map_b_lo : &map_b;
          uint8_t* dA = sA + s * SA + half * A_BYTES;
          uint8_t* dB = sB + s * SB + half * B_BYTES;
          if (!A_MN) {
            tma_load_2d(dA, pa, full + s, k0, m0);
          } else {
            for (int j = 0; j < GEMM_BM / 32; ++j) tma_load_2d(dA + j * 4096, pa, full + s, m0 + 32 * j, k0);
          }
          if (!B_MN) {
            tma_load_2d(dB, pb, full + s, k0, n0);
          } else {
            for (int j = 0; j < BN / 32; ++j) tma_load_2d(dB + j * 4096, pb, full + s, n0 + 32 * j, k0);
          }
        }
      }
    } else if (warp == 5 && lane == 0) {
      // ---------------- MMA issuer ----------------
      // instruction descriptor: fp32 accumulate, tf32 x tf32, majorness bits, N >> 3, M >> 4
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(GEMM_BM >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % NST;
        if (!mbar_wait(full + s, (i / NST) & 1)) { *abort_flag = 1; ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + s * SA), b_addr = smem_u32(sB + s * SB);
#pragma unroll
        for (int k = 0; k < GEMM_BK / 8; ++k) {
          // K-major: 32 bytes further inside the 128-byte row; MN-major: next 8 k-rows (two
          // 4-row atoms, 512 bytes apart; 32-element MN blocks are 4096 bytes apart)
          const uint64_t da = A_MN ? make_desc(a_addr + k * 1024, 4096, 512, 1) : make_desc(a_addr + k * 32, 16, 1024);
          const uint64_t db = B_MN ? make_desc(b_addr + k * 1024, 4096, 512, 1) : make_desc(b_addr + k * 32, 16, 1024);
          umma_tf32(tmem_base, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
          if (x3) {
            const uint32_t al = a_addr + A_BYTES, bl = b_addr + B_BYTES;
            const uint64_t dal = A_MN ? make_desc(al + k * 1024, 4096, 512, 1) : make_desc(al + k * 32, 16, 1024);
            const uint64_t dbl = B_MN ? make_desc(bl + k * 1024, 4096, 512, 1) : make_desc(bl + k * 32, 16, 1024);
            umma_tf32(tmem_base, da, dbl, idesc, 1u);   // hi . lo
            umma_tf32(tmem_base, dal, db, idesc, 1u);   // lo . hi
          }
        }
        tc_commit(empty + s);  // frees this stage once the MMAs above have read it
      }
      if (ok) tc_commit(acc_ready);
    } else if (warp < 4) {
      // ---------------- epilogue: TMEM -> registers -> global ----------------
      bool ok = mbar_wait(acc_ready, 0);
      if (!ok) *abort_flag = 1;
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const int row = m0 + warp * 32 + lane;
        const bool split = gridDim.z > 1;
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c, r);
          if (row < g.M) {
            float* out = g.d + (size_t)row * g.ldd + n0 + c;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int col = n0 + c + j;
              if (col < g.N) {
                float v = __uint_as_float(r[j]);
                if (g.bias != nullptr && blockIdx.z == 0) v += g.bias[col];
                if (split) atomicAdd(out + j, v);
                else out[j] = g.relu ? fmaxf(v, 0.f) : v;
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(g.error, GEMM_ERR_TIMEOUT);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- persistent variant ---------------------------------------------------------------------------
// One CTA per SM walks over output tiles (tile t = blockIdx.x, + gridDim.x, ...; M-tiles vary
// fastest so that the CTAs running at one time share B panels in L2).  The TMA producer keeps
// running ahead across tile boundaries and the accumulator is double-buffered in TMEM (2 x BN of
// the 512 columns), so the epilogue of tile t overlaps the multiplications of tile t + 1.
// Used when there is no split-K and the tile count covers the machine a few times.
__device__ __forceinline__ bool gemm_epi_bar_or(bool flag) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "r"((uint32_t)flag) : "memory");
  return r != 0;
}

// X3: the split-operand product with its three passes fused per k-block: a pipeline stage holds A_hi, A_lo,
// B_hi and B_lo of one k-block (four TMA loads) and feeds three MMA groups (hi.hi, hi.lo, lo.hi), so every
// operand tile is fetched once instead of twice: a third less L2 -> shared-memory traffic per FLOP.
template <int BN, bool A_MN, bool B_MN, bool X3>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tf32_persist_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b_lo,
                         GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int A_BYTES = GEMM_BM * GEMM_BK * 4;
  constexpr int B_BYTES = BN * GEMM_BK * 4;
  constexpr int NST = X3 ? GEMM_STAGES / 2 : GEMM_STAGES;       // stages (an X3 stage is twice as large)
  constexpr int SA = X3 ? 2 * A_BYTES : A_BYTES, SB = X3 ? 2 * B_BYTES : B_BYTES;
  uint8_t* sA = smem;
  uint8_t* sB = smem + NST * SA;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + NST * SB);
  uint64_t* empty = full + NST;
  uint64_t* acc_full = empty + NST;   // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (g.M + GEMM_BM - 1) / GEMM_BM, tiles_n = (g.N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb1 = (g.K + GEMM_BK - 1) / GEMM_BK;
  const int n_kb = X3 ? n_kb1 : n_kb1 * g.passes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
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
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ---------------- TMA producer: lane 0 waits and arms the barrier, lanes 0..P-1 issue one box each ------------
    constexpr int PA = A_MN ? GEMM_BM / 32 : 1, PB = B_MN ? BN / 32 : 1;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      const int m0 = (tile % tiles_m) * GEMM_BM, n0 = (tile / tiles_m) * BN;
      int ok = 1;
      for (int i = 0; i < n_kb; ++i, ++it) {
        const uint32_t s = it % NST;
        if (lane == 0) {
          if (it >= NST && !mbar_wait(empty + s, ((it / NST) - 1) & 1)) ok = 0;
          if (*abort_flag) ok = 0;
          if (ok) mbar_expect_tx(full + s, SA + SB);
          else *abort_flag = 1;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const int pass = X3 ? 0 : i / n_kb1;
        const int k0 = (i % n_kb1) * GEMM_BK;
        // lanes [0, PA + PB): the (hi) tiles of this iteration; X3: lanes [PA + PB, 2 (PA + PB)) the lo tiles
        const int half = X3 ? lane / (PA + PB) : 0, l = X3 ? lane % (PA + PB) : lane;
        const CUtensorMap* pa = (X3 ? half == 1 : pass == 2) ? &map_a_lo : &map_a;   // passes: (A, B), (A, B_lo), (A_lo, B)
        const CUtensorMap* pb = (X3 ? half == 1 : pass == 1) ? &map_b_lo : &map_b;
        if (half < (X3 ? 2 : 1)) {
          if (l < PA) {
            uint8_t* dst = sA + s * SA + half * A_BYTES;
            if (!A_MN) tma_load_2d(dst, pa, full + s, k0, m0);
            else tma_load_2d(dst + l * 4096, pa, full + s, m0 + 32 * l, k0);
          } else if (l < PA + PB) {
            const int j = l - PA;
            uint8_t* dst = sB + s * SB + half * B_BYTES;
            if (!B_MN) tma_load_2d(dst, pb, full + s, k0, n0);
            else tma_load_2d(dst + j * 4096, pb, full + s, n0 + 32 * j, k0);
          }
        }
        __syncwarp();
      }
      if (!ok) break;
    }
  } else if (warp == 5 && lane == 0) {
    // ---------------- MMA issuer ----------------
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(GEMM_BM >> 4) << 24);
    uint32_t it = 0, lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      if (lt >= 2 && !mbar_wait(acc_empty + buf, ((lt >> 1) - 1) & 1)) { *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      const uint32_t d = tmem_base + buf * BN;
      for (int i = 0; i < n_kb; ++i, ++it) {
        const uint32_t s = it % NST;
        if (!mbar_wait(full + s, (it / NST) & 1)) { *abort_flag = 1; ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + s * SA), b_addr = smem_u32(sB + s * SB);
#pragma unroll
        for (int k = 0; k < GEMM_BK / 8; ++k) {
          const uint64_t da = A_MN ? make_desc(a_addr + k * 1024, 4096, 512, 1) : make_desc(a_addr + k * 32, 16, 1024);
          const uint64_t db = B_MN ? make_desc(b_addr + k * 1024, 4096, 512, 1) : make_desc(b_addr + k * 32, 16, 1024);
          umma_tf32(d, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
          if (X3) {
            const uint32_t al = a_addr + A_BYTES, bl = b_addr + B_BYTES;
            const uint64_t dal = A_MN ? make_desc(al + k * 1024, 4096, 512, 1) : make_desc(al + k * 32, 16, 1024);
            const uint64_t dbl = B_MN ? make_desc(bl + k * 1024, 4096, 512, 1) : make_desc(bl + k * 32, 16, 1024);
            umma_tf32(d, da, dbl, idesc, 1u);   // hi . lo
            umma_tf32(d, dal, db, idesc, 1u);   // lo . hi
          }
        }
        tc_commit(empty + s);
      }
      if (ok) tc_commit(acc_full + buf);
    }
  } else if (warp < 4) {
    // ---------------- epilogue: TMEM -> registers -> global, overlapped with the next tile ----------------
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++lt) {
      const uint32_t buf = lt & 1;
      const bool bad = !mbar_wait(acc_full + buf, (lt >> 1) & 1) || *abort_flag != 0;
      if (gemm_epi_bar_or(bad)) {   // the same decision in all 128 epilogue threads
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int m0 = (tile % tiles_m) * GEMM_BM, n0 = (tile / tiles_m) * BN;
      const int row = m0 + warp * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BN + (uint32_t)c, r);
        if (row < g.M && n0 + c < g.N) {
          float* out = g.d + (size_t)row * g.ldd + n0 + c;
          if (n0 + c + 16 <= g.N && (g.ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(g.d) & 15) == 0 &&
              (reinterpret_cast<uintptr_t>(g.bias) & 15) == 0) {   // n0 + c is a multiple of 16
            // full chunk: four 16-byte stores
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
              float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                     __uint_as_float(r[j + 3]));
              if (g.bias != nullptr) {
                const float4 bv = *reinterpret_cast<const float4*>(g.bias + n0 + c + j);
                v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
              }
              if (g.relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
              *reinterpret_cast<float4*>(out + j) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int col = n0 + c + j;
              if (col < g.N) {
                float v = __uint_as_float(r[j]);
                if (g.bias != nullptr) v += g.bias[col];
                out[j] = g.relu ? fmaxf(v, 0.f) : v;
              }
            }
          }
        }
      }
      // the accumulator buffer may be overwritten by the tile after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buf);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(g.error, GEMM_ERR_TIMEOUT);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------- host side ----------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-d fp32 tensor map: inner (contiguous) extent `inner`, `outer` rows of `row_stride` elements
static int make_map_2d(CUtensorMap* map, const void* base, long long inner, long long outer, long long row_stride,
                       int box_inner, int box_outer, bool mn_major) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride * 4) % 16 != 0) return -11;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride * 4};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

static int* g_gemm_error[64];

static int* gemm_error_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (g_gemm_error[dev] == nullptr) {
    if (cudaMalloc(&g_gemm_error[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(g_gemm_error[dev], 0, sizeof(int));
  }
  return g_gemm_error[dev];
}

extern "C" int gemm_tf32_last_error() {
  int* w = gemm_error_word();
  int v = -1;
  if (w != nullptr) cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mal, const CUtensorMap& mbl,
                       const GemmArgs& g, int splits, cudaStream_t st) {
  constexpr int smem = GEMM_STAGES * (GEMM_BM * GEMM_BK * 4 + BN * GEMM_BK * 4) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_kernel<BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((g.M + GEMM_BM - 1) / GEMM_BM, (g.N + BN - 1) / BN, splits);
  gemm_tf32_kernel<BN, A_MN, B_MN><<<grid, GEMM_THREADS, smem, st>>>(ma, mb, mal, mbl, g);
  return (int)cudaGetLastError();
}

template <int BN, bool A_MN, bool B_MN, bool X3>
static int launch_gemm_persist_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mal,
                                 const CUtensorMap& mbl, const GemmArgs& g, int grid, cudaStream_t st) {
  constexpr int smem = GEMM_STAGES * (GEMM_BM * GEMM_BK * 4 + BN * GEMM_BK * 4) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_persist_kernel<BN, A_MN, B_MN, X3>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  gemm_tf32_persist_kernel<BN, A_MN, B_MN, X3><<<grid, GEMM_THREADS, smem, st>>>(ma, mb, mal, mbl, g);
  return (int)cudaGetLastError();
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm_persist(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mal,
                               const CUtensorMap& mbl, const GemmArgs& g, int grid, cudaStream_t st) {
  // the fused three-pass form needs 2 (PA + PB) producer lanes: 24 at most (MN-major 128 x 256 tiles)
  static int fused = -1;
  if (fused < 0) {
    const char* e = getenv("CHOCO_GEMM_X3_FUSED");
    fused = e == nullptr || atoi(e) != 0;
  }
  if (g.passes == 3 && fused) return launch_gemm_persist_t<BN, A_MN, B_MN, true>(ma, mb, mal, mbl, g, grid, st);
  return launch_gemm_persist_t<BN, A_MN, B_MN, false>(ma, mb, mal, mbl, g, grid, st);
}

template <int BN>
static int dispatch_persist(bool a_mn, bool b_mn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mal,
                            const CUtensorMap& mbl, const GemmArgs& g, int grid, cudaStream_t st) {
  if (!a_mn && !b_mn) return launch_gemm_persist<BN, false, false>(ma, mb, mal, mbl, g, grid, st);
  if (!a_mn && b_mn) return launch_gemm_persist<BN, false, true>(ma, mb, mal, mbl, g, grid, st);
  if (a_mn && !b_mn) return launch_gemm_persist<BN, true, false>(ma, mb, mal, mbl, g, grid, st);
  return launch_gemm_persist<BN, true, true>(ma, mb, mal, mbl, g, grid, st);
}

template <int BN>
static int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mal,
                          const CUtensorMap& mbl, const GemmArgs& g, int splits, cudaStream_t st) {
  if (!a_mn && !b_mn) return launch_gemm<BN, false, false>(ma, mb, mal, mbl, g, splits, st);
  if (!a_mn && b_mn) return launch_gemm<BN, false, true>(ma, mb, mal, mbl, g, splits, st);
  if (a_mn && !b_mn) return launch_gemm<BN, true, false>(ma, mb, mal, mbl, g, splits, st);
  return launch_gemm<BN, true, true>(ma, mb, mal, mbl, g, splits, st);
}

// D[M,N] = A . B^T (+ bias).  a_mn = 0: A is [M, K] (K contiguous, lda);  a_mn = 1: A is [K, M].
// Same for B with N rows.  split_k > 1 accumulates with atomics into D, which the caller zeroed.
// a_lo / b_lo non-null: three passes over K accumulate  A.B + A.B_lo + A_lo.B  into the same TMEM
// accumulator (operands given as exact TF32 values plus their fp32 remainders, see tf32_split_pad):
// products carry 2^-21 relative error instead of TF32's 2^-10, at three times the tensor-core work.
static int gemm_run(const void* a, const void* a_lo, const void* b, const void* b_lo, void* d, const void* bias, int M,
                    int N, int K, int lda, int ldb, int ldd, int a_mn, int b_mn, int split_k, int relu,
                    cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((a_lo == nullptr) != (b_lo == nullptr)) return -1;
  // 256-wide tiles when the grid still fills the machine: with 4-byte operands a 128 x 128 tile reads
  // shared memory as fast as the tensor core consumes it; 128 x 256 needs 25 % less per FLOP
  const long long tiles256 = (long long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + 255) / 256);
  const int BN = N <= 32 ? 32 : (N <= 64 ? 64 : ((N >= 256 && tiles256 >= 120 && split_k <= 1) ? 256 : 128));
  CUtensorMap ma, mb, mal, mbl;
  for (int which = 0; which < 2; ++which) {
    const void* pa = which ? a_lo : a;
    const void* pb = which ? b_lo : b;
    if (pa == nullptr) { mal = ma; mbl = mb; break; }
    int rc = a_mn ? make_map_2d(which ? &mal : &ma, pa, M, K, lda, 32, GEMM_BK, true)
                  : make_map_2d(which ? &mal : &ma, pa, K, M, lda, GEMM_BK, GEMM_BM, false);
    if (rc) return rc;
    rc = b_mn ? make_map_2d(which ? &mbl : &mb, pb, N, K, ldb, 32, GEMM_BK, true)
              : make_map_2d(which ? &mbl : &mb, pb, K, N, ldb, GEMM_BK, BN, false);
    if (rc) return rc;
  }
  GemmArgs g;
  g.d = reinterpret_cast<float*>(d);
  g.bias = reinterpret_cast<const float*>(bias);
  g.error = gemm_error_word();
  if (g.error == nullptr) return -13;
  g.M = M; g.N = N; g.K = K; g.ldd = ldd; g.relu = relu;
  g.passes = a_lo != nullptr ? 3 : 1;
  const int total_kb = (K + GEMM_BK - 1) / GEMM_BK;
  int splits = split_k < 1 ? 1 : split_k;
  if (splits > total_kb) splits = total_kb;
  g.k_blocks_per_split = (total_kb + splits - 1) / splits;
  splits = (total_kb + g.k_blocks_per_split - 1) / g.k_blocks_per_split;
  if (splits == 1 && (BN == 128 || BN == 256)) {
    // persistent form when the tiles cover the machine at least twice (epilogue / multiply overlap)
    static int sms = 0, enabled = -1;
    if (enabled < 0) {
      const char* e = getenv("CHOCO_GEMM_PERSISTENT");
      enabled = e == nullptr || atoi(e) != 0;   // 541 against 457 TFLOP/s at 4096^3, 605 against 596 at 8192^3
      int dev = 0;
      cudaGetDevice(&dev);
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
    }
    const long long tiles = (long long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
    if (enabled && tiles >= 2LL * sms) {
      const int grid = sms;
      return BN == 256 ? dispatch_persist<256>(a_mn, b_mn, ma, mb, mal, mbl, g, grid, stream)
                       : dispatch_persist<128>(a_mn, b_mn, ma, mb, mal, mbl, g, grid, stream);
    }
  }
  if (BN == 32) return dispatch_major<32>(a_mn, b_mn, ma, mb, mal, mbl, g, splits, stream);
  if (BN == 64) return dispatch_major<64>(a_mn, b_mn, ma, mb, mal, mbl, g, splits, stream);
  if (BN == 256) return dispatch_major<256>(a_mn, b_mn, ma, mb, mal, mbl, g, splits, stream);
  return dispatch_major<128>(a_mn, b_mn, ma, mb, mal, mbl, g, splits, stream);
}

extern "C" int gemm_tf32(const void* a, const void* b, void* d, const void* bias, int M, int N, int K, int lda, int ldb,
                         int ldd, int a_mn, int b_mn, int split_k, int relu, cudaStream_t stream) {
  return gemm_run(a, nullptr, b, nullptr, d, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, split_k, relu, stream);
}

// fp32-grade product on the TF32 tensor cores (the "3xTF32" scheme): operands come as (hi, lo) pairs
// from tf32_split_pad with the same leading dimension.
extern "C" int gemm_tf32x3(const void* a_hi, const void* a_lo, const void* b_hi, const void* b_lo, void* d,
                           const void* bias, int M, int N, int K, int lda, int ldb, int ldd, int a_mn, int b_mn,
                           int split_k, int relu, cudaStream_t stream) {
  if (a_lo == nullptr || b_lo == nullptr) return -1;
  return gemm_run(a_hi, a_lo, b_hi, b_lo, d, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, split_k, relu, stream);
}

// hi = x with the 13 low mantissa bits cleared (an exact TF32 value), lo = x - hi (exact in fp32), both
// written with `ldd` floats per row (ldd >= cols, a multiple of 4 so that rows are 16-byte aligned for
// TMA; the tail columns are zero).  One pass: 4 bytes read, 8 written per element.
__global__ void tf32_split_pad_kernel(const float* __restrict__ src, long long rows, int cols, long long lds,
                                      float* __restrict__ hi, float* __restrict__ lo, int ldd) {
  const long long total = rows * (long long)(ldd / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (ldd / 4);
    const int c = (int)(i % (ldd / 4)) * 4;
    float v[4], h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[e] = (c + e < cols) ? src[r * lds + c + e] : 0.f;
      h[e] = __uint_as_float(__float_as_uint(v[e]) & 0xFFFFE000u);
      l[e] = v[e] - h[e];
    }
    *reinterpret_cast<float4*>(hi + r * ldd + c) = make_float4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<float4*>(lo + r * ldd + c) = make_float4(l[0], l[1], l[2], l[3]);
  }
}

extern "C" int tf32_split_pad(const void* src, long long rows, int cols, long long lds, void* hi, void* lo, int ldd,
                              cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || ldd < cols || ldd % 4 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(hi) & 15) != 0 || (reinterpret_cast<uintptr_t>(lo) & 15) != 0) return -1;
  long long blocks = (rows * (ldd / 4) + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  tf32_split_pad_kernel<<<(int)blocks, 256, 0, st>>>(reinterpret_cast<const float*>(src), rows, cols, lds,
                                                    reinterpret_cast<float*>(hi), reinterpret_cast<float*>(lo), ldd);
  return (int)cudaGetLastError();
}
