// Persistent recurrent kernels of one LSTM layer (gate order i, f, g, o as in torch.nn.LSTM).
//
// The input projection of all time steps is one large GEMM outside; what remains is the chain
//   pre_t = proj_t + h_{t-1} W_hh^T ;  cell ;  h_t        (T dependent steps, [B, H] x [H, 4H] each)
// which a library runs as one small GEMM plus pointwise kernels per step (70 + 70 launches of
// 17 us for T = 35 and two layers).  Here ONE kernel per layer and direction walks over all steps:
//   * CTA c owns `upc` hidden units: the 4 upc rows of W_hh that produce their gates stay in shared
//     memory for the whole sequence (forward), and the matching upc columns of W_hh (backward);
//   * per step every CTA reads the full h_{t-1} (forward) or the full d(pre-activation) vector of
//     step t+1 (backward) that all CTAs wrote in the step before, separated by a grid-wide barrier
//     (one CTA per SM, all co-resident; the wait is bounded and reports through an error word);
//   * fp32 FMA arithmetic (the operation is bound by the barrier and the L2 reads, not by math).
// The cell state derivative lives in registers for the whole backward sweep.
// Replaces the per-step launches of dl_code/pcode/models/rnn_lm.py:29 (torch.nn.LSTM) on the
// native path; B <= 32, shared memory permitting (H = 650: 140 KB).
#include <cuda_runtime.h>
#include <stdint.h>

#define LP_THREADS 512     // 16 warps: four per scheduler hide the shared-memory and FMA latencies
#define LP_WARPS 16
#define LP_HSTRIDE 33      // h is kept transposed [k][b] with a padded row: conflict-free both ways
#define LP_UPC_MAX 8
#define LP_CHUNK 256        // rows of d(pre) per staged chunk (32 KB)

struct LstmRecArgs {
  float* gates;          // [T][B][4H]  fwd: projections in, activations out; bwd: activations in, d(pre) out
  const float* w_hh;     // [4H][H]
  float* hs;             // [T+1][B][H], hs[0] = h0
  float* cs;             // [T+1][B][H], cs[0] = c0
  const float* d_out;    // bwd: [T][B][H] or null
  float* dh;             // bwd: [B][H] in: d h_T, out: d h_0
  float* dc;             // bwd: [B][H] in: d c_T, out: d c_0
  float* dgt;            // bwd scratch: [2][4H][32] transposed d(pre) of the step just finished
  unsigned* barrier;     // [0] arrivals, [1] generation, [2] error flag
  int T, B, H, upc;
};

__device__ __forceinline__ float lp_sigm(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ unsigned lp_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier for co-resident CTAs; false when the bounded wait ran out.
__device__ __forceinline__ bool lp_grid_barrier(unsigned* bar, int* sh_ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    const unsigned gen = lp_ld_acquire(bar + 1);
    __threadfence();
    if (atomicAdd(bar, 1u) == gridDim.x - 1) {
      *bar = 0;
      __threadfence();
      atomicAdd(bar + 1, 1u);
    } else {
      unsigned spins = 0;
      while (lp_ld_acquire(bar + 1) == gen) {
        __nanosleep(20);
        if (++spins > (1u << 24)) { ok = 0; atomicExch(bar + 2, 1u); break; }
      }
    }
    *sh_ok = ok;
  }
  __syncthreads();
  return *sh_ok != 0;
}

__global__ void __launch_bounds__(LP_THREADS, 1) lstm_rec_fwd_kernel(LstmRecArgs a) {
  extern __shared__ float lp_smem[];
  __shared__ int sh_ok;
  const int H = a.H, B = a.B, upc = a.upc, rows = 4 * upc;   // rows is a multiple of 4
  const int HP = (H + 3) & ~3;
  float* Wk = lp_smem;                         // [HP][rows]: W_hh[row r][k] stored k-major (rows contiguous)
  float* hT = Wk + (size_t)HP * rows;          // [HP][LP_HSTRIDE]: h_{t-1} transposed
  float* part = hT + (size_t)HP * LP_HSTRIDE;  // [LP_WARPS][rows][32] partial dot products per K-slice
  const int u0 = blockIdx.x * upc;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int idx = threadIdx.x; idx < rows * HP; idx += LP_THREADS) {
    const int r = idx / HP, k = idx - r * HP;      // coalesced reads along k
    const int g = r / upc, u = u0 + (r - g * upc);
    Wk[(size_t)k * rows + r] = (u < H && k < H) ? a.w_hh[((size_t)g * H + u) * H + k] : 0.f;
  }
  for (int idx = threadIdx.x; idx < HP * LP_HSTRIDE; idx += LP_THREADS) hT[idx] = 0.f;
  __syncthreads();
  // warp w multiplies the K-slice [k_lo, k_hi) for ALL rows of the CTA (lane = sample)
  const int kpw = (HP + LP_WARPS - 1) / LP_WARPS;
  const int k_lo = warp * kpw, k_hi = min(HP, k_lo + kpw);

  for (int t = 0; t < a.T; ++t) {
    // h_{t-1} of all units (written by all CTAs in the previous step): every load of a thread is
    // issued before the first use, so the copy costs about one L2 round trip
    const float* hprev = a.hs + (size_t)t * B * H;
    for (int b = warp; b < B; b += LP_WARPS) {
      const float* row = hprev + (size_t)b * H;
      for (int k0 = lane; k0 < H; k0 += 32 * 8) {      // eight coalesced loads in flight per lane
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = k0 + q * 32 < H ? __ldcg(row + k0 + q * 32) : 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (k0 + q * 32 < H) hT[(k0 + q * 32) * LP_HSTRIDE + b] = v[q];
      }
    }
    float* gt = a.gates + (size_t)t * B * 4 * H;
    // projection values of this CTA's (unit, gate, sample) triples, fetched while the dot products run
    float proj[2] = {0.f, 0.f};
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int idx = threadIdx.x + q * LP_THREADS;       // idx -> (row r, sample b)
      const int r = idx >> 5, bb = idx & 31;
      if (r < rows) {
        const int g = r / upc, u = u0 + (r - g * upc);
        if (bb < B && u < H) proj[q] = __ldcg(gt + (size_t)bb * 4 * H + (size_t)g * H + u);
      }
    }
    __syncthreads();
    // partial[r] = sum over the warp's K-slice of h[lane][k] W[r][k]
    float acc[4 * LP_UPC_MAX];
#pragma unroll
    for (int r = 0; r < 4 * LP_UPC_MAX; ++r) acc[r] = 0.f;
    for (int k = k_lo; k < k_hi; ++k) {
      const float hv = hT[k * LP_HSTRIDE + lane];
      const float* wk = Wk + (size_t)k * rows;
#pragma unroll
      for (int r4 = 0; r4 < LP_UPC_MAX; ++r4) {
        if (r4 * 4 < rows) {
          const float4 w4 = *reinterpret_cast<const float4*>(wk + r4 * 4);
          acc[r4 * 4 + 0] = fmaf(hv, w4.x, acc[r4 * 4 + 0]);
          acc[r4 * 4 + 1] = fmaf(hv, w4.y, acc[r4 * 4 + 1]);
          acc[r4 * 4 + 2] = fmaf(hv, w4.z, acc[r4 * 4 + 2]);
          acc[r4 * 4 + 3] = fmaf(hv, w4.w, acc[r4 * 4 + 3]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 4 * LP_UPC_MAX; ++r)
      if (r < rows) part[((size_t)warp * rows + r) * 32 + lane] = acc[r];
    __syncthreads();
    // add the K-slices in a fixed order; thread idx -> (row, sample) as for proj
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int idx = threadIdx.x + q * LP_THREADS;
      const int r = idx >> 5;
      if (r < rows) {
        float sum = proj[q];
        for (int w = 0; w < LP_WARPS; ++w) sum += part[((size_t)w * rows + r) * 32 + (idx & 31)];
        part[(size_t)r * 32 + (idx & 31)] = sum;   // slice 0 is complete at this point for this element only
      }
    }
    __syncthreads();
    // cell for this CTA's units (pre-activations in part[row][sample])
    for (int idx = threadIdx.x; idx < upc * 32; idx += LP_THREADS) {
      const int j = idx >> 5, bq = idx & 31, u = u0 + j;
      if (bq < B && u < H) {
        const float i = lp_sigm(part[(0 * upc + j) * 32 + bq]), f = lp_sigm(part[(1 * upc + j) * 32 + bq]);
        const float gg = tanhf(part[(2 * upc + j) * 32 + bq]), o = lp_sigm(part[(3 * upc + j) * 32 + bq]);
        const size_t hi = (size_t)bq * H + u;
        const float cn = fmaf(f, __ldcg(a.cs + (size_t)t * B * H + hi), i * gg);
        a.cs[(size_t)(t + 1) * B * H + hi] = cn;
        a.hs[(size_t)(t + 1) * B * H + hi] = o * tanhf(cn);
        float* gb = gt + (size_t)bq * 4 * H + u;
        gb[0] = i; gb[(size_t)H] = f; gb[(size_t)2 * H] = gg; gb[(size_t)3 * H] = o;
      }
    }
    if (t + 1 < a.T && !lp_grid_barrier(a.barrier, &sh_ok)) return;
  }
}

__global__ void __launch_bounds__(LP_THREADS, 1) lstm_rec_bwd_kernel(LstmRecArgs a) {
  extern __shared__ float lp_smem[];
  __shared__ int sh_ok;
  const int H = a.H, B = a.B, upc = a.upc, R = 4 * H;
  const int RP = (R + LP_CHUNK - 1) / LP_CHUNK * LP_CHUNK;   // rows padded to whole chunks (zeros)
  float* WT = lp_smem;                             // [RP][LP_UPC_MAX]: W_hh[r][u0 + j]
  float* red = WT + (size_t)RP * LP_UPC_MAX;       // [LP_WARPS][upc][32]
  float* stage = red + (size_t)LP_WARPS * LP_UPC_MAX * 32;   // [2][LP_CHUNK][32]
  const int u0 = blockIdx.x * upc;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int idx = threadIdx.x; idx < RP * LP_UPC_MAX; idx += LP_THREADS) {
    const int r = idx / LP_UPC_MAX, j = idx - r * LP_UPC_MAX;
    WT[idx] = (r < R && j < upc && u0 + j < H) ? a.w_hh[(size_t)r * H + u0 + j] : 0.f;
  }
  for (int idx = threadIdx.x; idx < 2 * LP_CHUNK * 32; idx += LP_THREADS) stage[idx] = 0.f;   // rows past 4H stay zero
  __syncthreads();
  // thread (j, b) of the first upc warps owns unit u0 + j of sample b for the whole sweep
  const int oj = threadIdx.x >> 5, ob = lane;
  const bool owner = oj < upc && ob < B && u0 + oj < H;
  const size_t ohi = (size_t)ob * H + u0 + oj;
  float dc_reg = owner ? a.dc[ohi] : 0.f;
  float dh_rec = owner ? a.dh[ohi] : 0.f;

  for (int t = a.T - 1; t >= -1; --t) {
    if (t < a.T - 1) {
      // dh_rec[b][j] = sum_r dG_{t+1}[r][b] W_hh[r][u0 + j]; the barrier below made dG_{t+1} visible
      const float* dg = a.dgt + (size_t)((t + 1) & 1) * R * 32;
      float acc[LP_UPC_MAX];
#pragma unroll
      for (int j = 0; j < LP_UPC_MAX; ++j) acc[j] = 0.f;
      // the whole d(pre) vector of step t+1 ([4H][32], 333 KB for H = 650) streams through two
      // 32 KB shared-memory buffers with 16-byte asynchronous copies; warp w multiplies rows
      // [32 w, 32 w + 32) of each chunk
      const int n_chunks = (R + LP_CHUNK - 1) / LP_CHUNK;
      auto issue = [&](int c) {
        float* dst = stage + (size_t)(c & 1) * LP_CHUNK * 32;
        const int row0 = c * LP_CHUNK;
        for (int piece = threadIdx.x; piece < LP_CHUNK * 8; piece += LP_THREADS) {   // 8 pieces of 16 B per row
          const int rr = piece >> 3;
          if (row0 + rr < R) {
            const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst + (size_t)piece * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(dg + ((size_t)row0 * 32 + (size_t)piece * 4))
                         : "memory");
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      };
      issue(0);
      for (int c = 0; c < n_chunks; ++c) {
        if (c + 1 < n_chunks) {
          issue(c + 1);
          asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
          asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* src = stage + (size_t)(c & 1) * LP_CHUNK * 32;
        const int rbase = c * LP_CHUNK + warp * (LP_CHUNK / LP_WARPS);
#pragma unroll 8
        for (int q = 0; q < LP_CHUNK / LP_WARPS; ++q) {
          const int r = rbase + q;
          const float gval = src[(size_t)(warp * (LP_CHUNK / LP_WARPS) + q) * 32 + lane];
          const float4 w0 = *reinterpret_cast<const float4*>(WT + (size_t)r * LP_UPC_MAX);
          const float4 w1 = *reinterpret_cast<const float4*>(WT + (size_t)r * LP_UPC_MAX + 4);
          acc[0] = fmaf(gval, w0.x, acc[0]); acc[1] = fmaf(gval, w0.y, acc[1]);
          acc[2] = fmaf(gval, w0.z, acc[2]); acc[3] = fmaf(gval, w0.w, acc[3]);
          acc[4] = fmaf(gval, w1.x, acc[4]); acc[5] = fmaf(gval, w1.y, acc[5]);
          acc[6] = fmaf(gval, w1.z, acc[6]); acc[7] = fmaf(gval, w1.w, acc[7]);
        }
        __syncthreads();   // the buffer is refilled by the copy issued in the next iteration
      }
#pragma unroll
      for (int j = 0; j < LP_UPC_MAX; ++j)
        if (j < upc) red[(warp * upc + j) * 32 + lane] = acc[j];
      __syncthreads();
      if (oj < upc) {
        float s = 0.f;
        for (int w = 0; w < LP_WARPS; ++w) s += red[(w * upc + oj) * 32 + ob];   // fixed order
        dh_rec = s;
      }
      __syncthreads();
    }
    if (t < 0) break;   // dh_rec now holds d h_0
    if (owner) {
      float* gb = a.gates + (size_t)t * B * R + (size_t)ob * R + u0 + oj;
      const float i = gb[0], f = gb[(size_t)H], gg = gb[(size_t)2 * H], o = gb[(size_t)3 * H];
      const float c_prev = a.cs[(size_t)t * B * H + ohi], c = a.cs[(size_t)(t + 1) * B * H + ohi];
      const float dhv = dh_rec + (a.d_out != nullptr ? a.d_out[(size_t)t * B * H + ohi] : 0.f);
      const float tc = tanhf(c);
      const float dcv = fmaf(dhv * o, 1.f - tc * tc, dc_reg);
      const float di = dcv * gg * i * (1.f - i), df = dcv * c_prev * f * (1.f - f);
      const float dg_ = dcv * i * (1.f - gg * gg), d_o = dhv * tc * o * (1.f - o);
      gb[0] = di; gb[(size_t)H] = df; gb[(size_t)2 * H] = dg_; gb[(size_t)3 * H] = d_o;
      float* dgo = a.dgt + (size_t)(t & 1) * R * 32;
      const int u = u0 + oj;
      dgo[(size_t)(0 * H + u) * 32 + ob] = di;
      dgo[(size_t)(1 * H + u) * 32 + ob] = df;
      dgo[(size_t)(2 * H + u) * 32 + ob] = dg_;
      dgo[(size_t)(3 * H + u) * 32 + ob] = d_o;
      dc_reg = dcv * f;
    }
    if (!lp_grid_barrier(a.barrier, &sh_ok)) return;
  }
  if (owner) {
    a.dh[ohi] = dh_rec;
    a.dc[ohi] = dc_reg;
  }
}

// ---------------------------------- host side ----------------------------------------------
static unsigned* g_lp_barrier[64];

static unsigned* lp_barrier_words() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (g_lp_barrier[dev] == nullptr) {
    if (cudaMalloc(&g_lp_barrier[dev], 4 * sizeof(unsigned)) != cudaSuccess) return nullptr;
    cudaMemset(g_lp_barrier[dev], 0, 4 * sizeof(unsigned));
  }
  return g_lp_barrier[dev];
}

static int lp_units_per_cta(int H) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  return (H + sms - 1) / sms;
}
static size_t lp_fwd_smem(int H, int upc) {
  const int HP = (H + 3) & ~3;
  return ((size_t)4 * upc * HP + (size_t)HP * LP_HSTRIDE + (size_t)LP_WARPS * 4 * upc * 32) * sizeof(float);
}
static size_t lp_bwd_smem(int H, int upc) {
  (void)upc;
  const size_t RP = ((size_t)4 * H + LP_CHUNK - 1) / LP_CHUNK * LP_CHUNK;
  return (RP * LP_UPC_MAX + (size_t)LP_WARPS * LP_UPC_MAX * 32 + (size_t)2 * LP_CHUNK * 32) * sizeof(float);
}

extern "C" int lstm_rec_supported(int T, int B, int H) {
  if (T < 1 || B < 1 || B > 32 || H < 1) return 0;
  const int upc = lp_units_per_cta(H);
  return upc <= LP_UPC_MAX && lp_fwd_smem(H, upc) <= 200 * 1024 && lp_bwd_smem(H, LP_UPC_MAX) <= 200 * 1024;
}

// floats of the backward scratch (transposed d(pre) of two consecutive steps)
extern "C" long long lstm_rec_bwd_scratch(int H) { return 2LL * 4 * H * 32; }

extern "C" int lstm_rec_last_error() {
  unsigned* w = lp_barrier_words();
  unsigned v[4] = {0, 0, 0, 0};
  if (w == nullptr || cudaMemcpy(v, w, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)v[2];
}

extern "C" int lstm_rec_forward(void* gates, const void* w_hh, void* hs, void* cs, int T, int B, int H, cudaStream_t st) {
  if (!lstm_rec_supported(T, B, H)) return -1;
  LstmRecArgs a = {};
  a.gates = reinterpret_cast<float*>(gates);
  a.w_hh = reinterpret_cast<const float*>(w_hh);
  a.hs = reinterpret_cast<float*>(hs);
  a.cs = reinterpret_cast<float*>(cs);
  a.barrier = lp_barrier_words();
  if (a.barrier == nullptr) return -13;
  a.T = T; a.B = B; a.H = H; a.upc = lp_units_per_cta(H);
  const size_t smem = lp_fwd_smem(H, a.upc);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(lstm_rec_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = 200 * 1024;
  }
  const int grid = (H + a.upc - 1) / a.upc;
  lstm_rec_fwd_kernel<<<grid, LP_THREADS, smem, st>>>(a);
  return (int)cudaGetLastError();
}

// gates: activations in, d(pre-activations) out; dh / dc: [B][H] in (d h_T, d c_T) and out (d h_0, d c_0)
extern "C" int lstm_rec_backward(void* gates, const void* w_hh, const void* cs, const void* d_out, void* dh, void* dc,
                                 void* scratch, int T, int B, int H, cudaStream_t st) {
  if (!lstm_rec_supported(T, B, H)) return -1;
  LstmRecArgs a = {};
  a.gates = reinterpret_cast<float*>(gates);
  a.w_hh = reinterpret_cast<const float*>(w_hh);
  a.cs = const_cast<float*>(reinterpret_cast<const float*>(cs));
  a.d_out = reinterpret_cast<const float*>(d_out);
  a.dh = reinterpret_cast<float*>(dh);
  a.dc = reinterpret_cast<float*>(dc);
  a.dgt = reinterpret_cast<float*>(scratch);
  a.barrier = lp_barrier_words();
  if (a.barrier == nullptr) return -13;
  a.T = T; a.B = B; a.H = H; a.upc = LP_UPC_MAX;   // fewer, fatter CTAs: each reads the whole d(pre) vector per step
  const size_t smem = lp_bwd_smem(H, a.upc);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(lstm_rec_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = 200 * 1024;
  }
  const int grid = (H + a.upc - 1) / a.upc;
  lstm_rec_bwd_kernel<<<grid, LP_THREADS, smem, st>>>(a);
  return (int)cudaGetLastError();
}
