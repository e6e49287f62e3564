// Fused steps of the algorithms other than CHOCO-SGD, on the same arenas, segment tables,
// wire formats and peer mailboxes as the CHOCO kernels:
//
//   D-PSGD        x <- sum_j w_ij (x_j - lr d'_j)                    dl_code/pcode/optim/sgd.py:93-121
//   DCD-PSGD      q = Q(sum_j w_ij xh_j - lr d' - x); xh_j += q_j; x <- xh_i        dcd_psgd.py:96-144
//   ECD-PSGD      x <- sum_j w_ij xh_j - lr d'; z = (1 - t/2) x_old + (t/2) x;
//                 xh_j <- (1 - 2/t) xh_j + (2/t) Q(z_j)                              ecd_psgd.py:99-157
//   DeepSqueeze   x -= lr d'; e += x; c = Q(e); e -= c; x += gamma sum_j (w_ij - [j = i]) c_j
//                                                                                   deep_squeeze.py:94-127
//   DGC           v = d' + mem; c = top/random-k(v); mem = v outside the selection;
//                 x -= lr / n sum_j c_j   (quantizers: c = Q(d'), no memory)         dgc.py:118-252
//   EF-signSGD    p = d' + mem; c = ||p||_1 / n sign(p); mem = p - c; x -= lr / n sum_j c_j
//                                                                                   ef_sign_sgd.py:78-123
//
// One training step is
//   algo_prep        momentum-SGD direction, the algorithm's vector v (to the scratch buffer),
//                    state updates, per-tensor norm / first radix histogram; with the sign codec
//                    and for D-PSGD the payload is packed and pushed by this kernel too
//   (codec kernels)  QSGD pack / top-k select + emit / random-k emit of the CHOCO path: they
//                    compress the scratch buffer, push into the neighbours' mailboxes over NVLink,
//                    raise the flags and advance the device-resident step counter
//   algo_apply_*     bounded wait for the neighbours' flags of THIS step (these algorithms are
//                    blocking in the reference), decode every payload, apply the update
// The step index lives in device memory, so the sequence replays from a CUDA graph.
#include "common.cuh"
#include "launch.cuh"
#include "codec_dev.cuh"

#define ALGO_DCD 1
#define ALGO_ECD 2
#define ALGO_DSQ 3
#define ALGO_DGC 4
#define ALGO_EF 5
#define ALGO_DPSGD 6

#define CODEC_QSGD 0
#define CODEC_TOPK 1
#define CODEC_RANDK 2
#define CODEC_SIGN 3
#define CODEC_RAW 4

// Per logical rank, beside its ChocoParams block (mirrored by a ctypes.Structure).
struct AlgoParams {
  float* hat[CHOCO_MAX_PEERS + 1];  // DCD / ECD replicas: [0] own, [1 + k] of peer k
  float* mem;                       // error memory (DeepSqueeze, DGC, EF-signSGD)
  float inv_world;                  // 1 / n (DGC, EF-signSGD)
  int mask_momentum;                // DGC: zero the momentum at the selected coordinates
  int use_memory;                   // DGC keeps no memory with a quantizer
  int t_offset;                     // ECD-PSGD: its step index t is (pushes completed - t_offset)
};

extern "C" int algo_params_size() { return (int)sizeof(AlgoParams); }

__device__ __forceinline__ void ld4(const float* p, float* a) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
}
__device__ __forceinline__ void st4(float* p, const float* a) {
  *reinterpret_cast<float4*>(p) = make_float4(a[0], a[1], a[2], a[3]);
}

template <int ALGO>
__global__ void __launch_bounds__(CHOCO_THREADS) algo_prep_kernel(const ChocoParams* __restrict__ params,
                                                                const AlgoParams* __restrict__ aparams, int codec) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const AlgoParams& a = aparams[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = blockIdx.x;
  __shared__ float red[32];
  __shared__ int sh_flag;
  __shared__ uint32_t sh_hist[2048];

  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int span = (valid + 31) & ~31;
  const uint32_t t = p.step[0];
  const int PW = p.payload_words, body = p.body_off, par_cur = t & 1, n_peers = p.n_peers;
  if (t > 0 && p.step[2] < t && threadIdx.x == 0 && chunk == 0)
    report(p.status, CHOCO_BAD_STEP, -1, (int)t);  // the exchange of step t-1 was never applied

  const float lr = p.hyper[HYP_LR], mu = p.hyper[HYP_MOMENTUM];
  const bool nesterov = p.hyper[HYP_NESTEROV] != 0.f;
  const float gscale = p.hyper[HYP_GSCALE];
  const bool mom_init = p.step[1] != 0;
  const float wd = tb.seg_wd[seg];
  const float tt = (float)((int)t + 1 - a.t_offset);  // 1-based step index of ECD-PSGD
  const bool pushes = codec == CODEC_SIGN || codec == CODEC_RAW;

  if (codec == CODEC_TOPK) {
    for (int i = threadIdx.x; i < 2048; i += CHOCO_THREADS) sh_hist[i] = 0;
    __syncthreads();
  }

  float acc = 0.f;
  const int n_iter = (span + CHOCO_THREADS * 4 - 1) / (CHOCO_THREADS * 4);  // uniform over the CTA
  for (int it = 0; it < n_iter; ++it) {
    const int base = it * CHOCO_THREADS * 4 + threadIdx.x * 4;
    const bool active = base < span;
    const int pos = start + base;
    uint32_t nib = 0;
    if (active) {
      float x_a[4], g_a[4], m_a[4] = {0.f, 0.f, 0.f, 0.f}, v_a[4] = {0.f, 0.f, 0.f, 0.f};
      float mix[4] = {0.f, 0.f, 0.f, 0.f}, e_a[4] = {0.f, 0.f, 0.f, 0.f};
      ld4(p.x + pos, x_a);
      const float4 gv = load_grad4(p, seg, pos, base, valid);
      g_a[0] = gv.x; g_a[1] = gv.y; g_a[2] = gv.z; g_a[3] = gv.w;
      if (mu != 0.f && mom_init) ld4(p.m + pos, m_a);
      if (ALGO == ALGO_DCD || ALGO == ALGO_ECD) {
        float h[4];
        ld4(a.hat[0] + pos, h);
#pragma unroll
        for (int e = 0; e < 4; ++e) mix[e] = p.w_self * h[e];
        for (int k = 0; k < n_peers; ++k) {
          ld4(a.hat[1 + k] + pos, h);
          const float w = p.w_peer[k];
#pragma unroll
          for (int e = 0; e < 4; ++e) mix[e] = fmaf(w, h[e], mix[e]);
        }
      }
      const bool has_mem = ALGO == ALGO_DSQ || ALGO == ALGO_EF || (ALGO == ALGO_DGC && a.use_memory);
      if (has_mem) ld4(a.mem + pos, e_a);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (base + e < valid) {
          const float d = sgd_direction(x_a[e], g_a[e] * gscale, m_a[e], wd, mu, nesterov, mom_init);
          float v;
          if (ALGO == ALGO_DCD) {
            v = fmaf(-lr, d, mix[e]) - x_a[e];
          } else if (ALGO == ALGO_ECD) {
            const float xn = fmaf(-lr, d, mix[e]);
            v = (1.f - 0.5f * tt) * x_a[e] + (0.5f * tt) * xn;
            x_a[e] = xn;
          } else if (ALGO == ALGO_DSQ) {
            const float xn = fmaf(-lr, d, x_a[e]);
            x_a[e] = xn;
            v = e_a[e] + xn;
            e_a[e] = v;
          } else if (ALGO == ALGO_DPSGD) {
            v = fmaf(-lr, d, x_a[e]);
            x_a[e] = v;
          } else {  // DGC, EF-signSGD
            v = d + e_a[e];
            e_a[e] = v;
          }
          v_a[e] = v;
          if (codec == CODEC_QSGD) acc = fmaf(v, v, acc);
          else if (codec == CODEC_SIGN) {
            acc += fabsf(v);
            nib |= (v < 0.f ? 1u : 0u) << e;
          } else if (codec == CODEC_TOPK) atomicAdd(&sh_hist[(__float_as_uint(v) & 0x7FFFFFFFu) >> 20], 1u);
        }
      }
      if (ALGO != ALGO_DCD && ALGO != ALGO_DGC && ALGO != ALGO_EF) st4(p.x + pos, x_a);
      if (mu != 0.f) st4(p.m + pos, m_a);
      if (has_mem) st4(a.mem + pos, e_a);
      clear_grad4(p, pos);
      if (codec == CODEC_RAW) {
        const float4 o = make_float4(v_a[0], v_a[1], v_a[2], v_a[3]);
        for (int k = 0; k < n_peers; ++k) *reinterpret_cast<float4*>(p.peer_inbox[k] + par_cur * PW + pos) = o;
      } else if (codec != CODEC_SIGN) {
        st4(p.scratch_d + pos, v_a);
      }
    }
    if (codec == CODEC_SIGN) {
      // 8 consecutive lanes hold the 32 bits of one word (all lanes take part in the shuffles)
      uint32_t wbits = nib << ((threadIdx.x & 7) * 4);
      wbits |= __shfl_xor_sync(0xffffffffu, wbits, 1);
      wbits |= __shfl_xor_sync(0xffffffffu, wbits, 2);
      wbits |= __shfl_xor_sync(0xffffffffu, wbits, 4);
      if (active && (threadIdx.x & 7) == 0) p.outbox[par_cur * PW + body + (pos >> 5)] = wbits;
    }
  }
  if (codec == CODEC_SIGN) {
    // the chunk's sign words are contiguous: one coalesced copy per neighbour (see push_words)
    __syncthreads();
    push_words(p, par_cur * PW + body + (start >> 5), span >> 5);
  }

  if (codec == CODEC_TOPK) {
    __syncthreads();
    uint32_t* gh = p.hist + (size_t)seg * CHOCO_HIST_WORDS;
    for (int i = threadIdx.x; i < 2048; i += CHOCO_THREADS)
      if (sh_hist[i]) atomicAdd(gh + i, sh_hist[i]);
  }
  if (codec == CODEC_QSGD || codec == CODEC_SIGN) {
    // per-tensor norm: per-chunk partials, added in a fixed order by the segment's last CTA
    const float tot = block_sum(acc, red);
    if (threadIdx.x == 0) {
      p.partial[chunk] = tot;
      __threadfence();
      sh_flag = (atomicAdd(p.seg_count + seg, 1u) == (uint32_t)tb.seg_n_chunks[seg] - 1);
      if (sh_flag) __threadfence();
    }
    __syncthreads();
    if (sh_flag) {
      const int c0 = tb.seg_first_chunk[seg], nc = tb.seg_n_chunks[seg];
      float s = 0.f;
      for (int c = threadIdx.x; c < nc; c += CHOCO_THREADS) s += __ldcg(p.partial + c0 + c);
      float norm = block_sum(s, red);
      if (codec == CODEC_QSGD) norm = sqrtf(norm);
      if (threadIdx.x == 0) {
        const uint32_t nb = __float_as_uint(norm);
        p.outbox[par_cur * PW + seg] = nb;
        for (int k = 0; k < n_peers; ++k) p.peer_inbox[k][par_cur * PW + seg] = nb;
        p.seg_count[seg] = 0;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (pushes) {
      __threadfence_system();
      if (atomicAdd(p.done_count, 1u) == (uint32_t)tb.n_chunks - 1) {
        __threadfence_system();
        p.done_count[0] = 0;
        for (int k = 0; k < n_peers; ++k) st_release_sys(p.peer_flag[k], t + 1);
        p.step[1] = 1;
        __threadfence();
        p.step[0] = t + 1;
      }
    } else {
      __threadfence();
      if (atomicAdd(p.done_count + 1, 1u) == (uint32_t)tb.n_chunks - 1) {
        p.done_count[1] = 0;
        p.step[1] = 1;
      }
    }
  }
}

// Dense decode + update (QSGD, sign, raw).  T = pushes completed; the payloads of step T-1 sit
// in parity (T-1) & 1 of the own outbox and of the mailbox slots the neighbours write.
template <int ALGO>
__global__ void __launch_bounds__(CHOCO_THREADS) algo_apply_dense_kernel(const ChocoParams* __restrict__ params,
                                                                       const AlgoParams* __restrict__ aparams,
                                                                       int codec) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const AlgoParams& a = aparams[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = blockIdx.x;
  __shared__ int sh_flag;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int span = (valid + 31) & ~31;
  const int seg_n = tb.seg_size[seg];
  const uint32_t T = p.step[0];
  if (T == 0 || p.step[2] >= T) return;  // nothing published since the last apply (same answer in every CTA)
  const int PW = p.payload_words, body = p.body_off, n_peers = p.n_peers, par = (T - 1) & 1;
  const int nbits = p.qsgd_nbits, pl = nbits + 1;

  if (threadIdx.x == 0) {
    int ok = 1;
    for (int k = 0; k < n_peers; ++k)
      if (!wait_flag_ge(p.my_flag[k], T, p.wait_budget_ns)) {
        report(p.status, CHOCO_TIMEOUT, p.peer_rank[k], (int)T - 1);
        ok = 0;
        break;
      }
    sh_flag = ok;
  }
  __syncthreads();
  if (!sh_flag) return;

  const float lr = p.hyper[HYP_LR], gamma = p.hyper[HYP_GAMMA];
  const float tt = (float)((int)T - a.t_offset), ea = 1.f - 2.f / tt, eb = 2.f / tt;
  const uint32_t* own = p.outbox + par * PW;
  float unit_own = 0.f;
  if (codec == CODEC_SIGN) unit_own = __uint_as_float(__ldcg(own + seg)) / (float)seg_n;
  else if (codec == CODEC_QSGD)
    unit_own = (qsgd_scale_of(seg_n, p.qsgd_s, p.qsgd_biased) * __uint_as_float(__ldcg(own + seg))) / (float)p.qsgd_s;

  for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 4) {
    const int pos = start + base, group = pos >> 5, bit0 = pos & 31;
    const int nv = valid - base < 4 ? valid - base : 4;
    if (nv <= 0) continue;
    float q[4] = {0.f, 0.f, 0.f, 0.f}, accx[4] = {0.f, 0.f, 0.f, 0.f};
    // own payload (D-PSGD has none: the own term is x itself)
    if (codec == CODEC_SIGN) sign_accumulate4(__ldcg(own + body + group), bit0, nv, unit_own, q);
    else if (codec == CODEC_QSGD) qsgd_accumulate4(own + body + group * pl, nbits, bit0, nv, unit_own, q, nullptr, 0.f);
    if (ALGO == ALGO_DCD || ALGO == ALGO_ECD) {
      float h[4];
      ld4(a.hat[0] + pos, h);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < nv) h[e] = ALGO == ALGO_DCD ? h[e] + q[e] : fmaf(ea, h[e], eb * q[e]);
      st4(a.hat[0] + pos, h);
      if (ALGO == ALGO_DCD) st4(p.x + pos, h);
    } else if (ALGO == ALGO_DSQ) {
      float m[4];
      ld4(a.mem + pos, m);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        m[e] -= q[e];
        accx[e] = (p.w_self - 1.f) * q[e];
      }
      st4(a.mem + pos, m);
    } else if (ALGO == ALGO_EF) {
      float m[4];
      ld4(a.mem + pos, m);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        m[e] -= q[e];
        accx[e] = q[e];
      }
      st4(a.mem + pos, m);
    } else if (ALGO == ALGO_DGC) {
#pragma unroll
      for (int e = 0; e < 4; ++e) accx[e] = q[e];
    }
    for (int k = 0; k < n_peers; ++k) {
      const uint32_t* in = p.my_inbox[k] + par * PW;
      float qk[4] = {0.f, 0.f, 0.f, 0.f};
      if (codec == CODEC_SIGN) {
        sign_accumulate4(__ldcg(in + body + group), bit0, nv, __uint_as_float(__ldcg(in + seg)) / (float)seg_n, qk);
      } else if (codec == CODEC_QSGD) {
        const float unit =
            (qsgd_scale_of(seg_n, p.qsgd_s, p.qsgd_biased) * __uint_as_float(__ldcg(in + seg))) / (float)p.qsgd_s;
        qsgd_accumulate4(in + body + group * pl, nbits, bit0, nv, unit, qk, nullptr, 0.f);
      } else {  // raw fp32 (D-PSGD)
        const float4 v = __ldcg(reinterpret_cast<const float4*>(in + pos));
        qk[0] = v.x; qk[1] = v.y; qk[2] = v.z; qk[3] = v.w;
      }
      if (ALGO == ALGO_DCD || ALGO == ALGO_ECD) {
        float h[4];
        ld4(a.hat[1 + k] + pos, h);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (e < nv) h[e] = ALGO == ALGO_DCD ? h[e] + qk[e] : fmaf(ea, h[e], eb * qk[e]);
        st4(a.hat[1 + k] + pos, h);
      } else if (ALGO == ALGO_DSQ || ALGO == ALGO_DPSGD) {
        const float w = p.w_peer[k];
#pragma unroll
        for (int e = 0; e < 4; ++e) accx[e] = fmaf(w, qk[e], accx[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) accx[e] += qk[e];
      }
    }
    if (ALGO == ALGO_DSQ || ALGO == ALGO_EF || ALGO == ALGO_DGC || ALGO == ALGO_DPSGD) {
      float x_a[4];
      ld4(p.x + pos, x_a);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (e < nv) {
          if (ALGO == ALGO_DSQ) x_a[e] = fmaf(gamma, accx[e], x_a[e]);
          else if (ALGO == ALGO_DPSGD) x_a[e] = fmaf(p.w_self, x_a[e], accx[e]);
          else x_a[e] = fmaf(-lr * a.inv_world, accx[e], x_a[e]);
        }
      }
      st4(p.x + pos, x_a);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.done_count + 1, 1u) == (uint32_t)tb.n_chunks - 1) {
      p.done_count[1] = 0;
      p.step[2] = T;
    }
  }
}

__device__ __forceinline__ int algo_segment_of_entry(const SegTable& tb, int e) {
  int lo = 0, hi = tb.n_segments - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tb.seg_koff[mid] <= e) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Sparse decode + update of ONE source payload (src < 0: own).  Indices inside one payload are
// distinct and the sources are applied by consecutive launches, so no atomics are needed and the
// result is bitwise reproducible.  Preceded by choco_wait_flags, followed by the decoded mark.
template <int ALGO>
__global__ void __launch_bounds__(CHOCO_THREADS) algo_apply_sparse_kernel(const ChocoParams* __restrict__ params,
                                                                        const AlgoParams* __restrict__ aparams,
                                                                        int src, int codec) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const AlgoParams& a = aparams[blockIdx.y];
  const SegTable& tb = p.tab;
  const uint32_t T = p.step[0];
  if (T == 0 || p.step[2] >= T || p.status[0] != CHOCO_OK) return;
  if (src >= p.n_peers) return;
  const int PW = p.payload_words, par = (T - 1) & 1;
  const int sum_k = codec == CODEC_TOPK ? PW / 2 : PW;
  const uint32_t* pay = (src < 0 ? p.outbox : p.my_inbox[src]) + par * PW;
  const float w = src < 0 ? p.w_self : p.w_peer[src];
  const int src_rank = src < 0 ? p.rank : p.peer_rank[src];
  const uint32_t seed = p.seed - 7919u * (uint32_t)p.rank + 7919u * (uint32_t)src_rank;
  const float lr = p.hyper[HYP_LR], gamma = p.hyper[HYP_GAMMA];
  const float tt = (float)((int)T - a.t_offset), ea = 1.f - 2.f / tt, eb = 2.f / tt;
  for (int e = blockIdx.x * CHOCO_THREADS + threadIdx.x; e < sum_k; e += gridDim.x * CHOCO_THREADS) {
    const int seg = algo_segment_of_entry(tb, e);
    uint32_t idx;
    float v;
    if (codec == CODEC_TOPK) {
      idx = __ldcg(pay + e);
      v = __uint_as_float(__ldcg(pay + sum_k + e));
      if (idx >= (uint32_t)tb.seg_size[seg]) {  // corrupt payload: record and skip
        report(p.status, CHOCO_BAD_STEP, src_rank, (int)T - 1);
        continue;
      }
    } else {
      const uint32_t n = (uint32_t)tb.seg_size[seg];
      uint32_t keys[4];
#pragma unroll
      for (uint32_t r = 0; r < 4; ++r) keys[r] = feistel_key(seed, T - 1, (uint32_t)seg, r);
      idx = feistel_perm((uint32_t)(e - tb.seg_koff[seg]), n, feistel_half_bits(n), keys);
      v = __uint_as_float(__ldcg(pay + e));
    }
    const int pos = tb.seg_start[seg] + (int)idx;
    if (ALGO == ALGO_DCD) {
      float* h = a.hat[src + 1] + pos;
      const float hv = *h + v;
      *h = hv;
      if (src < 0) p.x[pos] = hv;
    } else if (ALGO == ALGO_ECD) {
      float* h = a.hat[src + 1] + pos;
      *h = fmaf(ea, *h, eb * v);
    } else if (ALGO == ALGO_DSQ) {
      if (src < 0) {
        a.mem[pos] -= v;
        p.x[pos] = fmaf(gamma * (w - 1.f), v, p.x[pos]);
      } else {
        p.x[pos] = fmaf(gamma * w, v, p.x[pos]);
      }
    } else {  // DGC
      if (src < 0) {
        if (a.use_memory) a.mem[pos] = 0.f;
        if (a.mask_momentum) p.m[pos] = 0.f;
      }
      p.x[pos] = fmaf(-lr * a.inv_world, v, p.x[pos]);
    }
  }
}

// ---- host entry points ------------------------------------------------------------------------------
#define ALGO_DISPATCH(KERNEL, ...)                                                   \
  switch (algo) {                                                                    \
    case ALGO_DCD: launch_k(KERNEL<ALGO_DCD>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, __VA_ARGS__); break;     \
    case ALGO_ECD: launch_k(KERNEL<ALGO_ECD>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, __VA_ARGS__); break;     \
    case ALGO_DSQ: launch_k(KERNEL<ALGO_DSQ>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, __VA_ARGS__); break;     \
    case ALGO_DGC: launch_k(KERNEL<ALGO_DGC>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, __VA_ARGS__); break;     \
    case ALGO_EF: launch_k(KERNEL<ALGO_EF>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, __VA_ARGS__); break;       \
    case ALGO_DPSGD: launch_k(KERNEL<ALGO_DPSGD>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, __VA_ARGS__); break; \
    default: return -1;                                                              \
  }

extern "C" int algo_prep(const void* params_dev, const void* aparams_dev, int n_chunks, int n_ranks, int algo, int codec,
                         cudaStream_t stream) {
  if (codec < 0 || codec > CODEC_RAW || (codec == CODEC_RAW) != (algo == ALGO_DPSGD)) return -1;
  dim3 grid(n_chunks, n_ranks);
  const ChocoParams* pp = reinterpret_cast<const ChocoParams*>(params_dev);
  const AlgoParams* ap = reinterpret_cast<const AlgoParams*>(aparams_dev);
  ALGO_DISPATCH(algo_prep_kernel, pp, ap, codec)
  return (int)cudaGetLastError();
}

extern "C" int algo_apply_dense(const void* params_dev, const void* aparams_dev, int n_chunks, int n_ranks, int algo,
                                int codec, cudaStream_t stream) {
  if (!(codec == CODEC_QSGD || codec == CODEC_SIGN || codec == CODEC_RAW)) return -1;
  dim3 grid(n_chunks, n_ranks);
  const ChocoParams* pp = reinterpret_cast<const ChocoParams*>(params_dev);
  const AlgoParams* ap = reinterpret_cast<const AlgoParams*>(aparams_dev);
  ALGO_DISPATCH(algo_apply_dense_kernel, pp, ap, codec)
  return (int)cudaGetLastError();
}

extern "C" int algo_apply_sparse(const void* params_dev, const void* aparams_dev, int n_blocks, int n_ranks, int algo,
                                 int src, int codec, cudaStream_t stream) {
  if (!(codec == CODEC_TOPK || codec == CODEC_RANDK) || algo == ALGO_EF || algo == ALGO_DPSGD) return -1;
  dim3 grid(n_blocks, n_ranks);
  const ChocoParams* pp = reinterpret_cast<const ChocoParams*>(params_dev);
  const AlgoParams* ap = reinterpret_cast<const AlgoParams*>(aparams_dev);
  switch (algo) {
    case ALGO_DCD: launch_k(algo_apply_sparse_kernel<ALGO_DCD>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, pp, ap, src, codec); break;
    case ALGO_ECD: launch_k(algo_apply_sparse_kernel<ALGO_ECD>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, pp, ap, src, codec); break;
    case ALGO_DSQ: launch_k(algo_apply_sparse_kernel<ALGO_DSQ>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, pp, ap, src, codec); break;
    case ALGO_DGC: launch_k(algo_apply_sparse_kernel<ALGO_DGC>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, pp, ap, src, codec); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}
