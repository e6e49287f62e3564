// CHOCO-SGD step with QSGD stochastic quantization: two kernels per training step.
//
//   choco_dense_prep   (decode of step t-1, fused as in the sign kernel)  ->  local SGD step
//                      -> consensus -> d = x - x_hat into the scratch buffer; per-chunk sum of
//                      squares; the last CTA of a segment publishes ||d_seg||_2 (own outbox
//                      + neighbours' mailboxes, NVLink stores)
//   choco_qsgd_pack    level = floor(s |d| / norm) + [u < frac], u from a counter hash of
//                      (seed, step, position); levels and signs are bit-sliced with warp
//                      ballots: every group of 32 positions becomes nbits + 1 words, stored to
//                      the outbox and pushed into each neighbour's mailbox; the last CTA raises
//                      the flags and advances the step counter
//
// Quantizer: dl_code/pcode/utils/sparsification.py:87-98 (which ships the de-quantized fp32
// tensor; here (nbits + 1) bits per element travel).  A zero tensor quantizes to zeros.
#include "common.cuh"
#include "launch.cuh"
#include "codec_dev.cuh"

#define MODE_DECODE 1

// Warp-cooperative form (nbits <= 7): a warp covers 128 consecutive positions = 4 groups; the
// 4 (nbits + 1) plane words are loaded ONCE (lane j loads word j) and handed out by shuffles, so
// the payload is read with one load per lane instead of nbits + 1 loads per thread.
// `words_valid` bounds the load at the end of a chunk / of the payload.  All 32 lanes must call.
__device__ __forceinline__ void qsgd_accumulate4_warp(const uint32_t* __restrict__ wsrc, int nbits, int lane,
                                                      int words_valid, int n_valid, float unit, float* acc,
                                                      float* acc2, float w2) {
  const int pl = nbits + 1;
  const uint32_t mine = lane < words_valid ? __ldcg(wsrc + lane) : 0u;
  const int gsel = (lane >> 3) * pl, bit0 = (lane & 7) * 4;
  uint32_t levels = 0, sgn = 0;
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const uint32_t w = __shfl_sync(0xffffffffu, mine, (gsel + b) & 31);
    const uint32_t nib = (w >> bit0) & 0xFu;
    if (b < nbits) levels |= ((nib * 0x00204081u) & 0x01010101u) << b;
    else if (b == nbits) sgn = nib;
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
}

// codec: 0 = qsgd (fused decode + L2 norm), 1 = top-k (first radix histogram), 2 = random-k
__global__ void __launch_bounds__(CHOCO_THREADS) choco_dense_prep_kernel(const ChocoParams* __restrict__ params,
                                                                       int mode, int codec) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = blockIdx.x;
  __shared__ float red[32];
  __shared__ int sh_flag;
  __shared__ uint32_t sh_hist[2048];

  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int span = (valid + 31) & ~31;
  const int seg_n = tb.seg_size[seg];
  const uint32_t t = p.step[0];
  const int PW = p.payload_words, body = p.body_off;
  const int n_peers = p.n_peers;
  const int nbits = p.qsgd_nbits, pl = nbits + 1;

  const bool do_decode = codec == 0 && (mode & MODE_DECODE) && t > 0 && p.step[2] < t;
  if (codec != 0 && t > 0 && p.step[2] < t && threadIdx.x == 0 && chunk == 0)
    report(p.status, CHOCO_BAD_STEP, -1, (int)t);
  if (do_decode) {
    if (threadIdx.x == 0) {
      int ok = 1;
      for (int k = 0; k < n_peers; ++k)
        if (!wait_flag_ge(p.my_flag[k], t, p.wait_budget_ns)) {
          report(p.status, CHOCO_TIMEOUT, p.peer_rank[k], (int)t - 1);
          ok = 0;
          break;
        }
      sh_flag = ok;
    }
    __syncthreads();
    if (!sh_flag) return;
  }
  if (codec == 1) {
    for (int i = threadIdx.x; i < 2048; i += CHOCO_THREADS) sh_hist[i] = 0;
    __syncthreads();
  }

  const int par_prev = (t - 1) & 1, par_cur = t & 1;
  float unit_own = 0.f, unit_peer[CHOCO_MAX_PEERS];
  if (do_decode) {
    const float sc = qsgd_scale_of(seg_n, p.qsgd_s, p.qsgd_biased);
    unit_own = (sc * __uint_as_float(__ldcg(p.outbox + par_prev * PW + seg))) / (float)p.qsgd_s;
    for (int k = 0; k < n_peers; ++k)
      unit_peer[k] =
          p.w_peer[k] * ((sc * __uint_as_float(__ldcg(p.my_inbox[k] + par_prev * PW + seg))) / (float)p.qsgd_s);
  }

  const float lr = p.hyper[HYP_LR], mu = p.hyper[HYP_MOMENTUM], gamma = p.hyper[HYP_GAMMA];
  const bool nesterov = p.hyper[HYP_NESTEROV] != 0.f;
  const float gscale = p.hyper[HYP_GSCALE];
  const bool mom_init = p.step[1] != 0;
  const float wd = tb.seg_wd[seg];

  float sq = 0.f;
  const int lane = threadIdx.x & 31;
  const bool warp_decode = do_decode && nbits <= 7;   // plane words shared through shuffles
  // all lanes of a warp iterate together (the cooperative decode shuffles across the warp)
  for (int wb = (threadIdx.x & ~31) * 4; wb < span; wb += CHOCO_THREADS * 4) {
    const int base = wb + lane * 4;
    const bool act = base < span;
    const int pos = start + (act ? base : wb);
    const int group = pos >> 5, bit0 = pos & 31;
    float4 xh = make_float4(0.f, 0.f, 0.f, 0.f), sv = xh;
    if (act) {
      xh = *reinterpret_cast<const float4*>(p.x_hat + pos);
      sv = *reinterpret_cast<const float4*>(p.s + pos);
    }
    float xh_a[4] = {xh.x, xh.y, xh.z, xh.w}, s_a[4] = {sv.x, sv.y, sv.z, sv.w};
    if (do_decode) {
      const int nv = !act ? 0 : (valid - base < 4 ? valid - base : 4);
      // own payload: x_hat += q, s += w_ii q ; neighbours: s += w_ij q_j (weight folded into unit)
      if (warp_decode) {
        const int wgroup = (start + wb) >> 5;
        const int groups_here = (span - wb) >= 128 ? 4 : ((span - wb + 31) >> 5);
        const int words_valid = groups_here * pl;
        qsgd_accumulate4_warp(p.outbox + par_prev * PW + body + wgroup * pl, nbits, lane, words_valid, nv, unit_own,
                              xh_a, s_a, p.w_self);
        for (int k = 0; k < n_peers; ++k)
          qsgd_accumulate4_warp(p.my_inbox[k] + par_prev * PW + body + wgroup * pl, nbits, lane, words_valid, nv,
                                unit_peer[k], s_a, nullptr, 0.f);
      } else if (act) {
        qsgd_accumulate4(p.outbox + par_prev * PW + body + group * pl, nbits, bit0, nv, unit_own, xh_a, s_a, p.w_self);
        for (int k = 0; k < n_peers; ++k)
          qsgd_accumulate4(p.my_inbox[k] + par_prev * PW + body + group * pl, nbits, bit0, nv, unit_peer[k], s_a, nullptr,
                           0.f);
      }
      if (act) {
        *reinterpret_cast<float4*>(p.x_hat + pos) = make_float4(xh_a[0], xh_a[1], xh_a[2], xh_a[3]);
        *reinterpret_cast<float4*>(p.s + pos) = make_float4(s_a[0], s_a[1], s_a[2], s_a[3]);
      }
    }
    if (!act) continue;
    const float4 xv = *reinterpret_cast<const float4*>(p.x + pos);
    const float4 gv = load_grad4(p, seg, pos, base, valid);
    float x_a[4] = {xv.x, xv.y, xv.z, xv.w}, g_a[4] = {gv.x, gv.y, gv.z, gv.w};
    float m_a[4] = {0.f, 0.f, 0.f, 0.f}, d_a[4] = {0.f, 0.f, 0.f, 0.f};
    if (mu != 0.f && mom_init) {
      const float4 mv = *reinterpret_cast<const float4*>(p.m + pos);
      m_a[0] = mv.x; m_a[1] = mv.y; m_a[2] = mv.z; m_a[3] = mv.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (base + e < valid) {
        const float d = sgd_direction(x_a[e], g_a[e] * gscale, m_a[e], wd, mu, nesterov, mom_init);
        float xn = fmaf(-lr, d, x_a[e]);
        xn = fmaf(gamma, s_a[e] - xh_a[e], xn);
        x_a[e] = xn;
        const float diff = xn - xh_a[e];
        d_a[e] = diff;
        sq = fmaf(diff, diff, sq);
        if (codec == 1) atomicAdd(&sh_hist[(__float_as_uint(diff) & 0x7FFFFFFFu) >> 20], 1u);
      }
    *reinterpret_cast<float4*>(p.x + pos) = make_float4(x_a[0], x_a[1], x_a[2], x_a[3]);
    if (mu != 0.f) *reinterpret_cast<float4*>(p.m + pos) = make_float4(m_a[0], m_a[1], m_a[2], m_a[3]);
    clear_grad4(p, pos);
    *reinterpret_cast<float4*>(p.scratch_d + pos) = make_float4(d_a[0], d_a[1], d_a[2], d_a[3]);
  }

  if (codec == 1) {
    __syncthreads();
    uint32_t* gh = p.hist + (size_t)seg * CHOCO_HIST_WORDS;
    for (int i = threadIdx.x; i < 2048; i += CHOCO_THREADS)
      if (sh_hist[i]) atomicAdd(gh + i, sh_hist[i]);
  }
  if (codec == 0) {
    const float tot = block_sum(sq, red);
    if (threadIdx.x == 0) {
      p.partial[chunk] = tot;
      __threadfence();
      sh_flag = (atomicAdd(p.seg_count + seg, 1u) == (uint32_t)tb.seg_n_chunks[seg] - 1);
      if (sh_flag) __threadfence();
    }
    __syncthreads();
    if (sh_flag) {
      const int c0 = tb.seg_first_chunk[seg], nc = tb.seg_n_chunks[seg];
      float acc = 0.f;
      for (int c = threadIdx.x; c < nc; c += CHOCO_THREADS) acc += __ldcg(p.partial + c0 + c);
      const float norm = sqrtf(block_sum(acc, red));
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
    __threadfence();
    if (atomicAdd(p.done_count + 1, 1u) == (uint32_t)tb.n_chunks - 1) {
      p.done_count[1] = 0;
      if (do_decode) p.step[2] = t;
      p.step[1] = 1;
    }
  }
}

extern "C" int choco_dense_prep(const void* params_dev, int n_chunks, int n_ranks, int mode, int codec,
                                cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  launch_k(choco_dense_prep_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev),
                                                             mode, codec);
  return (int)cudaGetLastError();
}

// ---- QSGD quantize + bit-slice + push ------------------------------------------------------
__global__ void __launch_bounds__(CHOCO_THREADS) choco_qsgd_pack_generic_kernel(const ChocoParams* __restrict__ params) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = blockIdx.x;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int span = (valid + 31) & ~31;
  const uint32_t t = p.step[0];
  const int PW = p.payload_words, body = p.body_off;
  const int par_cur = t & 1;
  const int nbits = p.qsgd_nbits, pl = nbits + 1;
  const int lane = threadIdx.x & 31;
  const float norm = __uint_as_float(__ldcg(p.outbox + par_cur * PW + seg));
  const float s_f = (float)p.qsgd_s;
  const uint32_t ubase = uniform_base(p.seed, t);

  // one warp per group of 32 positions (lane = position inside the group); four groups are
  // loaded before any of them is processed so that four loads per lane are in flight
  const int warp = threadIdx.x >> 5;
  for (int base0 = warp * 32; base0 < span; base0 += CHOCO_THREADS * 4) {
    float dv[4];
    bool okv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int base = base0 + u * CHOCO_THREADS;
      okv[u] = base < span && base + lane < valid;
      dv[u] = okv[u] ? p.scratch_d[start + base + lane] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int base = base0 + u * CHOCO_THREADS;
      if (base >= span) break;  // uniform over the warp
      const int pos = start + base + lane;
      const bool ok = okv[u];
      const float d = dv[u];
      uint32_t lv = 0;
      if (ok && norm > 0.f) {
        const float lvl = fabsf(d) * (s_f / norm);
        const float fl = floorf(lvl);
        const float u01 = counter_uniform(ubase, (uint32_t)pos);
        lv = (uint32_t)fl + ((u01 < (lvl - fl)) ? 1u : 0u);
      }
      uint32_t mine = 0;
      for (int b = 0; b < nbits; ++b) {
        const uint32_t w = __ballot_sync(0xffffffffu, (lv >> b) & 1u);
        if (lane == b) mine = w;
      }
      const uint32_t sgn = __ballot_sync(0xffffffffu, ok && d < 0.f);
      if (lane == nbits) mine = sgn;
      if (lane < pl) p.outbox[par_cur * PW + body + ((start + base) >> 5) * pl + lane] = mine;
    }
  }
  __syncthreads();
  push_words(p, par_cur * PW + body + (start >> 5) * pl, (span >> 5) * pl);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(p.done_count, 1u) == (uint32_t)tb.n_chunks - 1) {
      __threadfence_system();
      p.done_count[0] = 0;
      for (int k = 0; k < p.n_peers; ++k) st_release_sys(p.peer_flag[k], t + 1);
      __threadfence();
      p.step[0] = t + 1;
    }
  }
}

// Fast path, NBITS known at compile time (1..8): level = floor(|d| * (s / norm)) + [u < frac] with no
// branch (padding and zero-norm tensors come out as level 0 by construction), fully unrolled
// ballots, one multiply instead of a division per element.
template <int NBITS>
__global__ void __launch_bounds__(CHOCO_THREADS) choco_qsgd_pack_kernel(const ChocoParams* __restrict__ params) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = blockIdx.x;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int span = (valid + 31) & ~31;
  const uint32_t t = p.step[0];
  const int PW = p.payload_words;
  const int par_cur = t & 1;
  constexpr int PL = NBITS + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float norm = __uint_as_float(__ldcg(p.outbox + par_cur * PW + seg));
  const float scale = norm > 0.f ? (float)p.qsgd_s / norm : 0.f;
  const uint32_t ubase = uniform_base(p.seed, t);
  const float* dptr = p.scratch_d + start;
  const int out0 = par_cur * PW + p.body_off + (start >> 5) * PL + lane;
  const int n_peers = p.n_peers;

  for (int base0 = warp * 32; base0 < span; base0 += CHOCO_THREADS * 4) {
    float dv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = base0 + u * CHOCO_THREADS + lane;
      dv[u] = i < valid ? dptr[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int base = base0 + u * CHOCO_THREADS;
      if (base >= span) break;  // uniform over the warp
      const float d = dv[u];
      const float a = fabsf(d) * scale;
      const float fl = floorf(a);
      const float u01 = counter_uniform(ubase, (uint32_t)(start + base + lane));
      const uint32_t lv = (uint32_t)fl + ((u01 < (a - fl)) ? 1u : 0u);
      uint32_t mine = __ballot_sync(0xffffffffu, d < 0.f);   // plane NBITS: signs
#pragma unroll
      for (int b = 0; b < NBITS; ++b) {
        const uint32_t w = __ballot_sync(0xffffffffu, (lv >> b) & 1u);
        mine = (lane == b) ? w : mine;
      }
      if (lane < PL) p.outbox[out0 + (base >> 5) * PL] = mine;
    }
  }
  // push: the chunk's words are contiguous in the payload; copied to every neighbour's mailbox by the whole
  // CTA (128 contiguous bytes per warp instruction; 20-byte stores per warp crossed NVLink far below link rate)
  __syncthreads();
  push_words(p, par_cur * PW + p.body_off + (start >> 5) * PL, (span >> 5) * PL);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(p.done_count, 1u) == (uint32_t)tb.n_chunks - 1) {
      __threadfence_system();
      p.done_count[0] = 0;
      for (int k = 0; k < n_peers; ++k) st_release_sys(p.peer_flag[k], t + 1);
      __threadfence();
      p.step[0] = t + 1;
    }
  }
}

extern "C" int choco_qsgd_pack_nbits(const void* params_dev, int n_chunks, int n_ranks, int nbits, cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  const ChocoParams* pp = reinterpret_cast<const ChocoParams*>(params_dev);
  switch (nbits) {
#define QSGD_CASE(B) case B: launch_k(choco_qsgd_pack_kernel<B>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, pp); break;
    QSGD_CASE(1) QSGD_CASE(2) QSGD_CASE(3) QSGD_CASE(4) QSGD_CASE(5) QSGD_CASE(6) QSGD_CASE(7) QSGD_CASE(8)
#undef QSGD_CASE
    default: launch_k(choco_qsgd_pack_generic_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, pp);
  }
  return (int)cudaGetLastError();
}

// nbits unknown to the caller: the generic kernel (reads it from the parameter block)
extern "C" int choco_qsgd_pack(const void* params_dev, int n_chunks, int n_ranks, cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  launch_k(choco_qsgd_pack_generic_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev));
  return (int)cudaGetLastError();
}

// decode-only (flush after the last training step): x_hat, s += payloads of step t-1
__global__ void __launch_bounds__(CHOCO_THREADS) choco_qsgd_decode_kernel(const ChocoParams* __restrict__ params) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = blockIdx.x;
  __shared__ int sh_flag;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int span = (valid + 31) & ~31;
  const uint32_t t = p.step[0];
  const bool do_decode = t > 0 && p.step[2] < t;
  const int PW = p.payload_words, body = p.body_off, n_peers = p.n_peers;
  const int nbits = p.qsgd_nbits, pl = nbits + 1;
  if (do_decode) {
    if (threadIdx.x == 0) {
      int ok = 1;
      for (int k = 0; k < n_peers; ++k)
        if (!wait_flag_ge(p.my_flag[k], t, p.wait_budget_ns)) {
          report(p.status, CHOCO_TIMEOUT, p.peer_rank[k], (int)t - 1);
          ok = 0;
          break;
        }
      sh_flag = ok;
    }
    __syncthreads();
    if (!sh_flag) return;
    const int par_prev = (t - 1) & 1;
    const float sc = qsgd_scale_of(tb.seg_size[seg], p.qsgd_s, p.qsgd_biased);
    const float unit_own = (sc * __uint_as_float(__ldcg(p.outbox + par_prev * PW + seg))) / (float)p.qsgd_s;
    for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 4) {
      const int pos = start + base, group = pos >> 5, bit0 = pos & 31;
      const float4 xh = *reinterpret_cast<const float4*>(p.x_hat + pos);
      const float4 sv = *reinterpret_cast<const float4*>(p.s + pos);
      float xh_a[4] = {xh.x, xh.y, xh.z, xh.w}, s_a[4] = {sv.x, sv.y, sv.z, sv.w};
      const int nv = valid - base < 4 ? valid - base : 4;
      qsgd_accumulate4(p.outbox + par_prev * PW + body + group * pl, nbits, bit0, nv, unit_own, xh_a, s_a, p.w_self);
      for (int k = 0; k < n_peers; ++k) {
        const float unit =
            p.w_peer[k] * ((sc * __uint_as_float(__ldcg(p.my_inbox[k] + par_prev * PW + seg))) / (float)p.qsgd_s);
        qsgd_accumulate4(p.my_inbox[k] + par_prev * PW + body + group * pl, nbits, bit0, nv, unit, s_a, nullptr, 0.f);
      }
      *reinterpret_cast<float4*>(p.x_hat + pos) = make_float4(xh_a[0], xh_a[1], xh_a[2], xh_a[3]);
      *reinterpret_cast<float4*>(p.s + pos) = make_float4(s_a[0], s_a[1], s_a[2], s_a[3]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.done_count + 1, 1u) == (uint32_t)tb.n_chunks - 1) {
      p.done_count[1] = 0;
      if (do_decode) p.step[2] = t;
    }
  }
}

extern "C" int choco_qsgd_decode(const void* params_dev, int n_chunks, int n_ranks, cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  launch_k(choco_qsgd_decode_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev));
  return (int)cudaGetLastError();
}
