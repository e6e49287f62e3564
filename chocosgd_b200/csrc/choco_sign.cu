// Fused CHOCO-SGD step with sign + L1-norm compression: ONE kernel per training step.
//
// For every chunk of the flat arena a CTA does, in registers and in this order:
//   (decode, step t-1)  wait (bounded) for the neighbours' flags of step t-1, then
//                       x_hat += q_i ;  s += w_ii q_i + sum_j w_ij q_j
//                       with q = ||d_seg||_1 / n_seg * sign bits read from the mailboxes
//   (local step)        x -= lr d'   (Nesterov / momentum / weight decay, gradient zeroed)
//   (consensus)         x += gamma (s - x_hat)
//   (compress + push)   bits of (x - x_hat) -> own outbox AND, with plain 32-bit stores
//                       over NVLink, straight into each neighbour's mailbox; per-chunk |.|
//                       partial sums
// The last CTA of a segment reduces the partials in a fixed order (bitwise reproducible)
// and pushes the norm; the last CTA of the grid raises the neighbours' flags
// (st.release.sys) and advances the device-resident step counter.
//
// Semantics: dl_code/pcode/optim/parallel_choco_v.py:104-155 (step) and :476-558 (sign
// codec); the decode of step t-1 is deferred to the start of step t, exactly where the
// reference joins its helper thread.
//
// gridDim.y enumerates logical ranks whose state lives on this GPU (1 in production; n
// in the single-GPU loopback used by the tests, where "peer" pointers are local).
#include "common.cuh"
#include "launch.cuh"

#define MODE_DECODE 1
#define MODE_PUSH 2

__device__ __forceinline__ float sel_sign(uint32_t word, int bit, float mag) {
  return ((word >> bit) & 1u) ? -mag : mag;
}

// NP = number of peers known at compile time (unrolled register arrays), or -1 = runtime.
// chunk0: first chunk of this launch.  A step may be issued as several launches over disjoint chunk
// ranges (buckets of tensors, each as soon as its gradients exist): the arrival counters run over all
// chunks of the arena, so the CTA that completes the LAST range publishes the step.
template <int NP>
__global__ void __launch_bounds__(CHOCO_THREADS) choco_sign_kernel(const ChocoParams* __restrict__ params, int mode,
                                                                 int chunk0) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const SegTable& tb = p.tab;
  const int chunk = chunk0 + blockIdx.x;
  constexpr int MAXP = NP >= 0 ? (NP > 0 ? NP : 1) : CHOCO_MAX_PEERS;
  const int n_peers = NP >= 0 ? NP : p.n_peers;

  __shared__ float red[32];
  __shared__ int sh_flag;

  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int span = (valid + 31) & ~31;  // positions covered by this chunk (whole words)
  const int seg_n = tb.seg_size[seg];
  const uint32_t t = p.step[0];
  const int PW = p.payload_words;

  const bool do_decode = (mode & MODE_DECODE) && t > 0 && p.step[2] < t;
  const bool do_push = (mode & MODE_PUSH) != 0;
  if (do_push && !do_decode && t > 0 && p.step[2] < t && threadIdx.x == 0 && chunk == 0)
    report(p.status, CHOCO_BAD_STEP, -1, (int)t);  // push of step t before step t-1 was applied

  // ---- wait for the neighbours' payloads of step t-1 -----------------------------------
  if (do_decode) {
    if (threadIdx.x == 0) {
      int ok = 1;
      for (int k = 0; k < n_peers; ++k) {
        if (!wait_flag_ge(p.my_flag[k], t, p.wait_budget_ns)) {
          report(p.status, CHOCO_TIMEOUT, p.peer_rank[k], (int)t - 1);
          ok = 0;
          break;
        }
      }
      sh_flag = ok;
    }
    __syncthreads();
    if (!sh_flag) return;  // every CTA that times out leaves; the host raises an error
  }

  const int par_prev = (t - 1) & 1, par_cur = t & 1;
  float mag_own = 0.f, mag_peer[MAXP];
  const uint32_t* inbox_prev[MAXP];
  uint32_t* inbox_out[MAXP];
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    mag_peer[k] = 0.f;
    inbox_prev[k] = nullptr;
    inbox_out[k] = nullptr;
    if (k < n_peers) {
      inbox_prev[k] = p.my_inbox[k] + par_prev * PW;
      inbox_out[k] = p.peer_inbox[k] + par_cur * PW;
    }
  }
  if (do_decode) {
    const float inv_n = 1.0f / (float)seg_n;
    mag_own = __uint_as_float(__ldcg(p.outbox + par_prev * PW + seg)) * inv_n;
#pragma unroll
    for (int k = 0; k < MAXP; ++k)
      if (k < n_peers) mag_peer[k] = p.w_peer[k] * __uint_as_float(__ldcg(inbox_prev[k] + seg)) * inv_n;
  }

  const float lr = p.hyper[HYP_LR], mu = p.hyper[HYP_MOMENTUM], gamma = p.hyper[HYP_GAMMA];
  const bool nesterov = p.hyper[HYP_NESTEROV] != 0.f;
  const float gscale = p.hyper[HYP_GSCALE];
  const bool mom_init = p.step[1] != 0;
  const float wd = tb.seg_wd[seg];
  const float w_self = p.w_self;
  const uint32_t* own_prev = p.outbox + par_prev * PW + p.body_off;
  uint32_t* own_out = p.outbox + par_cur * PW + p.body_off;
  const int body = p.body_off;

  float l1 = 0.f;
  const int n_iter = (span + CHOCO_THREADS * 4 - 1) / (CHOCO_THREADS * 4);  // uniform over the CTA
  for (int it = 0; it < n_iter; ++it) {
    const int base = it * CHOCO_THREADS * 4 + threadIdx.x * 4;
    const bool active = base < span;
    const int pos = start + base;  // flat position of this thread's 4 elements
    const int word = pos >> 5;     // sign word index
    const int bit0 = pos & 31;     // bit of the first element
    float xh_a[4] = {0.f, 0.f, 0.f, 0.f}, s_a[4] = {0.f, 0.f, 0.f, 0.f};
    if (active) {
      const float4 xh = *reinterpret_cast<const float4*>(p.x_hat + pos);
      const float4 sv = *reinterpret_cast<const float4*>(p.s + pos);
      xh_a[0] = xh.x; xh_a[1] = xh.y; xh_a[2] = xh.z; xh_a[3] = xh.w;
      s_a[0] = sv.x; s_a[1] = sv.y; s_a[2] = sv.z; s_a[3] = sv.w;
    }
    if (do_decode && active) {
      const uint32_t w_own = __ldcg(own_prev + word);
      uint32_t w_peer[MAXP];
#pragma unroll
      for (int k = 0; k < MAXP; ++k) w_peer[k] = (k < n_peers) ? __ldcg(inbox_prev[k] + body + word) : 0u;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (base + e < valid) {
          const float q = sel_sign(w_own, bit0 + e, mag_own);
          xh_a[e] += q;
          float acc = w_self * q;
#pragma unroll
          for (int k = 0; k < MAXP; ++k)
            if (k < n_peers) acc += sel_sign(w_peer[k], bit0 + e, mag_peer[k]);
          s_a[e] += acc;
        }
      }
      *reinterpret_cast<float4*>(p.x_hat + pos) = make_float4(xh_a[0], xh_a[1], xh_a[2], xh_a[3]);
      *reinterpret_cast<float4*>(p.s + pos) = make_float4(s_a[0], s_a[1], s_a[2], s_a[3]);
    }
    if (do_push) {
      uint32_t nib = 0;
      if (active) {
        const float4 xv = *reinterpret_cast<const float4*>(p.x + pos);
        const float4 gv = load_grad4(p, seg, pos, base, valid);
        float x_a[4] = {xv.x, xv.y, xv.z, xv.w}, g_a[4] = {gv.x, gv.y, gv.z, gv.w};
        float m_a[4] = {0.f, 0.f, 0.f, 0.f};
        if (mu != 0.f && mom_init) {
          const float4 mv = *reinterpret_cast<const float4*>(p.m + pos);
          m_a[0] = mv.x; m_a[1] = mv.y; m_a[2] = mv.z; m_a[3] = mv.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (base + e < valid) {
            const float d = sgd_direction(x_a[e], g_a[e] * gscale, m_a[e], wd, mu, nesterov, mom_init);
            float xn = fmaf(-lr, d, x_a[e]);
            xn = fmaf(gamma, s_a[e] - xh_a[e], xn);
            x_a[e] = xn;
            const float diff = xn - xh_a[e];
            l1 += fabsf(diff);
            nib |= (diff < 0.f ? 1u : 0u) << e;
          }
        }
        *reinterpret_cast<float4*>(p.x + pos) = make_float4(x_a[0], x_a[1], x_a[2], x_a[3]);
        if (mu != 0.f) *reinterpret_cast<float4*>(p.m + pos) = make_float4(m_a[0], m_a[1], m_a[2], m_a[3]);
        clear_grad4(p, pos);
      }
      // 8 consecutive lanes hold the 32 bits of one word (all lanes take part in the shuffles)
      uint32_t wbits = nib << ((threadIdx.x & 7) * 4);
      wbits |= __shfl_xor_sync(0xffffffffu, wbits, 1);
      wbits |= __shfl_xor_sync(0xffffffffu, wbits, 2);
      wbits |= __shfl_xor_sync(0xffffffffu, wbits, 4);
      if (active && (threadIdx.x & 7) == 0) own_out[word] = wbits;
    }
  }
  if (do_push && n_peers > 0) {
    // push: this chunk's sign words are contiguous; the whole CTA copies them into each neighbour's mailbox
    // with consecutive words per thread (scattered 4-byte stores crossed NVLink far below link rate)
    __syncthreads();
    const int w0 = start >> 5, nw = span >> 5;
#pragma unroll
    for (int k = 0; k < MAXP; ++k)
      if (k < n_peers)
        for (int i = threadIdx.x; i < nw; i += CHOCO_THREADS) inbox_out[k][body + w0 + i] = own_out[w0 + i];
  }
  if (!do_push) {
    // decode-only launch: the last CTA records that step t-1 has been applied
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.done_count + 1, 1u) == (uint32_t)tb.n_chunks - 1) {
        p.done_count[1] = 0;
        if (do_decode) p.step[2] = t;
      }
    }
    return;
  }

  // ---- per-segment L1 norm: deterministic two-level reduction ----------------------------
  const float tot = block_sum(l1, red);
  if (threadIdx.x == 0) {
    p.partial[chunk] = tot;
    __threadfence();
    const uint32_t arrived = atomicAdd(p.seg_count + seg, 1u);
    sh_flag = (arrived == (uint32_t)tb.seg_n_chunks[seg] - 1);
    if (sh_flag) __threadfence();
  }
  __syncthreads();
  if (sh_flag) {
    const int c0 = tb.seg_first_chunk[seg], nc = tb.seg_n_chunks[seg];
    float acc = 0.f;
    for (int c = threadIdx.x; c < nc; c += CHOCO_THREADS) acc += __ldcg(p.partial + c0 + c);
    const float norm = block_sum(acc, red);
    if (threadIdx.x == 0) {
      const uint32_t nb = __float_as_uint(norm);
      p.outbox[par_cur * PW + seg] = nb;
#pragma unroll
      for (int k = 0; k < MAXP; ++k)
        if (k < n_peers) inbox_out[k][seg] = nb;
      p.seg_count[seg] = 0;
    }
  }
  // ---- publish: last CTA of the grid raises the neighbours' flags ------------------------
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(p.done_count, 1u) == (uint32_t)tb.n_chunks - 1) {
      __threadfence_system();
      p.done_count[0] = 0;
      for (int k = 0; k < n_peers; ++k) st_release_sys(p.peer_flag[k], t + 1);
      if (do_decode) p.step[2] = t;
      p.step[1] = 1;
      __threadfence();
      p.step[0] = t + 1;
    }
  }
}

// n_peers_hint: compile-time specialisation to use when every logical rank of this launch
// has that many peers (0, 1, 2, 3, 4, 7), anything else selects the runtime-loop variant.
// chunks [chunk0, chunk0 + n_chunks) of every logical rank
extern "C" int choco_sign_step_range(const void* params_dev, int chunk0, int n_chunks, int n_ranks, int mode,
                                     int n_peers_hint, cudaStream_t stream) {
  if (chunk0 < 0 || n_chunks < 1) return -1;
  dim3 grid(n_chunks, n_ranks);
  const ChocoParams* p = reinterpret_cast<const ChocoParams*>(params_dev);
  switch (n_peers_hint) {
    case 0: launch_k(choco_sign_kernel<0>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, p, mode, chunk0); break;
    case 1: launch_k(choco_sign_kernel<1>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, p, mode, chunk0); break;
    case 2: launch_k(choco_sign_kernel<2>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, p, mode, chunk0); break;
    case 3: launch_k(choco_sign_kernel<3>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, p, mode, chunk0); break;
    case 4: launch_k(choco_sign_kernel<4>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, p, mode, chunk0); break;
    case 7: launch_k(choco_sign_kernel<7>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, p, mode, chunk0); break;
    default: launch_k(choco_sign_kernel<-1>, dim3(grid), dim3(CHOCO_THREADS), 0, stream, p, mode, chunk0); break;
  }
  return (int)cudaGetLastError();
}

extern "C" int choco_sign_step(const void* params_dev, int n_chunks, int n_ranks, int mode, int n_peers_hint,
                               cudaStream_t stream) {
  return choco_sign_step_range(params_dev, 0, n_chunks, n_ranks, mode, n_peers_hint, stream);
}
