// Centralized SGD in one kernel: gradient all-reduce (average) over the peer-mapped mailboxes
// fused with the momentum-SGD update.  Replaces flatten + all_reduce + unflatten + the
// per-tensor update loop of dl_code/pcode/optim/sgd.py:68-92 and
// dl_code/pcode/utils/communication.py:173-181.
//
// Two-shot all-reduce on the complete graph, work split by chunk: chunk c belongs to rank
// c mod n and is its (c div n)-th local chunk.
//   phase 1  every rank stores its (clipped) gradient of the chunks owned by peer k into its
//            slot of k's mailbox, words [lc * chunk_elems, ...), then raises k's flag to 2t+1
//   phase 2  the owner waits for all flags, sums own + received gradients in a fixed order,
//            scales by 1/n, stores the average into every peer's slot at [S + lc * chunk_elems)
//            (S = words of one shard), applies the update to its own chunks, raises flags to 2t+2
//   phase 3  every rank waits, reads the averages of the chunks it does not own from its own
//            mailbox and applies the same update
// Each average is computed by exactly one rank, so all replicas stay bit-identical.
// t (number of completed all-reduces), the momentum flag and the arrival counters live in device
// memory: the launch takes no per-step host argument and can be replayed from a CUDA graph.
//
// The CTAs of all ranks wait on one another, so the grid must be co-resident: at most one CTA
// per SM in a distributed run; the single-device emulation (gridDim.y logical ranks in one
// launch) is a cooperative launch.  Every wait is bounded; a CTA that gives up records the peer
// and leaves, and the host raises an error before the state is used again.
#include "common.cuh"

struct ArPlan {
  int n_world;
  int my_rank;
  int shard_words;   // S
  int slot_of[CHOCO_MAX_PEERS + 1];  // rank -> index k into the peer arrays (-1 for self)
};

__device__ __forceinline__ bool wait_all(const ChocoParams& p, uint32_t want, int* sh_ok) {
  if (threadIdx.x == 0) {
    int good = 1;
    for (int k = 0; k < p.n_peers; ++k)
      if (!wait_flag_ge(p.my_flag[k], want, p.wait_budget_ns)) {
        report(p.status, CHOCO_TIMEOUT, p.peer_rank[k], (int)want);
        good = 0;
        break;
      }
    *sh_ok = good;
  }
  __syncthreads();
  const bool ok = *sh_ok != 0;
  __syncthreads();
  return ok;
}

// arrive on a counter; the last CTA of this logical rank runs `then`
template <class F>
__device__ __forceinline__ void arrive_last(uint32_t* counter, F then) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(counter, 1u) == gridDim.x - 1) {
      __threadfence_system();
      then();
    }
  }
}

__device__ __forceinline__ void sgd_apply4(const ChocoParams& p, int pos, int base, int valid, float4 gv, float wd,
                                           float lr, float mu, bool nesterov, bool mom_init) {
  const float4 xv = *reinterpret_cast<const float4*>(p.x + pos);
  float x_a[4] = {xv.x, xv.y, xv.z, xv.w}, g_a[4] = {gv.x, gv.y, gv.z, gv.w}, m_a[4] = {0.f, 0.f, 0.f, 0.f};
  if (mu != 0.f && mom_init) {
    const float4 mv = *reinterpret_cast<const float4*>(p.m + pos);
    m_a[0] = mv.x; m_a[1] = mv.y; m_a[2] = mv.z; m_a[3] = mv.w;
  }
#pragma unroll
  for (int e = 0; e < 4; ++e)
    if (base + e < valid) {
      const float d = sgd_direction(x_a[e], g_a[e], m_a[e], wd, mu, nesterov, mom_init);
      x_a[e] = fmaf(-lr, d, x_a[e]);
    }
  if (mu != 0.f) *reinterpret_cast<float4*>(p.m + pos) = make_float4(m_a[0], m_a[1], m_a[2], m_a[3]);
  *reinterpret_cast<float4*>(p.x + pos) = make_float4(x_a[0], x_a[1], x_a[2], x_a[3]);
  clear_grad4(p, pos);
}

__global__ void __launch_bounds__(CHOCO_THREADS) allreduce_sgd_kernel(const ChocoParams* __restrict__ params,
                                                                     const ArPlan* __restrict__ plans) {
  const ChocoParams& p = params[blockIdx.y];
  const ArPlan& pl = plans[blockIdx.y];
  const SegTable& tb = p.tab;
  __shared__ int sh_ok;
  const int n = pl.n_world, me = pl.my_rank, CE = tb.chunk_elems, S = pl.shard_words;
  const uint32_t t = p.step[0];
  const long long par = (long long)(t & 1u) * p.payload_words;
  const float lr = p.hyper[HYP_LR], mu = p.hyper[HYP_MOMENTUM], gscale = p.hyper[HYP_GSCALE];
  const bool nesterov = p.hyper[HYP_NESTEROV] != 0.f;
  const bool mom_init = p.step[1] != 0;
  const float inv_n = 1.0f / (float)n;

  // ---- phase 1: scatter my gradients to the chunk owners --------------------------------------
  for (int c = blockIdx.x; c < tb.n_chunks; c += gridDim.x) {
    const int owner = c % n;
    if (owner == me) continue;
    const int k = pl.slot_of[owner];
    const int seg = tb.chunk_seg[c], start = tb.chunk_start[c], valid = tb.chunk_valid[c];
    const int span = (valid + 3) & ~3;
    float* dst = reinterpret_cast<float*>(p.peer_inbox[k]) + par + (long long)(c / n) * CE;
    for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 4) {
      float4 g = load_grad4(p, seg, start + base, base, valid);
      g.x *= gscale; g.y *= gscale; g.z *= gscale; g.w *= gscale;
      *reinterpret_cast<float4*>(dst + base) = g;
    }
  }
  arrive_last(p.done_count + 0, [&] {
    for (int k = 0; k < p.n_peers; ++k) st_release_sys(p.peer_flag[k], 2u * t + 1u);
  });

  // ---- phase 2: reduce the chunks I own, publish the average, update them ------------------------
  if (!wait_all(p, 2u * t + 1u, &sh_ok)) return;
  for (int c = blockIdx.x; c < tb.n_chunks; c += gridDim.x) {
    if (c % n != me) continue;
    const int seg = tb.chunk_seg[c], start = tb.chunk_start[c], valid = tb.chunk_valid[c];
    const int span = (valid + 3) & ~3;
    const float wd = tb.seg_wd[seg];
    const long long off = par + (long long)(c / n) * CE;
    for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 4) {
      float4 a = load_grad4(p, seg, start + base, base, valid);
      a.x *= gscale; a.y *= gscale; a.z *= gscale; a.w *= gscale;
      for (int k = 0; k < p.n_peers; ++k) {
        const float4 q = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.my_inbox[k]) + off + base));
        a.x += q.x; a.y += q.y; a.z += q.z; a.w += q.w;
      }
      a.x *= inv_n; a.y *= inv_n; a.z *= inv_n; a.w *= inv_n;
      for (int k = 0; k < p.n_peers; ++k)
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.peer_inbox[k]) + off + S + base) = a;
      sgd_apply4(p, start + base, base, valid, a, wd, lr, mu, nesterov, mom_init);
    }
  }
  arrive_last(p.done_count + 1, [&] {
    for (int k = 0; k < p.n_peers; ++k) st_release_sys(p.peer_flag[k], 2u * t + 2u);
  });

  // ---- phase 3: update the chunks owned by the peers from the averages they published -------------
  if (!wait_all(p, 2u * t + 2u, &sh_ok)) return;
  for (int c = blockIdx.x; c < tb.n_chunks; c += gridDim.x) {
    const int owner = c % n;
    if (owner == me) continue;
    const int k = pl.slot_of[owner];
    const int seg = tb.chunk_seg[c], start = tb.chunk_start[c], valid = tb.chunk_valid[c];
    const int span = (valid + 3) & ~3;
    const float wd = tb.seg_wd[seg];
    const float* src = reinterpret_cast<const float*>(p.my_inbox[k]) + par + S + (long long)(c / n) * CE;
    for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 4) {
      const float4 a = __ldcg(reinterpret_cast<const float4*>(src + base));
      sgd_apply4(p, start + base, base, valid, a, wd, lr, mu, nesterov, mom_init);
    }
  }
  arrive_last(p.seg_count + 0, [&] {
    p.done_count[0] = 0;
    p.done_count[1] = 0;
    p.seg_count[0] = 0;
    p.step[0] = t + 1u;
    p.step[1] = 1u;
  });
}

extern "C" int ar_plan_size() { return (int)sizeof(ArPlan); }

// Largest grid.x such that grid.x * n_ranks CTAs are co-resident on the current device.
extern "C" int allreduce_sgd_max_grid(int n_ranks) {
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_sgd_kernel, CHOCO_THREADS, 0) != cudaSuccess)
    return -1;
  if (n_ranks <= 1) return sms;  // one CTA per SM
  const int cap = sms * per_sm / n_ranks;
  return cap < 1 ? 0 : cap;
}

extern "C" int allreduce_sgd_step(const void* params_dev, const void* plans_dev, int grid_x, int n_ranks,
                                  cudaStream_t stream) {
  if (grid_x < 1 || n_ranks < 1) return -1;
  dim3 grid(grid_x, n_ranks);
  if (n_ranks == 1) {
    allreduce_sgd_kernel<<<grid, CHOCO_THREADS, 0, stream>>>(reinterpret_cast<const ChocoParams*>(params_dev),
                                                            reinterpret_cast<const ArPlan*>(plans_dev));
    return (int)cudaGetLastError();
  }
  void* args[] = {(void*)&params_dev, (void*)&plans_dev};
  return (int)cudaLaunchCooperativeKernel((const void*)allreduce_sgd_kernel, grid, dim3(CHOCO_THREADS), args, 0, stream);
}
