// All-reduce (sum or average) through the NVSwitch: ONE kernel per rank over a symmetric buffer that is
// also mapped as an NVLink multicast object.
//
//   multimem.ld_reduce.add.v4.f32 [mc + i]   the switch reads element i of every rank's buffer and
//                                            returns the sum: one load instead of world - 1 peer loads
//   multimem.st.v4.f32 [mc + i], v           the switch writes v into every rank's buffer at i
//
// Two-shot form: rank r owns the r-th shard; it load-reduces its shard, scales it and multicasts the
// result, so every element crosses each GPU's links once in each direction and is computed by exactly
// one rank (all replicas end up bit-identical).  Replaces the averaged-model all-reduce and the
// centralized aggregators' all_reduce (dl_code/pcode/utils/communication.py:114-122, 173-181).
//
// Synchronisation: two exchanges of flags written into every rank's flag array with plain release
// stores over the peer mapping (slot = writer's rank, value = 2 e + 1 / 2 e + 2 for the e-th collective
// of this buffer): "my input is in place" before the first load, "my shard is everywhere" before the
// kernel ends.  Every wait is bounded; on expiry the kernel records {status, peer, epoch} and all CTAs
// leave.  CTAs spin while others still work, so the grid never exceeds what is co-resident.
#include "common.cuh"

struct NvlsArgs {
  float* mc;                                   // multicast address of the data region
  float* local;                                // this rank's own address of the data region
  uint32_t* flags_local;                       // [world] this rank's flag words
  uint32_t* flags_peer[CHOCO_MAX_PEERS + 1];   // every rank's flag array through the peer mapping (self included)
  uint32_t* epoch;                             // [4] local: {collectives done, arrivals 1, arrivals 2, unused}
  int32_t* status;                             // [4] {code, peer, epoch, aux}
  long long n;                                 // floats, a multiple of 4
  long long budget_ns;
  float scale;                                 // 1 (sum) or 1 / world (average)
  int rank, world;
};

__device__ __forceinline__ float4 multimem_ld_reduce_add(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(float* mc_addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w) : "memory");
}

// every CTA waits until all ranks' flags reached `want`
__device__ bool nvls_wait_all(const NvlsArgs& a, uint32_t want, uint32_t e, int* sh_ok) {
  if (threadIdx.x < a.world) {
    if (!wait_flag_ge(a.flags_local + threadIdx.x, want, a.budget_ns)) report(a.status, CHOCO_TIMEOUT, threadIdx.x, (int)e);
  }
  __syncthreads();
  if (threadIdx.x == 0) *sh_ok = __ldcg(a.status) == CHOCO_OK;
  __syncthreads();
  const bool ok = *sh_ok != 0;
  __syncthreads();
  return ok;
}

__global__ void __launch_bounds__(CHOCO_THREADS) nvls_allreduce_kernel(NvlsArgs a) {
  __shared__ int sh_ok;
  const uint32_t e = a.epoch[0];
  // ---- first flag exchange: every rank's input is in its buffer (it was written before this kernel started) ----
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(a.flags_peer[threadIdx.x] + a.rank, 2u * e + 1u);
  }
  if (!nvls_wait_all(a, 2u * e + 1u, e, &sh_ok)) return;
  // ---- reduce my shard in the switch, multicast the result ---------------------------------------
  const long long n4 = a.n / 4;
  const long long per = (n4 + a.world - 1) / a.world;
  const long long lo = per * a.rank, hi = lo + per < n4 ? lo + per : n4;
  // a load-reduce is a round trip through the switch (microseconds): NVLS_UNROLL of them are in flight per
  // thread before the first result is used
  constexpr int NVLS_UNROLL = 4;
  const long long stride = (long long)gridDim.x * CHOCO_THREADS;
  for (long long i0 = lo + (long long)blockIdx.x * CHOCO_THREADS + threadIdx.x; i0 < hi; i0 += stride * NVLS_UNROLL) {
    float4 v[NVLS_UNROLL];
#pragma unroll
    for (int u = 0; u < NVLS_UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < hi) v[u] = multimem_ld_reduce_add(a.mc + 4 * i);
    }
#pragma unroll
    for (int u = 0; u < NVLS_UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < hi) {
        v[u].x *= a.scale; v[u].y *= a.scale; v[u].z *= a.scale; v[u].w *= a.scale;
        multimem_st(a.mc + 4 * i, v[u]);
      }
    }
  }
  // ---- second flag exchange: my shard has been written everywhere ------------------------------------------------
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.epoch + 1, 1u) == gridDim.x - 1) {
      a.epoch[1] = 0;
      __threadfence_system();
      for (int r = 0; r < a.world; ++r) st_release_sys(a.flags_peer[r] + a.rank, 2u * e + 2u);
    }
  }
  if (!nvls_wait_all(a, 2u * e + 2u, e, &sh_ok)) return;
  if (threadIdx.x == 0 && atomicAdd(a.epoch + 2, 1u) == gridDim.x - 1) {
    a.epoch[2] = 0;
    __threadfence();
    a.epoch[0] = e + 1u;      // after every CTA of this launch has read e
  }
}

extern "C" int nvls_args_size() { return (int)sizeof(NvlsArgs); }

// largest co-resident grid of the kernel on the current device
extern "C" int nvls_max_grid() {
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, nvls_allreduce_kernel, CHOCO_THREADS, 0) != cudaSuccess) return -1;
  return sms * per_sm;
}

extern "C" int nvls_allreduce(const NvlsArgs* args, int grid, cudaStream_t st) {
  const NvlsArgs& a = *args;
  if (a.world < 1 || a.world > CHOCO_MAX_PEERS + 1 || a.rank < 0 || a.rank >= a.world || a.n < 4 || a.n % 4 != 0) return -1;
  if (a.mc == nullptr || a.local == nullptr || grid < 1) return -1;
  if ((reinterpret_cast<uintptr_t>(a.mc) & 15) != 0) return -1;
  nvls_allreduce_kernel<<<grid, CHOCO_THREADS, 0, st>>>(a);
  return (int)cudaGetLastError();
}
