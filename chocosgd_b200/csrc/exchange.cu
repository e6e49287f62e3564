// Generic neighbour exchange over the peer-mapped mailboxes, used by the algorithms that are
// not fused end to end (D-PSGD, DCD-/ECD-PSGD, DeepSqueeze; DGC / EF-signSGD on the complete
// graph as an all-gather by push), plus two small fused consumers.
//
//   mailbox_push   copy a payload into slot parity `seq & 1` of every neighbour's mailbox with
//                  16-byte NVLink stores; the last CTA raises the neighbours' flags to seq + 1
//   mailbox_wait   bounded wait until every neighbour has published payload `seq`
//   dpsgd_mix      x <- w_ii x + sum_k w_ik inbox_k   (full-precision gossip averaging,
//                  dl_code/pcode/optim/sgd.py:93-121) in one pass
//   sq_distance    deterministic ||a - b||^2 (consensus distance ||x_i - xbar||,
//                  dl_code/pcode/utils/auxiliary.py:18-24)
#include "common.cuh"
#include "launch.cuh"

struct ExchangeArgs {
  const uint32_t* src;                        // payload to publish
  uint32_t* peer_inbox[CHOCO_MAX_PEERS];      // remote slot base ([2][slot_words])
  uint32_t* peer_flag[CHOCO_MAX_PEERS];       // remote flag
  const uint32_t* my_inbox[CHOCO_MAX_PEERS];  // local slot base
  const uint32_t* my_flag[CHOCO_MAX_PEERS];   // local flag
  float w_peer[CHOCO_MAX_PEERS];
  float w_self;
  uint32_t* counter;                          // CTA arrival counter (self-resetting)
  int32_t* status;                            // {code, peer, seq}
  long long wait_budget_ns;
  long long n_words;                          // payload words (multiple of 4)
  long long slot_words;                       // words per parity buffer
  int n_peers;
  uint32_t seq;
  int peer_rank[CHOCO_MAX_PEERS];
};

__global__ void __launch_bounds__(CHOCO_THREADS) mailbox_push_kernel(ExchangeArgs a) {
  const long long n4 = a.n_words >> 2;
  const long long off = (long long)(a.seq & 1) * a.slot_words;
  const uint4* src = reinterpret_cast<const uint4*>(a.src);
  for (long long i = (long long)blockIdx.x * CHOCO_THREADS + threadIdx.x; i < n4; i += (long long)gridDim.x * CHOCO_THREADS) {
    const uint4 v = src[i];
    for (int k = 0; k < a.n_peers; ++k) reinterpret_cast<uint4*>(a.peer_inbox[k] + off)[i] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.counter, 1u) == gridDim.x - 1) {
      __threadfence_system();
      *a.counter = 0;
      for (int k = 0; k < a.n_peers; ++k) st_release_sys(a.peer_flag[k], a.seq + 1);
    }
  }
}

__global__ void mailbox_wait_kernel(ExchangeArgs a) {
  const int k = threadIdx.x;
  if (k < a.n_peers && !wait_flag_ge(a.my_flag[k], a.seq + 1, a.wait_budget_ns))
    report(a.status, CHOCO_TIMEOUT, a.peer_rank[k], (int)a.seq);
}

// x <- w_self x + sum_k w_k inbox_k   (n floats; waits for the neighbours first)
__global__ void __launch_bounds__(CHOCO_THREADS) dpsgd_mix_kernel(ExchangeArgs a, float* __restrict__ x, long long n) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    int good = 1;
    for (int k = 0; k < a.n_peers; ++k)
      if (!wait_flag_ge(a.my_flag[k], a.seq + 1, a.wait_budget_ns)) {
        report(a.status, CHOCO_TIMEOUT, a.peer_rank[k], (int)a.seq);
        good = 0;
        break;
      }
    ok = good;
  }
  __syncthreads();
  if (!ok) return;
  const long long off = (long long)(a.seq & 1) * a.slot_words;
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * CHOCO_THREADS + threadIdx.x; i < n4; i += (long long)gridDim.x * CHOCO_THREADS) {
    float4 v = reinterpret_cast<float4*>(x)[i];
    v.x *= a.w_self; v.y *= a.w_self; v.z *= a.w_self; v.w *= a.w_self;
    for (int k = 0; k < a.n_peers; ++k) {
      const float4 p = __ldcg(reinterpret_cast<const float4*>(a.my_inbox[k] + off) + i);
      const float w = a.w_peer[k];
      v.x = fmaf(w, p.x, v.x); v.y = fmaf(w, p.y, v.y); v.z = fmaf(w, p.z, v.z); v.w = fmaf(w, p.w, v.w);
    }
    reinterpret_cast<float4*>(x)[i] = v;
  }
}

static int grid_for_words(long long n4) {
  long long b = (n4 + CHOCO_THREADS - 1) / CHOCO_THREADS;
  if (b > sm_count() * 8) b = sm_count() * 8;
  return (int)(b < 1 ? 1 : b);
}

extern "C" int exchange_args_size() { return (int)sizeof(ExchangeArgs); }

extern "C" int mailbox_push(const ExchangeArgs* a, cudaStream_t st) {
  if (a->n_words % 4 != 0 || a->n_words > a->slot_words) return -1;
  mailbox_push_kernel<<<grid_for_words(a->n_words >> 2), CHOCO_THREADS, 0, st>>>(*a);
  return (int)cudaGetLastError();
}

extern "C" int mailbox_wait(const ExchangeArgs* a, cudaStream_t st) {
  mailbox_wait_kernel<<<1, 32, 0, st>>>(*a);
  return (int)cudaGetLastError();
}

extern "C" int dpsgd_mix(const ExchangeArgs* a, void* x, long long n, cudaStream_t st) {
  if (n % 4 != 0) return -1;
  dpsgd_mix_kernel<<<grid_for_words(n >> 2), CHOCO_THREADS, 0, st>>>(*a, reinterpret_cast<float*>(x), n);
  return (int)cudaGetLastError();
}

// ---- deterministic squared distance -------------------------------------------------------------
__global__ void __launch_bounds__(CHOCO_THREADS) sq_distance_kernel(const float* __restrict__ p, const float* __restrict__ q,
                                                                   long long n, double* partial, unsigned* counter,
                                                                   double* out) {
  __shared__ double red[CHOCO_THREADS];
  __shared__ int last;
  double acc = 0.0;
  for (long long i = (long long)blockIdx.x * CHOCO_THREADS + threadIdx.x; i < n; i += (long long)gridDim.x * CHOCO_THREADS) {
    const double d = (double)p[i] - (double)q[i];
    acc += d * d;
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = CHOCO_THREADS / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    partial[blockIdx.x] = red[0];
    __threadfence();
    last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    if (last) __threadfence();
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    double t = 0.0;
    for (unsigned b = 0; b < gridDim.x; ++b) t += partial[b];
    *out = t;
    *counter = 0;
  }
}

// scratch: (blocks + 2) doubles; out: 1 double
extern "C" int sq_distance_blocks(long long n) { return grid_for_words((n + 3) / 4) > 296 ? 296 : grid_for_words((n + 3) / 4); }

extern "C" int sq_distance(const void* p, const void* q, long long n, void* scratch, void* out, cudaStream_t st) {
  const int blocks = sq_distance_blocks(n);
  double* partial = reinterpret_cast<double*>(scratch);
  unsigned* counter = reinterpret_cast<unsigned*>(partial + blocks);
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(unsigned), st);
  if (e != cudaSuccess) return (int)e;
  sq_distance_kernel<<<blocks, CHOCO_THREADS, 0, st>>>(reinterpret_cast<const float*>(p), reinterpret_cast<const float*>(q),
                                                      n, partial, counter, reinterpret_cast<double*>(out));
  return (int)cudaGetLastError();
}
