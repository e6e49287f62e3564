// Shared device helpers of the gossip / optimizer kernels (sm_100a).
//
// Conventions
//  * flat fp32 arenas whose segments (= parameter tensors) start on 32-element
//    boundaries; a "chunk" is a run of CHUNK_ELEMS positions inside one segment, one
//    CTA per chunk, so per-segment reductions never need to split a CTA;
//  * everything that changes from step to step (step index, learning rate, momentum
//    state) lives in device memory, so a captured CUDA graph can be replayed unchanged;
//  * every wait on a word written by another GPU is bounded; on expiry the kernel records
//    {status, peer, step} and all CTAs leave normally (the host turns it into an error).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define CHOCO_MAX_PEERS 16
#define CHOCO_THREADS 256
// radix-select histograms per segment: 2048 (bits 30..20) + 2048 (bits 19..9) + 512 (bits 8..0)
#define CHOCO_HIST_WORDS 4608

// status codes written to ChocoParams::status[0]
#define CHOCO_OK 0
#define CHOCO_TIMEOUT 1
#define CHOCO_BAD_STEP 2

// hyper[] slots (device-resident floats, refreshed by the host when they change)
#define HYP_LR 0
#define HYP_MOMENTUM 1
#define HYP_GAMMA 2
#define HYP_NESTEROV 3
#define HYP_GSCALE 4   // multiplier applied to the gradient (global-norm clipping), 1 by default
#define HYP_N 8

struct SegTable {
  const int* chunk_seg;      // [n_chunks] segment of each chunk
  const int* chunk_start;    // [n_chunks] flat offset of the chunk's first element (multiple of 32)
  const int* chunk_valid;    // [n_chunks] number of valid (non padding) elements in the chunk
  const int* seg_start;      // [T] flat offset
  const int* seg_size;       // [T] logical element count
  const int* seg_first_chunk;  // [T]
  const int* seg_n_chunks;   // [T]
  const float* seg_wd;       // [T] weight decay
  const int* seg_k;          // [T] kept elements (sparsifiers)
  const int* seg_koff;       // [T] exclusive prefix sum of seg_k
  int n_chunks;
  int n_segments;
  int chunk_elems;           // multiple of 1024
  int total;                 // padded arena length
};

// One logical rank's view of the gossip state.  Layout is mirrored by a ctypes.Structure
// on the Python side: 8-byte members first, then 4-byte members.
struct ChocoParams {
  float* x;
  float* g;
  float* m;
  float* x_hat;
  float* s;
  float* scratch_d;                       // [total] difference buffer (multi-pass codecs)
  uint32_t* outbox;                       // [2][payload_words] own payloads (both parities)
  uint32_t* peer_inbox[CHOCO_MAX_PEERS];  // remote: base of my slot in peer k's mailbox ([2][payload_words])
  uint32_t* peer_flag[CHOCO_MAX_PEERS];   // remote: flag word of my slot in peer k's mailbox
  const uint32_t* my_inbox[CHOCO_MAX_PEERS];  // local: slot that peer k writes ([2][payload_words])
  const uint32_t* my_flag[CHOCO_MAX_PEERS];   // local: flag word that peer k raises
  const float* hyper;                     // [HYP_N]
  uint32_t* step;                         // [0] pushes completed, [1] momentum initialised, [2] decodes completed
  uint32_t* seg_count;                    // [T] chunk arrival counters (self-resetting)
  uint32_t* done_count;                   // [8] CTA arrival counters (self-resetting); [4], [5]: grid barrier
  float* partial;                         // [n_chunks] per-chunk partial norms
  uint32_t* hist;                         // [T][HIST_WORDS] radix-select histograms
  uint32_t* chunk_cnt;                    // [n_chunks][2] (#greater, #equal) per chunk
  uint32_t* sel;                          // [T][4] {threshold key, ties to take, prefix, remaining k}
  int32_t* status;                        // [4] {code, peer, step, aux}
  const float* const* seg_g;              // optional [T] per-tensor gradient pointers (null: use the flat g)
  long long wait_budget_ns;
  SegTable tab;
  float w_self;
  float w_peer[CHOCO_MAX_PEERS];
  int n_peers;
  int payload_words;                      // words per parity buffer
  int body_off;                           // first body word (after the per-segment header)
  int rank;
  int peer_rank[CHOCO_MAX_PEERS];
  uint32_t seed;
  int qsgd_s;
  int qsgd_nbits;
  int qsgd_biased;
  int pad_;
};

// ---- hashing shared bit for bit with compress/reference.py --------------------------------
__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}
__host__ __device__ __forceinline__ uint32_t uniform_base(uint32_t seed, uint32_t step) {
  return mix32(step * 0x9E3779B9u + 0x7F4A7C15u) ^ seed;
}
__host__ __device__ __forceinline__ float counter_uniform(uint32_t base, uint32_t pos) {
  // one round of the avalanche hash: consecutive positions under a per-step base decorrelate
  // well enough for stochastic rounding, and the quantizer is bound by its instruction count
  uint32_t h = mix32(pos ^ base);
  return (float)(h >> 8) * (1.0f / 16777216.0f);
}
__host__ __device__ __forceinline__ uint32_t feistel_key(uint32_t seed, uint32_t step, uint32_t seg, uint32_t r) {
  return mix32(seed ^ mix32(step * 0x9E3779B9u + seg * 0x85EBCA6Bu + r * 0xC2B2AE35u + 1u));
}
// image of j under the keyed permutation of [0, n) (4-round Feistel, cycle-walked)
__host__ __device__ __forceinline__ uint32_t feistel_perm(uint32_t j, uint32_t n, int half_bits, const uint32_t* keys) {
  if (n == 1) return 0;
  const uint32_t mask = (1u << half_bits) - 1u;
  uint32_t v = j;
  for (int it = 0; it < 64; ++it) {
    uint32_t l = v >> half_bits, r = v & mask;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t nl = r;
      r = l ^ (mix32(r ^ keys[k]) & mask);
      l = nl;
    }
    v = (l << half_bits) | r;
    if (v < n) break;
  }
  return v;
}
__host__ __device__ __forceinline__ int feistel_half_bits(uint32_t n) {
  int bits = 2;
  while (bits < 32 && (1ull << bits) < (unsigned long long)n) ++bits;
  if (bits & 1) ++bits;
  return bits / 2;
}

#ifdef __CUDACC__
// ---- system-scope loads / stores -----------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait until *flag >= want.  Returns true on success.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, long long budget_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  const long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
      __nanosleep(64);
    }
    if (global_ns() - t0 > budget_ns) return false;
  }
}

// Copy `n` payload words starting at word `off` of the own outbox into the same place of every
// neighbour's mailbox: consecutive threads store consecutive words (full NVLink packets).  The words must
// have been written by this CTA before a __syncthreads().
__device__ __forceinline__ void push_words(const ChocoParams& p, int off, int n) {
  for (int k = 0; k < p.n_peers; ++k) {
    uint32_t* dst = p.peer_inbox[k] + off;
    const uint32_t* src = p.outbox + off;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  }
}

// ---- reductions ----------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// deterministic block sum (fixed tree); result valid in every thread
__device__ __forceinline__ float block_sum(float v, float* smem /* >= 32 floats */) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  float r = (lane < (blockDim.x >> 5)) ? smem[lane] : 0.f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ void report(int32_t* status, int code, int peer, int step) {
  if (atomicCAS(status, CHOCO_OK, code) == CHOCO_OK) {
    status[1] = peer;
    status[2] = step;
  }
}

// Gradient of 4 consecutive positions.  With a pointer table the gradients stay where
// autograd produced them (one contiguous tensor per parameter) and are never packed.
__device__ __forceinline__ float4 load_grad4(const ChocoParams& p, int seg, int pos, int base, int valid) {
  if (p.seg_g == nullptr) return *reinterpret_cast<const float4*>(p.g + pos);
  const float* gp = p.seg_g[seg] + (pos - p.tab.seg_start[seg]);
  if (base + 4 <= valid) return *reinterpret_cast<const float4*>(gp);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (base + 0 < valid) v.x = gp[0];
  if (base + 1 < valid) v.y = gp[1];
  if (base + 2 < valid) v.z = gp[2];
  return v;
}
__device__ __forceinline__ void clear_grad4(const ChocoParams& p, int pos) {
  if (p.seg_g == nullptr) *reinterpret_cast<float4*>(p.g + pos) = make_float4(0.f, 0.f, 0.f, 0.f);
}

// Momentum-SGD direction for one element; updates m in place.
//   d = g + wd x;  m = d (first) | mu m + d;  d' = d + mu m (nesterov) | m;  mu == 0: d' = d
__device__ __forceinline__ float sgd_direction(float x, float g, float& m, float wd, float mu, bool nesterov,
                                               bool mom_init) {
  float d = fmaf(wd, x, g);
  if (mu != 0.f) {
    m = mom_init ? fmaf(mu, m, d) : d;
    d = nesterov ? fmaf(mu, m, d) : m;
  }
  return d;
}
#endif
