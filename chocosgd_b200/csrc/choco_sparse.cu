// CHOCO-SGD with sparsifying compressors (top-k, random-k): selection, compaction and push.
//
// top-k (per parameter tensor, exact k, ties to the lowest index, output ordered by index):
//   the keys are the bit patterns of |d| (monotone as unsigned integers); a 3-digit radix
//   select (11 + 11 + 9 bits) narrows the k-th largest key:
//     choco_dense_prep(codec=1)  histogram of digit 1 while d is produced
//     choco_topk_hist(pass=2|3)  histogram of the next digit among keys matching the prefix
//     choco_topk_count           threshold key known -> per-chunk (#greater, #equal)
//     choco_topk_emit            ordered compaction of (index, value) pairs into the own
//                                outbox AND the neighbours' mailboxes (NVLink stores); last CTA
//                                raises the flags
//   replaces per-tensor torch.topk + gather + cat (dl_code/pcode/utils/sparsification.py:18-31,
//   dl_code/pcode/optim/parallel_choco_v.py:229-269).
// random-k: the k indices of a tensor are the first k images of a keyed Feistel permutation
//   of [0, n), a function of (seed, step, tensor): only values travel.
// decode: one launch per source payload (indices inside one payload are distinct, so no
//   atomics are needed and the result is bitwise reproducible).
#include "common.cuh"
#include "launch.cuh"

__device__ __forceinline__ uint32_t key_of(float d) { return __float_as_uint(d) & 0x7FFFFFFFu; }
__device__ __forceinline__ uint32_t koff_of(const SegTable& tb, int seg) { return (uint32_t)tb.seg_koff[seg]; }

// Among `nbins` counts (global memory), find the bin B with  #(bins > B) < k <= #(bins >= B).
// Returns B and k_rem = k - #(bins > B) to every thread.  nbins is 2048 or 512.
__device__ void find_bucket(const uint32_t* __restrict__ hist, int nbins, uint32_t k, uint32_t* sh /*[256+2]*/,
                            uint32_t& bucket, uint32_t& k_rem) {
  const int per = nbins / CHOCO_THREADS;  // 8 or 2
  uint32_t local[8];
  uint32_t sum = 0;
  for (int j = 0; j < per; ++j) {
    local[j] = __ldcg(hist + threadIdx.x * per + j);
    sum += local[j];
  }
  // counts in the bins of all higher threads: suffix sums inside the warp by shuffles, then the totals
  // of the higher warps
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  uint32_t suf = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_down_sync(0xffffffffu, suf, o);
    if (lane + o < 32) suf += v;
  }
  __syncthreads();   // sh may still be read by a previous call
  if (lane == 0) sh[wid] = suf;
  __syncthreads();
  uint32_t above = suf - sum;
  for (int w = wid + 1; w < CHOCO_THREADS / 32; ++w) above += sh[w];
  for (int j = per - 1; j >= 0; --j) {
    if (above < k && k <= above + local[j]) {
      sh[CHOCO_THREADS] = threadIdx.x * per + j;
      sh[CHOCO_THREADS + 1] = k - above;
    }
    above += local[j];
  }
  __syncthreads();
  bucket = sh[CHOCO_THREADS];
  k_rem = sh[CHOCO_THREADS + 1];
  __syncthreads();
}

// pass 2: digit-2 histogram of keys whose digit 1 equals the selected bucket
// pass 3: digit-3 histogram of keys whose digits 1 and 2 equal the selected buckets
__device__ void topk_hist_chunk(const ChocoParams& p, int chunk, int pass, uint32_t* sh /*[258]*/,
                                uint32_t* sh_hist /*[2048]*/) {
  const SegTable& tb = p.tab;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const uint32_t k = (uint32_t)tb.seg_k[seg];
  uint32_t* gh = p.hist + (size_t)seg * CHOCO_HIST_WORDS;
  uint32_t b1, k1, b2 = 0, k2 = 0;
  find_bucket(gh, 2048, k, sh, b1, k1);
  if (pass == 3) find_bucket(gh + 2048, 2048, k1, sh, b2, k2);
  const int nb = pass == 2 ? 2048 : 512;
  for (int i = threadIdx.x; i < nb; i += CHOCO_THREADS) sh_hist[i] = 0;
  __syncthreads();
  // 2 x 16-byte loads in flight per thread; the padding behind `valid` holds zeros and is skipped
  const float* dptr = p.scratch_d + start;
  const int span = (valid + 3) & ~3;
  for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 8) {
    const int base2 = base + CHOCO_THREADS * 4;
    const float4 va = *reinterpret_cast<const float4*>(dptr + base);
    float4 vb = make_float4(0.f, 0.f, 0.f, 0.f);
    if (base2 < span) vb = *reinterpret_cast<const float4*>(dptr + base2);
    const float d8[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int i = (e < 4 ? base : base2 - 4) + e;
      const uint32_t key = key_of(d8[e]);
      if (i < valid && (key >> 20) == b1) {
        if (pass == 2) atomicAdd(&sh_hist[(key >> 9) & 2047u], 1u);
        else if (((key >> 9) & 2047u) == b2) atomicAdd(&sh_hist[key & 511u], 1u);
      }
    }
  }
  __syncthreads();
  uint32_t* out = gh + (pass == 2 ? 2048 : 4096);
  for (int i = threadIdx.x; i < nb; i += CHOCO_THREADS)
    if (sh_hist[i]) atomicAdd(out + i, sh_hist[i]);
  __syncthreads();   // sh_hist may be reused by the caller's next chunk
}

__global__ void __launch_bounds__(CHOCO_THREADS) choco_topk_hist_kernel(const ChocoParams* __restrict__ params,
                                                                      int pass) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t sh[CHOCO_THREADS + 2];
  __shared__ uint32_t sh_hist[2048];
  topk_hist_chunk(params[blockIdx.y], blockIdx.x, pass, sh, sh_hist);
}

extern "C" int choco_topk_hist(const void* params_dev, int n_chunks, int n_ranks, int pass, cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  launch_k(choco_topk_hist_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev), pass);
  return (int)cudaGetLastError();
}

// threshold key and per-chunk counts
__device__ void topk_count_chunk(const ChocoParams& p, int chunk, uint32_t* sh /*[258]*/) {
  const SegTable& tb = p.tab;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const uint32_t k = (uint32_t)tb.seg_k[seg];
  const uint32_t* gh = p.hist + (size_t)seg * CHOCO_HIST_WORDS;
  uint32_t b1, k1, b2, k2, b3, k3;
  find_bucket(gh, 2048, k, sh, b1, k1);
  find_bucket(gh + 2048, 2048, k1, sh, b2, k2);
  find_bucket(gh + 4096, 512, k2, sh, b3, k3);
  const uint32_t thr = (b1 << 20) | (b2 << 9) | b3;
  uint32_t gt = 0, eq = 0;
  const float* dptr = p.scratch_d + start;
  const int span = (valid + 3) & ~3;
  for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 8) {
    const int base2 = base + CHOCO_THREADS * 4;
    const float4 va = *reinterpret_cast<const float4*>(dptr + base);
    float4 vb = make_float4(0.f, 0.f, 0.f, 0.f);
    if (base2 < span) vb = *reinterpret_cast<const float4*>(dptr + base2);
    const float d8[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int i = (e < 4 ? base : base2 - 4) + e;
      const uint32_t key = key_of(d8[e]);
      if (i < valid) {
        gt += key > thr;
        eq += key == thr;
      }
    }
  }
  // exact integer block sums through the float reducer would lose bits: use shuffles on ints
  for (int o = 16; o > 0; o >>= 1) {
    gt += __shfl_xor_sync(0xffffffffu, gt, o);
    eq += __shfl_xor_sync(0xffffffffu, eq, o);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    sh[(threadIdx.x >> 5) * 2] = gt;
    sh[(threadIdx.x >> 5) * 2 + 1] = eq;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t g = 0, e = 0;
    for (int w = 0; w < CHOCO_THREADS / 32; ++w) {
      g += sh[w * 2];
      e += sh[w * 2 + 1];
    }
    p.chunk_cnt[chunk * 2] = g;
    p.chunk_cnt[chunk * 2 + 1] = e;
    if (chunk == tb.seg_first_chunk[seg]) {
      p.sel[seg * 4] = thr;
      p.sel[seg * 4 + 1] = k3;  // how many keys equal to thr are kept (lowest indices first)
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(CHOCO_THREADS) choco_topk_count_kernel(const ChocoParams* __restrict__ params) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t sh[CHOCO_THREADS + 2];
  topk_count_chunk(params[blockIdx.y], blockIdx.x, sh);
}

extern "C" int choco_topk_count(const void* params_dev, int n_chunks, int n_ranks, cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  launch_k(choco_topk_count_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev));
  return (int)cudaGetLastError();
}

// publish helper shared by the emit kernels: last CTA raises the flags and advances the step
__device__ __forceinline__ void publish_if_last(const ChocoParams& p, uint32_t n_ctas, uint32_t t) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(p.done_count, 1u) == n_ctas - 1) {
      __threadfence_system();
      p.done_count[0] = 0;
      for (int k = 0; k < p.n_peers; ++k) st_release_sys(p.peer_flag[k], t + 1);
      __threadfence();
      p.step[0] = t + 1;
    }
  }
}

// ordered compaction: payload = [sum_k int32 indices][sum_k fp32 values]
__device__ void topk_emit_chunk(const ChocoParams& p, int chunk, uint32_t* sh /*[258]*/, uint32_t* sh_base /*[2]*/) {
  const SegTable& tb = p.tab;
  const int seg = tb.chunk_seg[chunk];
  const int start = tb.chunk_start[chunk];
  const int valid = tb.chunk_valid[chunk];
  const int seg_start = tb.seg_start[seg];
  const uint32_t t = p.step[0];
  const int PW = p.payload_words, par_cur = t & 1;
  const int sum_k = PW / 2;
  const uint32_t thr = p.sel[seg * 4], need_eq = p.sel[seg * 4 + 1];
  const int c0 = tb.seg_first_chunk[seg];

  // totals of the preceding chunks of this segment
  uint32_t gt_b = 0, eq_b = 0;
  {
    const uint2* cc = reinterpret_cast<const uint2*>(p.chunk_cnt);
#pragma unroll 4
    for (int c = c0 + threadIdx.x; c < chunk; c += CHOCO_THREADS) {
      const uint2 v = __ldcg(cc + c);
      gt_b += v.x;
      eq_b += v.y;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    gt_b += __shfl_xor_sync(0xffffffffu, gt_b, o);
    eq_b += __shfl_xor_sync(0xffffffffu, eq_b, o);
  }
  if ((threadIdx.x & 31) == 0) {
    sh[(threadIdx.x >> 5) * 2] = gt_b;
    sh[(threadIdx.x >> 5) * 2 + 1] = eq_b;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t g = 0, e = 0;
    for (int w = 0; w < CHOCO_THREADS / 32; ++w) {
      g += sh[w * 2];
      e += sh[w * 2 + 1];
    }
    sh_base[0] = g;
    sh_base[1] = e;
  }
  __syncthreads();
  uint32_t G = sh_base[0], E = sh_base[1];  // running counts before the current tile
  const uint32_t slot_begin = koff_of(tb, seg) + G + (E < need_eq ? E : need_eq);   // first slot this chunk fills
  const int koff = tb.seg_koff[seg];
  uint32_t* out_idx = p.outbox + par_cur * PW;
  uint32_t* out_val = out_idx + sum_k;

  // tiles of 2048 elements, 8 consecutive elements per thread (two 16-byte loads): one block scan
  // of the packed (gt, eq) counts per tile keeps the output ordered by index
  constexpr int EPT = 8, TILE = CHOCO_THREADS * EPT;
  const float* dptr = p.scratch_d + start;
  const int span = (valid + 3) & ~3;
  const int n_tiles = (valid + TILE - 1) / TILE;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 na = zero4, nb = zero4;  // next tile, loaded one iteration ahead
  {
    const int i0 = threadIdx.x * EPT;
    if (i0 < span) na = *reinterpret_cast<const float4*>(dptr + i0);
    if (i0 + 4 < span) nb = *reinterpret_cast<const float4*>(dptr + i0 + 4);
  }
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int i0 = tile * TILE + threadIdx.x * EPT;
    const float4 va = na, vb = nb;
    na = zero4; nb = zero4;
    if (i0 + TILE < span) na = *reinterpret_cast<const float4*>(dptr + i0 + TILE);
    if (i0 + TILE + 4 < span) nb = *reinterpret_cast<const float4*>(dptr + i0 + TILE + 4);
    const float d8[EPT] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
    uint32_t gt_mask = 0, eq_mask = 0;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const uint32_t key = key_of(d8[e]);
      if (i0 + e < valid) {
        gt_mask |= (uint32_t)(key > thr) << e;
        eq_mask |= (uint32_t)(key == thr) << e;
      }
    }
    const uint32_t v = __popc(gt_mask) | (__popc(eq_mask) << 16);
    uint32_t inc = v;
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) sh[wid] = inc;
    __syncthreads();
    uint32_t warp_off = 0, tile_tot = 0;
    for (int w = 0; w < CHOCO_THREADS / 32; ++w) {
      const uint32_t sw = sh[w];
      if (w < wid) warp_off += sw;
      tile_tot += sw;
    }
    if (gt_mask | eq_mask) {
      const uint32_t exc = warp_off + inc - v;
      uint32_t g_run = G + (exc & 0xFFFFu), e_run = E + (exc >> 16);
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        const bool is_gt = (gt_mask >> e) & 1u, is_eq = (eq_mask >> e) & 1u;
        if (is_gt || (is_eq && e_run < need_eq)) {
          const uint32_t slot = koff + g_run + (e_run < need_eq ? e_run : need_eq);
          const uint32_t idx = (uint32_t)(start + i0 + e - seg_start);
          const uint32_t vbits = __float_as_uint(d8[e]);
          out_idx[slot] = idx;
          out_val[slot] = vbits;
        }
        g_run += is_gt;
        e_run += is_eq;
      }
    }
    G += tile_tot & 0xFFFFu;
    E += tile_tot >> 16;
  }
  // push: the chunk's entries occupy a contiguous range of slots; the CTA copies the index and the value
  // range into every neighbour's mailbox with consecutive words per thread
  {
    const uint32_t slot_end = koff_of(tb, seg) + G + (E < need_eq ? E : need_eq);
    __syncthreads();
    push_words(p, par_cur * PW + (int)slot_begin, (int)(slot_end - slot_begin));
    push_words(p, par_cur * PW + sum_k + (int)slot_begin, (int)(slot_end - slot_begin));
  }
  // the first chunk of a segment clears the segment's histograms for the next step
  if (chunk == c0) {
    uint32_t* gh = p.hist + (size_t)seg * CHOCO_HIST_WORDS;
    for (int i = threadIdx.x; i < CHOCO_HIST_WORDS; i += CHOCO_THREADS) gh[i] = 0;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(CHOCO_THREADS) choco_topk_emit_kernel(const ChocoParams* __restrict__ params) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  __shared__ uint32_t sh[CHOCO_THREADS + 2];
  __shared__ uint32_t sh_base[2];
  const uint32_t t = p.step[0];
  topk_emit_chunk(p, blockIdx.x, sh, sh_base);
  publish_if_last(p, (uint32_t)p.tab.n_chunks, t);
}

extern "C" int choco_topk_emit(const void* params_dev, int n_chunks, int n_ranks, cudaStream_t stream) {
  dim3 grid(n_chunks, n_ranks);
  launch_k(choco_topk_emit_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev));
  return (int)cudaGetLastError();
}

__device__ __forceinline__ int segment_of_entry(const SegTable& tb, int e) {
  int lo = 0, hi = tb.n_segments - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tb.seg_koff[mid] <= e) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// random-k: payload = [sum_k fp32 values]; entry e of tensor `seg` is element perm(e - koff)
__device__ void randk_emit_entries(const ChocoParams& p, uint32_t t) {
  const SegTable& tb = p.tab;
  const int PW = p.payload_words, par_cur = t & 1;
  const int sum_k = PW;
  for (int e = blockIdx.x * CHOCO_THREADS + threadIdx.x; e < sum_k; e += gridDim.x * CHOCO_THREADS) {
    const int seg = segment_of_entry(tb, e);
    const uint32_t n = (uint32_t)tb.seg_size[seg];
    uint32_t keys[4];
#pragma unroll
    for (uint32_t r = 0; r < 4; ++r) keys[r] = feistel_key(p.seed, t, (uint32_t)seg, r);
    const uint32_t idx = feistel_perm((uint32_t)(e - tb.seg_koff[seg]), n, feistel_half_bits(n), keys);
    const uint32_t vb = __float_as_uint(p.scratch_d[tb.seg_start[seg] + idx]);
    p.outbox[par_cur * PW + e] = vb;
    for (int k = 0; k < p.n_peers; ++k) p.peer_inbox[k][par_cur * PW + e] = vb;
  }
}

__global__ void __launch_bounds__(CHOCO_THREADS) choco_randk_emit_kernel(const ChocoParams* __restrict__ params) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const uint32_t t = p.step[0];
  randk_emit_entries(p, t);
  publish_if_last(p, gridDim.x, t);
}

extern "C" int choco_randk_emit(const void* params_dev, int n_blocks, int n_ranks, cudaStream_t stream) {
  dim3 grid(n_blocks, n_ranks);
  launch_k(choco_randk_emit_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev));
  return (int)cudaGetLastError();
}

// Bounded wait for the neighbours' flags of step t-1 (one CTA per logical rank).
__global__ void choco_wait_flags_kernel(const ChocoParams* __restrict__ params) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.x];
  const uint32_t t = p.step[0];
  if (t == 0 || p.step[2] >= t) return;
  const int k = threadIdx.x;
  if (k < p.n_peers && !wait_flag_ge(p.my_flag[k], t, p.wait_budget_ns))
    report(p.status, CHOCO_TIMEOUT, p.peer_rank[k], (int)t - 1);
}

extern "C" int choco_wait_flags(const void* params_dev, int n_ranks, cudaStream_t stream) {
  launch_k(choco_wait_flags_kernel, dim3(n_ranks), dim3(32), 0, stream, reinterpret_cast<const ChocoParams*>(params_dev));
  return (int)cudaGetLastError();
}

// Apply one source payload of step t-1:  src < 0: own (x_hat += v, s += w_ii v);  src = k: s += w_ik v.
// codec 1 = top-k (indices in the payload), 2 = random-k (indices regenerated from the sender's seed).
// mark_done: this is the last source; record that step t-1 has been applied.
__device__ void sparse_decode_entries(const ChocoParams& p, uint32_t t, int src, int codec) {
  const SegTable& tb = p.tab;
  const int PW = p.payload_words, par_prev = (t - 1) & 1;
  const int sum_k = codec == 1 ? PW / 2 : PW;
  const uint32_t* pay = (src < 0 ? p.outbox : p.my_inbox[src]) + par_prev * PW;
  const float w = src < 0 ? p.w_self : p.w_peer[src];
  const int src_rank = src < 0 ? p.rank : p.peer_rank[src];
  const uint32_t seed = p.seed - 7919u * (uint32_t)p.rank + 7919u * (uint32_t)src_rank;
  for (int e = blockIdx.x * CHOCO_THREADS + threadIdx.x; e < sum_k; e += gridDim.x * CHOCO_THREADS) {
    const int seg = segment_of_entry(tb, e);
    uint32_t idx;
    float v;
    if (codec == 1) {
      idx = __ldcg(pay + e);
      v = __uint_as_float(__ldcg(pay + sum_k + e));
      if (idx >= (uint32_t)tb.seg_size[seg]) {  // corrupt payload: record and skip
        report(p.status, CHOCO_BAD_STEP, src_rank, (int)t - 1);
        continue;
      }
    } else {
      const uint32_t n = (uint32_t)tb.seg_size[seg];
      uint32_t keys[4];
#pragma unroll
      for (uint32_t r = 0; r < 4; ++r) keys[r] = feistel_key(seed, t - 1, (uint32_t)seg, r);
      idx = feistel_perm((uint32_t)(e - tb.seg_koff[seg]), n, feistel_half_bits(n), keys);
      v = __uint_as_float(__ldcg(pay + e));
    }
    const int pos = tb.seg_start[seg] + (int)idx;
    if (src < 0) p.x_hat[pos] += v;
    p.s[pos] += w * v;
  }
}

// flags bit 0: every CTA first waits (bounded) for the neighbours' flags of step t-1 (the first launch of a
// chain); bit 1: this is the last launch of the chain: its last CTA records that step t-1 has been applied.
__global__ void __launch_bounds__(CHOCO_THREADS) choco_sparse_decode_kernel(const ChocoParams* __restrict__ params,
                                                                          int src, int codec, int flags) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.y];
  const uint32_t t = p.step[0];
  __shared__ int sh_ok;
  const bool due = t > 0 && p.step[2] < t;
  bool ok = due && __ldcg(p.status) == CHOCO_OK;
  if ((flags & 1) && ok) {
    if (threadIdx.x < p.n_peers && !wait_flag_ge(p.my_flag[threadIdx.x], t, p.wait_budget_ns))
      report(p.status, CHOCO_TIMEOUT, p.peer_rank[threadIdx.x], (int)t - 1);
    __syncthreads();
    if (threadIdx.x == 0) sh_ok = __ldcg(p.status) == CHOCO_OK;
    __syncthreads();
    ok = sh_ok != 0;
  }
  if (ok && src < p.n_peers) sparse_decode_entries(p, t, src, codec);   // (fewer neighbours than the launch covers: nothing)
  if (flags & 2) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.done_count + 1, 1u) == gridDim.x - 1) {
        p.done_count[1] = 0;
        if (due && __ldcg(p.status) == CHOCO_OK) p.step[2] = t;
      }
    }
  }
}

__global__ void choco_mark_decoded_kernel(const ChocoParams* __restrict__ params) {
  pdl_wait();
  pdl_trigger();
  const ChocoParams& p = params[blockIdx.x];
  const uint32_t t = p.step[0];
  if (threadIdx.x == 0 && t > 0 && p.step[2] < t && p.status[0] == CHOCO_OK) p.step[2] = t;
}

extern "C" int choco_sparse_decode(const void* params_dev, int n_blocks, int n_ranks, int src, int codec,
                                   cudaStream_t stream) {
  const ChocoParams* p = reinterpret_cast<const ChocoParams*>(params_dev);
  if (src == 1000) {  // all sources applied: record it
    launch_k(choco_mark_decoded_kernel, dim3(n_ranks), dim3(32), 0, stream, p);
    return (int)cudaGetLastError();
  }
  dim3 grid(n_blocks, n_ranks);
  launch_k(choco_sparse_decode_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream, p, src, codec, 0);
  return (int)cudaGetLastError();
}

// one launch of a decode chain with the flag wait (flags & 1) and / or the completion mark (flags & 2) folded in
extern "C" int choco_sparse_decode_ex(const void* params_dev, int n_blocks, int n_ranks, int src, int codec, int flags,
                                      cudaStream_t stream) {
  dim3 grid(n_blocks, n_ranks);
  launch_k(choco_sparse_decode_kernel, dim3(grid), dim3(CHOCO_THREADS), 0, stream,
           reinterpret_cast<const ChocoParams*>(params_dev), src, codec, flags);
  return (int)cudaGetLastError();
}

// ---- the whole step of a sparsifying codec as ONE cooperative kernel ---------------------------
// Phases, separated by grid barriers of this logical rank's CTAs (gridDim.x CTAs, all co-resident:
// a cooperative launch):
//   wait for the neighbours' payloads of step t-1 | apply own payload | apply each neighbour's |
//   SGD + consensus step, d = x - x_hat (+ first radix histogram) | [top-k: histogram 2 | histogram 3 |
//   threshold and per-chunk counts |] compaction + push | raise the flags.
// The work inside a phase is the same device code as the stand-alone kernels above, walked with a
// grid-stride loop; only the launch boundaries are replaced.  Sources are applied one after the other
// (not with atomics) so that s and x_hat stay bitwise reproducible.

// Bounded barrier of the gridDim.x CTAs with blockIdx.y == this rank: bar[0] arrivals, bar[1] generation.
// Returns false (in every thread of the CTA) when the budget ran out.
__device__ bool rank_grid_barrier(uint32_t* bar, long long budget_ns, int* sh_ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    uint32_t gen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(bar + 1) : "memory");
    __threadfence();
    if (atomicAdd(bar, 1u) == gridDim.x - 1) {
      bar[0] = 0;
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bar + 1), "r"(gen + 1u) : "memory");
    } else {
      // tight polling (a barrier is a few microseconds); the clock is read once per 256 polls only
      long long t0 = 0;
      for (bool done = false; !done;) {
        for (int i = 0; i < 256; ++i) {
          uint32_t now;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(now) : "l"(bar + 1) : "memory");
          if (now != gen) { done = true; break; }
        }
        if (done) break;
        const long long tn = global_ns();
        if (t0 == 0) t0 = tn;
        else if (tn - t0 > budget_ns) { ok = 0; break; }
      }
    }
    *sh_ok = ok;
  }
  __syncthreads();
  return *sh_ok != 0;   // (the next barrier's write to sh_ok comes after its own __syncthreads)
}

// SGD step + consensus step + difference for one chunk (the non-decoding path of choco_dense_prep)
__device__ void sparse_prep_chunk(const ChocoParams& p, int chunk, int codec, uint32_t* sh_hist /*[2048]*/) {
  const SegTable& tb = p.tab;
  const int seg = tb.chunk_seg[chunk], start = tb.chunk_start[chunk], valid = tb.chunk_valid[chunk];
  const int span = (valid + 31) & ~31;
  const float lr = p.hyper[HYP_LR], mu = p.hyper[HYP_MOMENTUM], gamma = p.hyper[HYP_GAMMA];
  const bool nesterov = p.hyper[HYP_NESTEROV] != 0.f;
  const float gscale = p.hyper[HYP_GSCALE];
  const bool mom_init = p.step[1] != 0;
  const float wd = tb.seg_wd[seg];
  if (codec == 1) {
    for (int i = threadIdx.x; i < 2048; i += CHOCO_THREADS) sh_hist[i] = 0;
    __syncthreads();
  }
  for (int base = threadIdx.x * 4; base < span; base += CHOCO_THREADS * 4) {
    const int pos = start + base;
    const float4 xh = *reinterpret_cast<const float4*>(p.x_hat + pos);
    const float4 sv = *reinterpret_cast<const float4*>(p.s + pos);
    const float4 xv = *reinterpret_cast<const float4*>(p.x + pos);
    const float4 gv = load_grad4(p, seg, pos, base, valid);
    const float xh_a[4] = {xh.x, xh.y, xh.z, xh.w}, s_a[4] = {sv.x, sv.y, sv.z, sv.w};
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
    __syncthreads();
  }
}

// mode bit 0: apply the payloads of step t-1; bit 1: take the step and push (0 alone = decode only)
__global__ void __launch_bounds__(CHOCO_THREADS) choco_sparse_coop_kernel(const ChocoParams* __restrict__ params, int codec,
                                                                        int mode) {
  const ChocoParams& p = params[blockIdx.y];
  const SegTable& tb = p.tab;
  __shared__ uint32_t sh[CHOCO_THREADS + 2];
  __shared__ uint32_t sh_base[2];
  __shared__ uint32_t sh_hist[2048];
  __shared__ int sh_ok;
  uint32_t* bar = p.done_count + 4;   // words 4 (arrivals) and 5 (generation)
  const uint32_t t = p.step[0];
  const long long budget = p.wait_budget_ns;
  // (a barrier may have to outwait CTA 0's flag wait: twice the budget plus a margin)
#define COOP_BARRIER()                                                      \
  if (!rank_grid_barrier(bar, 2 * budget + 1000000, &sh_ok)) {              \
    if (threadIdx.x == 0) report(p.status, CHOCO_TIMEOUT, p.rank, (int)t);  \
    return;                                                                 \
  }
  const bool decode = (mode & 1) && t > 0 && p.step[2] < t;
  if (decode) {
    if (blockIdx.x == 0 && threadIdx.x < p.n_peers &&
        !wait_flag_ge(p.my_flag[threadIdx.x], t, budget))
      report(p.status, CHOCO_TIMEOUT, p.peer_rank[threadIdx.x], (int)t - 1);
    COOP_BARRIER();
    if (__ldcg(p.status) != CHOCO_OK) return;      // the same answer in every CTA: written before the barrier
    for (int src = -1; src < p.n_peers; ++src) {
      sparse_decode_entries(p, t, src, codec);
      COOP_BARRIER();
    }
  } else if ((mode & 2) && t > 0 && p.step[2] < t) {
    if (blockIdx.x == 0 && threadIdx.x == 0) report(p.status, CHOCO_BAD_STEP, -1, (int)t);
  }
  if (!(mode & 2)) {
    if (decode && blockIdx.x == 0 && threadIdx.x == 0) p.step[2] = t;
    return;
  }
  for (int c = blockIdx.x; c < tb.n_chunks; c += gridDim.x) sparse_prep_chunk(p, c, codec, sh_hist);
  COOP_BARRIER();
  if (codec == 1) {
    for (int c = blockIdx.x; c < tb.n_chunks; c += gridDim.x) topk_hist_chunk(p, c, 2, sh, sh_hist);
    COOP_BARRIER();
    for (int c = blockIdx.x; c < tb.n_chunks; c += gridDim.x) topk_hist_chunk(p, c, 3, sh, sh_hist);
    COOP_BARRIER();
    for (int c = blockIdx.x; c < tb.n_chunks; c += gridDim.x) topk_count_chunk(p, c, sh);
    COOP_BARRIER();
    for (int c = blockIdx.x; c < tb.n_chunks; c += gridDim.x) topk_emit_chunk(p, c, sh, sh_base);
  } else {
    randk_emit_entries(p, t);
  }
  // every CTA's pushes are ordered before its arrival; one thread then raises the flags
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
  COOP_BARRIER();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int k = 0; k < p.n_peers; ++k) st_release_sys(p.peer_flag[k], t + 1);
    if (decode) p.step[2] = t;
    p.step[1] = 1;
    __threadfence();
    p.step[0] = t + 1;
  }
#undef COOP_BARRIER
}

// Largest gridDim.x such that gridDim.x * n_ranks CTAs are co-resident on the current device.
extern "C" int choco_sparse_coop_max_grid(int n_ranks) {
  int dev = 0, sms = 0, per_sm = 0;
  if (n_ranks < 1 || cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, choco_sparse_coop_kernel, CHOCO_THREADS, 0) != cudaSuccess)
    return -1;
  return sms * per_sm / n_ranks;
}

extern "C" int choco_sparse_coop_step(const void* params_dev, int grid_x, int n_ranks, int codec, int mode,
                                      cudaStream_t stream) {
  if (grid_x < 1 || n_ranks < 1 || !(codec == 1 || codec == 2)) return -1;
  dim3 grid(grid_x, n_ranks);
  void* args[] = {(void*)&params_dev, (void*)&codec, (void*)&mode};
  return (int)cudaLaunchCooperativeKernel((const void*)choco_sparse_coop_kernel, grid, dim3(CHOCO_THREADS), args, 0, stream);
}
