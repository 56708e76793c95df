// Nucleus (top-p) + temperature sampling, one 1024-thread block per row
// (reference: mesh_transformer/sampling.py:6-44).
//
// The reference sorts the row in descending order (higher index first among
// equal values, -0 == +0), removes every entry for which the cumulative softmax
// probability of the entries sorted BEFORE it exceeds top_p (the head always
// stays), and takes argmax((logit - 1e10 * removed) / temp + Gumbel(uniform)),
// lowest index on ties (jax.random.categorical).
//
// Here the softmax numerators e_i = exp(l_i - max) become fixed-point weights
// q_i = floor(e_i * 2^40); sums of weights are exact integers, so they do not
// depend on the order of addition and the test reads
//     (weight sorted before entry j)  >  T = floor(top_p * total weight).
// With exact sums the removed entries are a suffix of the sorted order: it is
// enough to find the entry whose weight interval [before, before + q) contains
// T.  That is a most-significant-digit radix SELECTION on the 32-bit sort key
// (four passes of weighted 256-bin histograms, no sort); entries with a larger
// key are removed, entries with the same key (equal logits) are ranked by
// descending index in a separate pass that only runs when the cut falls inside
// such a group.  exp and log are fixed polynomials of individually rounded
// fp32 operations (no FMA contraction), so a CPU restatement reproduces the
// token ids bit for bit.
//
// top_k (sampling.py:15-26) is a second selection, by COUNT instead of weight:
// the key of the entry with sorted rank top_k - 1 and, among entries with that
// key, the index below which they fall outside the first top_k.  Such an entry
// i loses 1e10 * i (the reference scatters the token INDEX, not a flag, into
// its mask, so token 0 is never masked by this branch); the cumulative
// probabilities of the top-p rule still come from the unmasked logits.
#include <math.h>

#include <algorithm>

#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

constexpr int kSampThreads = 1024;

__device__ __forceinline__ float exp_pinned(float x) {     // x <= 0
  const float xs = fmaxf(x, -87.0f);
  const float n = rintf(__fmul_rn(xs, 1.4426950408889634f));
  float r = __fsub_rn(xs, __fmul_rn(n, 0.693145751953125f));
  r = __fsub_rn(r, __fmul_rn(n, 1.42860682030941723212e-6f));
  float p = 1.9875691500e-4f;
  p = __fadd_rn(__fmul_rn(p, r), 1.3981999507e-3f);
  p = __fadd_rn(__fmul_rn(p, r), 8.3334519073e-3f);
  p = __fadd_rn(__fmul_rn(p, r), 4.1665795894e-2f);
  p = __fadd_rn(__fmul_rn(p, r), 1.6666665459e-1f);
  p = __fadd_rn(__fmul_rn(p, r), 5.0000001201e-1f);
  const float r2 = __fmul_rn(r, r);
  const float y = __fadd_rn(__fadd_rn(__fmul_rn(p, r2), r), 1.0f);
  const float scale = __int_as_float((static_cast<int>(n) + 127) << 23);
  return x < -87.0f ? 0.0f : __fmul_rn(y, scale);
}

__device__ __forceinline__ float log_pinned(float x) {     // positive, normal
  const int bits = __float_as_int(x);
  int e = ((bits >> 23) & 0xFF) - 126;
  const float m = __int_as_float((bits & 0x007FFFFF) | 0x3F000000);
  const bool small = m < 0.70710678118654752440f;
  const float ef = static_cast<float>(small ? e - 1 : e);
  const float f = __fsub_rn(small ? __fadd_rn(m, m) : m, 1.0f);
  const float z = __fmul_rn(f, f);
  float p = 7.0376836292e-2f;
  p = __fadd_rn(__fmul_rn(p, f), -1.1514610310e-1f);
  p = __fadd_rn(__fmul_rn(p, f), 1.1676998740e-1f);
  p = __fadd_rn(__fmul_rn(p, f), -1.2420140846e-1f);
  p = __fadd_rn(__fmul_rn(p, f), 1.4249322787e-1f);
  p = __fadd_rn(__fmul_rn(p, f), -1.6668057665e-1f);
  p = __fadd_rn(__fmul_rn(p, f), 2.0000714765e-1f);
  p = __fadd_rn(__fmul_rn(p, f), -2.4999993993e-1f);
  p = __fadd_rn(__fmul_rn(p, f), 3.3333331174e-1f);
  float y = __fmul_rn(__fmul_rn(p, f), z);
  y = __fadd_rn(y, __fmul_rn(ef, -2.12194440e-4f));
  y = __fsub_rn(y, __fmul_rn(0.5f, z));
  return __fadd_rn(__fadd_rn(f, y), __fmul_rn(ef, 0.693359375f));
}

__device__ __forceinline__ uint32_t sort_key(float v) {
  if (v == 0.0f) v = 0.0f;                                  // -0 and +0 compare equal
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);           // ascending integer order == ascending float order
  return ~u;                                                // ascending key == descending value
}

__device__ __forceinline__ float inv_sort_key(uint32_t key) {
  const uint32_t u = ~key;
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// q = floor(exp(l - vmax) * 2^40): a power-of-two scaling (exact) and a truncation
__device__ __forceinline__ unsigned long long weight_of(float l, float vmax) {
  return __float2ull_rz(__fmul_rn(exp_pinned(__fsub_rn(l, vmax)), 1099511627776.0f));
}

// h[dig] += q for the participating lanes of a warp; h belongs to this warp alone.  Lanes whose digit
// no other lane shares add directly (distinct addresses); the others are summed group by group.
__device__ __forceinline__ void warp_hist_add(unsigned long long* h, uint32_t dig, unsigned long long q, bool part,
                                              int lane) {
  const uint32_t same = __match_any_sync(0xffffffffu, dig);
  const bool alone = __popc(same) == 1;
  if (part && alone) h[dig] += q;
  uint32_t rem = __ballot_sync(0xffffffffu, part && !alone);
  while (rem) {
    const int src = __ffs(rem) - 1;
    const uint32_t dsel = __shfl_sync(0xffffffffu, dig, src);
    const bool member = dig == dsel;
    // q < 2^41: three 14-bit limbs, whose sums over 32 lanes fit 32 bits, one warp reduction each
    const unsigned long long qm = member ? q : 0ull;
    const uint32_t s0 = __reduce_add_sync(0xffffffffu, static_cast<uint32_t>(qm) & 0x3FFFu);
    const uint32_t s1 = __reduce_add_sync(0xffffffffu, static_cast<uint32_t>(qm >> 14) & 0x3FFFu);
    const uint32_t s2 = __reduce_add_sync(0xffffffffu, static_cast<uint32_t>(qm >> 28));
    if (lane == src)
      h[dsel] += static_cast<unsigned long long>(s0) + (static_cast<unsigned long long>(s1) << 14) +
                 (static_cast<unsigned long long>(s2) << 28);
    rem &= ~__ballot_sync(0xffffffffu, member);
  }
  __syncwarp();
}

// g = -log(-log(u)), the Gumbel noise of jax.random.categorical, for rows * V uniforms
__global__ void __launch_bounds__(256) gumbel_kernel(const float* __restrict__ u, float* __restrict__ g, size_t n) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * 256) {
    const float tl = log_pinned(u[i]);
    g[i] = -log_pinned(-tl);
  }
}

// Counter-based generator for the sampler's uniforms (Philox4x32-10, Salmon et al. 2011): stands in for the
// jax.random key stream of the generate scan (transformer_shard.py:200,327-335).  One call yields four 32-bit
// words = the uniforms of four consecutive vocabulary entries of one (position, sequence).
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u, kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(kM0, ctr.x), lo0 = kM0 * ctr.x;
    const uint32_t hi1 = __umulhi(kM1, ctr.z), lo1 = kM1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += kW0;
    key.y += kW1;
  }
  return ctr;
}
// 24 random bits -> [tiny, 1): jax.random.gumbel draws its uniforms with minval = tiny
__device__ __forceinline__ float rng_uniform(uint32_t w) {
  return fmaxf(static_cast<float>(w >> 8) * 5.9604644775390625e-08f, 1.17549435e-38f);
}

// uniforms (out_u) or their Gumbel noise (out_g) for rows x V entries at decode position *pos_dev (or pos_host)
__global__ void __launch_bounds__(256) rng_kernel(const uint32_t* __restrict__ seed, uint32_t seed_lo, uint32_t seed_hi,
                                                  const int32_t* pos_dev, int pos_host, float* out_u, float* out_g,
                                                  int rows, int V) {
  pdl_wait();
  pdl_launch_dependents();
  const uint2 key = seed ? make_uint2(seed[0], seed[1]) : make_uint2(seed_lo, seed_hi);
  const uint32_t pos = static_cast<uint32_t>(pos_dev ? *pos_dev : pos_host);
  const int groups = (V + 3) >> 2;
  for (size_t t = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; t < static_cast<size_t>(rows) * groups;
       t += static_cast<size_t>(gridDim.x) * 256) {
    const uint32_t row = static_cast<uint32_t>(t / groups), grp = static_cast<uint32_t>(t % groups);
    const uint4 w = philox4x32_10(make_uint4(grp, row, pos, 0x4d544au), key);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = static_cast<int>(grp) * 4 + e;
      if (col >= V) break;
      const float u = rng_uniform(ws[e]);
      const size_t i = static_cast<size_t>(row) * V + col;
      if (out_u) out_u[i] = u;
      if (out_g) out_g[i] = -log_pinned(-log_pinned(u));
    }
  }
}

constexpr int kBins = 256;
constexpr int kMaxCluster = 8;

// thread-block cluster helpers: the blocks of one row exchange small results through each other's shared memory
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_smem(const void* p, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
  return a;
}
__device__ __forceinline__ unsigned long long ld_peer_u64(const void* p, uint32_t rank) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(peer_smem(p, rank)) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_peer_u32(const void* p, uint32_t rank) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(peer_smem(p, rank)) : "memory");
  return v;
}

// One row = one cluster of C blocks (C = 1, 2, 4 or 8); block c owns the vocabulary slice
// [c * slice, (c + 1) * slice).  Every block computes the histogram of its slice, reads the other blocks'
// 256 bin sums through distributed shared memory and makes the same selection, so control flow stays
// uniform over the cluster (every block reaches every cluster barrier).
__global__ void __launch_bounds__(kSampThreads, 1) sample_top_p_kernel(const SampleArgs a) {
  extern __shared__ __align__(16) unsigned char samp_smem[];
  unsigned long long* hist = reinterpret_cast<unsigned long long*>(samp_smem);          // [32 warps][256]
  unsigned long long* bins = hist + 32 * kBins;                                         // [2][256] by level parity
  unsigned long long* gbins = bins + 2 * kBins;                                         // [256] sums over the cluster
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(gbins + kBins);                        // [ceil(slice / 32)]
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  __shared__ uint32_t wsum[33];
  __shared__ uint32_t sel_digit, sel_none;
  __shared__ unsigned long long sel_before, sel_sum, sel_T;
  __shared__ uint32_t x_max, x_ties, x_best_v, x_best_i;      // read by the other blocks of the cluster
  __shared__ uint32_t x_kties, x_kidx;

  const uint32_t C = cluster_size(), crank = cluster_rank();
  const int row = blockIdx.x / C, t = threadIdx.x, V = a.V;
  const int lane = t & 31, warp = t >> 5;
  const float* logits = a.logits + static_cast<size_t>(row) * V;
  const float* gum = a.gumbel ? a.gumbel + static_cast<size_t>(row) * V : nullptr;   // null: filter only
  const int slice = ((V + static_cast<int>(C) - 1) / static_cast<int>(C) + 31) & ~31;
  const int i_begin = min(V, static_cast<int>(crank) * slice), i_end = min(V, i_begin + slice);

  // ---- row maximum (the head of the sorted order) ----
  float vmax = -INFINITY;
  for (int i = i_begin + t; i < i_end; i += kSampThreads) vmax = fmaxf(vmax, logits[i]);
  vmax = warp_max(vmax);
  if (lane == 0) red_v[warp] = vmax;
  __syncthreads();
  vmax = red_v[0];
#pragma unroll
  for (int w = 1; w < 32; ++w) vmax = fmaxf(vmax, red_v[w]);
  if (t == 0) x_max = __float_as_uint(vmax);
  cluster_sync();
  for (uint32_t c = 0; c < C; ++c) vmax = fmaxf(vmax, __uint_as_float(ld_peer_u32(&x_max, c)));

  // ---- radix selection of the entry whose weight interval contains T ----
  const float top_p = a.top_p[row], temp = a.temp ? a.temp[row] : 1.0f;
  uint32_t prefix = 0;                     // the selected key's digits so far
  unsigned long long before = 0;           // weight of all keys below the selected prefix
  unsigned long long T = 0, group_sum = 0;
  bool cut = true;                         // false: nothing is removed
  unsigned long long* my_hist = hist + warp * kBins;
  for (int level = 0; level < 4 && cut; ++level) {
    const int shift = 24 - 8 * level;
    unsigned long long* lbins = bins + (level & 1) * kBins;
    for (int i = t; i < 32 * kBins; i += kSampThreads) hist[i] = 0ull;
    __syncthreads();
    for (int i0 = i_begin; i0 < i_end; i0 += 4 * kSampThreads) {
      float l[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kSampThreads + t;
        l[u] = i < i_end ? logits[i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + u * kSampThreads >= i_end) break;         // block-uniform
        const int i = i0 + u * kSampThreads + t;
        const uint32_t key = sort_key(l[u]);
        const bool part = i < i_end && (level == 0 || (key >> (shift + 8)) == prefix);
        const uint32_t dig = part ? ((key >> shift) & 255u) : 0xFFFFu;
        const unsigned long long q = part ? weight_of(l[u], vmax) : 0ull;
        warp_hist_add(my_hist, dig, q, part, lane);
      }
    }
    __syncthreads();
    if (t < kBins) {
      unsigned long long sum = 0ull;
#pragma unroll 8
      for (int w = 0; w < 32; ++w) sum += hist[w * kBins + t];
      lbins[t] = sum;
    }
    cluster_sync();                                        // every block's bin sums of this level are in place
    if (t < kBins) {
      unsigned long long sum = 0ull;
      for (uint32_t c = 0; c < C; ++c) sum += ld_peer_u64(lbins + t, c);
      gbins[t] = sum;
    }
    __syncthreads();
    if (warp == 0) {
      unsigned long long b[8], local = 0ull;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        b[k] = gbins[lane * 8 + k];
        local += b[k];
      }
      unsigned long long inc = local;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const unsigned long long y = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += y;
      }
      if (level == 0) {
        // the grand total gives the threshold T = floor(top_p * total), evaluated exactly (same in every lane)
        const unsigned long long total = __shfl_sync(0xffffffffu, inc, 31);
        bool none = false;
        const uint32_t pb = __float_as_uint(top_p);
        const int ex = static_cast<int>((pb >> 23) & 0xFFu);
        if (top_p != top_p || (ex == 255 && !(pb >> 31))) {
          none = true;                                     // NaN or +inf: nothing exceeds it
        } else if ((pb >> 31) || ex == 0) {
          T = 0ull;                                        // negative, zero or subnormal (top_p * total < 1)
        } else {
          const unsigned long long m = (pb & 0x007FFFFFu) | 0x00800000u;   // top_p = m * 2^(ex - 150)
          const unsigned long long lo = total * m, hi = __umul64hi(total, m);
          const int sh = 150 - ex;                         // right shift of the 128-bit product
          if (sh <= 0) {
            none = true;                                   // top_p >= 2^23
          } else if (sh >= 128) {
            T = 0ull;
          } else if (sh >= 64) {
            T = hi >> (sh - 64);
          } else {
            if (hi >> sh) none = true;                     // does not fit 64 bits: far above the total
            T = (lo >> sh) | (hi << (64 - sh));
          }
        }
        if (!none && T >= total) none = true;              // no entry has that much weight before it
        if (lane == 0) {
          sel_T = T;
          sel_none = none ? 1u : 0u;
        }
        if (none) cut = false;
      }
      if (cut) {
        // the bin whose weight interval [run, run + b) contains T
        unsigned long long run = before + inc - local;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (T >= run && T - run < b[k]) {
            sel_digit = static_cast<uint32_t>(lane * 8 + k);
            sel_before = run;
            sel_sum = b[k];
          }
          run += b[k];
        }
      }
    }
    __syncthreads();
    if (level == 0) {
      T = sel_T;
      cut = sel_none == 0u;
    }
    if (cut) {
      prefix = (prefix << 8) | sel_digit;
      before = sel_before;
      group_sum = sel_sum;
    }
    __syncthreads();
  }

  // ---- the selected key k0: larger keys are removed; equal keys by rank (descending index) ----
  const uint32_t k0 = prefix;
  bool tie_cut = false;
  unsigned long long r0 = 0ull;
  if (cut) {
    const unsigned long long qt = weight_of(inv_sort_key(k0), vmax);     // > 0: the interval contains T
    const unsigned long long cnt = group_sum / qt;
    r0 = (T - before) / qt;                                              // rank of the entry that holds T
    tie_cut = r0 + 1 < cnt;
  }
  if (tie_cut) {                                                         // uniform over the cluster
    // thread t owns a contiguous index range of this block's slice, thread 0 the highest indices
    const int n_own = i_end - i_begin;
    const int per = (n_own + kSampThreads - 1) / kSampThreads;
    const int hi_i = i_end - 1 - t * per, lo_i = max(i_begin - 1, hi_i - per);
    for (int i = t; i < (n_own + 31) / 32; i += kSampThreads) bitmap[i] = 0u;
    uint32_t mine = 0;
    for (int i = hi_i; i > lo_i; --i) mine += sort_key(logits[i]) == k0 ? 1u : 0u;
    uint32_t inc = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t y = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += y;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const uint32_t w = wsum[lane];
      uint32_t winc = w;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, winc, off);
        if (lane >= off) winc += y;
      }
      wsum[lane] = winc - w;
      if (lane == 31) x_ties = winc;                                     // equal keys in this block's slice
    }
    cluster_sync();
    unsigned long long rank = wsum[warp] + inc - mine;
    for (uint32_t c = crank + 1; c < C; ++c) rank += ld_peer_u32(&x_ties, c);   // slices with higher indices come first
    for (int i = hi_i; i > lo_i; --i) {
      if (sort_key(logits[i]) == k0) {
        if (rank > r0) atomicOr(bitmap + ((i - i_begin) >> 5), 1u << ((i - i_begin) & 31));
        ++rank;
      }
    }
    __syncthreads();
  }

  // ---- top_k: key kk of the entry of sorted rank top_k - 1; equal keys below index kidx are beyond it ----
  uint32_t kk = 0xFFFFFFFFu;
  int kidx = 0;                                            // defaults: no entry is beyond the first top_k
  if (a.top_k) {                                           // uniform over the grid
    const int k = a.top_k[row];
    if (k <= 0) {
      kk = 0u;
      kidx = V;                                            // every entry is beyond the first top_k
    } else if (k < V) {                                    // uniform over the cluster
      uint32_t* cnt = reinterpret_cast<uint32_t*>(hist);
      const unsigned long long R = static_cast<unsigned long long>(k - 1);
      uint32_t kprefix = 0;
      unsigned long long kbefore = 0, kgroup = 0;
      cluster_sync();                                      // the bin sums of the last top-p level have been read
      for (int level = 0; level < 4; ++level) {
        const int shift = 24 - 8 * level;
        unsigned long long* lbins = bins + (level & 1) * kBins;
        if (t < kBins) cnt[t] = 0u;
        __syncthreads();
        for (int i = i_begin + t; i < i_end; i += kSampThreads) {
          const uint32_t key = sort_key(logits[i]);
          if (level == 0 || (key >> (shift + 8)) == kprefix) atomicAdd(cnt + ((key >> shift) & 255u), 1u);
        }
        __syncthreads();
        if (t < kBins) lbins[t] = cnt[t];
        cluster_sync();
        if (t < kBins) {
          unsigned long long sum = 0ull;
          for (uint32_t c = 0; c < C; ++c) sum += ld_peer_u64(lbins + t, c);
          gbins[t] = sum;
        }
        __syncthreads();
        if (warp == 0) {
          unsigned long long b[8], local = 0ull;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            b[j] = gbins[lane * 8 + j];
            local += b[j];
          }
          unsigned long long inc = local;
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) {
            const unsigned long long y = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += y;
          }
          unsigned long long run = kbefore + inc - local;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (R >= run && R - run < b[j]) {
              sel_digit = static_cast<uint32_t>(lane * 8 + j);
              sel_before = run;
              sel_sum = b[j];
            }
            run += b[j];
          }
        }
        __syncthreads();
        kprefix = (kprefix << 8) | sel_digit;
        kbefore = sel_before;
        kgroup = sel_sum;
        __syncthreads();
      }
      kk = kprefix;
      const unsigned long long n_keep = R - kbefore + 1;   // entries with key kk inside the first top_k: 1..kgroup
      if (n_keep < kgroup) {                               // uniform over the cluster
        // the n_keep-th highest index among the entries with key kk; same ownership as the tie pass above
        const int n_own = i_end - i_begin;
        const int per = (n_own + kSampThreads - 1) / kSampThreads;
        const int hi_i = i_end - 1 - t * per, lo_i = max(i_begin - 1, hi_i - per);
        uint32_t mine = 0;
        for (int i = hi_i; i > lo_i; --i) mine += sort_key(logits[i]) == kk ? 1u : 0u;
        uint32_t inc = mine;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const uint32_t y = __shfl_up_sync(0xffffffffu, inc, off);
          if (lane >= off) inc += y;
        }
        if (t == 0) x_kidx = 0xFFFFFFFFu;
        __syncthreads();                                   // also: the tie pass above is done with wsum
        if (lane == 31) wsum[warp] = inc;
        __syncthreads();
        if (warp == 0) {
          const uint32_t w = wsum[lane];
          uint32_t winc = w;
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, winc, off);
            if (lane >= off) winc += y;
          }
          wsum[lane] = winc - w;
          if (lane == 31) x_kties = winc;
        }
        cluster_sync();
        unsigned long long rank = wsum[warp] + inc - mine;
        for (uint32_t c = crank + 1; c < C; ++c) rank += ld_peer_u32(&x_kties, c);
        for (int i = hi_i; i > lo_i; --i) {
          if (sort_key(logits[i]) == kk) {
            if (rank + 1 == n_keep) x_kidx = static_cast<uint32_t>(i);       // exactly one entry of the row
            ++rank;
          }
        }
        cluster_sync();
        uint32_t found = 0xFFFFFFFFu;
        for (uint32_t c = 0; c < C; ++c) found = min(found, ld_peer_u32(&x_kidx, c));
        kidx = static_cast<int>(found);
      }
    }
  }

  // ---- Gumbel-max over the filtered, tempered logits ----
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = i_begin + t; i < i_end; i += kSampThreads) {
    const float lg = logits[i];
    const uint32_t key = sort_key(lg);
    const int j = i - i_begin;
    const bool removed = cut && (key > k0 || (tie_cut && key == k0 && ((bitmap[j >> 5] >> (j & 31)) & 1u)));
    const bool beyond_k = key > kk || (key == kk && i < kidx);
    const float lk = beyond_k ? __fsub_rn(lg, __fmul_rn(1e10f, static_cast<float>(i))) : lg;
    const float lm = __fsub_rn(lk, removed ? 1e10f : 0.0f);
    if (a.filtered) a.filtered[static_cast<size_t>(row) * V + i] = lm;       // nucleaus_filter's return value
    const float score = __fadd_rn(__fdiv_rn(lm, temp), gum ? gum[i] : 0.0f);
    if (score > best) {                                    // ascending i: the first maximum stays
      best = score;
      best_i = i;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  if (lane == 0) {
    red_v[warp] = best;
    red_i[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    best = red_v[lane];
    best_i = red_i[lane];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, off);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (lane == 0) {
      x_best_v = __float_as_uint(best);
      x_best_i = static_cast<uint32_t>(best_i);
    }
  }
  cluster_sync();
  if (crank == 0 && t == 0) {
    for (uint32_t c = 1; c < C; ++c) {
      const float ov = __uint_as_float(ld_peer_u32(&x_best_v, c));
      const int oi = static_cast<int>(ld_peer_u32(&x_best_i, c));
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (a.tokens) a.tokens[row] = static_cast<uint32_t>(best_i);
    if (a.tokens_copy) a.tokens_copy[row] = static_cast<uint32_t>(best_i);
    if (a.cur_dev && row == 0) *a.cur_dev += 1;
  }
  cluster_sync();                                          // no block leaves while its shared memory may be read
}

inline int sample_cluster(int rows) { return rows <= 18 ? 8 : (rows <= 37 ? 4 : (rows <= 74 ? 2 : 1)); }
inline size_t sample_smem_bytes(int V, int cluster) {
  const int slice = ((V + cluster - 1) / cluster + 31) & ~31;
  return sizeof(unsigned long long) * (32 * kBins + 3 * kBins) + sizeof(uint32_t) * static_cast<size_t>((slice + 31) / 32);
}

}  // namespace

// one float per logit: the Gumbel noise derived from the uniforms
int64_t sample_scratch_bytes(int rows, int vocab) { return static_cast<int64_t>(rows) * vocab * 4; }

namespace {
// the attribute belongs to the device, not to the process
cudaError_t configure_sampler() {
  static DeviceOnce once;
  return once.run([] {
    return cudaFuncSetAttribute(sample_top_p_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  });
}

cudaError_t launch_selection(const SampleArgs& b, cudaStream_t s) {
  const int cluster = sample_cluster(b.rows);
  cudaLaunchAttribute cattr[1];
  cattr[0].id = cudaLaunchAttributeClusterDimension;
  cattr[0].val.clusterDim.x = cluster;
  cattr[0].val.clusterDim.y = 1;
  cattr[0].val.clusterDim.z = 1;
  cudaLaunchConfig_t scfg = {};
  scfg.gridDim = dim3(static_cast<unsigned>(b.rows * cluster));
  scfg.blockDim = dim3(kSampThreads);
  scfg.dynamicSmemBytes = sample_smem_bytes(b.V, cluster);
  scfg.stream = s;
  scfg.attrs = cattr;
  scfg.numAttrs = 1;
  return cudaLaunchKernelEx(&scfg, sample_top_p_kernel, b);
}
}  // namespace

cudaError_t launch_rng_uniforms(uint64_t seed, int position, int rows, int V, float* out, cudaStream_t s) {
  if (rows <= 0 || V <= 0 || !out) return cudaErrorInvalidValue;
  const size_t n = static_cast<size_t>(rows) * ((V + 3) / 4);
  const unsigned grid = static_cast<unsigned>(std::min<size_t>((n + 255) / 256, 148 * 8));
  rng_kernel<<<grid, 256, 0, s>>>(nullptr, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), nullptr,
                                  position, out, nullptr, rows, V);
  return cudaGetLastError();
}

// nucleaus_filter alone (sampling.py:10-38): filtered[r, i] = logits[r, i] - 1e10 * removed[r, i]
cudaError_t launch_nucleus_filter(const float* logits, const float* top_p, const int32_t* top_k, int rows, int V,
                                  float* filtered, cudaStream_t s) {
  if (rows <= 0 || V <= 0 || sample_smem_bytes(V, sample_cluster(rows)) > 220 * 1024) return cudaErrorInvalidValue;
  cudaError_t e = configure_sampler();
  if (e != cudaSuccess) return e;
  SampleArgs b = {};
  b.logits = logits;
  b.top_p = top_p;
  b.top_k = top_k;
  b.rows = rows;
  b.V = V;
  b.filtered = filtered;
  return launch_selection(b, s);
}

cudaError_t launch_sample_top_p(const SampleArgs& a, cudaStream_t s, bool pdl) {
  const int cluster = sample_cluster(a.rows);              // blocks per row: as many as keep one wave on 148 SMs
  const size_t smem = sample_smem_bytes(a.V, cluster);
  if (a.rows <= 0 || a.V <= 0 || smem > 220 * 1024 || !a.scratch) return cudaErrorInvalidValue;
  {
    cudaError_t e = configure_sampler();
    if (e != cudaSuccess) return e;
  }
  const size_t n = static_cast<size_t>(a.rows) * a.V;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(std::min<size_t>((n + 255) / 256, 148 * 8)));
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  float* g = static_cast<float*>(a.scratch);
  cudaError_t e;
  if (a.uniforms) {
    e = cudaLaunchKernelEx(&cfg, gumbel_kernel, a.uniforms, g, n);
  } else if (a.rng_seed) {                                 // no uniforms supplied: the device generator draws them
    cfg.gridDim = dim3(static_cast<unsigned>(std::min<size_t>((n / 4 + 255) / 256, 148 * 8)));
    e = cudaLaunchKernelEx(&cfg, rng_kernel, a.rng_seed, 0u, 0u, static_cast<const int32_t*>(a.cur_dev), 0,
                           static_cast<float*>(nullptr), g, a.rows, a.V);
  } else {
    return cudaErrorInvalidValue;
  }
  if (e != cudaSuccess) return e;
  SampleArgs b = a;
  b.gumbel = g;
  return launch_selection(b, s);
}

}  // namespace mtj
