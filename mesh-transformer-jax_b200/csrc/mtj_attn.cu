// Attention over the paged bf16 KV cache.
//
// decode_attn_kernel : one query per (sequence, head); the visible key range
//   [max(pad, cur-window+1), cur] is cut into one split per 64-token page, one
//   block per split: the page's K and V slabs of that head are contiguous and
//   arrive in shared memory by one bulk copy (TMA) each, issued before the wait
//   on the predecessor kernel for every page but the newest.  Partial (max,
//   sum, weighted V) triples are merged by the last block of each (sequence,
//   head) to finish.  HBM-bound: every K/V byte is read once.  (reference: layers.py:316-338 -- the sliding
//   window of seq-1 slots, left slots masked by tokens_decoded.)
// prefill_attn_kernel: causal multi-query attention used to build the decode
//   state and for eval (layers.py:275-283,299-313,347-366); CUDA-core version.
//
// Keys are stored already rotated at their absolute position, so the dot
// product depends only on the query/key distance, like the reference's
// re-rotation of the shifted window (layers.py:268-270,147).  Masked keys are
// skipped, which equals the reference's additive -1e10 whenever at least one
// key is visible (exp underflows to exactly 0 in fp32).
#include <math.h>
#include <stdlib.h>

#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;

template <int EPL>
struct KvVec;
template <>
struct KvVec<8> {
  uint4 v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = ld_stream16(p); }
  __device__ __forceinline__ void load_shared(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void get(float* f) const { unpack8(v, f); }
};
template <>
struct KvVec<2> {
  uint32_t v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = ld_stream4(p); }
  __device__ __forceinline__ void load_shared(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint32_t*>(p); }
  __device__ __forceinline__ void get(float* f) const {
    f[0] = bf16_lo(v);
    f[1] = bf16_hi(v);
  }
};

template <int DH>
__global__ void __launch_bounds__(kAttnThreads) decode_attn_kernel(const DecodeAttnArgs a) {
  constexpr int EPL = DH / 32;
  constexpr int TPW = kPageTokens / kAttnWarps;            // tokens per warp: 8
  constexpr uint32_t kSlab = kPageTokens * DH * 2;         // one (page, head) slab of K or V in bytes
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int split = blockIdx.x, head = blockIdx.y, b = blockIdx.z;

  extern __shared__ __align__(128) unsigned char attn_smem[];
  __nv_bfloat16* sk = reinterpret_cast<__nv_bfloat16*>(attn_smem);
  __nv_bfloat16* sv = reinterpret_cast<__nv_bfloat16*>(attn_smem + kSlab);
  __shared__ __align__(8) uint64_t bar;
  __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps];
  __shared__ float sm_o[kAttnWarps][DH];
  __shared__ bool is_last;

  // The step counter, the page table and every cached token except the newest
  // were written before the predecessor kernel started: the split geometry can
  // be worked out, and all pages but the one holding the newest token fetched,
  // before waiting for it.  One split = one 64-token page of one head, whose K
  // (and V) slab is contiguous: a single bulk copy each.
  const int cur = *a.cur_dev;
  const int start = max(a.kv.pad[b], cur - a.window + 1);
  const int end = cur + 1;
  const int first_page = start / kPageTokens;
  const int nsplit = cur / kPageTokens - first_page + 1;
  const int page_pos0 = (first_page + split) * kPageTokens;
  const bool active = split < nsplit;
  const bool newest_page = page_pos0 + kPageTokens > cur;
  const int t0 = max(start, page_pos0), t1 = min(end, page_pos0 + kPageTokens);
  const uint32_t bar_u32 = smem_u32(&bar);
  auto fetch = [&]() {
    const int32_t* table = a.kv.page_table + static_cast<size_t>(b) * a.kv.ring_pages;
    const int page = table[(first_page + split) % a.kv.ring_pages];
    const size_t off = (static_cast<size_t>(page) * a.heads + head) * kPageTokens * DH;
    const uint64_t pol = l2_evict_first_policy();
    mbar_expect_tx(bar_u32, 2 * kSlab);
    bulk_load(smem_u32(sk), a.kv.kpool + off, kSlab, bar_u32, pol);
    bulk_load(smem_u32(sv), a.kv.vpool + off, kSlab, bar_u32, pol);
  };
  if (threadIdx.x == 0) {
    mbar_init(bar_u32, 1);
    mbar_fence_init();
    if (active && !newest_page) fetch();
  }
  pdl_wait();
  pdl_launch_dependents();
  if (!active) return;
  if (threadIdx.x == 0 && newest_page) fetch();

  constexpr float scale = DH == 256 ? 0.0625f : 0.125f;   // 1 / sqrt(d_head), exact
  float q[EPL];
  {
    const float* qp = a.q + (static_cast<size_t>(b) * a.heads + head) * DH + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) q[e] = qp[e] * scale;
  }
  __syncthreads();                                         // the barrier's init is visible to every waiter
  const bool arrived = mbar_wait(bar_u32, 0);
  if (!arrived && threadIdx.x == 0 && a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);

  float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) o[e] = 0.f;
  {
    float s[TPW];
    bool ok[TPW];
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      const int tt = page_pos0 + warp * TPW + u;
      ok[u] = arrived && tt >= t0 && tt < t1;
      KvVec<EPL> kv;
      kv.load_shared(sk + static_cast<size_t>(warp * TPW + u) * DH + lane * EPL);
      float kf[EPL];
      kv.get(kf);
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) d = fmaf(q[e], kf[e], d);
      s[u] = d;
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1)
#pragma unroll
      for (int u = 0; u < TPW; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o2);
#pragma unroll
    for (int u = 0; u < TPW; ++u)
      if (ok[u]) m = fmaxf(m, s[u]);
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      if (!ok[u]) continue;
      const float p = __expf(s[u] - m);
      KvVec<EPL> vv;
      vv.load_shared(sv + static_cast<size_t>(warp * TPW + u) * DH + lane * EPL);
      float vf[EPL];
      vv.get(vf);
      l += p;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] = fmaf(p, vf[e], o[e]);
    }
  }

  // merge the warps of this split
  if (lane == 0) {
    sm_m[warp] = m;
    sm_l[warp] = l;
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) sm_o[warp][lane * EPL + e] = o[e];
  __syncthreads();
  const size_t pidx = (static_cast<size_t>(b) * a.heads + head) * a.max_splits + split;
  if (threadIdx.x < DH) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sm_m[w]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float f = sm_m[w] == -INFINITY ? 0.f : __expf(sm_m[w] - M);   // warps without a visible key
      L = fmaf(sm_l[w], f, L);
      O = fmaf(sm_o[w][threadIdx.x], f, O);
    }
    a.part_o[pidx * DH + threadIdx.x] = O;
    if (threadIdx.x == 0) {
      a.part_ml[pidx * 2] = M;
      a.part_ml[pidx * 2 + 1] = L;
    }
  }

  // the last split of this (sequence, head) to finish merges all of them
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t ticket = atomicAdd(a.counters + b * a.heads + head, 1u);
    is_last = (ticket == static_cast<uint32_t>(nsplit - 1));
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  {
    // Merge of the splits: the per-split weights are worked out by one warp with all its
    // loads in flight at once, then every output dimension sums its column with
    // independent loads (a serial walk over the splits would cost one L2 round trip each).
    __shared__ float wgt[64];
    __shared__ float inv_l;
    const size_t base = (static_cast<size_t>(b) * a.heads + head) * a.max_splits;
    if (warp == 0) {
      float ms[2], ls[2];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int sidx = lane + 32 * h2;
        ms[h2] = sidx < nsplit ? __ldcg(a.part_ml + (base + sidx) * 2) : -INFINITY;
        ls[h2] = sidx < nsplit ? __ldcg(a.part_ml + (base + sidx) * 2 + 1) : 0.f;
      }
      const float M = warp_max(fmaxf(ms[0], ms[1]));
      float lsum = 0.f;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const float f = ms[h2] == -INFINITY ? 0.f : __expf(ms[h2] - M);
        wgt[lane + 32 * h2] = f;
        lsum = fmaf(ls[h2], f, lsum);
      }
      lsum = warp_sum(lsum);
      if (lane == 0) inv_l = 1.0f / lsum;
    }
    __syncthreads();
    if (threadIdx.x < DH) {
      const float* po = a.part_o + base * DH + threadIdx.x;
      float O = 0.f;
      int sidx = 0;
      for (; sidx + 8 <= nsplit; sidx += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldcg(po + static_cast<size_t>(sidx + u) * DH);
#pragma unroll
        for (int u = 0; u < 8; ++u) O = fmaf(v[u], wgt[sidx + u], O);
      }
      for (; sidx < nsplit; ++sidx) O = fmaf(__ldcg(po + static_cast<size_t>(sidx) * DH), wgt[sidx], O);
      const size_t oi = static_cast<size_t>(b) * a.ld_out + head * DH + threadIdx.x;
      if (a.out_bf16) {
        const float y = O * inv_l;
        const __nv_bfloat16 hi = __float2bfloat16_rn(y);
        a.out_bf16[oi] = hi;
        if (a.out_lo) a.out_lo[oi] = __float2bfloat16_rn(y - __bfloat162float(hi));
      } else {
        a.out[oi] = O * inv_l;
      }
    }
  }
  if (threadIdx.x == 0) a.counters[b * a.heads + head] = 0u;
}

// The same decode attention for many sequences: one block walks a.stream_pages (1-4) consecutive pages of one
// (sequence, head) as half-page tiles (32 keys: 16 KB of K + 16 KB of V) through a 3-stage ring fed by a
// producer warp, so the block's loads stay in flight while its eight consumer warps work, and the
// per-block costs (launch, warp merge, partial write, ticket) are spread over up to 256 keys.  Each
// consumer warp keeps its own running (max, sum, weighted V) over the 4 keys it takes from every tile.
// The launcher picks the pages per block so that the grid fills whole waves of resident blocks: with few
// heads per GPU (tensor-parallel shards) four pages per block leave the last wave mostly empty.
constexpr int kStreamPages = 4;                            // most pages a block walks
constexpr int kStreamStages = 3;
constexpr int kTileTokens = 32;
constexpr int kStreamThreads = kAttnThreads + 32;

template <int DH>
__global__ void __launch_bounds__(kStreamThreads) decode_attn_stream_kernel(const DecodeAttnArgs a) {
  constexpr int EPL = DH / 32;
  constexpr int TPW = kTileTokens / kAttnWarps;            // keys per warp and tile: 4
  constexpr uint32_t kHalf = kTileTokens * DH * 2;         // bytes of K (or V) per tile
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int split = blockIdx.x, head = blockIdx.y, b = blockIdx.z;

  extern __shared__ __align__(128) unsigned char attn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * kStreamStages];
  __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps];
  __shared__ float sm_o[kAttnWarps][DH];
  __shared__ bool is_last;
  __shared__ uint32_t failed;

  const int cur = *a.cur_dev;                              // written before the predecessor kernel started
  const int start = max(a.kv.pad[b], cur - a.window + 1);
  const int end = cur + 1;
  const int first_page = start / kPageTokens;
  const int n_pages = cur / kPageTokens - first_page + 1;
  const int ppb = a.stream_pages;                          // pages per block
  const int nsplit = (n_pages + ppb - 1) / ppb;
  const int page0 = first_page + split * ppb;              // first page of this block
  const int my_pages = min(ppb, first_page + n_pages - page0);
  const int n_tiles = 2 * max(my_pages, 0);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int st) { return bar0 + 8u * st; };
  auto empty_bar = [&](int st) { return bar0 + 8u * (kStreamStages + st); };
  if (threadIdx.x == 0) {
    for (int st = 0; st < kStreamStages; ++st) {
      mbar_init(full_bar(st), 1);
      mbar_init(empty_bar(st), kAttnWarps);
    }
    mbar_fence_init();
    failed = 0;
  }
  __syncthreads();
  pdl_launch_dependents();
  if (split >= nsplit) return;                             // uniform for the block

  float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) o[e] = 0.f;

  if (warp == kAttnWarps) {
    // ---- producer ----
    if (lane == 0) {
      const int32_t* table = a.kv.page_table + static_cast<size_t>(b) * a.kv.ring_pages;
      const uint64_t pol = l2_evict_first_policy();
      bool waited = false;
      for (int tile = 0; tile < n_tiles; ++tile) {
        const int st = tile % kStreamStages;
        if (tile >= kStreamStages && !mbar_wait(empty_bar(st), ((tile / kStreamStages) - 1) & 1)) {
          atomicOr(&failed, 1u);
          break;
        }
        const int page_pos = (page0 + (tile >> 1)) * kPageTokens + (tile & 1) * kTileTokens;
        if (!waited && page_pos + kTileTokens > cur) {      // this tile holds the token the predecessor wrote
          pdl_wait();
          waited = true;
        }
        const int page = table[(page0 + (tile >> 1)) % a.kv.ring_pages];
        const size_t off = ((static_cast<size_t>(page) * a.heads + head) * kPageTokens + (tile & 1) * kTileTokens) * DH;
        const uint32_t dst = smem_u32(attn_smem) + st * 2 * kHalf;
        mbar_expect_tx(full_bar(st), 2 * kHalf);
        bulk_load(dst, a.kv.kpool + off, kHalf, full_bar(st), pol);
        bulk_load(dst + kHalf, a.kv.vpool + off, kHalf, full_bar(st), pol);
      }
    }
  } else {
    // ---- consumers ----
    pdl_wait();                                            // the query comes from the predecessor kernel
    constexpr float scale = DH == 256 ? 0.0625f : 0.125f;  // 1 / sqrt(d_head), exact
    float q[EPL];
    {
      const float* qp = a.q + (static_cast<size_t>(b) * a.heads + head) * DH + lane * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) q[e] = qp[e] * scale;
    }
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int st = tile % kStreamStages;
      if (!mbar_wait(full_bar(st), (tile / kStreamStages) & 1)) {
        atomicOr(&failed, 1u);
        break;
      }
      const __nv_bfloat16* sk = reinterpret_cast<const __nv_bfloat16*>(attn_smem + st * 2 * kHalf);
      const __nv_bfloat16* sv = reinterpret_cast<const __nv_bfloat16*>(attn_smem + st * 2 * kHalf + kHalf);
      const int pos0 = (page0 + (tile >> 1)) * kPageTokens + (tile & 1) * kTileTokens + warp * TPW;
      float sc[TPW];
      bool ok[TPW];
#pragma unroll
      for (int u = 0; u < TPW; ++u) {
        ok[u] = pos0 + u >= start && pos0 + u < end;
        KvVec<EPL> kv;
        kv.load_shared(sk + static_cast<size_t>(warp * TPW + u) * DH + lane * EPL);
        float kf[EPL];
        kv.get(kf);
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) d = fmaf(q[e], kf[e], d);
        sc[u] = d;
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1)
#pragma unroll
        for (int u = 0; u < TPW; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o2);
      float m_new = m;
#pragma unroll
      for (int u = 0; u < TPW; ++u)
        if (ok[u]) m_new = fmaxf(m_new, sc[u]);
      if (m_new > -INFINITY) {
        const float corr = m == -INFINITY ? 0.f : __expf(m - m_new);
        l *= corr;
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[e] *= corr;
#pragma unroll
        for (int u = 0; u < TPW; ++u) {
          if (!ok[u]) continue;
          const float pw = __expf(sc[u] - m_new);
          KvVec<EPL> vv;
          vv.load_shared(sv + static_cast<size_t>(warp * TPW + u) * DH + lane * EPL);
          float vf[EPL];
          vv.get(vf);
          l += pw;
#pragma unroll
          for (int e = 0; e < EPL; ++e) o[e] = fmaf(pw, vf[e], o[e]);
        }
        m = m_new;
      }
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(st)) : "memory");
      }
    }
    if (lane == 0) {
      sm_m[warp] = m;
      sm_l[warp] = l;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_o[warp][lane * EPL + e] = o[e];
  }
  __syncthreads();
  if (threadIdx.x == 0 && failed && a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
  const size_t pidx = (static_cast<size_t>(b) * a.heads + head) * a.max_splits + split;
  if (threadIdx.x < DH) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sm_m[w]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float f = sm_m[w] == -INFINITY ? 0.f : __expf(sm_m[w] - M);
      L = fmaf(sm_l[w], f, L);
      O = fmaf(sm_o[w][threadIdx.x], f, O);
    }
    a.part_o[pidx * DH + threadIdx.x] = O;
    if (threadIdx.x == 0) {
      a.part_ml[pidx * 2] = M;
      a.part_ml[pidx * 2 + 1] = L;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t ticket = atomicAdd(a.counters + b * a.heads + head, 1u);
    is_last = (ticket == static_cast<uint32_t>(nsplit - 1));
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  {
    __shared__ float wgt[64];
    __shared__ float inv_l;
    const size_t base = (static_cast<size_t>(b) * a.heads + head) * a.max_splits;
    if (warp == 0) {
      float ms[2], ls[2];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int sidx = lane + 32 * h2;
        ms[h2] = sidx < nsplit ? __ldcg(a.part_ml + (base + sidx) * 2) : -INFINITY;
        ls[h2] = sidx < nsplit ? __ldcg(a.part_ml + (base + sidx) * 2 + 1) : 0.f;
      }
      const float M = warp_max(fmaxf(ms[0], ms[1]));
      float lsum = 0.f;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const float f = ms[h2] == -INFINITY ? 0.f : __expf(ms[h2] - M);
        wgt[lane + 32 * h2] = f;
        lsum = fmaf(ls[h2], f, lsum);
      }
      lsum = warp_sum(lsum);
      if (lane == 0) inv_l = 1.0f / lsum;
    }
    __syncthreads();
    if (threadIdx.x < DH) {
      const float* po = a.part_o + base * DH + threadIdx.x;
      float O = 0.f;
      for (int sidx = 0; sidx < nsplit; ++sidx) O = fmaf(__ldcg(po + static_cast<size_t>(sidx) * DH), wgt[sidx], O);
      const size_t oi = static_cast<size_t>(b) * a.ld_out + head * DH + threadIdx.x;
      if (a.out_bf16) {
        const float y = O * inv_l;
        const __nv_bfloat16 hi = __float2bfloat16_rn(y);
        a.out_bf16[oi] = hi;
        if (a.out_lo) a.out_lo[oi] = __float2bfloat16_rn(y - __bfloat162float(hi));
      } else {
        a.out[oi] = O * inv_l;
      }
    }
  }
  if (threadIdx.x == 0) a.counters[b * a.heads + head] = 0u;
}

// Causal attention for a chunk of rows; one warp owns QPW consecutive queries
// of one (sequence, head) and walks the keys once for all of them.
template <int DH, int QPW>
__global__ void __launch_bounds__(kAttnThreads) prefill_attn_kernel(const PrefillAttnArgs a) {
  constexpr int EPL = DH / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y, bi = blockIdx.z;
  const int tl0 = (blockIdx.x * kAttnWarps + warp) * QPW;   // first query of this warp in the chunk
  if (tl0 >= a.rows.Tc) return;
  const int b = a.rows.b0 + bi;
  const int pos0 = a.rows.pos0_host;
  const int nq = min(QPW, a.rows.Tc - tl0);
  const int32_t* table = a.kv.page_table + static_cast<size_t>(b) * a.kv.ring_pages;
  const int kstart = a.kv.pad[b];
  const int klimit = a.key_limit ? a.key_limit[b] : 0x7fffffff;

  constexpr float scale = DH == 256 ? 0.0625f : 0.125f;   // 1 / sqrt(d_head), exact
  float q[QPW][EPL], o[QPW][EPL], m[QPW], l[QPW];
#pragma unroll
  for (int i = 0; i < QPW; ++i) {
    const int row = bi * a.rows.Tc + tl0 + (i < nq ? i : 0);
    const float* qp = a.q + (static_cast<size_t>(row) * a.heads + head) * DH + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      q[i][e] = qp[e] * scale;
      o[i][e] = 0.f;
    }
    m[i] = -INFINITY;
    l[i] = 0.f;
  }
  const int last_pos = min(pos0 + tl0 + nq - 1, klimit);
  for (int kp = kstart; kp <= last_pos; ++kp) {
    const size_t off = kv_offset(table, a.kv.ring_pages, a.heads, DH, head, kp) + lane * EPL;
    KvVec<EPL> kv, vv;
    kv.load(a.kv.kpool + off);
    vv.load(a.kv.vpool + off);
    float kf[EPL], vf[EPL];
    kv.get(kf);
    vv.get(vf);
    float s[QPW];
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) d = fmaf(q[i][e], kf[e], d);
      s[i] = d;
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1)
#pragma unroll
      for (int i = 0; i < QPW; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], o2);
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
      if (kp > pos0 + tl0 + i) continue;       // causal
      const float mn = fmaxf(m[i], s[i]);
      const float corr = __expf(m[i] - mn);
      const float p = __expf(s[i] - mn);
      l[i] = fmaf(l[i], corr, p);
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[i][e] = fmaf(o[i][e], corr, p * vf[e]);
      m[i] = mn;
    }
  }
#pragma unroll
  for (int i = 0; i < QPW; ++i) {
    if (i >= nq) break;
    const int row = bi * a.rows.Tc + tl0 + i;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;   // rows with no visible key (left pad) give 0
    const size_t o_off = static_cast<size_t>(row) * a.ld_out + head * DH + lane * EPL;
    if (a.out_bf16) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) a.out_bf16[o_off + e] = __float2bfloat16_rn(o[i][e] * inv);
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) a.out[o_off + e] = o[i][e] * inv;
    }
  }
}

template <typename K, typename A>
cudaError_t launch_cfg(K kernel, dim3 grid, dim3 block, cudaStream_t s, bool pdl, const A& a) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

}  // namespace

template <int DH>
cudaError_t launch_decode_dh(const DecodeAttnArgs& a, cudaStream_t s, bool pdl) {
  constexpr int smem = 2 * kPageTokens * DH * 2;
  static DeviceOnce once;
  {
    cudaError_t e = once.run([&] { return cudaFuncSetAttribute(decode_attn_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.grid_splits, a.heads, a.B);
  cfg.blockDim = dim3(kAttnThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, decode_attn_kernel<DH>, a);
}

template <int DH>
cudaError_t launch_decode_stream_dh(const DecodeAttnArgs& a, cudaStream_t s, bool pdl) {
  constexpr int smem = kStreamStages * 2 * kTileTokens * DH * 2;
  static DeviceOnce once;
  {
    cudaError_t e = once.run([&] { return cudaFuncSetAttribute(decode_attn_stream_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  // Pages per block: the grid should be whole waves of resident blocks.  est_pages is the number of pages the
  // sequences hold now (the grid must cover grid_splits, but blocks past a sequence's last page leave at once).
  int sms = 148, dev = 0, per_sm = 1;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_attn_stream_kernel<DH>, kStreamThreads, smem);
  const int resident = sms * (per_sm < 1 ? 1 : per_sm);
  const int pages = a.est_pages > 0 ? (a.est_pages < a.grid_splits ? a.est_pages : a.grid_splits) : a.grid_splits;
  DecodeAttnArgs b = a;
  float best = 0.f;
  for (int p = kStreamPages; p >= 1; --p) {
    const long blocks = static_cast<long>((pages + p - 1) / p) * a.heads * a.B;
    const float cost = static_cast<float>((blocks + resident - 1) / resident) * (p + 0.3f);   // 0.3: per-block overhead in page times
    if (p == kStreamPages || cost < best * 0.97f) {
      best = cost;
      b.stream_pages = p;
    }
  }
  if ((a.grid_splits + b.stream_pages - 1) / b.stream_pages > 64) b.stream_pages = kStreamPages;   // merge buffer: 64 splits
  cfg.gridDim = dim3((a.grid_splits + b.stream_pages - 1) / b.stream_pages, a.heads, a.B);
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, decode_attn_stream_kernel<DH>, b);
}

// Splits of the visible window: one per 64-token page it can touch.
int decode_attn_splits(int window) { return (window + kPageTokens - 1) / kPageTokens + 1; }

cudaError_t launch_decode_attn(const DecodeAttnArgs& a, cudaStream_t s, bool pdl) {
  if (a.B <= 0 || a.grid_splits <= 0 || a.grid_splits > a.max_splits || a.kv.ring_pages < a.grid_splits ||
      (a.grid_splits < decode_attn_splits(a.window) && a.grid_splits < a.kv.ring_pages))
    return cudaErrorInvalidValue;
  // many sequences: enough blocks even with several pages per block, which keeps each block streaming
  static int stream_min_b = -1;
  if (stream_min_b < 0) {
    const char* e = getenv("MTJ_ATTN_STREAM_MIN_B");
    stream_min_b = e ? atoi(e) : 8;
  }
  if (a.B >= stream_min_b) {
    if (a.d_head == 256) return launch_decode_stream_dh<256>(a, s, pdl);
    if (a.d_head == 64) return launch_decode_stream_dh<64>(a, s, pdl);
  }
  if (a.d_head == 256) return launch_decode_dh<256>(a, s, pdl);
  if (a.d_head == 64) return launch_decode_dh<64>(a, s, pdl);
  return cudaErrorInvalidValue;
}

cudaError_t launch_prefill_attn(const PrefillAttnArgs& a, cudaStream_t s) {
  if (a.M <= 0 || a.rows.Tc <= 0 || a.M % a.rows.Tc != 0) return cudaErrorInvalidValue;
  constexpr int QPW = 4;
  const dim3 grid((a.rows.Tc + kAttnWarps * QPW - 1) / (kAttnWarps * QPW), a.heads, a.M / a.rows.Tc);
  const dim3 block(kAttnThreads);
  if (a.d_head == 256) return launch_cfg(prefill_attn_kernel<256, QPW>, grid, block, s, false, a);
  if (a.d_head == 64) return launch_cfg(prefill_attn_kernel<64, QPW>, grid, block, s, false, a);
  return cudaErrorInvalidValue;
}

}  // namespace mtj
