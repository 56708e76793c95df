// Attention over the paged bf16 KV cache.
//
// decode_attn_kernel : one query per (sequence, head); the visible key range
//   [max(pad, cur-window+1), cur] is cut into splits, one block per split;
//   partial (max, sum, weighted V) triples are merged by the last block of each
//   (sequence, head) to finish.  HBM-bound: every K/V byte is read once with
//   coalesced 16-byte loads.  (reference: layers.py:316-338 -- the sliding
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
  __device__ __forceinline__ void get(float* f) const { unpack8(v, f); }
};
template <>
struct KvVec<2> {
  uint32_t v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = ld_stream4(p); }
  __device__ __forceinline__ void get(float* f) const {
    f[0] = bf16_lo(v);
    f[1] = bf16_hi(v);
  }
};

template <int DH>
__global__ void __launch_bounds__(kAttnThreads) decode_attn_kernel(const DecodeAttnArgs a) {
  constexpr int EPL = DH / 32;
  constexpr int U = 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int split = blockIdx.x, head = blockIdx.y, b = blockIdx.z;

  __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps];
  __shared__ float sm_o[kAttnWarps][DH];
  __shared__ bool is_last;

  // The step counter, the page table and every cached token except the newest
  // were written before the predecessor kernel started, so they may be read
  // (and the old keys/values pulled into L2) before waiting for it.
  const int cur = *a.cur_dev;
  const int start = max(a.kv.pad[b], cur - a.window + 1);
  const int end = cur + 1;
  const int nsplit = (end - start + a.split_tokens - 1) / a.split_tokens;
  const int t0 = start + split * a.split_tokens;
  const int t1 = min(end, t0 + a.split_tokens);
  const int32_t* table = a.kv.page_table + static_cast<size_t>(b) * a.kv.ring_pages;
  if (split < nsplit) {
    constexpr int kLines = DH * 2 / 128;                    // 128-byte lines per token row
    for (int i = threadIdx.x; i < (t1 - t0) * kLines; i += kAttnThreads) {
      const int tt = t0 + i / kLines;
      if (tt == cur) continue;                              // written by the predecessor
      const size_t off = kv_offset(table, a.kv.ring_pages, a.heads, DH, head, tt) + (i % kLines) * 64;
      prefetch_l2(a.kv.kpool + off);
      prefetch_l2(a.kv.vpool + off);
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  if (split >= nsplit) return;

  constexpr float scale = DH == 256 ? 0.0625f : 0.125f;   // 1 / sqrt(d_head), exact
  float q[EPL];
  {
    const float* qp = a.q + (static_cast<size_t>(b) * a.heads + head) * DH + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) q[e] = qp[e] * scale;
  }

  float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) o[e] = 0.f;

  for (int t = t0 + warp; t < t1; t += kAttnWarps * U) {
    KvVec<EPL> kv[U], vv[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tt = t + u * kAttnWarps;
      ok[u] = tt < t1;
      const size_t off = kv_offset(table, a.kv.ring_pages, a.heads, DH, head, ok[u] ? tt : t) + lane * EPL;
      kv[u].load(a.kv.kpool + off);
      vv[u].load(a.kv.vpool + off);
    }
    float s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[EPL];
      kv[u].get(kf);
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) d = fmaf(q[e], kf[e], d);
      s[u] = d;
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1)
#pragma unroll
      for (int u = 0; u < U; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o2);
    float mn = m;
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (ok[u]) mn = fmaxf(mn, s[u]);
    const float corr = __expf(m - mn);
    l *= corr;
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] *= corr;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!ok[u]) continue;
      const float p = __expf(s[u] - mn);
      float vf[EPL];
      vv[u].get(vf);
      l += p;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] = fmaf(p, vf[e], o[e]);
    }
    m = mn;
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
      const float f = __expf(sm_m[w] - M);     // exp(-inf) = 0 for idle warps
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
  if (threadIdx.x < DH) {
    const size_t base = (static_cast<size_t>(b) * a.heads + head) * a.max_splits;
    float M = -INFINITY;
    for (int sidx = 0; sidx < nsplit; ++sidx) M = fmaxf(M, __ldcg(a.part_ml + (base + sidx) * 2));
    float L = 0.f, O = 0.f;
    for (int sidx = 0; sidx < nsplit; ++sidx) {
      const float f = __expf(__ldcg(a.part_ml + (base + sidx) * 2) - M);
      L = fmaf(__ldcg(a.part_ml + (base + sidx) * 2 + 1), f, L);
      O = fmaf(__ldcg(a.part_o + (base + sidx) * DH + threadIdx.x), f, O);
    }
    a.out[static_cast<size_t>(b) * a.ld_out + head * DH + threadIdx.x] = O / L;
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

cudaError_t launch_decode_attn(const DecodeAttnArgs& a, cudaStream_t s, bool pdl) {
  if (a.B <= 0 || a.split_tokens <= 0 || a.grid_splits <= 0 || a.grid_splits > a.max_splits ||
      static_cast<long long>(a.grid_splits) * a.split_tokens < a.window)
    return cudaErrorInvalidValue;
  const dim3 grid(a.grid_splits, a.heads, a.B), block(kAttnThreads);
  if (a.d_head == 256) return launch_cfg(decode_attn_kernel<256>, grid, block, s, pdl, a);
  if (a.d_head == 64) return launch_cfg(decode_attn_kernel<64>, grid, block, s, pdl, a);
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
