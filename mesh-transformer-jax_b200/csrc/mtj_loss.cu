// Vocab-sharded softmax cross-entropy of ProjectionShard.loss (layers.py:569-593).
//
// ce_partial : per row of this shard's logits: local max, sum of exp(l - local
//              max) and the target's logit if the target id falls into this
//              shard's vocabulary range (the one-hot product of :578-579).
// ce_rescale : after the cross-shard max (pmax, :575): sums rescaled to the
//              global max, target logit shifted by it.
// ce_finalize: after the cross-shard sums (:580,:585): loss = log(sum_exp) -
//              target logit; correct = (shifted target logit == 0), i.e. the
//              target holds the global maximum (:591).  z_loss is 0 in eval.
#include <math.h>

#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; ++i) t = is_max ? fmaxf(t, red[i]) : t + red[i];
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(kThreads) ce_partial_kernel(const CeArgs a) {
  __shared__ float red[kThreads / 32];
  const int r = blockIdx.x;
  const float* row = a.logits + static_cast<size_t>(r) * a.vl;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < a.vl; i += kThreads) m = fmaxf(m, row[i]);
  m = block_reduce(m, red, true);
  float s = 0.f;
  for (int i = threadIdx.x; i < a.vl; i += kThreads) s += expf(row[i] - m);
  s = block_reduce(s, red, false);
  if (threadIdx.x == 0) {
    const int mrow = a.row0 + r;
    const int b = a.rows.b0 + mrow / a.rows.Tc, t = a.rows.pos0_host + mrow % a.rows.Tc;
    const int64_t local = static_cast<int64_t>(a.targets[static_cast<size_t>(b) * a.T + t]) - a.vocab_start;
    const bool hit = local >= 0 && local < a.vl;
    a.pmax[mrow] = m;
    a.psum[2 * mrow] = s;
    a.psum[2 * mrow + 1] = hit ? row[local] : 0.f;
    a.hit[mrow] = hit ? 1 : 0;
  }
}

// Combines the per-group (max, sum of exp) pairs that the fused logits epilogue leaves (one group = 32
// vocabulary entries) into this shard's per-row local max and sum: the same three results ce_partial gives.
// Block = 32 token rows x 8 warps; the warps split the groups, lanes are rows (coalesced loads).
__global__ void __launch_bounds__(256) ce_combine_kernel(const CeArgs a, const float* __restrict__ gmax,
                                                         const float* __restrict__ gsum, int n_groups, int ld,
                                                         const float* __restrict__ tlogit,
                                                         const uint8_t* __restrict__ ghit, int rows) {
  __shared__ float sm[8][32], ss[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.x * 32 + lane;
  float m = -INFINITY, s = 0.f;
  if (r < rows) {
    for (int g = warp; g < n_groups; g += 8) {
      const float gm = gmax[static_cast<size_t>(g) * ld + r], gs = gsum[static_cast<size_t>(g) * ld + r];
      if (gm == -INFINITY) continue;                       // a group beyond the end of the vocabulary slice
      const float nm = fmaxf(m, gm);
      s = s * expf(m - nm) + gs * expf(gm - nm);          // m = -inf only while s = 0: exp(-inf) = 0
      m = nm;
    }
  }
  sm[warp][lane] = m;
  ss[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && r < rows) {
    float M = sm[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) M = fmaxf(M, sm[w][lane]);
    float S = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) S += sm[w][lane] == -INFINITY ? 0.f : ss[w][lane] * expf(sm[w][lane] - M);
    const int mrow = a.row0 + r;
    const bool hit = ghit[r] != 0;
    a.pmax[mrow] = M;
    a.psum[2 * mrow] = S;
    a.psum[2 * mrow + 1] = hit ? tlogit[r] : 0.f;
    a.hit[mrow] = hit ? 1 : 0;
  }
}

__global__ void ce_rescale_kernel(const CeArgs a, const float* __restrict__ lmax, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float g = a.pmax[i];                 // global max after the all-reduce
  a.psum[2 * i] = a.psum[2 * i] * expf(lmax[i] - g);
  a.psum[2 * i + 1] = a.hit[i] ? a.psum[2 * i + 1] - g : 0.f;
}

__global__ void ce_finalize_kernel(const CeArgs a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int b = a.rows.b0 + i / a.rows.Tc, t = a.rows.pos0_host + i % a.rows.Tc;
  const float predicted = a.psum[2 * i + 1];
  a.loss_out[static_cast<size_t>(b) * a.T + t] = logf(a.psum[2 * i]) - predicted;
  a.correct_out[static_cast<size_t>(b) * a.T + t] = (predicted == 0.0f) ? 1 : 0;
}

}  // namespace

cudaError_t launch_ce_partial(const CeArgs& a, int rows, cudaStream_t s) {
  ce_partial_kernel<<<rows, kThreads, 0, s>>>(a);
  return cudaGetLastError();
}
cudaError_t launch_ce_combine(const CeArgs& a, const float* gmax, const float* gsum, int n_groups, int ld,
                              const float* tlogit, const uint8_t* ghit, int rows, cudaStream_t s) {
  ce_combine_kernel<<<(rows + 31) / 32, 256, 0, s>>>(a, gmax, gsum, n_groups, ld, tlogit, ghit, rows);
  return cudaGetLastError();
}
cudaError_t launch_ce_rescale(const CeArgs& a, const float* lmax, int n, cudaStream_t s) {
  ce_rescale_kernel<<<(n + 255) / 256, 256, 0, s>>>(a, lmax, n);
  return cudaGetLastError();
}
cudaError_t launch_ce_finalize(const CeArgs& a, int n, cudaStream_t s) {
  ce_finalize_kernel<<<(n + 255) / 256, 256, 0, s>>>(a, n);
  return cudaGetLastError();
}

}  // namespace mtj
