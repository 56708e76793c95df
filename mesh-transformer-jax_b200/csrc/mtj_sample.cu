// Nucleus (top-p) + temperature sampling, one 1024-thread block per row
// (reference: mesh_transformer/sampling.py:6-44).
//
//   1. descending stable sort of the row (value desc, higher index first among
//      equal values, -0 == +0): LSD radix sort, 4-bit digits, on a key that is
//      the bitwise complement of the order-preserving integer image of the
//      logit, starting from positions laid out by descending index;
//   2. softmax of the sorted values, cumulative sum, "remove where the
//      cumulative probability of the PREVIOUS entry exceeds top_p";
//   3. argmax over (logit - 1e10*removed) / temp + Gumbel(uniform), lowest
//      index on ties (jax.random.categorical).
//
// Every floating-point operation is individually rounded (no FMA contraction)
// and sums follow a fixed association -- 1024 consecutive runs, a Hillis-Steele
// scan over the 32 run totals of each warp, then over the 32 warp totals -- so
// that the token ids can be reproduced bit for bit by a CPU restatement.
#include <math.h>

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

// Hillis-Steele inclusive scan over the 32 lanes of a warp (x[i] += x[i-off]).
__device__ __forceinline__ float warp_scan_hs(float x, int lane) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float y = __shfl_up_sync(0xffffffffu, x, off);
    if (lane >= off) x = __fadd_rn(x, y);
  }
  return x;
}

// Prefix of this thread's run and the grand total, in the pinned association.
__device__ __forceinline__ float block_prefix(float run_total, float* warp_tot, float* total_out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inc = warp_scan_hs(run_total, lane);
  float exc = __shfl_up_sync(0xffffffffu, inc, 1);
  if (lane == 0) exc = 0.f;
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const float ginc = warp_scan_hs(warp_tot[lane], lane);
    float gexc = __shfl_up_sync(0xffffffffu, ginc, 1);
    if (lane == 0) gexc = 0.f;
    warp_tot[lane] = gexc;
    if (lane == 31) warp_tot[32] = ginc;
  }
  __syncthreads();
  const float prefix = __fadd_rn(warp_tot[warp], exc);
  *total_out = warp_tot[32];
  __syncthreads();
  return prefix;
}

__global__ void __launch_bounds__(kSampThreads) sample_top_p_kernel(const SampleArgs a) {
  __shared__ uint16_t cnt[16][kSampThreads];
  __shared__ uint32_t wsum[33];
  __shared__ float warp_tot[33];
  __shared__ float last_cum[kSampThreads];
  __shared__ float red_v[32];
  __shared__ int red_i[32];

  pdl_wait();
  pdl_launch_dependents();

  const int row = blockIdx.x, t = threadIdx.x, V = a.V;
  const int lane = t & 31, warp = t >> 5;
  const float* logits = a.logits + static_cast<size_t>(row) * V;
  const float* unif = a.uniforms + static_cast<size_t>(row) * V;
  uint32_t* base = reinterpret_cast<uint32_t*>(a.scratch) + static_cast<size_t>(row) * 5 * V;
  uint32_t* key_a = base;
  uint32_t* key_b = base + V;
  uint32_t* idx_a = base + 2 * static_cast<size_t>(V);
  uint32_t* idx_b = base + 3 * static_cast<size_t>(V);
  float* val = reinterpret_cast<float*>(base + 4 * static_cast<size_t>(V));
  const int per = (V + kSampThreads - 1) / kSampThreads;
  const int j0 = min(V, t * per), j1 = min(V, j0 + per);

  // start from descending index order so that the stable sort puts the higher index first
  for (int j = j0; j < j1; ++j) {
    const int i = V - 1 - j;
    key_a[j] = sort_key(logits[i]);
    idx_a[j] = static_cast<uint32_t>(i);
  }
  __syncthreads();

  uint32_t *kin = key_a, *kout = key_b, *iin = idx_a, *iout = idx_b;
  for (int shift = 0; shift < 32; shift += 4) {
#pragma unroll
    for (int d = 0; d < 16; ++d) cnt[d][t] = 0;
    for (int j = j0; j < j1; ++j) cnt[(kin[j] >> shift) & 15][t]++;
    __syncthreads();
    // exclusive scan over the flattened [digit][thread] counts; thread t owns 16 consecutive entries
    uint16_t* flat = &cnt[0][0] + t * 16;
    uint32_t s = 0;
#pragma unroll
    for (int k = 0; k < 16; ++k) s += flat[k];
    uint32_t inc = s;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t y = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += y;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      uint32_t w = wsum[lane];
      uint32_t winc = w;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, winc, off);
        if (lane >= off) winc += y;
      }
      wsum[lane] = winc - w;
    }
    __syncthreads();
    uint32_t run = wsum[warp] + inc - s;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t c = flat[k];
      flat[k] = static_cast<uint16_t>(run);
      run += c;
    }
    __syncthreads();
    for (int j = j0; j < j1; ++j) {
      const uint32_t k = kin[j];
      const uint32_t pos = cnt[(k >> shift) & 15][t]++;
      kout[pos] = k;
      iout[pos] = iin[j];
    }
    __syncthreads();
    uint32_t* tk = kin; kin = kout; kout = tk;
    uint32_t* ti = iin; iin = iout; iout = ti;
  }
  // eight passes: the sorted order is back in (key_a, idx_a)

  // softmax numerators of the sorted values and their total
  const float vmax = logits[idx_a[0]];
  float run_sum = 0.f;
  for (int j = j0; j < j1; ++j) {
    const float e = exp_pinned(__fsub_rn(logits[idx_a[j]], vmax));
    val[j] = e;
    run_sum = __fadd_rn(run_sum, e);
  }
  float denom;
  block_prefix(run_sum, warp_tot, &denom);

  // probabilities and their cumulative sum
  run_sum = 0.f;
  for (int j = j0; j < j1; ++j) {
    const float p = __fdiv_rn(val[j], denom);
    val[j] = p;
    run_sum = __fadd_rn(run_sum, p);
  }
  float unused;
  const float prefix = block_prefix(run_sum, warp_tot, &unused);
  float c = prefix;
  for (int j = j0; j < j1; ++j) {
    c = __fadd_rn(c, val[j]);
    val[j] = c;
  }
  last_cum[t] = c;
  __syncthreads();

  // Gumbel-max over the filtered, tempered logits
  const float top_p = a.top_p[row], temp = a.temp[row];
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  float prev = (t > 0 && j0 < j1) ? last_cum[t - 1] : 0.f;
  for (int j = j0; j < j1; ++j) {
    const bool removed = (j > 0) && (prev > top_p);        // shifted by one: the head always stays
    prev = val[j];
    const int i = static_cast<int>(idx_a[j]);
    const float lm = __fsub_rn(logits[i], removed ? 1e10f : 0.0f);
    const float tl = log_pinned(unif[i]);
    const float g = -log_pinned(-tl);
    const float score = __fadd_rn(__fdiv_rn(lm, temp), g);
    if (score > best || (score == best && i < best_i)) {
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
      a.tokens[row] = static_cast<uint32_t>(best_i);
      if (a.tokens_copy) a.tokens_copy[row] = static_cast<uint32_t>(best_i);
      if (a.cur_dev && row == 0) *a.cur_dev += 1;
    }
  }
}

}  // namespace

int64_t sample_scratch_bytes(int rows, int vocab) {
  return static_cast<int64_t>(rows) * 5 * vocab * 4;
}

cudaError_t launch_sample_top_p(const SampleArgs& a, cudaStream_t s, bool pdl) {
  if (a.rows <= 0 || a.V <= 0 || a.V > 65535) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.rows);
  cfg.blockDim = dim3(kSampThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, sample_top_p_kernel, a);
}

}  // namespace mtj
