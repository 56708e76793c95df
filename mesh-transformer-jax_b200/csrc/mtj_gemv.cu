// Weight-streaming GEMV family for small token counts (decode): HBM-bound.
//
// A group of KS warps owns RW consecutive output rows; each warp walks its
// share of the K extent with 16-byte streaming loads (32 lanes x 8 bf16 = 256
// elements per step), the activations are fp32 and shared by all warps through
// L1.  There is no block-level synchronisation on the streaming path; the KS
// partial sums meet once in shared memory and are added in a fixed order.
// Three epilogues share the loop:
//   in-proj : LayerNorm prologue, [Q|K|V|FF-in] rows, interleaved RoPE on Q/K,
//             bf16 K/V written straight into the paged cache, bias + GELU on FF
//             (reference: layers.py:12-36,128-148,261-273,288-289,292-297)
//   out-proj: [attn | gelu(ff)] x [W_o ; W_ff_out] + bias + residual, and the
//             LayerNorm statistics of the finished rows computed by the last
//             block to arrive (layers.py:285,290,313; transformer_shard.py:60)
//   logits  : final LayerNorm prologue + bias (layers.py:561-564)
#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kGemvWarps; ++i) t += red[i];
  __syncthreads();
  return t;
}

template <int BT, int RW, int EPI, int KS>
__global__ void __launch_bounds__(kGemvThreads, BT == 1 ? (EPI == kEpiOut ? 4 : 3) : 2) gemv_kernel(const GemvArgs a) {
  constexpr bool kLN = (EPI != kEpiOut);
  constexpr int kGroups = kGemvWarps / KS;      // row groups per block; KS warps share one group's K extent
  static_assert(RW * BT <= 32 && (RW & 1) == 0, "one lane finishes one (row, token) pair");
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int grp = warp / KS, kpart = warp % KS;
  const int row0 = (blockIdx.x * kGroups + grp) * RW;
  const bool active = row0 < a.N;
  const int m0 = blockIdx.y * BT;
  const int nb = min(BT, a.M - m0);

  // N is a multiple of RW (checked at launch), so an active group has RW valid rows
  const __nv_bfloat16* wbase = a.W + static_cast<size_t>(active ? row0 : 0) * a.K + lane * 8;

  float acc[RW][BT];
#pragma unroll
  for (int r = 0; r < RW; ++r)
#pragma unroll
    for (int bt = 0; bt < BT; ++bt) acc[r][bt] = 0.f;

  const int nch = (a.K + 255) >> 8;             // the last chunk may be partial (K is a multiple of 8)
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  uint4 wnext[RW];
  if (active && kpart < nch) {
    // weights do not depend on the predecessor kernel: start streaming before the wait
#pragma unroll
    for (int r = 0; r < RW; ++r)
      wnext[r] = (kpart * 256 + lane * 8 < a.K) ? ld_stream16(wbase + static_cast<size_t>(r) * a.K + kpart * 256) : zero4;
#pragma unroll
    for (int r = 0; r < RW; ++r)
      if ((kpart + KS) * 256 + lane * 8 < a.K) prefetch_l2(wbase + static_cast<size_t>(r) * a.K + (kpart + KS) * 256);
  }
  pdl_wait();
  pdl_launch_dependents();

  const float* xr[BT];
  float mean[BT], rstd[BT];
#pragma unroll
  for (int bt = 0; bt < BT; ++bt) {
    const int m = m0 + (bt < nb ? bt : 0);
    const int src = a.row_select ? a.row_select[m] : m;
    xr[bt] = a.x + static_cast<size_t>(src) * a.ldx + lane * 8;
    if (kLN) {
      mean[bt] = a.stats[2 * src];
      rstd[bt] = a.stats[2 * src + 1];
    }
  }

  if (active) {
    for (int c = kpart; c < nch; c += KS) {
      uint4 wcur[RW];
#pragma unroll
      for (int r = 0; r < RW; ++r) wcur[r] = wnext[r];
      if (c + KS < nch) {
#pragma unroll
        for (int r = 0; r < RW; ++r)
          wnext[r] = ((c + KS) * 256 + lane * 8 < a.K)
                         ? ld_stream16(wbase + static_cast<size_t>(r) * a.K + (c + KS) * 256)
                         : zero4;
      }
      const int k = c * 256;
      const bool in_k = k + lane * 8 < a.K;       // lanes past the end of a partial chunk contribute zeros
      float sc[8], of[8];
      if (kLN && !in_k) {
#pragma unroll
        for (int e = 0; e < 8; ++e) sc[e] = of[e] = 0.f;
      }
      if (kLN && in_k) {
        const float4 s0 = *reinterpret_cast<const float4*>(a.ln_scale + k + lane * 8);
        const float4 s1 = *reinterpret_cast<const float4*>(a.ln_scale + k + lane * 8 + 4);
        const float4 o0 = *reinterpret_cast<const float4*>(a.ln_offset + k + lane * 8);
        const float4 o1 = *reinterpret_cast<const float4*>(a.ln_offset + k + lane * 8 + 4);
        sc[0] = s0.x; sc[1] = s0.y; sc[2] = s0.z; sc[3] = s0.w;
        sc[4] = s1.x; sc[5] = s1.y; sc[6] = s1.z; sc[7] = s1.w;
        of[0] = o0.x; of[1] = o0.y; of[2] = o0.z; of[3] = o0.w;
        of[4] = o1.x; of[5] = o1.y; of[6] = o1.z; of[7] = o1.w;
      }
      float xv[BT][8];
#pragma unroll
      for (int bt = 0; bt < BT; ++bt) {
        const float4 zf = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 x0 = in_k ? *reinterpret_cast<const float4*>(xr[bt] + k) : zf;
        const float4 x1 = in_k ? *reinterpret_cast<const float4*>(xr[bt] + k + 4) : zf;
        xv[bt][0] = x0.x; xv[bt][1] = x0.y; xv[bt][2] = x0.z; xv[bt][3] = x0.w;
        xv[bt][4] = x1.x; xv[bt][5] = x1.y; xv[bt][6] = x1.z; xv[bt][7] = x1.w;
        if (kLN) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            xv[bt][e] = fmaf(sc[e] * rstd[bt], xv[bt][e] - mean[bt], of[e]);
        }
      }
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        float w8[8];
        unpack8(wcur[r], w8);
#pragma unroll
        for (int bt = 0; bt < BT; ++bt)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[r][bt] = fmaf(w8[e], xv[bt][e], acc[r][bt]);
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
      for (int bt = 0; bt < BT; ++bt) acc[r][bt] = warp_sum(acc[r][bt]);
  }
  // lane (bt*RW + r) finishes output (row0 + r, m0 + bt)
  float val = 0.f;
#pragma unroll
  for (int r = 0; r < RW; ++r)
#pragma unroll
    for (int bt = 0; bt < BT; ++bt)
      if (lane == bt * RW + r) val = acc[r][bt];
  if (KS > 1) {
    // fixed-order sum of the KS partial results of this row group
    __shared__ float part[kGroups][KS][32];
    part[grp][kpart][lane] = val;
    __syncthreads();
    if (kpart == 0) {
      val = 0.f;
#pragma unroll
      for (int kp = 0; kp < KS; ++kp) val += part[grp][kp][lane];
    }
  }
  if (active && kpart == 0) {
    const float partner = __shfl_xor_sync(0xffffffffu, val, 1);   // the other row of the RoPE pair
    const int r = lane % RW, bt = lane / RW;
    const int n = a.n0 + row0 + r;                 // row index within the full projection
    if (lane < RW * BT && bt < nb && row0 + r < a.N) {
      const int m = m0 + bt;
      if (EPI == kEpiInProj) {
        const int seq = a.rows.b0 + m / a.rows.Tc;
        const int pos = (a.rows.pos0_dev ? *a.rows.pos0_dev : a.rows.pos0_host) + m % a.rows.Tc;
        if (n < 3 * a.dl) {
          const int region = n / a.dl;          // 0 = Q, 1 = K, 2 = V
          const int nn = n - region * a.dl;
          const int head = nn / a.d_head, j = nn % a.d_head;
          float y = val;
          if (region < 2 && j < a.rot) {
            const float2 sc2 = a.sincos[static_cast<size_t>(pos) * (a.rot >> 1) + (j >> 1)];
            y = (j & 1) ? (val * sc2.y + partner * sc2.x) : (val * sc2.y - partner * sc2.x);
          }
          if (region == 0) {
            a.q_out[static_cast<size_t>(m) * a.dl + nn] = y;
          } else if (pos >= a.kv.pad[seq]) {
            __nv_bfloat16* pool = region == 1 ? a.kv.kpool : a.kv.vpool;
            const size_t off = kv_offset(a.kv.page_table + static_cast<size_t>(seq) * a.kv.ring_pages,
                                         a.kv.ring_pages, a.heads, a.d_head, head, pos);
            pool[off + j] = __float2bfloat16_rn(y);
          }
        } else {
          const int f = n - 3 * a.dl;
          a.act2[static_cast<size_t>(m) * (a.dl + a.ffl) + a.dl + f] = gelu_tanh(val + a.b_ff[f]);
        }
      } else if (EPI == kEpiOut) {
        float y = val + a.bias[n];
        if (a.residual) y += a.residual[static_cast<size_t>(m) * a.N + n];
        float* outp = a.out + (a.slot_sel ? static_cast<size_t>(*a.slot_sel & 1u) * a.slot_stride : 0);
        outp[static_cast<size_t>(m) * a.N + n] = y;
      } else {
        a.logits[static_cast<size_t>(m) * a.ld_logits + n] = val + a.bias[n];
      }
    }
  }

  if (EPI == kEpiOut) {
    if (a.stats_out == nullptr) return;
    // The last block of this token tile to finish computes the LayerNorm
    // statistics of the completed rows for the next layer's prologue.
    __shared__ float red[kGemvWarps];
    __shared__ bool is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t ticket = atomicAdd(a.counters + blockIdx.y, 1u);
      is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int bt = 0; bt < nb; ++bt) {
      const float* row = a.out + static_cast<size_t>(m0 + bt) * a.N;
      float s = 0.f;
#pragma unroll 8
      for (int i = threadIdx.x; i < a.N; i += kGemvThreads) s += __ldcg(row + i);
      const float mu = block_sum(s, red) / static_cast<float>(a.N);
      float v = 0.f;
#pragma unroll 8
      for (int i = threadIdx.x; i < a.N; i += kGemvThreads) {
        const float dlt = __ldcg(row + i) - mu;
        v = fmaf(dlt, dlt, v);
      }
      const float var = block_sum(v, red) / static_cast<float>(a.N);
      if (threadIdx.x == 0) {
        a.stats_out[2 * (m0 + bt)] = mu;
        a.stats_out[2 * (m0 + bt) + 1] = 1.0f / sqrtf(var + 1e-5f);
      }
    }
    if (threadIdx.x == 0) a.counters[blockIdx.y] = 0u;
  }
}

template <int BT, int RW, int EPI, int KS>
cudaError_t launch_one(const GemvArgs& a, cudaStream_t s, bool pdl) {
  constexpr int rows_per_block = RW * (kGemvWarps / KS);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.N + rows_per_block - 1) / rows_per_block, (a.M + BT - 1) / BT, 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemv_kernel<BT, RW, EPI, KS>, a);
}

template <int BT, int EPI>
cudaError_t launch_ks(const GemvArgs& a, cudaStream_t s, bool pdl) {
  // Split K over the warps of a block until there are enough blocks to fill
  // the GPU several times over (148 SMs x ~4 resident blocks).
  const int nch = (a.K + 255) >> 8;
  const long long tiles = (a.M + BT - 1) / BT;
  int ks = 1;
  while (ks < 8 && ks * 2 <= nch && tiles * ((a.N + 4 * (8 / ks) - 1) / (4 * (8 / ks))) < 148 * 6) ks *= 2;
  if (a.ks_override > 0) ks = a.ks_override;
  if (BT == 1 && a.rw_override == 8 && (a.N & 7) == 0) {
    switch (ks) {
      case 1: return launch_one<1, 8, EPI, 1>(a, s, pdl);
      case 2: return launch_one<1, 8, EPI, 2>(a, s, pdl);
      case 4: return launch_one<1, 8, EPI, 4>(a, s, pdl);
      default: return launch_one<1, 8, EPI, 8>(a, s, pdl);
    }
  }
  switch (ks) {
    case 1: return launch_one<BT, 4, EPI, 1>(a, s, pdl);
    case 2: return launch_one<BT, 4, EPI, 2>(a, s, pdl);
    case 4: return launch_one<BT, 4, EPI, 4>(a, s, pdl);
    default: return launch_one<BT, 4, EPI, 8>(a, s, pdl);
  }
}

template <int EPI>
cudaError_t launch_epi(const GemvArgs& a, cudaStream_t s, bool pdl) {
  if (a.M == 1) return launch_ks<1, EPI>(a, s, pdl);
  if (a.M == 2) return launch_ks<2, EPI>(a, s, pdl);
  return launch_ks<4, EPI>(a, s, pdl);
}

}  // namespace

cudaError_t launch_gemv(GemvEpilogue epi, const GemvArgs& a, cudaStream_t s, bool pdl) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || (a.K & 7) != 0 || (a.N & 3) != 0) return cudaErrorInvalidValue;
  if (a.ks_override != 0 && a.ks_override != 1 && a.ks_override != 2 && a.ks_override != 4 &&
      a.ks_override != 8)
    return cudaErrorInvalidValue;
  switch (epi) {
    case kEpiInProj: return launch_epi<kEpiInProj>(a, s, pdl);
    case kEpiOut: return launch_epi<kEpiOut>(a, s, pdl);
    default: return launch_epi<kEpiLogits>(a, s, pdl);
  }
}

}  // namespace mtj
