// One persistent kernel for a whole decode step (1-4 sequences, one GPU):
// embedding, every layer (LayerNorm + [Q|K|V|FF-in] projection with RoPE / KV
// write / GELU, split-KV attention over the paged cache, output projection +
// residual) and the final LayerNorm + logits -- the work of generate_once
// (transformer_shard.py:97-115; layers.py:187-193,316-344,561-564).
//
// Why: as separate kernels a 6B decode step is ~115 launches of 25-60 us, and
// every launch boundary drains and refills the HBM pipeline.  Here all blocks
// are resident at once (cooperative launch) and walk the same fixed list of
// phases; a phase that needs another phase's results waits on a global arrival
// counter instead of a kernel boundary:
//     x ready (layer l)      <- all blocks finished the out-projection of l-1
//     attention (layer l)    <- all blocks finished their Q/K/V rows of l
//     out-projection (l)     <- all blocks finished FF-in rows and attention of l
// Q/K/V rows are processed before the FF-in rows, so the attention dependency
// is normally satisfied long before a block gets there, and each block asks
// for its next weights (L2 prefetch) before it waits.  Waits are bounded: a
// wait that runs out sets the device error word and the block carries on, so
// the kernel always terminates.  The math of each phase is that of the
// stand-alone kernels (mtj_gemv.cu, mtj_attn.cu).
#include <math.h>

#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

constexpr int kMT = 256;                 // threads per block
constexpr int kMW = kMT / 32;            // warps per block
constexpr int kWaitLimit = 1 << 22;

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All threads of the block call these.
__device__ __forceinline__ void phase_arrive(uint32_t* counter) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
  }
}
__device__ __forceinline__ void phase_wait(const uint32_t* counter, uint32_t target, uint32_t* dev_err) {
  if (threadIdx.x == 0) {
    int spins = 0;
    while (ld_acquire_gpu(counter) < target) {
      if (++spins > kWaitLimit) {
        if (dev_err) atomicOr(dev_err, kDevErrTimeout);
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kMW; ++i) t += red[i];
  __syncthreads();
  return t;
}

// LayerNorm of the BT rows of x into shared memory, laid out so that lane l of a warp reads the
// two halves of its 8-element chunk from two conflict-free float4 arrays: lo[c*32 + l], hi[c*32 + l].
template <int BT>
__device__ __forceinline__ void layer_norm_to_smem(const float* __restrict__ x, int B, int d,
                                                   const float* __restrict__ scale,
                                                   const float* __restrict__ offset, float4* xn, float* red) {
  const int n8 = d >> 3;
#pragma unroll
  for (int bt = 0; bt < BT; ++bt) {
    float4* lo = xn + static_cast<size_t>(bt) * 2 * n8;
    float4* hi = lo + n8;
    if (bt >= B) {
      for (int c = threadIdx.x; c < n8; c += kMT) lo[c] = hi[c] = make_float4(0.f, 0.f, 0.f, 0.f);
      continue;
    }
    const float* xr = x + static_cast<size_t>(bt) * d;
    // each thread keeps its chunks (8 floats each, up to kLnChunks of them) in registers: one read of x
    constexpr int kLnChunks = 4;                   // d <= 256 threads * 4 chunks * 8 = 8192
    float4 va[kLnChunks], vb[kLnChunks];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kLnChunks; ++i) {
      const int c = threadIdx.x + i * kMT;
      if (c < n8) {
        va[i] = __ldcg(reinterpret_cast<const float4*>(xr) + 2 * c);
        vb[i] = __ldcg(reinterpret_cast<const float4*>(xr) + 2 * c + 1);
        s += (va[i].x + va[i].y) + (va[i].z + va[i].w) + (vb[i].x + vb[i].y) + (vb[i].z + vb[i].w);
      }
    }
    const float mu = block_sum(s, red) / static_cast<float>(d);
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < kLnChunks; ++i) {
      const int c = threadIdx.x + i * kMT;
      if (c < n8) {
        const float e0 = va[i].x - mu, e1 = va[i].y - mu, e2 = va[i].z - mu, e3 = va[i].w - mu;
        const float e4 = vb[i].x - mu, e5 = vb[i].y - mu, e6 = vb[i].z - mu, e7 = vb[i].w - mu;
        v += e0 * e0 + e1 * e1 + e2 * e2 + e3 * e3 + e4 * e4 + e5 * e5 + e6 * e6 + e7 * e7;
      }
    }
    const float rstd = 1.0f / sqrtf(block_sum(v, red) / static_cast<float>(d) + 1e-5f);
#pragma unroll
    for (int i = 0; i < kLnChunks; ++i) {
      const int c = threadIdx.x + i * kMT;
      if (c < n8) {
        const float4 s0 = reinterpret_cast<const float4*>(scale)[2 * c], s1 = reinterpret_cast<const float4*>(scale)[2 * c + 1];
        const float4 o0 = reinterpret_cast<const float4*>(offset)[2 * c], o1 = reinterpret_cast<const float4*>(offset)[2 * c + 1];
        lo[c] = make_float4(fmaf(s0.x * rstd, va[i].x - mu, o0.x), fmaf(s0.y * rstd, va[i].y - mu, o0.y),
                            fmaf(s0.z * rstd, va[i].z - mu, o0.z), fmaf(s0.w * rstd, va[i].w - mu, o0.w));
        hi[c] = make_float4(fmaf(s1.x * rstd, vb[i].x - mu, o1.x), fmaf(s1.y * rstd, vb[i].y - mu, o1.y),
                            fmaf(s1.z * rstd, vb[i].z - mu, o1.z), fmaf(s1.w * rstd, vb[i].w - mu, o1.w));
      }
    }
  }
  __syncthreads();
}

// Two weight rows x BT activation rows over chunks c = c0, c0 + cs, ... (< nch) of 256 elements.
// XS: activations come from the shared-memory layout above; otherwise from global fp32 rows.
template <int BT, bool XS>
__device__ __forceinline__ void warp_gemv2(const __nv_bfloat16* __restrict__ w, int K, int nch, int c0, int cs,
                                           const float4* xn, const float* xg, int ldx, int lane,
                                           float (&acc)[2][BT]) {
  const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
  const __nv_bfloat16* wl = w + lane * 8;
  constexpr int NC = 4;                      // chunks per pipeline stage (two stages in flight)
  auto load2 = [&](uint4 (&buf)[NC][2], int c) {
#pragma unroll
    for (int u = 0; u < NC; ++u) {
      const int cc = c + u * cs;
      const bool ok = cc < nch && cc * 256 + lane * 8 < K;
      buf[u][0] = ok ? ld_stream16(wl + static_cast<size_t>(cc) * 256) : z4;
      buf[u][1] = ok ? ld_stream16(wl + K + static_cast<size_t>(cc) * 256) : z4;
    }
  };
  uint4 nxt[NC][2];
  load2(nxt, c0);
  for (int c = c0; c < nch; c += NC * cs) {
    uint4 cur[NC][2];
#pragma unroll
    for (int u = 0; u < NC; ++u) {
      cur[u][0] = nxt[u][0];
      cur[u][1] = nxt[u][1];
    }
    if (c + NC * cs < nch) load2(nxt, c + NC * cs);
#pragma unroll
    for (int u = 0; u < NC; ++u) {
      const int cc = c + u * cs;
      if (cc >= nch) break;
      const bool in_k = cc * 256 + lane * 8 < K;
      float w0[8], w1[8];
      unpack8(cur[u][0], w0);
      unpack8(cur[u][1], w1);
#pragma unroll
      for (int bt = 0; bt < BT; ++bt) {
        float4 a, b;
        if (XS) {
          const float4* lo = xn + static_cast<size_t>(bt) * 2 * (K >> 3);
          a = lo[cc * 32 + lane];
          b = lo[(K >> 3) + cc * 32 + lane];
        } else {
          const float* xr = xg + static_cast<size_t>(bt) * ldx + cc * 256 + lane * 8;
          a = in_k ? *reinterpret_cast<const float4*>(xr) : make_float4(0.f, 0.f, 0.f, 0.f);
          b = in_k ? *reinterpret_cast<const float4*>(xr + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const float xv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          acc[0][bt] = fmaf(w0[e], xv[e], acc[0][bt]);
          acc[1][bt] = fmaf(w1[e], xv[e], acc[1][bt]);
        }
      }
    }
  }
}

template <int BT>
__device__ __forceinline__ float pick_lane_value(const float (&acc)[2][BT], int lane) {
  float val = 0.f;
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int bt = 0; bt < BT; ++bt)
      if (lane == bt * 2 + r) val = acc[r][bt];
  return val;
}

template <int BT, int DH>
__global__ void __launch_bounds__(kMT, BT == 1 ? 2 : 1) decode_mega_kernel(const MegaArgs a) {
  extern __shared__ __align__(128) unsigned char mega_smem[];
  __shared__ float red[kMW];

  __shared__ __align__(8) uint64_t bar;
  __shared__ float sm_m[kMW], sm_l[kMW];
  __shared__ float sm_o[kMW][DH];
  __shared__ float wgt[64];
  __shared__ float inv_l;
  __shared__ bool is_last;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = gridDim.x;
  const int gw = blockIdx.x * kMW + warp;            // global warp index
  const int GW = G * kMW;
  const int B = a.B, d = a.d, dl = a.dl, ffl = a.ffl, L = a.L;
  float4* xn = reinterpret_cast<float4*>(mega_smem);
  uint32_t* c_x = a.sync;                            // [L + 1]
  uint32_t* c_qkv = a.sync + (L + 1);                // [L]
  uint32_t* c_af = a.sync + (2 * L + 1);             // [L]
  uint32_t* c_end = a.sync + (3 * L + 1);
  const uint32_t target = static_cast<uint32_t>(G);
  const uint32_t bar_u32 = smem_u32(&bar);
  uint32_t bar_phase = 0;
  if (threadIdx.x == 0) {
    mbar_init(bar_u32, 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int cur = *a.cur;                            // absolute position of this step's token

  // ---- embedding: x[b] = table[token_b] + bias ------------------------------------------------
  for (int b = blockIdx.x; b < B; b += G) {
    const uint32_t id = a.tokens[b];
    const bool hit = id < static_cast<uint32_t>(a.V);
    const __nv_bfloat16* row = a.emb_w + static_cast<size_t>(hit ? id : 0) * d;
    for (int i = threadIdx.x; i < d; i += kMT)
      a.x[static_cast<size_t>(b) * d + i] = (hit ? __bfloat162float(row[i]) : 0.f) + a.emb_b[i];
  }
  phase_arrive(c_x);

  for (int l = 0; l < L; ++l) {
    const MegaLayer& lw = a.layers[l];
    const int N1 = 3 * dl + ffl;
    const int nq = (3 * dl) >> 1, n1 = N1 >> 1;      // warp units (2 rows each): Q/K/V first, then FF-in
    // ask for the first weights of this block's first unit before waiting for x
    if (gw < n1) {
      prefetch_l2(lw.w_in + static_cast<size_t>(2 * gw) * d + lane * 8);
      prefetch_l2(lw.w_in + static_cast<size_t>(2 * gw + 1) * d + lane * 8);
    }
    phase_wait(c_x + l, target, a.dev_err);
    layer_norm_to_smem<BT>(a.x, B, d, lw.ln_scale, lw.ln_offset, xn, red);

    // ---- in-projection ------------------------------------------------------------------------
    const int nch = (d + 255) >> 8;
    bool qkv_signalled = false;
    for (int u0 = 0; u0 < n1; u0 += GW) {
      const int u = u0 + gw;
      if (u < n1) {
        float acc[2][BT];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int bt = 0; bt < BT; ++bt) acc[r][bt] = 0.f;
        warp_gemv2<BT, true>(lw.w_in + static_cast<size_t>(2 * u) * d, d, nch, 0, 1, xn, nullptr, 0, lane, acc);
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int bt = 0; bt < BT; ++bt) acc[r][bt] = warp_sum(acc[r][bt]);
        const float val = pick_lane_value<BT>(acc, lane);
        const float partner = __shfl_xor_sync(0xffffffffu, val, 1);
        const int r = lane & 1, bt = lane >> 1;
        const int n = 2 * u + r;
        if (lane < 2 * BT && bt < B) {
          if (n < 3 * dl) {
            const int region = n / dl;
            const int nn = n - region * dl;
            const int head = nn / DH, j = nn % DH;
            float y = val;
            if (region < 2 && j < a.rot) {
              const float2 sc = a.sincos[static_cast<size_t>(cur) * (a.rot >> 1) + (j >> 1)];
              y = (j & 1) ? (val * sc.y + partner * sc.x) : (val * sc.y - partner * sc.x);
            }
            if (region == 0) {
              a.q[static_cast<size_t>(bt) * dl + nn] = y;
            } else if (cur >= a.pad[bt]) {
              __nv_bfloat16* pool = region == 1 ? lw.kpool : lw.vpool;
              const size_t off = kv_offset(a.page_table + static_cast<size_t>(bt) * a.ring_pages, a.ring_pages,
                                           a.heads, DH, head, cur);
              pool[off + j] = __float2bfloat16_rn(y);
            }
          } else {
            const int f = n - 3 * dl;
            a.act2[static_cast<size_t>(bt) * (dl + ffl) + dl + f] = gelu_tanh(val + lw.b_ff[f]);
          }
        }
      }
      // once every Q/K/V unit of this block is behind it, tell the attention phase
      if (!qkv_signalled && u0 + GW >= nq) {
        phase_arrive(c_qkv + l);
        qkv_signalled = true;
      }
    }
    if (!qkv_signalled) phase_arrive(c_qkv + l);

    // ---- attention: one unit = (sequence, head, 64-token page) ---------------------------------
    phase_wait(c_qkv + l, target, a.dev_err);          // also: every warp of this block left shared x
    {
      constexpr int EPL = DH / 32;
      constexpr int TPW = kPageTokens / kMW;
      constexpr uint32_t kSlab = kPageTokens * DH * 2;
      __nv_bfloat16* sk = reinterpret_cast<__nv_bfloat16*>(mega_smem);
      __nv_bfloat16* sv = reinterpret_cast<__nv_bfloat16*>(mega_smem + kSlab);
      const int splits = a.grid_splits;
      const int units = B * a.heads * splits;
      for (int unit = blockIdx.x; unit < units; unit += G) {
        const int split = unit % splits, head = (unit / splits) % a.heads, b = unit / (splits * a.heads);
        const int start = max(a.pad[b], cur - a.window + 1);
        const int first_page = start / kPageTokens;
        const int nsplit = cur / kPageTokens - first_page + 1;
        if (split >= nsplit) continue;                 // uniform for the block
        const int page_pos0 = (first_page + split) * kPageTokens;
        const int t0 = max(start, page_pos0), t1 = min(cur + 1, page_pos0 + kPageTokens);
        if (threadIdx.x == 0) {
          const int32_t* table = a.page_table + static_cast<size_t>(b) * a.ring_pages;
          const int page = table[(first_page + split) % a.ring_pages];
          const size_t off = (static_cast<size_t>(page) * a.heads + head) * kPageTokens * DH;
          const uint64_t pol = l2_evict_first_policy();
          // generic-proxy reads of the previous unit are ordered before these async writes by the block barrier
          mbar_expect_tx(bar_u32, 2 * kSlab);
          bulk_load(smem_u32(sk), lw.kpool + off, kSlab, bar_u32, pol);
          bulk_load(smem_u32(sv), lw.vpool + off, kSlab, bar_u32, pol);
        }
        constexpr float scale = DH == 256 ? 0.0625f : 0.125f;
        float q[EPL];
        {
          const float* qp = a.q + (static_cast<size_t>(b) * a.heads + head) * DH + lane * EPL;
#pragma unroll
          for (int e = 0; e < EPL; ++e) q[e] = __ldcg(qp + e) * scale;
        }
        const bool arrived = mbar_wait(bar_u32, bar_phase & 1);
        bar_phase++;
        if (!arrived && threadIdx.x == 0 && a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
        float m = -INFINITY, lsum = 0.f, o[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[e] = 0.f;
        {
          float s[TPW];
          bool ok[TPW];
#pragma unroll
          for (int t = 0; t < TPW; ++t) {
            const int tt = page_pos0 + warp * TPW + t;
            ok[t] = arrived && tt >= t0 && tt < t1;
            const __nv_bfloat16* kp = sk + static_cast<size_t>(warp * TPW + t) * DH + lane * EPL;
            float kf[EPL];
            if (EPL == 8) unpack8(*reinterpret_cast<const uint4*>(kp), kf);
            else { const uint32_t w2 = *reinterpret_cast<const uint32_t*>(kp); kf[0] = bf16_lo(w2); kf[1] = bf16_hi(w2); }
            float dsum = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) dsum = fmaf(q[e], kf[e], dsum);
            s[t] = dsum;
          }
#pragma unroll
          for (int o2 = 16; o2 > 0; o2 >>= 1)
#pragma unroll
            for (int t = 0; t < TPW; ++t) s[t] += __shfl_xor_sync(0xffffffffu, s[t], o2);
#pragma unroll
          for (int t = 0; t < TPW; ++t)
            if (ok[t]) m = fmaxf(m, s[t]);
#pragma unroll
          for (int t = 0; t < TPW; ++t) {
            if (!ok[t]) continue;
            const float p = __expf(s[t] - m);
            const __nv_bfloat16* vp = sv + static_cast<size_t>(warp * TPW + t) * DH + lane * EPL;
            float vf[EPL];
            if (EPL == 8) unpack8(*reinterpret_cast<const uint4*>(vp), vf);
            else { const uint32_t w2 = *reinterpret_cast<const uint32_t*>(vp); vf[0] = bf16_lo(w2); vf[1] = bf16_hi(w2); }
            lsum += p;
#pragma unroll
            for (int e = 0; e < EPL; ++e) o[e] = fmaf(p, vf[e], o[e]);
          }
        }
        if (lane == 0) {
          sm_m[warp] = m;
          sm_l[warp] = lsum;
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) sm_o[warp][lane * EPL + e] = o[e];
        __syncthreads();
        const size_t pbase = (static_cast<size_t>(b) * a.heads + head) * a.max_splits;
        if (threadIdx.x < DH) {
          float M = -INFINITY;
#pragma unroll
          for (int w = 0; w < kMW; ++w) M = fmaxf(M, sm_m[w]);
          float Ls = 0.f, O = 0.f;
#pragma unroll
          for (int w = 0; w < kMW; ++w) {
            const float f = sm_m[w] == -INFINITY ? 0.f : __expf(sm_m[w] - M);
            Ls = fmaf(sm_l[w], f, Ls);
            O = fmaf(sm_o[w][threadIdx.x], f, O);
          }
          a.part_o[(pbase + split) * DH + threadIdx.x] = O;
          if (threadIdx.x == 0) {
            a.part_ml[(pbase + split) * 2] = M;
            a.part_ml[(pbase + split) * 2 + 1] = Ls;
          }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
          const uint32_t ticket = atomicAdd(a.head_counters + b * a.heads + head, 1u);
          is_last = (ticket == static_cast<uint32_t>(nsplit - 1));
        }
        __syncthreads();
        if (is_last) {                                  // uniform: merge the splits of this (sequence, head)
          __threadfence();
          if (warp == 0) {
            float ms[2], ls[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int sidx = lane + 32 * h2;
              ms[h2] = sidx < nsplit ? __ldcg(a.part_ml + (pbase + sidx) * 2) : -INFINITY;
              ls[h2] = sidx < nsplit ? __ldcg(a.part_ml + (pbase + sidx) * 2 + 1) : 0.f;
            }
            const float M = warp_max(fmaxf(ms[0], ms[1]));
            float lt = 0.f;
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const float f = ms[h2] == -INFINITY ? 0.f : __expf(ms[h2] - M);
              wgt[lane + 32 * h2] = f;
              lt = fmaf(ls[h2], f, lt);
            }
            lt = warp_sum(lt);
            if (lane == 0) inv_l = 1.0f / lt;
          }
          __syncthreads();
          if (threadIdx.x < DH) {
            const float* po = a.part_o + pbase * DH + threadIdx.x;
            float O = 0.f;
            int sidx = 0;
            for (; sidx + 8 <= nsplit; sidx += 8) {
              float v[8];
#pragma unroll
              for (int t = 0; t < 8; ++t) v[t] = __ldcg(po + static_cast<size_t>(sidx + t) * DH);
#pragma unroll
              for (int t = 0; t < 8; ++t) O = fmaf(v[t], wgt[sidx + t], O);
            }
            for (; sidx < nsplit; ++sidx) O = fmaf(__ldcg(po + static_cast<size_t>(sidx) * DH), wgt[sidx], O);
            a.act2[static_cast<size_t>(b) * (dl + ffl) + head * DH + threadIdx.x] = O * inv_l;
          }
          if (threadIdx.x == 0) a.head_counters[b * a.heads + head] = 0u;
        }
        __syncthreads();                                // shared buffers are free for the next unit
      }
    }
    // prefetch this block's first out-projection rows, then wait for attention + FF-in everywhere
    {
      const int K2 = dl + ffl;
      const int rg = gw;
      if (rg < (d >> 1)) {
        prefetch_l2(lw.w_out + static_cast<size_t>(2 * rg) * K2 + lane * 8);
        prefetch_l2(lw.w_out + static_cast<size_t>(2 * rg + 1) * K2 + lane * 8);
      }
    }
    phase_arrive(c_af + l);
    phase_wait(c_af + l, target, a.dev_err);

    // ---- out-projection + bias + residual: a block owns two rows, its warps split K ------------
    {
      const int K2 = dl + ffl;
      const int nch2 = (K2 + 255) >> 8;
      for (int rg = gw; rg < (d >> 1); rg += GW) {     // a warp owns two output rows over the whole K
        float acc[2][BT];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int bt = 0; bt < BT; ++bt) acc[r][bt] = 0.f;
        warp_gemv2<BT, false>(lw.w_out + static_cast<size_t>(2 * rg) * K2, K2, nch2, 0, 1, nullptr, a.act2, K2,
                              lane, acc);
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int bt = 0; bt < BT; ++bt) acc[r][bt] = warp_sum(acc[r][bt]);
        const float val = pick_lane_value<BT>(acc, lane);
        const int r = lane & 1, bt = lane >> 1;
        const int n = 2 * rg + r;
        if (lane < 2 * BT && bt < B) {
          float* xp = a.x + static_cast<size_t>(bt) * d + n;
          *xp = val + lw.b_out[n] + *xp;
        }
      }
    }
    phase_arrive(c_x + l + 1);
  }

  // ---- final LayerNorm + logits ------------------------------------------------------------------
  {
    const int nv = a.V >> 1;
    if (gw < nv) {
      prefetch_l2(a.proj_w + static_cast<size_t>(2 * gw) * d + lane * 8);
      prefetch_l2(a.proj_w + static_cast<size_t>(2 * gw + 1) * d + lane * 8);
    }
    phase_wait(c_x + L, target, a.dev_err);
    layer_norm_to_smem<BT>(a.x, B, d, a.lnf_scale, a.lnf_offset, xn, red);
    const int nch = (d + 255) >> 8;
    for (int u = gw; u < nv; u += GW) {
      float acc[2][BT];
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int bt = 0; bt < BT; ++bt) acc[r][bt] = 0.f;
      warp_gemv2<BT, true>(a.proj_w + static_cast<size_t>(2 * u) * d, d, nch, 0, 1, xn, nullptr, 0, lane, acc);
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int bt = 0; bt < BT; ++bt) acc[r][bt] = warp_sum(acc[r][bt]);
      const float val = pick_lane_value<BT>(acc, lane);
      const int r = lane & 1, bt = lane >> 1;
      const int n = 2 * u + r;
      if (lane < 2 * BT && bt < B) a.logits[static_cast<size_t>(bt) * a.V + n] = val + a.proj_b[n];
    }
  }

  // ---- the last block to finish resets the arrival counters for the next launch -----------------
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(c_end, 1u);
    is_last = (ticket == target - 1);
  }
  __syncthreads();
  if (is_last)
    for (int i = threadIdx.x; i < 3 * L + 2; i += kMT) a.sync[i] = 0u;
}

template <int BT, int DH>
cudaError_t launch_mega_t(const MegaArgs& a, cudaStream_t s, int* grid_out) {
  const int smem_attn = 2 * kPageTokens * DH * 2;
  const int smem_x = BT * a.d * 4;
  const int smem = smem_attn > smem_x ? smem_attn : smem_x;
  static int cached_blocks = 0, cached_smem = -1;
  if (cached_smem != smem) {
    cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel<BT, DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel<BT, DH>, kMT, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    cached_blocks = sms * per_sm;
    cached_smem = smem;
  }
  if (grid_out) *grid_out = cached_blocks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cached_blocks);
  cfg.blockDim = dim3(kMT);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;      // all blocks resident: the phase waits cannot starve
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_mega_kernel<BT, DH>, a);
}

}  // namespace

cudaError_t launch_decode_mega(const MegaArgs& a, cudaStream_t s, int* grid_out) {
  if (a.B < 1 || a.B > 4 || (a.d & 255) || a.d > 8192 || (a.dl & 1) || (a.V & 1) || ((3 * a.dl + a.ffl) & 1) ||
      ((a.dl + a.ffl) & 7) || a.grid_splits > 64)
    return cudaErrorInvalidValue;
  if (a.dh == 256) {
    if (a.B == 1) return launch_mega_t<1, 256>(a, s, grid_out);
    if (a.B == 2) return launch_mega_t<2, 256>(a, s, grid_out);
    return launch_mega_t<4, 256>(a, s, grid_out);
  }
  if (a.dh == 64) {
    if (a.B == 1) return launch_mega_t<1, 64>(a, s, grid_out);
    if (a.B == 2) return launch_mega_t<2, 64>(a, s, grid_out);
    return launch_mega_t<4, 64>(a, s, grid_out);
  }
  return cudaErrorInvalidValue;
}

}  // namespace mtj
