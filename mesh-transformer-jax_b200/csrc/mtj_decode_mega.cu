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

#include <cstdlib>

#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

// This file is compiled twice: with 256 threads per block (two blocks per SM), and with MTJ_MEGA_MT=512 (one block
// of 16 warps per SM) for one sequence on one GPU, where halving the arrivals per grid-wide hand-over is worth
// 1.2 % of the step; with tensor-parallel slices the wider block loses more in the attention phase than it gains.
#ifndef MTJ_MEGA_MT
#define MTJ_MEGA_MT 256
#endif
constexpr int kMT = MTJ_MEGA_MT;         // threads per block
constexpr int kMW = kMT / 32;            // warps per block
#ifndef MTJ_MEGA_NC
#define MTJ_MEGA_NC 4
#endif

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void trace(unsigned long long* t, int slot) {
  // phase time stamps of block 0 (nanoseconds), for the profiling read-out
  if (t && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long v;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
    t[slot] = v;
  }
}

// All threads of the block call these.
__device__ __forceinline__ void phase_arrive(uint32_t* counter) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
  }
}
__device__ __forceinline__ void phase_wait(const uint32_t* counter, uint32_t target, uint32_t* dev_err, int limit) {
  if (threadIdx.x == 0) {
    int spins = 0;
    while (ld_acquire_gpu(counter) < target) {
      if (++spins > limit) {
        if (dev_err) atomicOr(dev_err, kDevErrTimeout);
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
}

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// g_psum over the "shard" axis inside the persistent kernel (tensor parallel decode).  Every rank
// has written its [B, d] partial sums into slot (k & 1) of its exchange buffer (k = all-reduces done
// so far).  The last block to arrive publishes flag[rank] = k + 1 to all peers; every block waits
// (bounded) for the peers' flags, then adds its slice of the peers' slots in rank order into x
// (x += sum, or x = sum when `accumulate` is false).  Same protocol as mtj_p2p.cu.
__device__ __forceinline__ void mega_all_reduce(const MegaArgs& a, uint32_t k, uint32_t* c_local, uint32_t target,
                                                int n_elems, bool accumulate) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(c_local, 1u);
    if (ticket == target - 1) {                      // every block's partial sums are in place
      __threadfence_system();
      for (int r = 0; r < a.world; ++r)
        if (r != a.rank) st_release_sys_u32(a.peer_flags[r] + a.rank, k + 1);
    }
  }
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    const uint32_t* f = a.local_flags + threadIdx.x;
    int spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys_u32(f) - (k + 1)) < 0) {
      if (++spins > a.wait_limit) {
        if (a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
        break;
      }
    }
  } else if (threadIdx.x == a.rank) {
    // this rank's own partial sums are read below like a peer's: a peer's flag says nothing about them, so
    // wait until every block of THIS rank has arrived as well (the flag towards the peers is sent by the last)
    int spins = 0;
    while (ld_acquire_gpu(c_local) < target) {
      if (++spins > a.wait_limit) {
        if (a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
  const size_t slot = static_cast<size_t>(k & 1u) * a.slot_elems;
  for (int i = (blockIdx.x * kMT + threadIdx.x) * 4; i < n_elems; i += gridDim.x * kMT * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < a.world; ++r) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(a.peer_data[r] + slot + i));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float4* xp = reinterpret_cast<float4*>(a.x + i);
    if (accumulate) {
      const float4 o = *xp;
      acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    *xp = acc;
  }
}

// The layer's g_psum without flags, fences or a grid-wide hand-over.  Block b of every rank computes
// the same 2 * kMW output rows.  Each partial sum (bias included) travels as one 8-byte packet
// (value, k + 1) stored straight into every rank's receive buffer [slot k & 1][source rank]; an aligned
// 8-byte store is indivisible, so a packet whose second word reads k + 1 carries this exchange's value.
// The block then polls (bounded) the `world` packets of each of its rows and adds them in rank order to
// x.  A receive row is written by the peers' block b and read by this rank's block b alone, and a peer
// reaches exchange k + 2 only after it has seen this block's packets of exchange k + 1, which are sent
// after slot k & 1 was read: two slots suffice.  Only blocks that own rows take part.
__device__ __forceinline__ void st_packet(uint2* p, float v, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_packet(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mega_push_reduce(const MegaArgs& a, uint32_t k, int B, int d) {
  const int n_first = blockIdx.x * 2 * kMW;
  if (n_first >= d) return;
  const int rows = min(2 * kMW, d - n_first);
  if (threadIdx.x < rows * B) {
    const int n = n_first + threadIdx.x % rows, bt = threadIdx.x / rows;
    const uint2* src = a.peer_recv[a.rank] + static_cast<size_t>(k & 1u) * a.world * kMegaPushRows * d +
                       static_cast<size_t>(bt) * d + n;
    float* xp = a.x + static_cast<size_t>(bt) * d + n;
    float acc = *xp;
    for (int r = 0; r < a.world; ++r) {
      const uint2* p = src + static_cast<size_t>(r) * kMegaPushRows * d;
      uint2 v = ld_packet(p);
      int spins = 0;
      while (v.y != k + 1) {
        if (++spins > a.wait_limit) {
          if (a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
          break;
        }
        v = ld_packet(p);
      }
      acc += __uint_as_float(v.x);
    }
    *xp = acc;
  }
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

// acc += rows (w, w + K) x activations over chunks [c_begin, c_end) of 256 elements, two stages of
// NC chunks in flight.  XS: activations in the shared-memory layout, otherwise global fp32 rows.
template <int BT, bool XS>
__device__ __forceinline__ void warp_rows2(const __nv_bfloat16* __restrict__ w, int K, int c_begin, int c_end,
                                           const float4* xn, const float* xg, int ldx, int lane,
                                           float (&acc)[2][BT]) {
  constexpr int NC = MTJ_MEGA_NC;
  const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
  const __nv_bfloat16* wl = w + lane * 8;
  auto load = [&](uint4 (&buf)[NC][2], int c) {
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int cc = c + i;
      const bool ok = cc < c_end && cc * 256 + lane * 8 < K;
      buf[i][0] = ok ? ld_stream16(wl + static_cast<size_t>(cc) * 256) : z4;
      buf[i][1] = ok ? ld_stream16(wl + K + static_cast<size_t>(cc) * 256) : z4;
    }
  };
  if (c_begin >= c_end) return;
  uint4 nxt[NC][2];
  load(nxt, c_begin);
  for (int c = c_begin; c < c_end; c += NC) {
    uint4 cur[NC][2];
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      cur[i][0] = nxt[i][0];
      cur[i][1] = nxt[i][1];
    }
    if (c + NC < c_end) load(nxt, c + NC);
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int cc = c + i;
      if (cc >= c_end) break;
      const bool in_k = cc * 256 + lane * 8 < K;
      float w0[8], w1[8];
      unpack8(cur[i][0], w0);
      unpack8(cur[i][1], w1);
#pragma unroll
      for (int bt = 0; bt < BT; ++bt) {
        float4 a, b;
        if (XS) {
          // K need not be a multiple of 256 (tensor-parallel slices): the last chunk's upper lanes hold nothing
          const float4* lo = xn + static_cast<size_t>(bt) * 2 * (K >> 3);
          a = in_k ? lo[cc * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
          b = in_k ? lo[(K >> 3) + cc * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
          const float* xr = xg + static_cast<size_t>(bt) * ldx + cc * 256 + lane * 8;
          a = in_k ? __ldcg(reinterpret_cast<const float4*>(xr)) : make_float4(0.f, 0.f, 0.f, 0.f);
          b = in_k ? __ldcg(reinterpret_cast<const float4*>(xr + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
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

// The same two-row product for a whole list of units u = u_first, u_first + u_step, ... (< u_end),
// rows 2u and 2u + 1 of W, as ONE software pipeline: the loads of the next unit's first chunks are
// already in flight while the current unit is reduced and finished by epi(u, value-of-this-lane).
template <int BT, bool XS, typename Epi>
__device__ __forceinline__ void warp_stream(const __nv_bfloat16* __restrict__ W, int K, int nch, int u_first,
                                            int u_step, int u_end, const float4* xn, const float* xg, int ldx,
                                            int lane, Epi epi) {
  constexpr int NC = MTJ_MEGA_NC;            // chunks per pipeline stage (two stages in flight)
  if (u_first >= u_end) return;
  const int spu = (nch + NC - 1) / NC;       // stages per unit
  const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
  auto load = [&](uint4 (&buf)[NC][2], int u, int st) {
    const __nv_bfloat16* wl = W + static_cast<size_t>(2 * u) * K + lane * 8;
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int cc = st * NC + i;
      const bool ok = cc < nch && cc * 256 + lane * 8 < K;
      buf[i][0] = ok ? ld_stream16(wl + static_cast<size_t>(cc) * 256) : z4;
      buf[i][1] = ok ? ld_stream16(wl + K + static_cast<size_t>(cc) * 256) : z4;
    }
  };
  float acc[2][BT];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int bt = 0; bt < BT; ++bt) acc[r][bt] = 0.f;
  uint4 nxt[NC][2];
  int u = u_first, st = 0;
  load(nxt, u, st);
  while (u < u_end) {
    uint4 cur[NC][2];
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      cur[i][0] = nxt[i][0];
      cur[i][1] = nxt[i][1];
    }
    int un = u, sn = st + 1;                 // the stage after this one
    if (sn == spu) {
      sn = 0;
      un = u + u_step;
    }
    if (un < u_end) load(nxt, un, sn);
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int cc = st * NC + i;
      if (cc >= nch) break;
      const bool in_k = cc * 256 + lane * 8 < K;
      float w0[8], w1[8];
      unpack8(cur[i][0], w0);
      unpack8(cur[i][1], w1);
#pragma unroll
      for (int bt = 0; bt < BT; ++bt) {
        float4 a, b;
        if (XS) {
          // K need not be a multiple of 256 (tensor-parallel slices): the last chunk's upper lanes hold nothing
          const float4* lo = xn + static_cast<size_t>(bt) * 2 * (K >> 3);
          a = in_k ? lo[cc * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
          b = in_k ? lo[(K >> 3) + cc * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
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
    if (st == spu - 1) {
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int bt = 0; bt < BT; ++bt) acc[r][bt] = warp_sum(acc[r][bt]);
      epi(u, pick_lane_value<BT>(acc, lane));
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int bt = 0; bt < BT; ++bt) acc[r][bt] = 0.f;
    }
    u = un;
    st = sn;
  }
}

#if MTJ_MEGA_MT == 256
// The same pipeline for units of ONE row of W (2 * NC chunks of the row per stage): rows r = r_first, r_first +
// r_step, ... (< r_end); epi(r, acc) gets the BT sums of the row in every lane.  Used for the FF-in rows of
// tensor-parallel slices, where whole row pairs leave the warps too unevenly loaded.
template <int BT, typename Epi>
__device__ __forceinline__ void warp_stream1(const __nv_bfloat16* __restrict__ W, int K, int nch, int r_first,
                                             int r_step, int r_end, const float4* xn, int lane, Epi epi) {
  constexpr int NC = 2 * MTJ_MEGA_NC;
  if (r_first >= r_end) return;
  const int spu = (nch + NC - 1) / NC;       // stages per row
  const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
  auto load = [&](uint4 (&buf)[NC], int r, int st) {
    const __nv_bfloat16* wl = W + static_cast<size_t>(r) * K + lane * 8;
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int cc = st * NC + i;
      const bool ok = cc < nch && cc * 256 + lane * 8 < K;
      buf[i] = ok ? ld_stream16(wl + static_cast<size_t>(cc) * 256) : z4;
    }
  };
  float acc[BT];
#pragma unroll
  for (int bt = 0; bt < BT; ++bt) acc[bt] = 0.f;
  uint4 nxt[NC];
  int r = r_first, st = 0;
  load(nxt, r, st);
  while (r < r_end) {
    uint4 cur[NC];
#pragma unroll
    for (int i = 0; i < NC; ++i) cur[i] = nxt[i];
    int rn = r, sn = st + 1;
    if (sn == spu) {
      sn = 0;
      rn = r + r_step;
    }
    if (rn < r_end) load(nxt, rn, sn);
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int cc = st * NC + i;
      if (cc >= nch) break;
      const bool in_k = cc * 256 + lane * 8 < K;
      float w0[8];
      unpack8(cur[i], w0);
#pragma unroll
      for (int bt = 0; bt < BT; ++bt) {
        const float4* lo = xn + static_cast<size_t>(bt) * 2 * (K >> 3);
        const float4 xa = in_k ? lo[cc * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 xb = in_k ? lo[(K >> 3) + cc * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[bt] = fmaf(w0[e], xv[e], acc[bt]);
      }
    }
    if (st == spu - 1) {
#pragma unroll
      for (int bt = 0; bt < BT; ++bt) acc[bt] = warp_sum(acc[bt]);
      epi(r, acc);
#pragma unroll
      for (int bt = 0; bt < BT; ++bt) acc[bt] = 0.f;
    }
    r = rn;
    st = sn;
  }
}
#endif

template <int BT, int DH>
__global__ void __launch_bounds__(kMT, (BT == 1 && kMT == 256) ? 2 : 1) decode_mega_kernel(const MegaArgs a) {
  extern __shared__ __align__(128) unsigned char mega_smem[];
  __shared__ float red[kMW];

  __shared__ float sm_m[kMW], sm_l[kMW];
  __shared__ float sm_o[kMW][DH];
  __shared__ float wgt[64];
  __shared__ float inv_l;
  __shared__ bool is_last;
  __shared__ unsigned long long blk_amax[4];         // greedy token: this block's best (logit order key, index) per row

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = gridDim.x;
  const int gw = blockIdx.x * kMW + warp;            // global warp index
  const int GW = G * kMW;
  const int B = a.B, d = a.d, dl = a.dl, ffl = a.ffl, L = a.L;
  float4* xn = reinterpret_cast<float4*>(mega_smem);
  uint32_t* c_x = a.sync;                            // [L + 1]
  uint32_t* c_qkv = a.sync + (L + 1);                // [L]
  uint32_t* c_af = a.sync + (2 * L + 1);             // [L] attention (incl. merges) done
  uint32_t* c_ff = a.sync + (3 * L + 1);             // [L] FF-in rows done
  uint32_t* c_end = a.sync + (4 * L + 1);
  uint32_t* c_red = a.sync + (4 * L + 2);            // [L + 1] partial sums written (tensor parallel)
  const bool tp = a.world > 1;
  const uint32_t seq0 = tp ? *a.seq : 0u;            // all-reduces completed before this step
  float* partial = tp ? a.slot_base : nullptr;       // this rank's exchange buffer (two slots)
  const uint32_t target = static_cast<uint32_t>(G);
  // the push exchange needs one pass of row pairs over the grid's warps (block b owns rows [16 b, 16 b + 16))
  const bool push = tp && a.peer_recv[0] != nullptr && (d >> 1) <= GW && B <= kMegaPushRows;

  const int cur = *a.cur;                            // absolute position of this step's token

  // ---- embedding: x[b] = table[token_b] + bias ------------------------------------------------
  for (int b = blockIdx.x; b < B; b += G) {
    const int64_t id = static_cast<int64_t>(a.tokens[b]) - a.vocab_start;
    const bool hit = id >= 0 && id < a.V;
    const __nv_bfloat16* row = a.emb_w + static_cast<size_t>(hit ? id : 0) * d;
    float* dst = tp ? partial + static_cast<size_t>(seq0 & 1u) * a.slot_elems : a.x;
    for (int i = threadIdx.x; i < d; i += kMT)
      dst[static_cast<size_t>(b) * d + i] = (hit ? __bfloat162float(row[i]) : 0.f) + a.emb_b[i];
  }
  if (tp) mega_all_reduce(a, seq0, c_red, target, B * d, false);
  phase_arrive(c_x);

  for (int l = 0; l < L; ++l) {
    const MegaLayer& lw = a.layers[l];
    const int N1 = 3 * dl + ffl;
    const int nq = (3 * dl) >> 1, n1 = N1 >> 1;      // warp units (2 rows each): Q/K/V first, then FF-in
    // ask for the first weights of this block's first unit before waiting for x
    if (gw < n1) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c * 256 + lane * 8 < d) {
          prefetch_l2(lw.w_in + static_cast<size_t>(2 * gw) * d + c * 256 + lane * 8);
          prefetch_l2(lw.w_in + static_cast<size_t>(2 * gw + 1) * d + c * 256 + lane * 8);
        }
      }
    }
    trace(a.trace, 6 * l + 0);
    phase_wait(c_x + l, target, a.dev_err, a.wait_limit);
    trace(a.trace, 6 * l + 1);
    layer_norm_to_smem<BT>(a.x, B, d, lw.ln_scale, lw.ln_offset, xn, red);

    // this block's attention unit is known already: pull its keys / values (all but the newest token)
    // towards L2 while the projections stream
    {
      const int splits = a.grid_splits;
      const int unit = blockIdx.x;
      if (unit < B * a.heads * splits) {
        const int split = unit % splits, head = (unit / splits) % a.heads, b = unit / (splits * a.heads);
        const int start = max(a.pad[b], cur - a.window + 1);
        const int t0 = start + split * a.split_tokens, t1 = min(cur, t0 + a.split_tokens);
        const int32_t* table = a.page_table + static_cast<size_t>(b) * a.ring_pages;
        constexpr int kLines = DH * 2 / 128;
        for (int i = threadIdx.x; i < (t1 - t0) * kLines; i += kMT) {
          const size_t off = kv_offset(table, a.ring_pages, a.heads, DH, head, t0 + i / kLines) + (i % kLines) * 64;
          prefetch_l2(lw.kpool + off);
          prefetch_l2(lw.vpool + off);
        }
      }
    }

    // ---- in-projection ------------------------------------------------------------------------
    const int nch = (d + 255) >> 8;
    auto in_epi = [&](int u, float val) {
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
    };
    // Q/K/V rows first; once this block's share is behind it the attention phase may count on it
    warp_stream<BT, true>(lw.w_in, d, nch, gw, GW, nq, xn, nullptr, 0, lane, in_epi);
    phase_arrive(c_qkv + l);
#if MTJ_MEGA_MT == 256
    if (a.ff_row_units) {
      // Tensor-parallel slices have too few row pairs per warp for pairs to spread evenly (a quarter of GPT-J-6B:
      // 3584 pairs on 2368 warps, i.e. two pairs for half of the warps and one for the rest).  The warps that are a
      // Q/K/V pair short take one FF pair first; the remaining FF rows then go round ONE row at a time.
      const int q_rem = nq % GW, ffu = ffl >> 1;
      const int lvl = q_rem > 0 ? min(ffu, GW - q_rem) : 0;
      if (q_rem > 0 && gw >= q_rem && gw - q_rem < lvl) {
        const int u = nq + (gw - q_rem);
        warp_stream<BT, true>(lw.w_in, d, nch, u, GW, u + 1, xn, nullptr, 0, lane, in_epi);
      }
      warp_stream1<BT>(lw.w_in + static_cast<size_t>(3 * dl) * d, d, nch, 2 * lvl + gw, GW, ffl, xn, lane,
                       [&](int f, const float (&acc)[BT]) {
                         float val = 0.f;
#pragma unroll
                         for (int bt = 0; bt < BT; ++bt)
                           if (lane == bt) val = acc[bt];
                         if (lane < BT && lane < B)
                           a.act2[static_cast<size_t>(lane) * (dl + ffl) + dl + f] = gelu_tanh(val + lw.b_ff[f]);
                       });
    } else {
#endif
    // FF-in rows: continue the round-robin where the Q/K/V units stopped, so the load stays even
    const int ff_first = nq + ((gw - nq % GW) + GW) % GW;
    // The units of the last, partial round do not go to the first warps of the grid but to the last ones: with more
    // warps than out-projection row pairs those belong to blocks that have no out-projection rows, so being late
    // here delays nothing, whereas a block that is late into attention is late out of the out-projection, and the
    // next layer waits for it.
    const int n_full = (n1 / GW) * GW;
    const bool tail_swap = n_full >= nq && (d >> 1) <= GW - (n1 - n_full);
    warp_stream<BT, true>(lw.w_in, d, nch, ff_first, GW, tail_swap ? n_full : n1, xn, nullptr, 0, lane, in_epi);
    if (tail_swap && gw >= GW - (n1 - n_full)) {
      const int u = n_full + (GW - 1 - gw);
      warp_stream<BT, true>(lw.w_in, d, nch, u, GW, u + 1, xn, nullptr, 0, lane, in_epi);
    }
#if MTJ_MEGA_MT == 256
    }
#endif
    phase_arrive(c_ff + l);

    // ---- attention: one unit = (sequence, head, contiguous range of up to a.split_tokens keys) ------
    // Every block gets at most one unit per round; its warps read their keys / values straight from the
    // paged cache with all loads of a batch in flight at once (no staging, no block-level waits).
    __syncthreads();
    trace(a.trace, 6 * l + 2);                         // this block's in-projection rows are done
    phase_wait(c_qkv + l, target, a.dev_err, a.wait_limit);
    {
      constexpr int EPL = DH / 32;
      constexpr int TB = 8;                            // keys per batch and warp
      constexpr float scale = DH == 256 ? 0.0625f : 0.125f;
      const int splits = a.grid_splits;
      const int units = B * a.heads * splits;
      // The merge of a (sequence, head)'s splits takes 4-5 us.  Left to whichever block finishes a head last, it
      // makes that block late into the out-projection, late out of it, and the next layer waits for it.  With more
      // blocks than the out-projection has rows for, the merges go to blocks that have no out-projection rows:
      // block first_idle + (sequence, head) waits (bounded) for that head's splits and merges them.
      const int first_idle = ((d >> 1) + kMW - 1) / kMW;
      const bool dedicated = G - first_idle >= B * a.heads;
      auto merge_head = [&](int b, int head, int nsplit) {   // all threads of the block
        const size_t pbase = (static_cast<size_t>(b) * a.heads + head) * a.max_splits;
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
      };
      for (int unit = blockIdx.x; unit < units; unit += G) {
        const int split = unit % splits, head = (unit / splits) % a.heads, b = unit / (splits * a.heads);
        const int start = max(a.pad[b], cur - a.window + 1);
        const int len = cur + 1 - start;
        const int nsplit = (len + a.split_tokens - 1) / a.split_tokens;
        if (split >= nsplit) continue;                 // uniform for the block
        const int t0 = start + split * a.split_tokens, t1 = min(cur + 1, t0 + a.split_tokens);
        const int32_t* table = a.page_table + static_cast<size_t>(b) * a.ring_pages;
        float q[EPL];
        {
          const float* qp = a.q + (static_cast<size_t>(b) * a.heads + head) * DH + lane * EPL;
#pragma unroll
          for (int e = 0; e < EPL; ++e) q[e] = __ldcg(qp + e) * scale;
        }
        float m = -INFINITY, lsum = 0.f, o[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[e] = 0.f;
        // warp w takes keys t0 + w*per .. of this range, in batches of TB
        const int per = (t1 - t0 + kMW - 1) / kMW;
        const int w0 = t0 + warp * per, w1 = min(t1, w0 + per);
        for (int tb = w0; tb < w1; tb += TB) {
          uint4 kraw[TB], vraw[TB];
          bool ok[TB];
#pragma unroll
          for (int t = 0; t < TB; ++t) {
            const int tt = tb + t;
            ok[t] = tt < w1;
            const size_t off = kv_offset(table, a.ring_pages, a.heads, DH, head, ok[t] ? tt : tb) + lane * EPL;
            if (EPL == 8) {
              kraw[t] = ld_stream16(lw.kpool + off);
              vraw[t] = ld_stream16(lw.vpool + off);
            } else {
              kraw[t].x = ld_stream4(lw.kpool + off);
              vraw[t].x = ld_stream4(lw.vpool + off);
            }
          }
          float sc[TB];
#pragma unroll
          for (int t = 0; t < TB; ++t) {
            float kf[8];
            if (EPL == 8) unpack8(kraw[t], kf);
            else { kf[0] = bf16_lo(kraw[t].x); kf[1] = bf16_hi(kraw[t].x); }
            float dsum = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) dsum = fmaf(q[e], kf[e], dsum);
            sc[t] = dsum;
          }
#pragma unroll
          for (int o2 = 16; o2 > 0; o2 >>= 1)
#pragma unroll
            for (int t = 0; t < TB; ++t) sc[t] += __shfl_xor_sync(0xffffffffu, sc[t], o2);
          float mn = m;
#pragma unroll
          for (int t = 0; t < TB; ++t)
            if (ok[t]) mn = fmaxf(mn, sc[t]);
          const float corr = m == -INFINITY ? 0.f : __expf(m - mn);
          lsum *= corr;
#pragma unroll
          for (int e = 0; e < EPL; ++e) o[e] *= corr;
#pragma unroll
          for (int t = 0; t < TB; ++t) {
            if (!ok[t]) continue;
            const float p = __expf(sc[t] - mn);
            float vf[8];
            if (EPL == 8) unpack8(vraw[t], vf);
            else { vf[0] = bf16_lo(vraw[t].x); vf[1] = bf16_hi(vraw[t].x); }
            lsum += p;
#pragma unroll
            for (int e = 0; e < EPL; ++e) o[e] = fmaf(p, vf[e], o[e]);
          }
          m = mn;
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
          is_last = !dedicated && (ticket == static_cast<uint32_t>(nsplit - 1));
        }
        __syncthreads();
        if (is_last) merge_head(b, head, nsplit);       // uniform
        __syncthreads();                                // shared buffers are free for the next unit
      }
      if (dedicated && static_cast<int>(blockIdx.x) >= first_idle &&
          static_cast<int>(blockIdx.x) - first_idle < B * a.heads) {
        const int hb = static_cast<int>(blockIdx.x) - first_idle;
        const int b = hb / a.heads, head = hb % a.heads;
        const int start = max(a.pad[b], cur - a.window + 1);
        const int nsplit = (cur + 1 - start + a.split_tokens - 1) / a.split_tokens;
        if (threadIdx.x == 0) {
          int spins = 0;
          while (ld_acquire_gpu(a.head_counters + hb) < static_cast<uint32_t>(nsplit)) {
            if (++spins > a.wait_limit) {
              if (a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
              break;
            }
          }
        }
        __syncthreads();
        merge_head(b, head, nsplit);
        __syncthreads();
      }
    }
    // prefetch this block's first out-projection rows, then wait for attention + FF-in everywhere
    {
      const int K2 = dl + ffl;
      const int rg = gw;
      if (rg < (d >> 1)) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          if (c * 256 + lane * 8 < K2) {
            prefetch_l2(lw.w_out + static_cast<size_t>(2 * rg) * K2 + c * 256 + lane * 8);
            prefetch_l2(lw.w_out + static_cast<size_t>(2 * rg + 1) * K2 + c * 256 + lane * 8);
          }
        }
      }
    }
    trace(a.trace, 6 * l + 3);                         // attention units done
    phase_arrive(c_af + l);

    // ---- out-projection + bias + residual: a warp owns two output rows over the whole K ---------
    // K = [attention vector | gelu(ff)].  The FF columns only need every block's FF-in rows, which were
    // finished before attention started, so they are accumulated first; the attention columns follow
    // once every (sequence, head) has been merged -- the wait for the slowest attention unit is spent
    // streaming weights.  For one sequence the activations are staged in shared memory.
    {
      const int K2 = dl + ffl;
      const int nch2 = (K2 + 255) >> 8;
      constexpr bool kStage = (BT == 1);
      const int cS = (dl & 255) == 0 ? (dl >> 8) : 0;  // chunks [0, cS) are attention columns (0: no split)
      const int n8 = K2 >> 3;
      auto stage = [&](int e8_begin, int e8_end) {     // copy act2[8*e8_begin .. 8*e8_end) into the smem layout
        if (kStage) {
          float4* lo = xn;
          float4* hi = xn + n8;
          for (int c = e8_begin + threadIdx.x; c < e8_end; c += kMT) {
            lo[c] = __ldcg(reinterpret_cast<const float4*>(a.act2) + 2 * c);
            hi[c] = __ldcg(reinterpret_cast<const float4*>(a.act2) + 2 * c + 1);
          }
        }
        __syncthreads();
      };
      auto finish = [&](int rg, float (&acc)[2][BT]) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int bt = 0; bt < BT; ++bt) acc[r][bt] = warp_sum(acc[r][bt]);
        const float val = pick_lane_value<BT>(acc, lane);
        const int r = lane & 1, bt = lane >> 1;
        const int n = 2 * rg + r;
        if (lane < 2 * BT && bt < B) {
          if (push) {
            const float v = val + lw.b_out[n];
            const size_t off = (static_cast<size_t>(((seq0 + 1 + l) & 1u) * a.world + a.rank) * kMegaPushRows + bt) * d + n;
            for (int r = 0; r < a.world; ++r) st_packet(a.peer_recv[r] + off, v, seq0 + 2 + l);
          } else if (tp) {
            partial[static_cast<size_t>((seq0 + 1 + l) & 1u) * a.slot_elems + static_cast<size_t>(bt) * d + n] =
                val + lw.b_out[n];
          } else {
            float* xp = a.x + static_cast<size_t>(bt) * d + n;
            *xp = val + lw.b_out[n] + *xp;
          }
        }
      };
      const int nrg = d >> 1;
      const __nv_bfloat16* wrow = lw.w_out + static_cast<size_t>(2 * (gw < nrg ? gw : 0)) * K2;
      float acc[2][BT];
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int bt = 0; bt < BT; ++bt) acc[r][bt] = 0.f;
      phase_wait(c_ff + l, target, a.dev_err, a.wait_limit);
      const int sS = cS > 0 ? cS * 32 : n8;           // no split: everything is staged after the attention wait
      stage(sS, n8);
      if (gw < nrg && cS > 0) warp_rows2<BT, kStage>(wrow, K2, cS, nch2, xn, a.act2, K2, lane, acc);
      phase_wait(c_af + l, target, a.dev_err, a.wait_limit);
      trace(a.trace, 6 * l + 4);
      stage(0, sS);
      if (gw < nrg) {
        warp_rows2<BT, kStage>(wrow, K2, 0, cS > 0 ? cS : nch2, xn, a.act2, K2, lane, acc);
        finish(gw, acc);
      }
      // more row pairs than warps: everything is ready, plain passes
      for (int rg = gw + GW; rg < nrg; rg += GW) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int bt = 0; bt < BT; ++bt) acc[r][bt] = 0.f;
        warp_rows2<BT, kStage>(lw.w_out + static_cast<size_t>(2 * rg) * K2, K2, 0, nch2, xn, a.act2, K2, lane, acc);
        finish(rg, acc);
      }
    }
    __syncthreads();
    trace(a.trace, 6 * l + 5);                         // out-projection rows done
    if (push)
      mega_push_reduce(a, seq0 + 1 + l, B, d);
    else if (tp)
      mega_all_reduce(a, seq0 + 1 + l, c_red + 1 + l, target, B * d, true);
    phase_arrive(c_x + l + 1);
  }

  // ---- final LayerNorm + logits ------------------------------------------------------------------
  {
    const int nv = a.V >> 1;
    if (gw < nv) {
      prefetch_l2(a.proj_w + static_cast<size_t>(2 * gw) * d + lane * 8);
      prefetch_l2(a.proj_w + static_cast<size_t>(2 * gw + 1) * d + lane * 8);
    }
    trace(a.trace, 6 * L + 0);
    phase_wait(c_x + L, target, a.dev_err, a.wait_limit);
    trace(a.trace, 6 * L + 1);
    if (threadIdx.x < 4) blk_amax[threadIdx.x] = 0ull;             // (the LayerNorm below has block barriers)
    layer_norm_to_smem<BT>(a.x, B, d, a.lnf_scale, a.lnf_offset, xn, red);
    const int nch = (d + 255) >> 8;
    // The greedy token (nucleaus_sample with top_p -> 0: the arg-max, highest index among equal logits) is picked
    // on the way: every lane keeps the best logit it has written as (order key << 32 | index); the blocks fold
    // theirs into a.amax with a 64-bit atomic max and the last block to finish writes the token.
    unsigned long long best = 0ull;
    warp_stream<BT, true>(a.proj_w, d, nch, gw, GW, nv, xn, nullptr, 0, lane, [&](int u, float val) {
      const int r = lane & 1, bt = lane >> 1;
      const int n = 2 * u + r;
      if (lane < 2 * BT && bt < B) {
        float y = val + a.proj_b[n];
        a.logits[static_cast<size_t>(bt) * a.V + n] = y;
        if (a.amax) {
          if (y == 0.0f) y = 0.0f;                                   // -0 and +0 compare equal
          uint32_t k = __float_as_uint(y);
          k = (k & 0x80000000u) ? ~k : (k | 0x80000000u);            // ascending integer order == ascending float order
          const unsigned long long cand = (static_cast<unsigned long long>(k) << 32) | static_cast<uint32_t>(n);
          best = cand > best ? cand : best;
        }
      }
    });
    if (a.amax) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, 1);
      best = other > best ? other : best;
      if (lane < 2 * BT && (lane & 1) == 0 && (lane >> 1) < B && best) atomicMax(&blk_amax[lane >> 1], best);
    }
  }

  // ---- the last block to finish resets the arrival counters for the next launch -----------------
  __syncthreads();
  trace(a.trace, 6 * L + 2);
  if (a.amax && threadIdx.x < B && blk_amax[threadIdx.x]) atomicMax(a.amax + threadIdx.x, blk_amax[threadIdx.x]);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(c_end, 1u);
    is_last = (ticket == target - 1);
  }
  __syncthreads();
  if (is_last) {
    for (int i = threadIdx.x; i < 5 * L + 3; i += kMT) a.sync[i] = 0u;
    if (tp && threadIdx.x == 0) *a.seq = seq0 + 1 + L;
    if (a.amax) {
      // every block's maxima were published before its ticket: the token of the step, then the position moves on
      __threadfence();
      if (threadIdx.x < B) {
        const unsigned long long win = *reinterpret_cast<volatile unsigned long long*>(a.amax + threadIdx.x);
        a.tokens_out[threadIdx.x] = static_cast<uint32_t>(win);
        a.amax[threadIdx.x] = 0ull;
      }
      if (threadIdx.x == 0 && a.cur_out) *a.cur_out += 1;
    }
  }
}

template <int BT, int DH>
cudaError_t launch_mega_t(const MegaArgs& a, cudaStream_t s, int* grid_out) {
  const int smem_x = BT * a.d * 4;                                  // LayerNorm output of BT rows
  const int smem_o = BT == 1 ? (a.dl + a.ffl) * 4 : 0;             // staged out-projection input (one sequence)
  const int smem = smem_o > smem_x ? smem_o : smem_x;
  // the shared memory limit and the resident block count belong to the (kernel, device) pair
  static int blocks_of[64] = {}, smem_of[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (smem_of[dev] != smem + 1) {
    cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel<BT, DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    int sms = 0, per_sm = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel<BT, DH>, kMT, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    if (const char* lim = getenv("MTJ_MEGA_BLOCKS_PER_SM")) {      // measurement only
      const int v = atoi(lim);
      if (v >= 1 && v < per_sm) per_sm = v;
    }
    blocks_of[dev] = sms * per_sm;
    smem_of[dev] = smem + 1;
  }
  const int cached_blocks = blocks_of[dev];
  if (grid_out) *grid_out = cached_blocks;
  // attention: one round of units over the resident blocks, at most 64 splits per (sequence, head)
  MegaArgs b = a;
  int want = cached_blocks / (a.B * a.heads);
  want = want < 1 ? 1 : (want > 64 ? 64 : want);
  if (want > a.max_splits) want = a.max_splits;
  b.split_tokens = (a.window + want - 1) / want;
  b.grid_splits = (a.window + b.split_tokens - 1) / b.split_tokens;
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
  return cudaLaunchKernelEx(&cfg, decode_mega_kernel<BT, DH>, b);
}

}  // namespace

#if MTJ_MEGA_MT == 512
cudaError_t launch_decode_mega_wide(const MegaArgs& a, cudaStream_t s, int* grid_out) {
  if (a.B != 1) return cudaErrorInvalidValue;
  if (a.dh == 256) return launch_mega_t<1, 256>(a, s, grid_out);
  if (a.dh == 64) return launch_mega_t<1, 64>(a, s, grid_out);
  return cudaErrorInvalidValue;
}
#else
cudaError_t launch_decode_mega(const MegaArgs& a, cudaStream_t s, int* grid_out) {
  if (a.world < 1 || a.world > 8 || a.B < 1 || a.B > 4 || (a.d & 255) || a.d > 8192 || (a.dl & 1) || (a.V & 1) || ((3 * a.dl + a.ffl) & 1) ||
      ((a.dl + a.ffl) & 7) || a.max_splits < 1 || (a.dl + a.ffl) * 4 > 200 * 1024)
    return cudaErrorInvalidValue;
  if (a.world == 1 && a.B == 1 && !getenv("MTJ_MEGA_NARROW")) return launch_decode_mega_wide(a, s, grid_out);
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
#endif

}  // namespace mtj
