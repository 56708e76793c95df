// Tensor-core GEMM for many token rows (prefill / eval): tcgen05.mma with the
// accumulator in tensor memory, operands staged in shared memory by TMA.
//
//   Y^T[n, m] = sum_k W[n, k] * X[m, k]      W: bf16 [N, K] (packed weights)
//                                            X: bf16 [M, K] (activations)
//
// The WEIGHT rows are the MMA's M dimension (128 per tile) and the token rows
// its N dimension (BN per tile), so an epilogue thread owns one output feature
// (one TMEM lane) for BN tokens: the RoPE partner feature sits in the
// neighbouring lane, and for a fixed token the 32 lanes of a warp write 32
// consecutive features (coalesced).  The epilogues are those of the GEMV
// family (in-proj: RoPE / KV-cache write / bias + GELU; out-proj: bias +
// residual; logits: bias) -- reference lines are cited there.
//
// One tile per block; 6 warps: warp 0 = TMA producer, warp 1 = TMEM allocator
// and MMA issuer (one elected thread), warps 2-5 = epilogue (one TMEM lane
// quadrant each).  Two blocks fit on an SM, so one block's epilogue overlaps
// the other's main loop.  Every mbarrier wait is bounded; a wait that runs out
// sets the device error word and the block drains and frees its TMEM.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

#include <algorithm>

#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

constexpr int kBM = 128;          // weight rows per tile (UMMA M)
constexpr int kBK = 64;           // bf16 per 128-byte swizzled row
constexpr int kTcThreads = 192;

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(1) << 16;                 // leading byte offset (unused with swizzle) = 16 B
  d |= static_cast<uint64_t>(1024 >> 4) << 32;         // stride between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                 // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                 // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- two-SM forms (cta_group::2): the two blocks of a cluster of 2 work on ONE tile of 256 weight rows.  Each
// block holds its own 128 weight rows (A) and half of the token rows (B); the tensor cores of both SMs read both
// halves, so a block stages 32 KB per k-step instead of 48 KB.  The MMA is issued by the cluster's block 0.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t bar_cluster) {
  // bar_cluster: shared::cluster address of block 0's barrier (the peer's copy completes bytes there too)
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {      // arrives on `bar` in both blocks of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(static_cast<uint16_t>(3))
               : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ uint32_t tc_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t tc_map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

// thread-block cluster helpers (split-K over a cluster: the blocks of one tile add their accumulators through
// the leader's shared memory)
__device__ __forceinline__ void tc_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t tc_leader_smem(uint32_t addr) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(0u));
  return r;
}
__device__ __forceinline__ void tc_st_cluster(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tc_ld_shared(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// HILO: the activations arrive as two bf16 operands, x = hi + lo (lo = the rounding error of hi), both
// multiplied into the same accumulator: the product carries the activations to about 16 mantissa bits,
// which is what keeps few-sequence decode on the tensor cores as accurate as the fp32-activation path.
template <int BN, int STAGES, int EPI, bool HILO>
__global__ void __launch_bounds__(kTcThreads) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                             const __grid_constant__ CUtensorMap map_x,
                                                             const __grid_constant__ CUtensorMap map_xlo,
                                                             const GemmTcArgs a) {
  constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = BN * kBK * 2,
                     kStageBytes = kABytes + (HILO ? 2 : 1) * kBBytes;
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                              (static_cast<uint32_t>(kBM >> 4) << 24);
  extern __shared__ unsigned char tc_smem_raw[];
  const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;   // swizzled tiles need 1024-byte alignment
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t acc_bar = bar0 + 8u * (2 * STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2 * STAGES + 1; ++s) mbar_init(bar0 + 8u * s, 1);
    mbar_fence_init();
    failed = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(static_cast<uint32_t>(BN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_slot;

  pdl_wait();                      // the activations come from the predecessor kernel
  pdl_launch_dependents();

  // Token tiles vary fastest: the blocks that run together share one weight tile (read from HBM once,
  // then served by L2) and walk the activations, which stay L2-resident.
  const int n0 = blockIdx.y * kBM;           // first weight row of the tile
  const int m0 = blockIdx.x * BN;            // first token row of the tile
  // split-K: block z covers k-blocks [kb0, kb0 + nk) and leaves a partial sum
  const int nk_total = a.K / kBK;
  const int per_z = (nk_total + gridDim.z - 1) / gridDim.z;
  const int kb0 = blockIdx.z * per_z;
  const int nk = max(0, min(per_z, nk_total - kb0));
  // Split-K without a trip through global memory (few tiles, fused epilogue): the gridDim.z blocks of a tile
  // form one cluster along z; block z accumulates its K range, the others hand their accumulators to block 0
  // through its shared memory, and block 0 runs the epilogue.  (With a.partial the planes go to global memory.)
  const uint32_t cs = (!a.partial && gridDim.z > 1) ? gridDim.z : 1u;
  const uint32_t crank = cs > 1 ? blockIdx.z : 0u;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < nk; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !mbar_wait(empty_bar(s), ((kb / STAGES) - 1) & 1)) {
          atomicOr(&failed, 1u);
          break;
        }
        mbar_expect_tx(full_bar(s), kStageBytes);
        const uint32_t dst = smem_base + s * kStageBytes;
        tma_load_2d(dst, &map_w, (kb0 + kb) * kBK, n0, full_bar(s));
        tma_load_2d(dst + kABytes, &map_x, (kb0 + kb) * kBK, a.x_row0 + m0, full_bar(s));
        if (HILO) tma_load_2d(dst + kABytes + kBBytes, &map_xlo, (kb0 + kb) * kBK, a.x_row0 + m0, full_bar(s));
      }
    }
    __syncwarp();
    if (cs > 1) {                                    // the two cluster barriers of the epilogue warps
      tc_cluster_sync();
      tc_cluster_sync();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < nk; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(full_bar(s), (kb / STAGES) & 1)) {
          atomicOr(&failed, 1u);
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_base + s * kStageBytes;
        const uint64_t adesc = smem_desc_sw128(sa), bdesc = smem_desc_sw128(sa + kABytes);
        const uint64_t bdesc_lo = smem_desc_sw128(sa + kABytes + kBBytes);
#pragma unroll
        for (int k4 = 0; k4 < kBK / 16; ++k4) {    // UMMA K = 16 bf16 = 32 bytes = 2 descriptor units
          tc_mma_bf16(tmem_acc, adesc + 2 * k4, bdesc + 2 * k4, kIdesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          if (HILO) tc_mma_bf16(tmem_acc, adesc + 2 * k4, bdesc_lo + 2 * k4, kIdesc, 1u);
        }
        tc_commit(empty_bar(s));                   // frees the stage once these MMAs have read it
      }
      tc_commit(acc_bar);                          // accumulator complete
    }
    __syncwarp();
    if (cs > 1) {
      tc_cluster_sync();
      tc_cluster_sync();
    }
  } else {
    const int quad = warp & 3;                     // TMEM lanes this warp may read
    const int n = n0 + quad * 32 + lane;
    const bool n_ok = n < a.N;
    // per-feature constants of the epilogue
    int region = 0, nn = 0, head = 0, j = 0;
    float bias = 0.f;
    if (EPI == kEpiInProj) {
      if (n_ok) {
        if (n < 3 * a.dl) {
          region = n / a.dl;
          nn = n - region * a.dl;
          head = nn / a.d_head;
          j = nn % a.d_head;
        } else {
          region = 3;
          nn = n - 3 * a.dl;
          bias = a.b_ff[nn];
        }
      }
    } else if (n_ok) {
      bias = a.bias[n];
    }
    // decode (row m = sequence b0 + m, every row at the same position): the rotation factors, and per
    // 32-row chunk the left-pad limit and cache page of the sequence this LANE's index names, are fetched
    // now, while the main loop runs; the store loop gets them by shuffle instead of dependent loads
    constexpr int kChunks = BN / 32;
    const bool dec = EPI == kEpiInProj && a.rows.Tc == 1;
    int dpos = 0, dpad[kChunks], dpage[kChunks];
    float2 dsc = make_float2(0.f, 1.f);
    const bool rotary = EPI == kEpiInProj && n_ok && region < 2 && j < a.rot;
    const bool kv_lane = EPI == kEpiInProj && n_ok && (region == 1 || region == 2);
    const bool kv_warp = __any_sync(0xffffffffu, kv_lane);
    if (dec) {
      dpos = a.rows.pos0_dev ? *a.rows.pos0_dev : a.rows.pos0_host;
      if (rotary) dsc = a.sincos[static_cast<size_t>(dpos) * (a.rot >> 1) + (j >> 1)];
      const int slot = (dpos / kPageTokens) % a.kv.ring_pages;
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        const int m = m0 + c * 32 + lane;
        const bool have = kv_warp && m < a.M;
        dpad[c] = have ? a.kv.pad[a.rows.b0 + m] : 0x7fffffff;
        dpage[c] = have ? a.kv.page_table[static_cast<size_t>(a.rows.b0 + m) * a.kv.ring_pages + slot] : 0;
      }
    }
    const bool ok = nk > 0 && mbar_wait(acc_bar, 0);
    if (!ok && nk > 0) atomicOr(&failed, 1u);
    tc_fence_after();
    auto do_chunk = [&](int cc, uint32_t (&r)[32]) {
        const int c0 = cc * 32;
        if (dec) {
          const int pos = dpos;
          const bool any_rot = __any_sync(0xffffffffu, rotary);
          if (any_rot) {
            const float sx = (j & 1) ? dsc.x : -dsc.x;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float v = __uint_as_float(r[i]);
              const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
              if (rotary) r[i] = __float_as_uint(fmaf(v, dsc.y, partner * sx));
            }
          }
          const int valid = min(32, a.M - (m0 + c0));
          if (n_ok && valid > 0 && region == 3) {
            __nv_bfloat16* dst = a.act_out + static_cast<size_t>(m0 + c0) * (a.dl + a.ffl) + a.dl + nn;
            const size_t ld = static_cast<size_t>(a.dl + a.ffl);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (i < valid) {
                const float g = gelu_tanh(__uint_as_float(r[i]) + bias);
                const __nv_bfloat16 hi = __float2bfloat16_rn(g);
                dst[i * ld] = hi;
                if (a.act_lo)
                  a.act_lo[static_cast<size_t>(m0 + c0 + i) * ld + a.dl + nn] = __float2bfloat16_rn(g - __bfloat162float(hi));
              }
            }
          } else if (n_ok && valid > 0 && region == 0) {
            float* dst = a.q_out + static_cast<size_t>(m0 + c0) * a.dl + nn;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < valid) dst[static_cast<size_t>(i) * a.dl] = __uint_as_float(r[i]);
            if (a.q_bf16) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < valid)
                  a.q_bf16[static_cast<size_t>(m0 + c0 + i) * a.dl + nn] = __float2bfloat16_rn(__uint_as_float(r[i]));
            }
          }
          if (kv_warp) {                               // warp-uniform: the shuffles below need every lane
            __nv_bfloat16* pool = (region == 1 ? a.kv.kpool : a.kv.vpool) +
                                  (static_cast<size_t>(head) * kPageTokens + (pos % kPageTokens)) * a.d_head + j;
            const size_t page_stride = static_cast<size_t>(a.heads) * kPageTokens * a.d_head;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int padv = __shfl_sync(0xffffffffu, dpad[cc], i);
              const int page = __shfl_sync(0xffffffffu, dpage[cc], i);
              if (kv_lane && i < valid && pos >= padv)
                pool[page * page_stride] = __float2bfloat16_rn(__uint_as_float(r[i]));
            }
          }
          return;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int m = m0 + c0 + i;
          const float v = __uint_as_float(r[i]);
          const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
          if (m >= a.M || !n_ok) continue;
          if (EPI == kEpiInProj) {
            const int seq = a.rows.b0 + m / a.rows.Tc;
            const int pos = (a.rows.pos0_dev ? *a.rows.pos0_dev : a.rows.pos0_host) + m % a.rows.Tc;
            if (region < 3) {
              float y = v;
              if (region < 2 && j < a.rot) {
                const float2 sc = a.sincos[static_cast<size_t>(pos) * (a.rot >> 1) + (j >> 1)];
                y = (j & 1) ? (v * sc.y + partner * sc.x) : (v * sc.y - partner * sc.x);
              }
              if (region == 0) {
                a.q_out[static_cast<size_t>(m) * a.dl + nn] = y;
                if (a.q_bf16) a.q_bf16[static_cast<size_t>(m) * a.dl + nn] = __float2bfloat16_rn(y);
              } else if (pos >= a.kv.pad[seq]) {
                __nv_bfloat16* pool = region == 1 ? a.kv.kpool : a.kv.vpool;
                const size_t off = kv_offset(a.kv.page_table + static_cast<size_t>(seq) * a.kv.ring_pages,
                                             a.kv.ring_pages, a.heads, a.d_head, head, pos);
                pool[off + j] = __float2bfloat16_rn(y);
              }
            } else {
              a.act_out[static_cast<size_t>(m) * (a.dl + a.ffl) + a.dl + nn] =
                  __float2bfloat16_rn(gelu_tanh(v + bias));
            }
          } else if (a.partial) {
            // split-K: raw partial sum; bias / residual are added by the reduction kernel
            a.partial[(static_cast<size_t>(blockIdx.z) * a.M + m) * a.N + n] = v;
          } else if (EPI == kEpiOut) {
            float y = v + bias;
            if (a.residual) y += a.residual[static_cast<size_t>(m) * a.N + n];
            a.out[static_cast<size_t>(m) * a.N + n] = y;
          } else {
            a.out[static_cast<size_t>(m) * a.ld_out + n] = v + bias;
          }
        }
    };
    if (cs > 1) {
      // every block of the cluster: accumulator -> registers; blocks 1.. -> block 0's shared memory; block 0
      // adds them in block order and finishes the tile.  The first barrier says "all accumulators are
      // complete", i.e. no block's operand ring is in use any more: block 0's ring is the landing zone,
      // laid out [source block - 1][token column][weight row] so that a warp's stores are conflict-free.
      static_assert(BN > 64 || 3u * BN * kBM * 4u <= STAGES * kStageBytes, "landing zone exceeds the operand ring");
      uint32_t racc[kChunks][32];
#pragma unroll
      for (int cc = 0; cc < kChunks; ++cc) {
        if (ok) {
          tmem_ld32(tmem_acc + (static_cast<uint32_t>(quad * 32) << 16) + cc * 32, racc[cc]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) racc[cc][i] = 0u;   // an empty K range (or a failed wait) adds nothing
        }
      }
      const uint32_t row4 = static_cast<uint32_t>(quad * 32 + lane) * 4u;
      tc_cluster_sync();
      if (crank != 0) {
        const uint32_t dst = tc_leader_smem(smem_base) + (crank - 1u) * (BN * kBM * 4u) + row4;
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc)
#pragma unroll
          for (int i = 0; i < 32; ++i) tc_st_cluster(dst + static_cast<uint32_t>(cc * 32 + i) * (kBM * 4u), racc[cc][i]);
      }
      tc_cluster_sync();
      if (crank == 0) {
        for (uint32_t p = 0; p + 1 < cs; ++p) {
          const uint32_t src = smem_base + p * (BN * kBM * 4u) + row4;
#pragma unroll
          for (int cc = 0; cc < kChunks; ++cc)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              racc[cc][i] = __float_as_uint(__uint_as_float(racc[cc][i]) +
                                            __uint_as_float(tc_ld_shared(src + static_cast<uint32_t>(cc * 32 + i) * (kBM * 4u))));
        }
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc) do_chunk(cc, racc[cc]);
      }
    } else if (ok || (nk == 0 && a.partial)) {
#pragma unroll
      for (int cc = 0; cc < kChunks; ++cc) {
        uint32_t r[32];
        if (ok) {
          tmem_ld32(tmem_acc + (static_cast<uint32_t>(quad * 32) << 16) + cc * 32, r);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;      // an empty K range contributes zeros
        }
        do_chunk(cc, r);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc),
                 "r"(static_cast<uint32_t>(BN))
                 : "memory");
  }
  if (threadIdx.x == 0 && failed && a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
}

// ---------------------------------------------------------------------------------------------------
// Persistent variant for many token rows (prefill / eval): one block per SM walks the tile list, a
// tile is 128 weight rows x 256 token rows (UMMA 128 x 256 x 16), and the accumulator is double
// buffered in tensor memory (2 x 256 columns) so that the epilogue of tile i runs while the tensor
// core works on tile i + 1.  Warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-9 = epilogue
// (lane quadrant = warp % 4, column half = (warp - 2) / 4).  Token tiles vary fastest in the tile
// list, so the blocks that run together share weight tiles through L2.
//
// PAIR: the blocks come as clusters of 2 and a tile is 256 weight rows x 256 token rows, computed by
// tcgen05.mma.cta_group::2 (UMMA 256 x 256 x 16).  Block r of the pair holds weight rows [128 r, 128 r + 128) and
// token rows [128 r, 128 r + 128) of the tile in its shared memory and the accumulator of its own 128 weight
// rows in its tensor memory, so the epilogue is the same as without PAIR.  Both producers complete their bytes
// on block 0's "full" barrier; block 0 issues the MMAs and its commits arrive on the "empty" and "accumulator
// full" barriers of both blocks; the epilogue warps of both blocks arrive on block 0's "accumulator empty".
constexpr int kPBN = 256;
constexpr int kPStages = 4;
constexpr int kPEpiWarps = 8;
constexpr int kPThreads = 64 + 32 * kPEpiWarps;
constexpr int kPMaxStages = 6;
template <int EPI, bool PAIR>
struct PersistCfg {
  static constexpr int kStages = PAIR ? (EPI == kEpiLogitsCE ? 5 : 6) : kPStages;
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = (PAIR ? kPBN / 2 : kPBN) * kBK * 2;     // per block
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr int kSmem = kStages * kStageBytes + 1024 + (EPI == kEpiLogitsCE ? kPEpiWarps * 4096 : 0);
};

__device__ __forceinline__ void mbar_arrive_cta(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// tanh-form GELU written as x * sigmoid(2u), u = sqrt(2/pi) (x + 0.044715 x^3)
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float u2 = 1.5957691216057308f * x * fmaf(0.044715f * x, x, 1.0f);
  return __fdividef(x, 1.0f + __expf(-u2));
}

template <int EPI, bool PAIR>
__global__ void __launch_bounds__(kPThreads, 1) gemm_tc_persist_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                       const __grid_constant__ CUtensorMap map_x,
                                                                       const GemmTcArgs a) {
  using Cfg = PersistCfg<EPI, PAIR>;
  constexpr int kStages = Cfg::kStages;
  constexpr uint32_t kABytes = Cfg::kABytes, kStageBytes = Cfg::kStageBytes;
  constexpr int kTileN = PAIR ? 2 * kBM : kBM;       // weight rows per tile (of the pair)
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kPBN >> 3) << 17) |
                              (static_cast<uint32_t>(kTileN >> 4) << 24);
  extern __shared__ unsigned char tc_smem_raw[];
  const uint32_t smem_base = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
  __shared__ __align__(8) uint64_t bars[2 * kPMaxStages + 4];
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = PAIR ? tc_cluster_rank() : 0u;              // block of the pair
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto acc_full = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };
  volatile uint32_t* failed_v = &failed;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2 * kStages + 2; ++s) mbar_init(bar0 + 8u * s, 1);
    mbar_init(acc_empty(0), PAIR ? 2 * kPEpiWarps : kPEpiWarps);      // PAIR: the epilogue warps of both blocks
    mbar_init(acc_empty(1), PAIR ? 2 * kPEpiWarps : kPEpiWarps);
    mbar_fence_init();
    failed = 0;
  }
  if (warp == 1) {
    if (PAIR) {
      // the same warp of both blocks takes part; the columns are allocated in both
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                   "r"(512u)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                   "r"(512u)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  if (PAIR) tc_cluster_sync();                       // both blocks' barriers exist before either is signalled
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_slot;

  pdl_wait();
  pdl_launch_dependents();

  const int m_tiles = (a.M + kPBN - 1) / kPBN;
  const int n_tiles = (a.N + kTileN - 1) / kTileN;
  const int total = m_tiles * n_tiles;
  const int nk = a.K / kBK;
  const int tile_first = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int tile_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (int t = tile_first; t < total && alive; t += tile_step) {
        const int n0 = (t / m_tiles) * kTileN + static_cast<int>(crank) * kBM, m0 = (t % m_tiles) * kPBN;
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % kStages;
          if (it >= kStages && !mbar_wait(empty_bar(s), ((it / kStages) - 1) & 1)) {
            atomicOr(&failed, 1u);
            alive = false;
            break;
          }
          const uint32_t dst = smem_base + s * kStageBytes;
          if (PAIR) {
            // block 0's barrier counts the bytes of both blocks; the activation box has 128 token rows
            if (crank == 0) mbar_expect_tx(full_bar(s), 2 * kStageBytes);
            const uint32_t fb = tc_map_to_rank(full_bar(s), 0);
            tma_load_2d_pair(dst, &map_w, kb * kBK, n0, fb);
            tma_load_2d_pair(dst + kABytes, &map_x, kb * kBK, a.x_row0 + m0 + static_cast<int>(crank) * (kPBN / 2), fb);
          } else {
            mbar_expect_tx(full_bar(s), kStageBytes);
            tma_load_2d(dst, &map_w, kb * kBK, n0, full_bar(s));
            tma_load_2d(dst + kABytes, &map_x, kb * kBK, a.x_row0 + m0, full_bar(s));
            tma_load_2d(dst + kABytes + (kPBN / 2) * kBK * 2, &map_x, kb * kBK, a.x_row0 + m0 + kPBN / 2, full_bar(s));
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && crank == 0) {
      uint32_t it = 0;
      bool alive = true;
      int i = 0;
      for (int t = tile_first; t < total && alive; t += tile_step, ++i) {
        const int b = i & 1;
        if (i >= 2 && !mbar_wait(acc_empty(b), ((i >> 1) - 1) & 1)) {
          atomicOr(&failed, 1u);
          break;
        }
        tc_fence_after();
        const uint32_t d = tmem_acc + static_cast<uint32_t>(b * kPBN);
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(full_bar(s), (it / kStages) & 1)) {
            atomicOr(&failed, 1u);
            alive = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + s * kStageBytes;
          const uint64_t adesc = smem_desc_sw128(sa), bdesc = smem_desc_sw128(sa + kABytes);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4) {
            if (PAIR) tc_mma_bf16_pair(d, adesc + 2 * k4, bdesc + 2 * k4, kIdesc, (kb > 0 || k4 > 0) ? 1u : 0u);
            else tc_mma_bf16(d, adesc + 2 * k4, bdesc + 2 * k4, kIdesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          }
          if (PAIR) tc_commit_pair(empty_bar(s));
          else tc_commit(empty_bar(s));
        }
        if (alive) {
          if (PAIR) tc_commit_pair(acc_full(b));
          else tc_commit(acc_full(b));
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int Tc = a.rows.Tc;
    int pos0 = 0;
    if (EPI == kEpiInProj) pos0 = a.rows.pos0_dev ? *a.rows.pos0_dev : a.rows.pos0_host;
    int i = 0;
    for (int t = tile_first; t < total; t += tile_step, ++i) {
      const int b = i & 1;
      if (*failed_v || !mbar_wait(acc_full(b), (i >> 1) & 1)) {
        atomicOr(&failed, 1u);
        break;
      }
      tc_fence_after();
      const int n0 = (t / m_tiles) * kTileN + static_cast<int>(crank) * kBM,
                m0 = (t % m_tiles) * kPBN + half * (kPBN / 2);
      const int n = n0 + quad * 32 + lane;
      const bool n_ok = n < a.N;
      int region = 0, nn = 0, head = 0, j = 0;
      float bias = 0.f;
      if (EPI == kEpiInProj) {
        if (n_ok) {
          if (n < 3 * a.dl) {
            region = n / a.dl;
            nn = n - region * a.dl;
            head = nn / a.d_head;
            j = nn - head * a.d_head;
          } else {
            region = 3;
            nn = n - 3 * a.dl;
            bias = a.b_ff[nn];
          }
        }
      } else if (n_ok) {
        bias = a.bias[n];
      }
      // (sequence, position) of the chunk's first row, advanced chunk by chunk (uniform over the warp)
      int seq = 0, tin = 0;
      if (EPI == kEpiInProj) {
        seq = a.rows.b0 + m0 / Tc;
        tin = m0 % Tc;
      }
      const bool rotary = EPI == kEpiInProj && n_ok && region < 2 && j < a.rot;
      const bool any_rot = __any_sync(0xffffffffu, rotary);
      const float sgn = (j & 1) ? 1.f : -1.f;
      const int half_rot = a.rot >> 1;
      const size_t ld_act = static_cast<size_t>(a.dl + a.ffl);
      const uint32_t tbase = tmem_acc + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(b * kPBN + half * (kPBN / 2));
#pragma unroll 1
      for (int c0 = 0; c0 < kPBN / 2; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tbase + c0, r);
        if (c0 + 32 == kPBN / 2) {
          // this warp has read its part of the accumulator: hand the buffer back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) mbar_arrive_cluster(tc_map_to_rank(acc_empty(b), 0));
            else mbar_arrive_cta(acc_empty(b));
          }
        }
        const int mc = m0 + c0;                          // first token row of the chunk
        const int valid = min(32, a.M - mc);             // rows of the chunk that exist
        if (EPI == kEpiInProj) {
          if (valid == 32 && tin + 32 <= Tc) {
            // all 32 rows exist and belong to one sequence: positions pos .. pos + 31
            const int pos = pos0 + tin;
            if (any_rot) {
              const float2* sc = a.sincos + static_cast<size_t>(pos) * half_rot + (rotary ? (j >> 1) : 0);
#pragma unroll
              for (int q = 0; q < 32; ++q) {
                const float v = __uint_as_float(r[q]);
                const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
                if (rotary) {
                  const float2 t = sc[q * half_rot];
                  r[q] = __float_as_uint(fmaf(v, t.y, (sgn * partner) * t.x));
                }
              }
            }
            if (!n_ok) {
            } else if (region == 3) {
              __nv_bfloat16* dst = a.act_out + static_cast<size_t>(mc) * ld_act + a.dl + nn;
#pragma unroll
              for (int q = 0; q < 32; ++q)
                dst[q * ld_act] = __float2bfloat16_rn(gelu_tanh_fast(__uint_as_float(r[q]) + bias));
            } else if (region == 0) {
              if (a.q_bf16) {
                __nv_bfloat16* dst = a.q_bf16 + static_cast<size_t>(mc) * a.dl + nn;
#pragma unroll
                for (int q = 0; q < 32; ++q) dst[static_cast<size_t>(q) * a.dl] = __float2bfloat16_rn(__uint_as_float(r[q]));
              } else {
                float* dst = a.q_out + static_cast<size_t>(mc) * a.dl + nn;
#pragma unroll
                for (int q = 0; q < 32; ++q) dst[static_cast<size_t>(q) * a.dl] = __uint_as_float(r[q]);
              }
            } else {
              __nv_bfloat16* pool = (region == 1 ? a.kv.kpool : a.kv.vpool) + j;
              const int32_t* trow = a.kv.page_table + static_cast<size_t>(seq) * a.kv.ring_pages;
              const int padv = a.kv.pad[seq];
              const size_t slab = static_cast<size_t>(kPageTokens) * a.d_head;
              int pg = pos / kPageTokens, off = pos % kPageTokens;
              __nv_bfloat16* dst = pool + (static_cast<size_t>(trow[pg % a.kv.ring_pages]) * a.heads + head) * slab;
#pragma unroll
              for (int q = 0; q < 32; ++q) {
                if (off == kPageTokens) {
                  off = 0;
                  ++pg;
                  dst = pool + (static_cast<size_t>(trow[pg % a.kv.ring_pages]) * a.heads + head) * slab;
                }
                if (pos + q >= padv) dst[off * a.d_head] = __float2bfloat16_rn(__uint_as_float(r[q]));
                ++off;
              }
            }
            tin += 32;
            if (tin == Tc) {
              tin = 0;
              ++seq;
            }
          } else {
            // ragged chunk (end of the rows, or a sequence boundary inside it): element by element
#pragma unroll
            for (int q = 0; q < 32; ++q) {
              const int m = mc + q;
              const float v = __uint_as_float(r[q]);
              const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
              const int pos = pos0 + tin;
              if (m < a.M && n_ok) {
                if (region < 3) {
                  float y = v;
                  if (rotary) {
                    const float2 t = a.sincos[static_cast<size_t>(pos) * half_rot + (j >> 1)];
                    y = fmaf(v, t.y, (sgn * partner) * t.x);
                  }
                  if (region == 0) {
                    if (a.q_bf16)
                      a.q_bf16[static_cast<size_t>(m) * a.dl + nn] = __float2bfloat16_rn(y);
                    else
                      a.q_out[static_cast<size_t>(m) * a.dl + nn] = y;
                  } else if (pos >= a.kv.pad[seq]) {
                    __nv_bfloat16* pool = region == 1 ? a.kv.kpool : a.kv.vpool;
                    const size_t o = kv_offset(a.kv.page_table + static_cast<size_t>(seq) * a.kv.ring_pages,
                                               a.kv.ring_pages, a.heads, a.d_head, head, pos);
                    pool[o + j] = __float2bfloat16_rn(y);
                  }
                } else {
                  a.act_out[static_cast<size_t>(m) * ld_act + a.dl + nn] = __float2bfloat16_rn(gelu_tanh_fast(v + bias));
                }
              }
              if (++tin == Tc) {
                tin = 0;
                ++seq;
              }
            }
          }
        } else if (EPI == kEpiLogitsCE) {
          // Cross-entropy without the logits.  The accumulator arrives with lane = vocabulary entry and q = token
          // row; a reduction over the vocabulary would cross lanes, so the warp's 32 x 32 block is turned through
          // shared memory (XOR-swizzled, conflict-free both ways): afterwards lane = token row, and the 32 logits
          // of the group are walked in registers -- max, then sum of exp(l - max), and the target's logit if its
          // id falls into the group (layers.py:575-585 per group; ce_combine_kernel merges the groups).
          // (a pair's second block may hold a tile that lies entirely beyond the last weight row: no groups there)
          if (valid > 0 && n0 < a.N) {
            float* tsm = reinterpret_cast<float*>(tc_smem_raw + (smem_base - smem_u32(tc_smem_raw)) +
                                                  kStages * kStageBytes) + (warp - 2) * 1024;
#pragma unroll
            for (int q = 0; q < 32; ++q) tsm[q * 32 + (lane ^ q)] = n_ok ? __uint_as_float(r[q]) + bias : -INFINITY;
            __syncwarp();
            const float* mine = tsm + lane * 32;
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, mine[i ^ lane]);
            float sum = 0.f;
            if (mx > -INFINITY) {                                  // -inf only for a group past the end of the vocabulary
#pragma unroll
              for (int i = 0; i < 32; ++i) sum += __expf(mine[i ^ lane] - mx);
            }
            if (lane < valid) {
              const int crow = a.x_row0 + mc + lane;               // chunk row of this lane's token
              const int sq = a.rows.b0 + crow / Tc, tp = a.rows.pos0_host + crow % Tc;
              const uint32_t tgt = a.ce_targets[static_cast<size_t>(sq) * a.ce_T + tp];
              const uint32_t off = tgt - static_cast<uint32_t>(a.ce_vocab_start + n0 + quad * 32);
              if (off < 32u && n0 + quad * 32 + static_cast<int>(off) < a.N) {
                a.ce_tlogit[mc + lane] = mine[off ^ lane];
                a.ce_hit[mc + lane] = 1;
              }
              const size_t g = (static_cast<size_t>(n0 / kBM) * 4 + quad) * a.ce_ld + mc + lane;
              a.ce_gmax[g] = mx;
              a.ce_gsum[g] = sum;
            }
            __syncwarp();                                          // the next chunk overwrites the block
          }
        } else if (n_ok && valid > 0) {
          const size_t ldo = EPI == kEpiOut ? static_cast<size_t>(a.N) : static_cast<size_t>(a.ld_out);
          float* dst = a.out + static_cast<size_t>(mc) * ldo + n;
          if (EPI == kEpiOut && a.residual) {
            // all residual loads first (the output may alias the residual, which pins the order otherwise)
            const float* res = a.residual + static_cast<size_t>(mc) * ldo + n;
#pragma unroll
            for (int q = 0; q < 32; ++q)
              if (q < valid) r[q] = __float_as_uint(__uint_as_float(r[q]) + res[q * ldo]);
          }
#pragma unroll
          for (int q = 0; q < 32; ++q)
            if (q < valid) dst[q * ldo] = __uint_as_float(r[q]) + bias;
        }
      }
    }
  }
  tc_fence_before();
  if (PAIR) tc_cluster_sync();                       // neither block leaves, or frees, while the other may still signal it
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(512u) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(512u) : "memory");
  }
  if (threadIdx.x == 0 && failed && a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
}

// LayerNorm of fp32 rows into bf16 (the GEMM's activation operand), layers.py:17-36.
__global__ void __launch_bounds__(256) ln_rows_kernel(const float* __restrict__ x, const float* __restrict__ scale,
                                                      const float* __restrict__ offset,
                                                      __nv_bfloat16* __restrict__ out, __nv_bfloat16* out_lo, int d) {
  __shared__ float red[8];
  pdl_wait();
  pdl_launch_dependents();
  const float* xr = x + static_cast<size_t>(blockIdx.x) * d;
  __nv_bfloat16* o = out + static_cast<size_t>(blockIdx.x) * d;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto block_sum = [&](float v) {
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i];
    __syncthreads();
    return t;
  };
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += 256) s += xr[i];
  const float mu = block_sum(s) / static_cast<float>(d);
  float v = 0.f;
  for (int i = threadIdx.x; i < d; i += 256) {
    const float t = xr[i] - mu;
    v = fmaf(t, t, v);
  }
  const float rstd = 1.0f / sqrtf(block_sum(v) / static_cast<float>(d) + 1e-5f);
  for (int i = threadIdx.x; i < d; i += 256) {
    const float y = fmaf(scale[i] * rstd, xr[i] - mu, offset[i]);
    const __nv_bfloat16 hi = __float2bfloat16_rn(y);
    o[i] = hi;
    if (out_lo) out_lo[static_cast<size_t>(blockIdx.x) * d + i] = __float2bfloat16_rn(y - __bfloat162float(hi));
  }
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  return fn;
}

template <int BN, int STAGES, int EPI, bool HILO = false>
cudaError_t launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const GemmTcArgs& a, cudaStream_t s, bool pdl,
                      const CUtensorMap* mxlo = nullptr) {
  constexpr int smem = STAGES * (kBM * kBK * 2 + (HILO ? 2 : 1) * BN * kBK * 2) + 1024;
  static DeviceOnce once;
  {
    cudaError_t e = once.run([&] { return cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, EPI, HILO>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  // cluster split-K (no global partial planes): 2 or 4 blocks per tile, token tiles of at most 64 rows
  const int ck = (!a.partial && BN <= 64 && (a.cluster_k == 2 || a.cluster_k == 4)) ? a.cluster_k : 1;
  cfg.gridDim = dim3((a.M + BN - 1) / BN, (a.N + kBM - 1) / kBM, a.partial ? a.ksplit : ck);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (ck > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = ck;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, STAGES, EPI, HILO>, mw, mx, mxlo ? *mxlo : mx, a);
}

template <int EPI>
cudaError_t launch_tc_persist(const CUtensorMap& mw, const CUtensorMap& mx, const GemmTcArgs& a, cudaStream_t s) {
  // the cross-entropy epilogue turns each epilogue warp's 32 x 32 block through 4 KB of shared memory
  constexpr int smem = PersistCfg<EPI, false>::kSmem, smem_pair = PersistCfg<EPI, true>::kSmem;
  static DeviceOnce once;
  static int sms_of[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  e = once.run([&] {
    cudaError_t e2 = cudaFuncSetAttribute(gemm_tc_persist_kernel<EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e2 != cudaSuccess) return e2;
    e2 = cudaFuncSetAttribute(gemm_tc_persist_kernel<EPI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pair);
    if (e2 != cudaSuccess) return e2;
    return cudaDeviceGetAttribute(&sms_of[dev], cudaDevAttrMultiProcessorCount, dev);
  });
  if (e != cudaSuccess) return e;
  const int m_tiles = (a.M + kPBN - 1) / kPBN;
  if (a.pair && a.N >= 2 * kBM && sms_of[dev] >= 2) {
    // clusters of 2 blocks, one 256 x 256 tile per pair at a time
    const int total = m_tiles * ((a.N + 2 * kBM - 1) / (2 * kBM));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * std::min(total, sms_of[dev] / 2)));
    cfg.blockDim = dim3(kPThreads);
    cfg.dynamicSmemBytes = smem_pair;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_persist_kernel<EPI, true>, mw, mx, a);
  }
  const int total = m_tiles * ((a.N + kBM - 1) / kBM);
  gemm_tc_persist_kernel<EPI, false><<<std::min(total, sms_of[dev]), kPThreads, smem, s>>>(mw, mx, a);
  return cudaGetLastError();
}

}  // namespace

int gemm_tc_token_tile() { return 128; }
// Batched decode streams each weight tile once, and a block keeps only its TMA ring in flight: with fewer tiles
// than the GPU holds blocks (two per SM), K is split over a cluster of 2 or 4 blocks per tile so that the
// bytes in flight -- and with them the HBM rate -- do not fall with the tile count (tensor-parallel slices).
int gemm_tc_decode_cluster_k(int weight_rows, int M, int K) {
  if (M > 64) return 1;
  const int tiles = (weight_rows + kBM - 1) / kBM;      // one token tile
  int ck = 1;
  while (ck < 4 && tiles * ck * 2 <= 296 && K / kBK >= ck * 2 * 2) ck *= 2;
  return ck;
}

int gemm_tc_token_tile_for(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }
int gemm_tc_wide_token_tile() { return kPBN / 2; }     // rows of the activation box: a tile takes two of them

cudaError_t launch_gemm_tc_wide(GemvEpilogue epi, const void* map_w, const void* map_x, const GemmTcArgs& a,
                                cudaStream_t s) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.K % kBK || a.partial) return cudaErrorInvalidValue;
  const CUtensorMap& mw = *static_cast<const CUtensorMap*>(map_w);
  const CUtensorMap& mx = *static_cast<const CUtensorMap*>(map_x);
  switch (epi) {
    case kEpiInProj: return launch_tc_persist<kEpiInProj>(mw, mx, a, s);
    case kEpiOut: return launch_tc_persist<kEpiOut>(mw, mx, a, s);
    case kEpiLogitsCE:
      if (!a.ce_gmax || !a.ce_gsum || !a.ce_tlogit || !a.ce_hit || !a.ce_targets || a.ce_ld < a.M) return cudaErrorInvalidValue;
      return launch_tc_persist<kEpiLogitsCE>(mw, mx, a, s);
    default: return launch_tc_persist<kEpiLogits>(mw, mx, a, s);
  }
}

cudaError_t make_tensor_map_bf16(void* map_out, const void* base, int64_t rows, int64_t K, int box_rows) {
  PFN_cuTensorMapEncodeTiled_v12000 fn = encode_fn();
  if (!fn) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (K * 2) % 16 || box_rows > 256) return cudaErrorInvalidValue;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(static_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t launch_gemm_tc(GemvEpilogue epi, const void* map_w, const void* map_x, const GemmTcArgs& a,
                           cudaStream_t s, bool pdl, const void* map_x_lo) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.K % kBK) return cudaErrorInvalidValue;
  const CUtensorMap& mw = *static_cast<const CUtensorMap*>(map_w);
  const CUtensorMap& mx = *static_cast<const CUtensorMap*>(map_x);
  if (map_x_lo) {
    // hi + lo activations: token tiles of 32 or 64 rows only (few-sequence decode)
    const CUtensorMap* ml = static_cast<const CUtensorMap*>(map_x_lo);
    const int bnl = gemm_tc_token_tile_for(a.M);
    if (bnl == 32) {
      switch (epi) {
        case kEpiInProj: return launch_tc<32, 4, kEpiInProj, true>(mw, mx, a, s, pdl, ml);
        case kEpiOut: return launch_tc<32, 4, kEpiOut, true>(mw, mx, a, s, pdl, ml);
        default: return launch_tc<32, 4, kEpiLogits, true>(mw, mx, a, s, pdl, ml);
      }
    }
    if (bnl == 64) {
      switch (epi) {
        case kEpiInProj: return launch_tc<64, 3, kEpiInProj, true>(mw, mx, a, s, pdl, ml);
        case kEpiOut: return launch_tc<64, 3, kEpiOut, true>(mw, mx, a, s, pdl, ml);
        default: return launch_tc<64, 3, kEpiLogits, true>(mw, mx, a, s, pdl, ml);
      }
    }
    return cudaErrorInvalidValue;
  }
  // Few token rows (batched decode) stream the weights once: a narrower token tile leaves room for a
  // deeper TMA ring, i.e. more weight bytes in flight per block.
  const int bn = gemm_tc_token_tile_for(a.M);
  if (bn == 32) {
    switch (epi) {
      case kEpiInProj: return launch_tc<32, 5, kEpiInProj>(mw, mx, a, s, pdl);
      case kEpiOut: return launch_tc<32, 5, kEpiOut>(mw, mx, a, s, pdl);
      default: return launch_tc<32, 5, kEpiLogits>(mw, mx, a, s, pdl);
    }
  }
  if (bn == 64) {
    switch (epi) {
      case kEpiInProj: return launch_tc<64, 4, kEpiInProj>(mw, mx, a, s, pdl);
      case kEpiOut: return launch_tc<64, 4, kEpiOut>(mw, mx, a, s, pdl);
      default: return launch_tc<64, 4, kEpiLogits>(mw, mx, a, s, pdl);
    }
  }
  switch (epi) {
    case kEpiInProj: return launch_tc<128, 3, kEpiInProj>(mw, mx, a, s, pdl);
    case kEpiOut: return launch_tc<128, 3, kEpiOut>(mw, mx, a, s, pdl);
    default: return launch_tc<128, 3, kEpiLogits>(mw, mx, a, s, pdl);
  }
}

namespace {
// out[m, n] = sum_z partial[z, m, n] + bias[n] (+ residual[m, n]); fixed summation order
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int ksplit, int M, int N,
                                     const float* __restrict__ bias, const float* residual, float* out, int ld_out,
                                     const uint32_t* slot_sel, size_t slot_stride) {
  const size_t total = static_cast<size_t>(M) * N;
  pdl_wait();                      // the partial sums come from the predecessor kernel
  pdl_launch_dependents();
  if (slot_sel) out += static_cast<size_t>(*slot_sel & 1u) * slot_stride;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(i % N);
    const size_t m = i / N;
    float acc = 0.f;
    for (int z = 0; z < ksplit; ++z) acc += partial[static_cast<size_t>(z) * total + i];
    if (bias) acc += bias[n];
    if (residual) acc += residual[i];
    out[m * ld_out + n] = acc;
  }
}
}  // namespace

cudaError_t launch_splitk_reduce(const float* partial, int ksplit, int M, int N, const float* bias,
                                 const float* residual, float* out, int ld_out, const uint32_t* slot_sel,
                                 size_t slot_stride, cudaStream_t s, bool pdl) {
  const size_t total = static_cast<size_t>(M) * N;
  const int grid = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 8));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, partial, ksplit, M, N, bias, residual, out, ld_out, slot_sel,
                            slot_stride);
}

cudaError_t launch_ln_rows(const float* x, const float* scale, const float* offset, __nv_bfloat16* out, int rows,
                           int d, cudaStream_t s, bool pdl, __nv_bfloat16* out_lo) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, ln_rows_kernel, x, scale, offset, out, out_lo, d);
}

}  // namespace mtj
