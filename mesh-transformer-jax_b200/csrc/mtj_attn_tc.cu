// Causal flash-style attention for prefill / eval on the tensor cores
// (d_head = 256): tcgen05.mma with S and O in tensor memory, Q / K / V tiles
// staged by TMA, fp32 online softmax in registers.  Reference semantics:
// layers.py:275-283 (logits / sqrt(d_head), additive masks, softmax, weighted
// V) with the causal mask of :305-308, the left-pad mask of :353-360 and the
// eval key mask of transformer_shard.py:130.
//
// One block = one (sequence, head, 128-query tile).  Keys are walked in blocks
// of 64 (= one page of the KV cache, whose (page, head) slab is a dense
// [64, 256] matrix):
//     S[128, 64]   = Q[128, 256] . K^T          16 MMAs (K-major operands from shared memory)
//     P            = exp2(S*c - m)              8 softmax warps, a query row shared by two threads
//     O[128, 256] += P[128, 64] . V[64, 256]    4 MMAs (P from tensor memory, V MN-major: no transpose)
// Tensor memory: S0 | S1 (fp32) | O (256 columns) | P0 | P1 (bf16, two keys per column).  Warp 0 feeds TMA
// (Q once; K through a three-slot ring, V through a two-slot ring), warp 1 issues the S products, warp 2 the
// P.V products, warps 3-10 do the softmax and the epilogue: warps w and w + 4 read the same tensor-memory
// lanes, each taking 32 of the block's 64 key columns and half of the 256 output columns; the two threads of a
// row exchange their row maxima through shared memory behind a 64-thread named barrier.
// S_j is issued as soon as the softmax warps have READ S_{j-2} out of its buffer (not when P_{j-2} is
// written), so the scores of a block exist before the softmax warps ask for them; P is double buffered, so
// P_j does not wait for P.V of block j-1 either.  Key blocks that every row of a warp sees in full skip the
// mask arithmetic.  O is only rescaled when a row's running maximum grows by more than 2^8 (the stale maximum
// stays the reference, which is exact because the final normalisation uses the same reference).  Masked keys
// are excluded, which equals the reference's -1e10 whenever a row sees at least one key; rows that see none
// (left padding) give zeros.  Every wait is bounded.
//
// Measured and not kept: two softmax warp groups taking the key blocks in turn, the reference maximum handed
// from one to the other after its max pass (correct, 1.81 against 1.88 ms of attention per GPT-J-6B prefill and
// the same eval rate: the softmax warps are not what the tensor core waits for), four threads per row (same time), L2 prefetches of the pages three blocks ahead
// (10 % slower), the next block's scores loaded from tensor memory into a second register set while the
// current block is worked on (5 % slower), pairing a long and a short query tile in one block (17 % slower).
#include <cuda.h>
#include <math.h>

#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

constexpr int kQT = 128;                 // queries per block
constexpr int kKB = 64;                  // keys per block (one cache page)
constexpr int kDH = 256;
// threads sharing a query row (each 64 / kParts key columns and 256 / kParts output columns): 2 and 4 measure the
// same (1.88 / 1.87 ms of attention per GPT-J-6B prefill); 1 was 25 % slower
constexpr int kParts = 2;
constexpr int kSoftWarps = 4 * kParts;          // softmax warps: TMEM lane quadrant = warp % 4, part = (warp - 3) / 4
constexpr int kThreadsTc = 96 + 32 * kSoftWarps;   // TMA warp, two MMA warps (S; P.V), softmax warps
constexpr int kPartKeys = kKB / kParts, kPartCols = kDH / kParts;
constexpr uint32_t kQBytes = kQT * kDH * 2;          // 64 KB
constexpr uint32_t kKBytes = kKB * kDH * 2;          // 32 KB
constexpr int kKSlots = 3, kVSlots = 2;              // ring depths: a K slot is wanted again one key block sooner than a V slot
constexpr uint32_t kSmemTc = kQBytes + (kKSlots + kVSlots) * kKBytes;   // 224 KB: the dynamic buffer is 1024-byte aligned
// tensor memory: S0 | S1 (64 fp32 columns each) | O (256) | P0 | P1 (64 bf16 keys = 32 columns each)
constexpr uint32_t kColS = 0, kColO = 128, kColP = 384, kPCols = kKB / 2, kTmemCols = 512;

__device__ __forceinline__ void tma2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_bf16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
// shared-memory matrix descriptor, 128-byte swizzle; lbo / sbo in bytes
// the same with the A operand (bf16, K-major, two elements per 32-bit column) in tensor memory
__device__ __forceinline__ void mma_bf16_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ uint64_t sdesc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tm_ld32(uint32_t taddr, uint32_t* r) {
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
__device__ __forceinline__ void tm_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tm_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tm_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
__device__ __forceinline__ void tm_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__global__ void __launch_bounds__(kThreadsTc, 1) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                     const __grid_constant__ CUtensorMap map_k,
                                                                     const __grid_constant__ CUtensorMap map_v,
                                                                     const PrefillAttnTcArgs a) {
  extern __shared__ __align__(1024) unsigned char att_smem_raw[];
  const uint32_t base = smem_u32(att_smem_raw);       // swizzled tiles need 1024-byte alignment
  const uint32_t sQ = base, sK = base + kQBytes, sV = sK + kKSlots * kKBytes;
  __shared__ __align__(8) uint64_t bars[20];
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t failed;
  __shared__ float xmax[kParts][kQT];      // [part][row]: row maxima, at the end denominators, of the threads sharing a row

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0, k_full0 = bar0 + 8, k_empty0 = bar0 + 32, v_full0 = bar0 + 56,
                 v_empty0 = bar0 + 72, s_full0 = bar0 + 88, p_full0 = bar0 + 104, p_empty0 = bar0 + 120,
                 o_done = bar0 + 136, s_read0 = bar0 + 144;

  if (base & 1023u) {                                  // cannot happen with the declared alignment; checked, not assumed
    if (threadIdx.x == 0 && a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < 20; ++i) mbar_init(bar0 + 8u * i, 1);
    mbar_init(p_full0, 32 * kSoftWarps);
    mbar_init(p_full0 + 8, 32 * kSoftWarps);
    mbar_init(s_read0, 32 * kSoftWarps);
    mbar_init(s_read0 + 8, 32 * kSoftWarps);
    mbar_fence_init();
    failed = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;

  // causal: later query tiles walk more key blocks; the block order is longest tile first, heads
  // within a tile, so the tail of the grid is made of the short tiles
  const int tile = gridDim.y - 1 - blockIdx.y, head = blockIdx.x, bi = blockIdx.z;
  const int b = a.rows.b0 + bi;
  const int pos0 = a.rows.pos0_host;
  const int Tc = a.rows.Tc;
  const int row0 = bi * Tc + tile * kQT;                  // first chunk row of this tile
  const int q_rows = min(kQT, Tc - tile * kQT);
  const int pad = a.kv.pad[b];
  const int limit = a.key_limit ? a.key_limit[b] : 0x7fffffff;
  const int last_key = min(pos0 + tile * kQT + q_rows - 1, limit);
  const int first_blk = pad / kKB;
  const int nb = last_key >= pad ? last_key / kKB - first_blk + 1 : 0;

  if (warp == 0) {
    if (lane == 0 && nb > 0) {
      mbar_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) tma2d(sQ + kb * (kQT * 128), &map_q, head * kDH + kb * 64, row0, q_full);
      const int32_t* table = a.kv.page_table + static_cast<size_t>(b) * a.kv.ring_pages;
      auto slab_row = [&](int j) { return (table[(first_blk + j) % a.kv.ring_pages] * a.heads + head) * kKB; };
      auto load_k = [&](int j) {
        const int st = j % kKSlots;
        if (j >= kKSlots && !mbar_wait(k_empty0 + 8 * st, ((j / kKSlots) - 1) & 1)) return false;
        const int row = slab_row(j);
        const uint32_t dk = sK + st * kKBytes;
        mbar_expect_tx(k_full0 + 8 * st, kKBytes);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) tma2d(dk + kb * (kKB * 128), &map_k, kb * 64, row, k_full0 + 8 * st);
        return true;
      };
      auto load_v = [&](int j) {
        const int st = j & 1;
        if (j >= 2 && !mbar_wait(v_empty0 + 8 * st, ((j >> 1) - 1) & 1)) return false;
        const int row = slab_row(j);
        const uint32_t dv = sV + st * kKBytes;
        mbar_expect_tx(v_full0 + 8 * st, kKBytes);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) tma2d(dv + kb * (kKB * 128), &map_v, kb * 64, row, v_full0 + 8 * st);
        return true;
      };
      // the waits follow the tensor core's order: S0 S1 | PV0 S2 | PV1 S3 | ...
      bool okp = load_k(0);
      for (int j = 1; okp && j < kKSlots && j < nb; ++j) okp = load_k(j);
      for (int j = 0; okp && j < nb; ++j) {
        okp = load_v(j);
        if (okp && j + kKSlots < nb) okp = load_k(j + kKSlots);   // its slot is free once S_j is done
      }
      if (!okp) atomicOr(&failed, 1u);
    }
  } else if (warp == 1) {
    // S = Q . K^T, issued two key blocks ahead.  The products of a block are issued by two warps (this one and the
    // next): a single thread building descriptors and issuing all 20 MMAs of a block was the longest chain of
    // the kernel.
    if (lane == 0 && nb > 0) {
      constexpr uint32_t kIdS = (1u << 4) | (1u << 7) | (1u << 10) | ((kKB >> 3) << 17) | ((kQT >> 4) << 24);
      uint64_t qd[4];
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) qd[kb] = sdesc(sQ + kb * (kQT * 128), 16, 1024);
      auto issue_s = [&](int j) {
        const uint32_t dk = sK + (j % kKSlots) * kKBytes;
        const uint32_t ds = tmem + kColS + (j & 1) * kKB;
        const uint64_t kd = sdesc(dk, 16, 1024);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const uint64_t bd = kd + static_cast<uint64_t>((kb * (kKB * 128)) >> 4);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) mma_bf16(ds, qd[kb] + 2 * k4, bd + 2 * k4, kIdS, (kb | k4) ? 1u : 0u);
        }
        commit(s_full0 + 8 * (j & 1));
        commit(k_empty0 + 8 * (j % kKSlots));                  // the K slot is free once S_j is done
      };
      bool ok = mbar_wait(q_full, 0);
      for (int j = 0; ok && j < nb; ++j) {
        // S_j goes into the buffer of S_{j-2} as soon as the softmax warps have READ S_{j-2} into registers: it
        // does not wait for P_{j-2}, so the scores are ready before the softmax warps ask for them
        if (j >= 2) ok = mbar_wait(s_read0 + 8 * (j & 1), ((j - 2) >> 1) & 1);
        if (ok) ok = mbar_wait(k_full0 + 8 * (j % kKSlots), (j / kKSlots) & 1);
        if (!ok) break;
        fence_after();
        issue_s(j);
      }
      if (!ok) atomicOr(&failed, 1u);
    }
  } else if (warp == 2) {
    // O += P . V
    if (lane == 0 && nb > 0) {
      constexpr uint32_t kIdO = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((kDH >> 3) << 17) | ((kQT >> 4) << 24);
      bool ok = true;
      for (int j = 0; ok && j < nb; ++j) {
        // P_j written, V_j landed
        ok = mbar_wait(p_full0 + 8 * (j & 1), (j >> 1) & 1) && mbar_wait(v_full0 + 8 * (j & 1), (j >> 1) & 1);
        if (!ok) break;
        fence_after();
        // P from tensor memory (16 keys = 8 columns per MMA), V tile is [64 keys][256 dh] -> MN-major B operand,
        // 64-column blocks 8 KB apart
        const uint64_t vd = sdesc(sV + (j & 1) * kKBytes, kKB * 128, 1024);
        const uint32_t pa = tmem + kColP + (j & 1) * kPCols;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          mma_bf16_ts(tmem + kColO, pa + 8 * k4, vd + static_cast<uint64_t>((k4 * 2048) >> 4), kIdO, (j | k4) ? 1u : 0u);
        commit(v_empty0 + 8 * (j & 1));
        commit(p_empty0 + 8 * (j & 1));                          // P buffer j & 1 is free, O holds key blocks 0 .. j
        if (j == nb - 1) commit(o_done);
      }
      if (!ok) atomicOr(&failed, 1u);
    }
  } else {
    const int quad = warp & 3;                                 // the TMEM lane quadrant this warp may access
    const int part = (warp - 3) >> 2;                          // key columns [kPartKeys part, +kPartKeys) / O columns [kPartCols part, +kPartCols)
    const int r = quad * 32 + lane;                            // query row within the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t pair_bar = 1u + static_cast<uint32_t>(quad);   // named barrier of the warps sharing these rows
    auto pair_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(pair_bar), "n"(32 * kParts) : "memory"); };
    const float c2 = 0.0625f * 1.4426950408889634f;            // 1/sqrt(256) * log2(e)
    const bool row_ok = r < q_rows;
    const int qpos = pos0 + tile * kQT + r;
    float m_ref = -INFINITY, l = 0.f;
    const int warp_qpos0 = pos0 + tile * kQT + quad * 32;       // smallest query position of this warp
    bool ok = nb > 0;
    for (int j = 0; j < nb; ++j) {
      const int g = j;
      // a wait that runs out is remembered, but the thread keeps meeting its partner at the pair barrier
      if (ok) ok = mbar_wait(s_full0 + 8 * (g & 1), (g >> 1) & 1);
      fence_after();
      uint32_t sr[kPartKeys];
      const uint32_t s_addr = tmem + lane_addr + kColS + (g & 1) * kKB + part * kPartKeys;
      if (ok) {
        if (kPartKeys == 32) tm_ld32(s_addr, sr);
        else tm_ld16(s_addr, sr);
        fence_before();
        mbar_arrive(s_read0 + 8 * (g & 1));                    // the scores are in registers: the buffer may be refilled
      } else {
#pragma unroll
        for (int c = 0; c < kPartKeys; ++c) sr[c] = 0xff800000u;      // -inf
      }
      const int kbase = (first_blk + j) * kKB + part * kPartKeys;
      // every row of this warp sees all of its keys: no mask arithmetic.  Rows past the end of a partial query tile
      // do not exist and are never stored, so they do not force the masked path (with 2047 rows they would, in
      // one warp pair of the LONGEST tile, which paces the whole kernel: the masked pass costs 800 cycles a block).
      const bool full_blk = ok && kbase >= pad && kbase + kPartKeys - 1 <= min(warp_qpos0, limit);
      float mx = -INFINITY;
      if (full_blk) {
        float mxa = -INFINITY, mxb = -INFINITY;               // two chains
#pragma unroll
        for (int c = 0; c < kPartKeys; c += 2) {
          mxa = fmaxf(mxa, __uint_as_float(sr[c]));
          mxb = fmaxf(mxb, __uint_as_float(sr[c + 1]));
        }
        mx = fmaxf(mxa, mxb) * c2;
      } else {
        // the visible columns of this row are one range [lo_c, hi_c] of the block (empty for a row that does not
        // exist): two compares against constants per score instead of the full predicate
        const int lo_c = pad - kbase;
        const int hi_c = (ok && row_ok) ? min(qpos, limit) - kbase : -1;
        float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
        for (int c = 0; c < kPartKeys; c += 2) {
          const float v0 = (c >= lo_c && c <= hi_c) ? __uint_as_float(sr[c]) : -INFINITY;
          const float v1 = (c + 1 >= lo_c && c + 1 <= hi_c) ? __uint_as_float(sr[c + 1]) : -INFINITY;
          sr[c] = __float_as_uint(v0);
          sr[c + 1] = __float_as_uint(v1);
          mxa = fmaxf(mxa, v0);
          mxb = fmaxf(mxb, v1);
        }
        mx = fmaxf(mxa, mxb) * c2;                             // c2 > 0; (-inf) * c2 stays -inf
      }
      // the row's maximum over all 64 keys: the partner threads hold the other parts
      xmax[part][r] = mx;
      pair_sync();
#pragma unroll
      for (int q = 1; q < kParts; ++q) mx = fmaxf(mx, xmax[(part + q) % kParts][r]);
      pair_sync();                                             // all have read: the next block may overwrite
      float m_new = m_ref;
      if (mx > m_ref + 8.0f || (m_ref == -INFINITY && mx > -INFINITY)) m_new = mx;
      const float corr = (m_new == m_ref || m_ref == -INFINITY) ? 1.0f : exp2f(m_ref - m_new);
      // p = 2^(s c - m); a masked score is -inf and gives 0; a row that has seen no key yet (m = -inf)
      // takes a finite stand-in so that -inf - (-inf) does not appear
      const float neg_m = m_new == -INFINITY ? 0.f : -m_new;
      float psum0 = 0.f, psum1 = 0.f;
      uint32_t pk[kPartKeys / 2];
#pragma unroll
      for (int c = 0; c < kPartKeys; c += 2) {
        const float p0 = ex2_fast(fmaf(__uint_as_float(sr[c]), c2, neg_m));
        const float p1 = ex2_fast(fmaf(__uint_as_float(sr[c + 1]), c2, neg_m));
        psum0 += p0;
        psum1 += p1;
        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
      }
      l = l * corr + (psum0 + psum1);                          // this thread's part of the denominator
      // P is double buffered in tensor memory: buffer j & 1 is free once PV(j - 2) has read it
      if (j >= 2 && ok) ok = mbar_wait(p_empty0 + 8 * (j & 1), ((j >> 1) - 1) & 1);
      if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {    // the warps sharing a row see the same corr per row
        // O changes scale: PV(j - 1) must have landed (PV(j) cannot start before this thread has written P_j)
        if (ok) ok = mbar_wait(p_empty0 + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1);
        fence_after();
        if (ok) {
#pragma unroll 1
          for (int c0 = part * kPartCols; c0 < (part + 1) * kPartCols; c0 += 32) {
            uint32_t o[32];
            tm_ld32(tmem + lane_addr + kColO + c0, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            tm_st32(tmem + lane_addr + kColO + c0, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      // this thread's keys of the P row -> tensor memory, two bf16 per column: the A operand of P . V
      fence_after();
      if (kPartKeys == 32) tm_st16(tmem + lane_addr + kColP + (j & 1) * kPCols + part * (kPartKeys / 2), pk);
      else tm_st8(tmem + lane_addr + kColP + (j & 1) * kPCols + part * (kPartKeys / 2), pk);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      fence_before();
      mbar_arrive(p_full0 + 8 * (j & 1));
      m_ref = m_new;
    }
    if (nb > 0 && ok) ok = mbar_wait(o_done, 0);
    if (nb > 0 && !ok) atomicOr(&failed, 1u);
    fence_after();
    xmax[part][r] = l;
    pair_sync();
    l = 0.f;
#pragma unroll
    for (int q = 0; q < kParts; ++q) l += xmax[q][r];        // the same order in every thread of the row
    {
      // the TMEM loads are warp-wide: every lane takes part, only the stores are per row
      __nv_bfloat16* dst = a.out_bf16 + static_cast<size_t>(row0 + (row_ok ? r : 0)) * a.ld_out + head * kDH;
      const bool have = nb > 0 && ok;
      const float inv = (have && l > 0.f) ? 1.0f / l : 0.f;
#pragma unroll 1
      for (int c0 = part * kPartCols; c0 < (part + 1) * kPartCols; c0 += 32) {
        uint32_t o[32];
        if (have) {
          tm_ld32(tmem + lane_addr + kColO + c0, o);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c0 + i) = w;
          }
        }
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && failed && a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
}

}  // namespace

// Blocks are issued longest query tile first, which the hardware's dynamic block scheduling turns into a
// near-even finish (longest-processing-time order).  Pairing a long and a short tile inside one block, to get
// one even wave of blocks, was measured slower (2.35 ms against 2.01 ms per GPT-J-6B prefill): the pipeline
// drains and refills between a block's two tiles.
cudaError_t launch_prefill_attn_tc(const void* map_q, const void* map_k, const void* map_v,
                                   const PrefillAttnTcArgs& a, cudaStream_t s) {
  if (a.M <= 0 || a.rows.Tc <= 0 || a.M % a.rows.Tc != 0 || a.d_head != kDH) return cudaErrorInvalidValue;
  static DeviceOnce once;
  {
    cudaError_t e = once.run([&] { return cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kSmemTc)); });
    if (e != cudaSuccess) return e;
  }
  const dim3 grid(a.heads, (a.rows.Tc + kQT - 1) / kQT, a.M / a.rows.Tc);
  prefill_attn_tc_kernel<<<grid, kThreadsTc, kSmemTc, s>>>(*static_cast<const CUtensorMap*>(map_q),
                                                           *static_cast<const CUtensorMap*>(map_k),
                                                           *static_cast<const CUtensorMap*>(map_v), a);
  return cudaGetLastError();
}

}  // namespace mtj
