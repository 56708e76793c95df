// Tensor-parallel decode exchanges over NVLink peer memory, push style (stand in for jax.lax.psum on
// the "shard" axis, util.py:134-136 / layers.py:313, and for the all_gather of ProjectionShard.__call__,
// layers.py:565-567, when the step only needs the greedy token).
//
// tp_push_reduce_kernel -- one launch per layer does what took three (split-K reduction, peer all-reduce,
// LayerNorm to the next GEMM's operand) and one NVLink round trip less:
//   block m owns token row m.  It (1) sums this rank's split-K partial sums of the out-projection and adds
//   the rank's bias, (2) STORES the row into every peer's receive area [slot][source rank][row] with plain
//   16-byte stores, fences, and publishes one flag per (peer, row), (3) waits -- bounded -- for the flags of
//   the peers' copies of the same row, which by then sit in this GPU's own memory, (4) adds the world's rows
//   in rank order (identical on every rank, so the replicated residual stream stays bit-identical), adds
//   the residual, leaves the LayerNorm statistics and writes the normalised row as the bf16 (hi [+ lo])
//   operand of the next projection.
// Exchange number k lives on the device (the step is a replayed graph); slot = k & 1.  A rank can finish
// exchange k + 1 only after every peer has pushed k + 1, which a peer does after it has read exchange k:
// two slots suffice.  Flags carry k + 1 and only grow, so a peer that is one exchange ahead does no harm.
//
// tp_argmax_kernel -- greedy sampling without gathering the logits: every rank finds the arg-max of its
// vocabulary slice (highest index among equal logits, sampling.py:11-12), pushes (value, global index) as
// two tagged 8-byte packets to every rank, and all ranks pick the same winner.
//
// Every wait has an iteration limit; when it runs out the kernel sets the device error word and returns.
#include <cuda_runtime.h>
#include <math.h>

#include "mtj_comm.h"
#include "mtj_common.cuh"

namespace mtj {
namespace {

constexpr int kPushThreads = 1024;        // one 16-byte column group per thread at d_model 4096: every load in flight at once

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_packet(uint2* p, uint32_t v, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_packet(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kPushThreads / 32; ++i) t += red[i];
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(kPushThreads) tp_push_reduce_kernel(const TpReduceArgs a) {
  extern __shared__ __align__(16) float own[];         // this rank's finished partial row [d]
  __shared__ float red[kPushThreads / 32];
  __shared__ int timed_out;
  __shared__ bool is_last;
  pdl_wait();                                           // the partial sums come from the predecessor kernel
  pdl_launch_dependents();
  const int row = blockIdx.x, M = gridDim.x, d = a.d;
  const uint32_t k = *a.seq, want = k + 1;
  const size_t slot_off = static_cast<size_t>(k & 1u) * a.world * a.rows_cap * d;
  const size_t my_row_off = slot_off + (static_cast<size_t>(a.rank) * a.rows_cap + row) * d;
  if (threadIdx.x == 0) timed_out = 0;

  // (1) + (2): finish this rank's row and push it
  const size_t plane = static_cast<size_t>(M) * d;
  for (int i = threadIdx.x * 4; i < d; i += kPushThreads * 4) {
    float4 acc = a.bias ? *reinterpret_cast<const float4*>(a.bias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* pz = reinterpret_cast<const float4*>(a.partial + static_cast<size_t>(row) * d + i);
    float4 v[8];
#pragma unroll
    for (int z = 0; z < 8; ++z)                        // the planes' loads are independent: issue them together
      v[z] = z < a.ksplit ? __ldcg(pz + z * (plane >> 2)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int z = 0; z < 8; ++z) { acc.x += v[z].x; acc.y += v[z].y; acc.z += v[z].z; acc.w += v[z].w; }
    for (int z = 8; z < a.ksplit; ++z) {
      const float4 w = __ldcg(pz + z * (plane >> 2));
      acc.x += w.x; acc.y += w.y; acc.z += w.z; acc.w += w.w;
    }
    *reinterpret_cast<float4*>(own + i) = acc;
    for (int r = 0; r < a.world; ++r)
      if (r != a.rank) *reinterpret_cast<float4*>(a.peer_recv[r] + my_row_off + i) = acc;
  }
  __syncthreads();
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    __threadfence_system();                             // the row (all threads' stores) before its flag
    st_release_sys(a.peer_flags[threadIdx.x] + a.rank * a.rows_cap + row, want);
    // (3) the peer's copy of this row
    const uint32_t* f = a.peer_flags[a.rank] + threadIdx.x * a.rows_cap + row;
    int spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(f) - want) < 0) {
      if (++spins > a.wait_limit) {
        atomicExch(&timed_out, 1);
        break;
      }
    }
  }
  __syncthreads();
  if (timed_out) {
    if (threadIdx.x == 0 && a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
  } else {
    // (4) sum in rank order, residual, statistics, normalised operand
    const float* recv = a.peer_recv[a.rank] + slot_off + static_cast<size_t>(row) * d;
    float* xr = a.x + static_cast<size_t>(row) * d;
    float s = 0.f;
    for (int i = threadIdx.x * 4; i < d; i += kPushThreads * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < a.world; ++r) {
        const float4 v = r == a.rank ? *reinterpret_cast<const float4*>(own + i)
                                     : __ldcg(reinterpret_cast<const float4*>(recv + static_cast<size_t>(r) * a.rows_cap * d + i));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (a.accumulate) {
        const float4 o = *reinterpret_cast<const float4*>(xr + i);
        acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
      }
      *reinterpret_cast<float4*>(xr + i) = acc;
      *reinterpret_cast<float4*>(own + i) = acc;        // the finished row stays in shared memory
      s += acc.x + acc.y + acc.z + acc.w;
    }
    const float mu = block_sum(s, red) / static_cast<float>(d);
    float var = 0.f;
    for (int i = threadIdx.x * 4; i < d; i += kPushThreads * 4) {
      const float4 o = *reinterpret_cast<const float4*>(own + i);
      const float d0 = o.x - mu, d1 = o.y - mu, d2 = o.z - mu, d3 = o.w - mu;
      var += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
    }
    const float rstd = 1.0f / sqrtf(block_sum(var, red) / static_cast<float>(d) + 1e-5f);
    if (threadIdx.x == 0 && a.stats) {
      a.stats[2 * row] = mu;
      a.stats[2 * row + 1] = rstd;
    }
    if (a.xn) {
      for (int i = threadIdx.x; i < d; i += kPushThreads) {
        const float y = fmaf(a.ln_scale[i] * rstd, own[i] - mu, a.ln_offset[i]);
        const __nv_bfloat16 hi = __float2bfloat16_rn(y);
        a.xn[static_cast<size_t>(row) * d + i] = hi;
        if (a.xn_lo) a.xn_lo[static_cast<size_t>(row) * d + i] = __float2bfloat16_rn(y - __bfloat162float(hi));
      }
    }
  }
  // the last block to finish counts this exchange as done (selects the other slot next time)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t ticket = atomicAdd(a.ticket, 1u);
    is_last = (ticket == static_cast<uint32_t>(M) - 1);
  }
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    *a.ticket = 0u;
    *a.seq = want;
  }
}

__global__ void __launch_bounds__(1024) tp_argmax_kernel(const TpArgmaxArgs a) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float pv[kP2pMaxWorld];
  __shared__ uint32_t pi[kP2pMaxWorld];
  __shared__ int timed_out;
  __shared__ bool is_last;
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, B = gridDim.x;
  const uint32_t k = *a.seq, want = k + 1;
  if (threadIdx.x == 0) timed_out = 0;
  const float* rowp = a.logits + static_cast<size_t>(b) * a.Vl;
  float best = -INFINITY;
  int bi = -1;
  for (int i = threadIdx.x; i < a.Vl; i += blockDim.x) {
    const float v = rowp[i];
    if (bi < 0 || v > best || (v == best && i > bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) {
        best = ov;
        bi = oi;
      }
    }
    // packets of (slot, source rank, sequence): {value, tag}, {global index, tag}
    const size_t mine = ((static_cast<size_t>(k & 1u) * a.world + a.rank) * a.rows_cap + b) * 2;
    if (lane < a.world) {
      st_packet(a.peer_amax[lane] + mine, __float_as_uint(best), want);
      st_packet(a.peer_amax[lane] + mine + 1, static_cast<uint32_t>(a.vocab_start + bi), want);
      const uint2* src = a.peer_amax[a.rank] + ((static_cast<size_t>(k & 1u) * a.world + lane) * a.rows_cap + b) * 2;
      uint2 v0 = ld_packet(src), v1 = ld_packet(src + 1);
      int spins = 0;
      while (v0.y != want || v1.y != want) {
        if (++spins > a.wait_limit) {
          atomicExch(&timed_out, 1);
          break;
        }
        v0 = ld_packet(src);
        v1 = ld_packet(src + 1);
      }
      pv[lane] = __uint_as_float(v0.x);
      pi[lane] = v1.x;
    }
    __syncwarp();
    if (lane == 0) {
      if (timed_out) {
        if (a.dev_err) atomicOr(a.dev_err, kDevErrTimeout);
      } else {
        float wv = pv[0];
        uint32_t wi = pi[0];
        for (int r = 1; r < a.world; ++r)               // slices ascend with the rank: a later equal value wins
          if (pv[r] >= wv) {
            wv = pv[r];
            wi = pi[r];
          }
        a.tokens[b] = wi;
      }
      if (a.cur_dev && b == 0) *a.cur_dev += 1;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t ticket = atomicAdd(a.ticket, 1u);
    is_last = (ticket == static_cast<uint32_t>(B) - 1);
  }
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    *a.ticket = 0u;
    *a.seq = want;
  }
}

}  // namespace

cudaError_t launch_tp_push_reduce(const TpReduceArgs& a, int rows, cudaStream_t s, bool pdl) {
  if (rows <= 0 || rows > a.rows_cap || (a.d & 3) || a.ksplit < 1) return cudaErrorInvalidValue;
  const size_t smem = static_cast<size_t>(a.d) * sizeof(float);
  if (smem > 48 * 1024) {
    static DeviceOnce once;
    cudaError_t e = once.run([&] {
      return cudaFuncSetAttribute(tp_push_reduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    });
    if (e != cudaSuccess) return e;
    if (smem > 96 * 1024) return cudaErrorInvalidValue;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(kPushThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tp_push_reduce_kernel, a);
}

cudaError_t launch_tp_argmax(const TpArgmaxArgs& a, int B, cudaStream_t s, bool pdl) {
  if (B <= 0 || B > a.rows_cap || a.world > 32) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(B);
  cfg.blockDim = dim3(1024);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tp_argmax_kernel, a);
}

}  // namespace mtj
