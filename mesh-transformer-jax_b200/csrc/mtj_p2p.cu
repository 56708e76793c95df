// Small-message all-reduce over NVLink peer memory for the decode path
// (stands in for jax.lax.psum on the "shard" axis, util.py:134-136, where the
// payload is [batch, d_model] fp32 and latency, not bandwidth, decides).
//
// Every rank owns a buffer (IPC-shared with its peers) with two data slots and
// a row of arrival flags.  For all-reduce number k (counted on the device so a
// captured step can be replayed):
//   * the producer kernel has written this rank's partial sums into slot k & 1;
//   * one kernel per rank then (1) publishes flag[rank] = k + 1 in every
//     peer's buffer, (2) waits -- with an iteration limit -- until all peers
//     have published k + 1 here, (3) reads the peers' slots with plain loads
//     over NVLink, adds them in rank order (identical on every rank, so the
//     replicated residual stream stays bit-identical), adds the residual and
//     leaves the LayerNorm statistics of each finished row (layers.py:18-19,32).
// A rank can only be one all-reduce ahead of its slowest peer (it needs that
// peer's next flag), so two slots suffice.  A wait that runs out sets the
// device error word and the kernel returns; nothing spins forever.
#include <cuda_runtime.h>

#include <string>

#include "mtj_comm.h"
#include "mtj_common.cuh"

namespace mtj {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ float block_sum256(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) t += red[i];
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(kThreads) p2p_allreduce_kernel(const P2pArgs a) {
  __shared__ float red[kThreads / 32];
  __shared__ bool is_last;
  __shared__ int timed_out;
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const uint32_t k = *a.seq;                         // all-reduces completed so far on this rank
  const uint32_t want = k + 1;
  const size_t slot_off = static_cast<size_t>(k & 1u) * a.slot_elems;
  if (threadIdx.x == 0) timed_out = 0;
  __syncthreads();
  // (1) publish: the producer kernel finished before this kernel started, so the data is in place
  if (blockIdx.x == 0 && threadIdx.x < a.world && threadIdx.x != a.rank) {
    __threadfence_system();
    st_release_sys(a.peer_flags[threadIdx.x] + a.rank, want);
  }
  // (2) wait for every peer's partial sums
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    const uint32_t* f = a.local_flags + threadIdx.x;
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
    // (3) reduce this row in rank order, add the residual, keep the row for the statistics
    float* xr = a.x + static_cast<size_t>(row) * a.d;
    float s = 0.f;
    for (int i = threadIdx.x * 4; i < a.d; i += kThreads * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < a.world; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(a.peer_data[r] + slot_off +
                                                          static_cast<size_t>(row) * a.d + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (a.accumulate) {
        const float4 o = *reinterpret_cast<const float4*>(xr + i);
        acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
      }
      *reinterpret_cast<float4*>(xr + i) = acc;
      s += acc.x + acc.y + acc.z + acc.w;
    }
    const float mu = block_sum256(s, red) / static_cast<float>(a.d);
    float var = 0.f;
    for (int i = threadIdx.x * 4; i < a.d; i += kThreads * 4) {
      const float4 o = *reinterpret_cast<const float4*>(xr + i);     // this thread's own writes
      const float d0 = o.x - mu, d1 = o.y - mu, d2 = o.z - mu, d3 = o.w - mu;
      var += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
    }
    var = block_sum256(var, red) / static_cast<float>(a.d);
    if (threadIdx.x == 0) {
      a.stats[2 * row] = mu;
      a.stats[2 * row + 1] = 1.0f / sqrtf(var + 1e-5f);
    }
  }
  // the last block to finish counts this all-reduce as done (selects the other slot next time)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t ticket = atomicAdd(a.ticket, 1u);
    is_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    *a.ticket = 0u;
    *a.seq = want;
  }
}

}  // namespace

cudaError_t launch_p2p_allreduce(const P2pArgs& a, int rows, cudaStream_t s, bool pdl) {
  if (rows <= 0 || (a.d & 3)) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, p2p_allreduce_kernel, a);
}

}  // namespace mtj
