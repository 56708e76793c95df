// Embedding gather, greedy arg-max and weight repacking kernels.
#include <math.h>

#include <algorithm>

#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace mtj {
namespace {

constexpr int kThreads = 256;

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

// EmbeddingShard.__call__ (layers.py:187-193): the one-hot matmul is a row
// gather; ids outside this shard's vocabulary range contribute zero rows; the
// shard's bias is added on every shard (summed later by the all-reduce).
__global__ void __launch_bounds__(kThreads) embed_kernel(const EmbedArgs a) {
  __shared__ float red[kThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x;
  const uint32_t id = a.ids[static_cast<size_t>(a.rows.b0 + m / a.rows.Tc) * a.ids_ld +
                            a.rows.pos0_host + m % a.rows.Tc];
  const int64_t local = static_cast<int64_t>(id) - a.vocab_start;
  const bool hit = local >= 0 && local < a.vocab_local;
  const __nv_bfloat16* row = a.table + static_cast<size_t>(hit ? local : 0) * a.d;
  float* xo = a.x + (a.slot_sel ? static_cast<size_t>(*a.slot_sel & 1u) * a.slot_stride : 0) +
              static_cast<size_t>(m) * a.d;
  float s = 0.f;
  for (int i = threadIdx.x; i < a.d; i += kThreads) {
    const float v = (hit ? __bfloat162float(row[i]) : 0.f) + a.bias[i];
    xo[i] = v;
    s += v;
  }
  if (a.stats == nullptr) return;
  const float mu = block_sum256(s, red) / static_cast<float>(a.d);
  float var = 0.f;
  for (int i = threadIdx.x; i < a.d; i += kThreads) {
    const float dlt = xo[i] - mu;      // each thread re-reads only what it wrote
    var = fmaf(dlt, dlt, var);
  }
  var = block_sum256(var, red) / static_cast<float>(a.d);
  if (threadIdx.x == 0) {
    a.stats[2 * m] = mu;
    a.stats[2 * m + 1] = 1.0f / sqrtf(var + 1e-5f);
  }
}

// nucleaus_sample with top_p -> 0 keeps only the head of the descending stable
// sort (sampling.py:11-12,29-36): the arg-max, highest index among equal logits.
__global__ void __launch_bounds__(1024) argmax_kernel(const ArgmaxArgs a) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const float* row = a.logits + static_cast<size_t>(b) * a.V;
  float best = -INFINITY;
  int bi = -1;
  for (int i0 = threadIdx.x; i0 < a.V; i0 += 8 * blockDim.x) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {            // eight independent loads in flight
      const int i = i0 + u * blockDim.x;
      v[u] = i < a.V ? row[i] : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < a.V && (v[u] > best || (v[u] == best && i > bi) || bi < 0)) {
        best = v[u];
        bi = i;
      }
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
    if (lane == 0) {
      a.tokens[b] = static_cast<uint32_t>(bi);
      if (a.tokens_copy) a.tokens_copy[b] = static_cast<uint32_t>(bi);
      if (a.cur_dev && b == 0) *a.cur_dev += 1;
    }
  }
}

template <typename T>
__device__ __forceinline__ float ldf(const T* p, size_t i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __bfloat162float(p[i]);
}

// src [K, N] row-major -> dst[n * ld_dst + k_offset + k] (bf16)
template <typename T>
__global__ void pack_transpose_kernel(const T* __restrict__ src, int K, int N,
                                      __nv_bfloat16* __restrict__ dst, int ld_dst, int k_offset) {
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int k = k0 + j, n = n0 + threadIdx.x;
    tile[j][threadIdx.x] = (k < K && n < N) ? ldf<T>(src, static_cast<size_t>(k) * N + n) : 0.f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int n = n0 + j, k = k0 + threadIdx.x;
    if (n < N && k < K)
      dst[static_cast<size_t>(n) * ld_dst + k_offset + k] = __float2bfloat16_rn(tile[threadIdx.x][j]);
  }
}

template <typename T, typename O>
__global__ void convert_kernel(const T* __restrict__ src, int64_t n, O* __restrict__ dst) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = ldf<T>(src, i);
    if constexpr (sizeof(O) == 4) dst[i] = v;
    else dst[i] = __float2bfloat16_rn(v);
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

cudaError_t launch_embed(const EmbedArgs& a, cudaStream_t s, bool pdl) {
  if (a.M <= 0) return cudaErrorInvalidValue;
  return launch_cfg(embed_kernel, dim3(a.M), dim3(kThreads), s, pdl, a);
}

cudaError_t launch_argmax(const ArgmaxArgs& a, cudaStream_t s, bool pdl) {
  if (a.B <= 0) return cudaErrorInvalidValue;
  return launch_cfg(argmax_kernel, dim3(a.B), dim3(1024), s, pdl, a);
}

cudaError_t launch_pack_transpose(const void* src, int src_is_bf16, int K, int N,
                                  __nv_bfloat16* dst, int ld_dst, int k_offset, cudaStream_t s) {
  const dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
  if (src_is_bf16)
    pack_transpose_kernel<__nv_bfloat16><<<grid, block, 0, s>>>(
        static_cast<const __nv_bfloat16*>(src), K, N, dst, ld_dst, k_offset);
  else
    pack_transpose_kernel<float><<<grid, block, 0, s>>>(static_cast<const float*>(src), K, N, dst,
                                                        ld_dst, k_offset);
  return cudaGetLastError();
}

cudaError_t launch_to_f32(const void* src, int src_is_bf16, int64_t n, float* dst, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int grid = static_cast<int>(std::min<int64_t>((n + 255) / 256, 4096));
  if (src_is_bf16)
    convert_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), n, dst);
  else
    convert_kernel<float, float><<<grid, 256, 0, s>>>(static_cast<const float*>(src), n, dst);
  return cudaGetLastError();
}

cudaError_t launch_to_bf16(const void* src, int src_is_bf16, int64_t n, __nv_bfloat16* dst,
                           cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int grid = static_cast<int>(std::min<int64_t>((n + 255) / 256, 4096));
  if (src_is_bf16)
    convert_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(src), n, dst);
  else
    convert_kernel<float, __nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const float*>(src), n, dst);
  return cudaGetLastError();
}

}  // namespace mtj
