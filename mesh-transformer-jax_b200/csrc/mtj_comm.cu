// "shard"-axis collectives (jax.lax.psum / all_gather in the reference:
// util.py:134-136, layers.py:193,313,565,575-585) over NCCL, plus the small
// kernels that consume their results.  NCCL is resolved at run time from the
// process (torch has normally loaded it already), so the library carries no
// link-time dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <string>

#include "mtj_comm.h"
#include "mtj_common.cuh"

namespace mtj {
namespace {

struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;
};

NcclApi* api() {
  static NcclApi a;
  if (a.lib || !a.error.empty()) return &a;
  for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
    a.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (a.lib) break;
  }
  if (!a.lib) {
    a.error = "libnccl.so.2 could not be loaded (import torch first, or put NCCL on the library path)";
    return &a;
  }
  auto sym = [&](const char* n) {
    void* p = dlsym(a.lib, n);
    if (!p) a.error = std::string("NCCL symbol missing: ") + n;
    return p;
  };
  a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
  a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
  a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
  a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
  a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
  a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
  return &a;
}

std::string nccl_msg(const char* what, ncclResult_t r) {
  NcclApi* a = api();
  return std::string(what) + ": " + (a->GetErrorString ? a->GetErrorString(r) : "NCCL error");
}

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

// x[m] = (accumulate ? x[m] : 0) + reduced[m], then the LayerNorm statistics of
// the row (layers.py:18-19,32): what follows every g_psum on the residual path.
__global__ void __launch_bounds__(kThreads) residual_stats_kernel(float* __restrict__ x,
                                                                  const float* __restrict__ reduced,
                                                                  float* __restrict__ stats, int d,
                                                                  int accumulate) {
  __shared__ float red[kThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x;
  float* xr = x + static_cast<size_t>(m) * d;
  const float* rr = reduced + static_cast<size_t>(m) * d;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += kThreads) {
    const float v = (accumulate ? xr[i] : 0.f) + rr[i];
    xr[i] = v;
    s += v;
  }
  const float mu = block_sum256(s, red) / static_cast<float>(d);
  float var = 0.f;
  for (int i = threadIdx.x; i < d; i += kThreads) {
    const float dlt = xr[i] - mu;
    var = fmaf(dlt, dlt, var);
  }
  var = block_sum256(var, red) / static_cast<float>(d);
  if (threadIdx.x == 0) {
    stats[2 * m] = mu;
    stats[2 * m + 1] = 1.0f / sqrtf(var + 1e-5f);
  }
}

// all-gather result [mp][rows][vl] -> [rows][mp*vl] (vocabulary order is shard-major, layers.py:565-567)
__global__ void gather_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int mp, int rows,
                                   int vl) {
  const size_t n = static_cast<size_t>(mp) * rows * vl;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vl);
    const int r = static_cast<int>((i / vl) % rows);
    const int s = static_cast<int>(i / (static_cast<size_t>(vl) * rows));
    dst[(static_cast<size_t>(r) * mp + s) * vl + v] = src[i];
  }
}

}  // namespace

int32_t comm_unique_id(uint8_t* out128, std::string* err) {
  NcclApi* a = api();
  if (!a->error.empty()) {
    *err = a->error;
    return 6;
  }
  ncclUniqueId id;
  ncclResult_t r = a->GetUniqueId(&id);
  if (r != ncclSuccess) {
    *err = nccl_msg("ncclGetUniqueId", r);
    return 6;
  }
  memcpy(out128, id.internal, NCCL_UNIQUE_ID_BYTES);
  return 0;
}

int32_t comm_init(const uint8_t* id128, int rank, int world, void** comm_out, std::string* err) {
  NcclApi* a = api();
  if (!a->error.empty()) {
    *err = a->error;
    return 6;
  }
  ncclUniqueId id;
  memcpy(id.internal, id128, NCCL_UNIQUE_ID_BYTES);
  ncclComm_t c = nullptr;
  ncclResult_t r = a->CommInitRank(&c, world, id, rank);
  if (r != ncclSuccess) {
    *err = nccl_msg("ncclCommInitRank", r);
    return 6;
  }
  *comm_out = c;
  return 0;
}

void comm_destroy(void* comm) {
  NcclApi* a = api();
  if (comm && a->CommDestroy) a->CommDestroy(static_cast<ncclComm_t>(comm));
}

int32_t comm_all_reduce(void* comm, float* buf, size_t count, bool max_op, cudaStream_t s, std::string* err) {
  NcclApi* a = api();
  ncclResult_t r = a->AllReduce(buf, buf, count, ncclFloat32, max_op ? ncclMax : ncclSum,
                                static_cast<ncclComm_t>(comm), s);
  if (r != ncclSuccess) {
    *err = nccl_msg("ncclAllReduce", r);
    return 6;
  }
  return 0;
}

int32_t comm_all_gather(void* comm, const float* send, float* recv, size_t count, cudaStream_t s,
                        std::string* err) {
  NcclApi* a = api();
  ncclResult_t r = a->AllGather(send, recv, count, ncclFloat32, static_cast<ncclComm_t>(comm), s);
  if (r != ncclSuccess) {
    *err = nccl_msg("ncclAllGather", r);
    return 6;
  }
  return 0;
}

cudaError_t launch_residual_stats(float* x, const float* reduced, float* stats, int rows, int d,
                                  bool accumulate, cudaStream_t s, bool pdl) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, residual_stats_kernel, x, reduced, stats, d, accumulate ? 1 : 0);
}

cudaError_t launch_gather_rows(const float* src, float* dst, int mp, int rows, int vl, cudaStream_t s) {
  const size_t n = static_cast<size_t>(mp) * rows * vl;
  const int grid = static_cast<int>(std::min<size_t>((n + 255) / 256, 2048));
  gather_rows_kernel<<<grid, 256, 0, s>>>(src, dst, mp, rows, vl);
  return cudaGetLastError();
}

}  // namespace mtj
