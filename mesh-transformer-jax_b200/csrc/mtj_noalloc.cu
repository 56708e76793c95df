// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot hand it a scratch buffer and cannot let it
// call cudaMalloc either: a framework custom-call handler whose buffers are
// planned ahead by the framework's own allocator, a process in which another
// runtime has already reserved nearly all of the GPU's memory (an allocation
// would fail or force that runtime to give memory back), or a latency-critical
// serving loop in which the implicit device synchronisation of an allocation
// is not acceptable.  For them the split-KV decode attention is offered once
// more with its scratch (arrival counters and per-split partial results) in a
// fixed array that is part of the library image.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "../../include/mtj_b200.h"
#include "mtj_kernels.h"
#include "mtj_units.h"

namespace {

// Every GPU that loads the library holds this array until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MTJ_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// In host code `g_noalloc_scratch` is only a stand-in for the device array; the
// address a kernel may use has to be asked for, per device, with that device
// current.  Done once per device on the first call.  The address is kept for the
// life of the process: a host that calls cudaDeviceReset() destroys the context
// the address belongs to, and must not call this entry point on that device
// afterwards (the kept address would be stale).
int32_t scratch_for_current_device(char** out, std::string* err) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *err = "cudaGetDevice failed or device index out of range";
    return MTJ_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *err = std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e);
      return MTJ_ERR_CUDA;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = static_cast<char*>(g_scratch_ptr[dev]);
  return MTJ_OK;
}

}  // namespace

extern "C" {

int32_t mtj_set_error(int32_t code, const char* msg);

int32_t mtj_k_decode_attn_noalloc(const float* q, const void* kpool, const void* vpool,
                                  const int32_t* page_table, const int32_t* pad, const int32_t* cur,
                                  int32_t batch, int32_t heads, int32_t d_head, int32_t window,
                                  int32_t ring_pages, int32_t split_tokens, float* out, int32_t ld_out,
                                  mtj_stream s) {
  if (!q || !kpool || !vpool || !page_table || !pad || !cur || !out || ring_pages <= 0)
    return mtj_set_error(MTJ_ERR_INVALID, "null argument");
  mtj::DecodeAttnPlan p;
  std::string err;
  int32_t rc = mtj::plan_decode_attn(batch, heads, d_head, window, split_tokens, &p, &err);
  if (rc) return mtj_set_error(rc, err.c_str());
  if (p.total > MTJ_NOALLOC_SCRATCH_BYTES) {
    err = "mtj_k_decode_attn_noalloc: this shape needs " + std::to_string(p.total) +
          " bytes of scratch, the built-in array holds " + std::to_string(MTJ_NOALLOC_SCRATCH_BYTES) +
          "; use fewer sequences / larger splits or mtj_k_decode_attn with caller scratch";
    return mtj_set_error(MTJ_ERR_INVALID, err.c_str());
  }
  char* scratch = nullptr;
  rc = scratch_for_current_device(&scratch, &err);
  if (rc) return mtj_set_error(rc, err.c_str());
  // run_decode_attn zeroes the arrival counters (the array keeps whatever the
  // previous call left) and overwrites every partial result it later reads.
  rc = mtj::run_decode_attn(p, scratch, q, kpool, vpool, page_table, pad, cur, batch, heads, d_head,
                            window, ring_pages, split_tokens, out, ld_out, static_cast<cudaStream_t>(s), &err);
  return rc ? mtj_set_error(rc, err.c_str()) : MTJ_OK;
}

}  // extern "C"
