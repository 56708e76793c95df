// Handle-free unit entry points of the C ABI (one kernel family each), used by
// the parity tests and by callers that drive single kernels.
#include <cuda_runtime.h>

#include <cstdlib>
#include <string>

#include "../../include/mtj_b200.h"
#include "mtj_common.cuh"
#include "mtj_kernels.h"
#include "mtj_units.h"

namespace mtj {

int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

int32_t plan_decode_attn(int32_t batch, int32_t heads, int32_t d_head, int32_t window,
                         int32_t split_tokens, DecodeAttnPlan* p, std::string* err) {
  if (batch <= 0 || heads <= 0 || window <= 0 || split_tokens <= 0 || (split_tokens & 7)) {
    *err = "batch, heads, window must be positive and split_tokens a positive multiple of 8";
    return MTJ_ERR_INVALID;
  }
  if (d_head != 64 && d_head != 256) {
    *err = "d_head must be 64 or 256";
    return MTJ_ERR_UNSUPPORTED;
  }
  p->splits = decode_attn_splits(window);      // one split per 64-token page; split_tokens is only validated
  const int64_t rows = static_cast<int64_t>(batch) * heads;
  p->counters_bytes = align256(rows * 4);
  p->ml_off = p->counters_bytes;
  p->o_off = p->ml_off + align256(rows * p->splits * 2 * 4);
  p->total = p->o_off + align256(rows * p->splits * d_head * 4);
  return MTJ_OK;
}

int32_t run_decode_attn(const DecodeAttnPlan& p, char* scratch, const float* q, const void* kpool,
                        const void* vpool, const int32_t* page_table, const int32_t* pad,
                        const int32_t* cur, int32_t batch, int32_t heads, int32_t d_head, int32_t window,
                        int32_t ring_pages, int32_t split_tokens, float* out, int32_t ld_out,
                        cudaStream_t s, std::string* err) {
  // the arrival counters must start at zero; everything else is overwritten
  cudaError_t e = cudaMemsetAsync(scratch, 0, p.counters_bytes, s);
  if (e == cudaSuccess) {
    DecodeAttnArgs a = {};
    a.q = q;
    a.kv.kpool = static_cast<__nv_bfloat16*>(const_cast<void*>(kpool));
    a.kv.vpool = static_cast<__nv_bfloat16*>(const_cast<void*>(vpool));
    a.kv.page_table = page_table;
    a.kv.ring_pages = ring_pages;
    a.kv.pad = pad;
    a.B = batch;
    a.heads = heads;
    a.d_head = d_head;
    a.window = window;
    a.cur_dev = cur;
    a.max_splits = p.splits;
    a.grid_splits = p.splits;
    a.counters = reinterpret_cast<uint32_t*>(scratch);
    a.part_ml = reinterpret_cast<float*>(scratch + p.ml_off);
    a.part_o = reinterpret_cast<float*>(scratch + p.o_off);
    a.out = out;
    a.ld_out = ld_out;
    e = launch_decode_attn(a, s, false);
  }
  if (e != cudaSuccess) {
    *err = std::string("decode attention launch: ") + cudaGetErrorString(e);
    return MTJ_ERR_CUDA;
  }
  return MTJ_OK;
}

}  // namespace mtj

extern "C" {

int32_t mtj_set_error(int32_t code, const char* msg);   // defined next to mtj_last_error

int64_t mtj_k_decode_attn_scratch_bytes(int32_t batch, int32_t heads, int32_t d_head, int32_t window,
                                        int32_t split_tokens) {
  mtj::DecodeAttnPlan p;
  std::string err;
  if (mtj::plan_decode_attn(batch, heads, d_head, window, split_tokens, &p, &err)) return -1;
  return p.total;
}

int32_t mtj_k_decode_attn(const float* q, const void* kpool, const void* vpool, const int32_t* page_table,
                          const int32_t* pad, const int32_t* cur, int32_t batch, int32_t heads,
                          int32_t d_head, int32_t window, int32_t ring_pages, int32_t split_tokens,
                          void* scratch, int64_t scratch_bytes, float* out, int32_t ld_out, mtj_stream s) {
  if (!q || !kpool || !vpool || !page_table || !pad || !cur || !scratch || !out || ring_pages <= 0)
    return mtj_set_error(MTJ_ERR_INVALID, "null argument");
  mtj::DecodeAttnPlan p;
  std::string err;
  int32_t rc = mtj::plan_decode_attn(batch, heads, d_head, window, split_tokens, &p, &err);
  if (rc) return mtj_set_error(rc, err.c_str());
  if (scratch_bytes < p.total || (reinterpret_cast<uintptr_t>(scratch) & 255))
    return mtj_set_error(MTJ_ERR_INVALID, "scratch too small or not 256-byte aligned");
  rc = mtj::run_decode_attn(p, static_cast<char*>(scratch), q, kpool, vpool, page_table, pad, cur, batch,
                            heads, d_head, window, ring_pages, split_tokens, out, ld_out,
                            static_cast<cudaStream_t>(s), &err);
  return rc ? mtj_set_error(rc, err.c_str()) : MTJ_OK;
}


int32_t mtj_k_ln_gemv(const void* w, const float* x, const float* stats, const float* ln_scale,
                      const float* ln_offset, const float* bias, int32_t M, int32_t N, int32_t K,
                      int32_t k_split, int32_t rows_per_group, float* out, mtj_stream s) {
  if (!w || !x || !stats || !ln_scale || !ln_offset || !bias || !out)
    return mtj_set_error(MTJ_ERR_INVALID, "null argument");
  mtj::GemvArgs a = {};
  a.W = static_cast<const __nv_bfloat16*>(w);
  a.N = N;
  a.K = K;
  a.M = M;
  a.x = x;
  a.ldx = K;
  a.ln_scale = ln_scale;
  a.ln_offset = ln_offset;
  a.stats = stats;
  a.bias = bias;
  a.logits = out;
  a.ld_logits = N;
  a.ks_override = k_split;
  a.rw_override = rows_per_group;
  cudaError_t e = mtj::launch_gemv(mtj::kEpiLogits, a, static_cast<cudaStream_t>(s), false);
  if (e != cudaSuccess) return mtj_set_error(MTJ_ERR_CUDA, cudaGetErrorString(e));
  return MTJ_OK;
}


int32_t mtj_k_gemm_tc(const void* w, const void* x, const float* bias, int32_t M, int32_t N, int32_t K,
                      float* out, mtj_stream s) {
  if (!w || !x || !bias || !out) return mtj_set_error(MTJ_ERR_INVALID, "null argument");
  if (M <= 0 || N <= 0 || K <= 0 || K % 64) return mtj_set_error(MTJ_ERR_INVALID, "K must be a positive multiple of 64");
  struct alignas(64) Map { unsigned char b[128]; } mw, mx;
  const bool wide = M > 192;     // same rule as the model: long chunks take the persistent 128 x 256 kernel
  if (mtj::make_tensor_map_bf16(&mw, w, N, K, 128) != cudaSuccess ||
      mtj::make_tensor_map_bf16(&mx, x, M, K, wide ? mtj::gemm_tc_wide_token_tile() : mtj::gemm_tc_token_tile_for(M)) !=
          cudaSuccess)
    return mtj_set_error(MTJ_ERR_CUDA, "cuTensorMapEncodeTiled failed (pointers must be 16-byte aligned)");
  mtj::GemmTcArgs a = {};
  a.M = M;
  a.N = N;
  a.K = K;
  a.bias = bias;
  a.out = out;
  a.ld_out = N;
  a.cluster_k = mtj::gemm_tc_decode_cluster_k(N, M, K);     // the rule the decode step uses (1 for M > 64)
  a.pair = 1;
  cudaError_t e = wide ? mtj::launch_gemm_tc_wide(mtj::kEpiLogits, &mw, &mx, a, static_cast<cudaStream_t>(s))
                       : mtj::launch_gemm_tc(mtj::kEpiLogits, &mw, &mx, a, static_cast<cudaStream_t>(s), false);
  if (e != cudaSuccess) return mtj_set_error(MTJ_ERR_CUDA, cudaGetErrorString(e));
  return MTJ_OK;
}


int32_t mtj_k_rng_uniforms(uint64_t seed, int32_t position, int32_t rows, int32_t vocab, float* out, mtj_stream s) {
  if (!out || rows <= 0 || vocab <= 0 || position < 0) return mtj_set_error(MTJ_ERR_INVALID, "bad argument");
  cudaError_t e = mtj::launch_rng_uniforms(seed, position, rows, vocab, out, static_cast<cudaStream_t>(s));
  if (e != cudaSuccess) return mtj_set_error(MTJ_ERR_CUDA, cudaGetErrorString(e));
  return MTJ_OK;
}

int32_t mtj_nucleus_filter(const float* logits, const float* top_p, const int32_t* top_k, int32_t rows, int32_t vocab,
                           float* filtered_out, mtj_stream s) {
  if (!logits || !top_p || !filtered_out) return mtj_set_error(MTJ_ERR_INVALID, "null argument");
  if (rows <= 0 || vocab <= 0) return mtj_set_error(MTJ_ERR_INVALID, "rows and vocab must be positive");
  cudaError_t e = mtj::launch_nucleus_filter(logits, top_p, top_k, rows, vocab, filtered_out, static_cast<cudaStream_t>(s));
  if (e != cudaSuccess) return mtj_set_error(MTJ_ERR_CUDA, cudaGetErrorString(e));
  return MTJ_OK;
}

int32_t mtj_k_prefill_attn(const void* q_bf16, const void* kpool, const void* vpool, int32_t n_pages,
                           const int32_t* page_table, const int32_t* pad, const int32_t* key_limit,
                           int32_t batch, int32_t T, int32_t pos0, int32_t heads, int32_t d_head,
                           int32_t ring_pages, void* out_bf16, int32_t ld_out, uint32_t* status,
                           mtj_stream s) {
  if (!q_bf16 || !kpool || !vpool || !page_table || !pad || !out_bf16)
    return mtj_set_error(MTJ_ERR_INVALID, "null argument");
  if (d_head != 256) return mtj_set_error(MTJ_ERR_UNSUPPORTED, "the tensor-core attention is built for d_head 256");
  if (batch <= 0 || T <= 0 || pos0 < 0 || heads <= 0 || n_pages <= 0 || ring_pages <= 0 ||
      ld_out < heads * d_head || (ld_out & 7))
    return mtj_set_error(MTJ_ERR_INVALID, "bad shape (ld_out must cover heads * d_head and be a multiple of 8)");
  if (pos0 + T > ring_pages * mtj::kPageTokens)
    return mtj_set_error(MTJ_ERR_INVALID, "pos0 + T exceeds the positions the page ring holds");
  struct alignas(64) Map { unsigned char b[128]; } mq, mk, mv;
  const int64_t M = static_cast<int64_t>(batch) * T;
  const int64_t pool_rows = static_cast<int64_t>(n_pages) * heads * mtj::kPageTokens;
  if (mtj::make_tensor_map_bf16(&mq, q_bf16, M, static_cast<int64_t>(heads) * d_head, 128) != cudaSuccess ||
      mtj::make_tensor_map_bf16(&mk, kpool, pool_rows, d_head, 64) != cudaSuccess ||
      mtj::make_tensor_map_bf16(&mv, vpool, pool_rows, d_head, 64) != cudaSuccess)
    return mtj_set_error(MTJ_ERR_CUDA, "cuTensorMapEncodeTiled failed (pointers must be 16-byte aligned)");
  mtj::PrefillAttnTcArgs p = {};
  p.kv.kpool = static_cast<__nv_bfloat16*>(const_cast<void*>(kpool));
  p.kv.vpool = static_cast<__nv_bfloat16*>(const_cast<void*>(vpool));
  p.kv.page_table = page_table;
  p.kv.ring_pages = ring_pages;
  p.kv.pad = pad;
  p.rows = {0, T, pos0, nullptr};
  p.M = static_cast<int>(M);
  p.heads = heads;
  p.d_head = d_head;
  p.key_limit = key_limit;
  p.out_bf16 = static_cast<__nv_bfloat16*>(out_bf16);
  p.ld_out = ld_out;
  p.dev_err = status;
  cudaError_t e = mtj::launch_prefill_attn_tc(&mq, &mk, &mv, p, static_cast<cudaStream_t>(s));
  if (e != cudaSuccess) return mtj_set_error(MTJ_ERR_CUDA, cudaGetErrorString(e));
  return MTJ_OK;
}

}  // extern "C"
