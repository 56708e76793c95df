// Shared between the unit entry points: scratch layout of the split-KV decode
// attention (arrival counters | per-split (max, sum) | per-split weighted V).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace mtj {

struct DecodeAttnPlan {
  int32_t splits;
  int64_t counters_bytes, ml_off, o_off, total;
};

int32_t plan_decode_attn(int32_t batch, int32_t heads, int32_t d_head, int32_t window,
                         int32_t split_tokens, DecodeAttnPlan* p, std::string* err);

int32_t run_decode_attn(const DecodeAttnPlan& p, char* scratch, const float* q, const void* kpool,
                        const void* vpool, const int32_t* page_table, const int32_t* pad,
                        const int32_t* cur, int32_t batch, int32_t heads, int32_t d_head, int32_t window,
                        int32_t ring_pages, int32_t split_tokens, float* out, int32_t ld_out,
                        cudaStream_t s, std::string* err);

}  // namespace mtj
