// Host-side launcher interface of the sm_100a kernels (internal to libmtj_b200).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mtj {

// Rows of a forward chunk: row m belongs to sequence b0 + m / Tc and sits at
// absolute position pos0 + m % Tc, where pos0 = *pos0_dev when that pointer is
// set (decode: the step counter lives on the device so that a captured graph
// can be replayed) and pos0_host otherwise (prefill / eval).
struct RowMap {
  int b0;
  int Tc;
  int pos0_host;
  const int32_t* pos0_dev;
};

struct KvCache {
  __nv_bfloat16* kpool;        // [pages][heads][kPageTokens][d_head], one layer
  __nv_bfloat16* vpool;
  const int32_t* page_table;   // [batch][ring_pages]
  int ring_pages;
  const int32_t* pad;          // [batch] first valid absolute position
};

enum GemvEpilogue { kEpiInProj = 0, kEpiOut = 1, kEpiLogits = 2,
                    kEpiLogitsCE = 3 };   // logits that are never stored: per (128-entry vocabulary group, token) max and
                                          // sum of exp instead, plus the target's logit (persistent GEMM only)

struct GemvArgs {
  // y[m, n] = sum_k W[n, k] * act(x[m, k]);  W is bf16 [N, K] (K contiguous).
  const __nv_bfloat16* W;      // first row of this launch
  int N, K, M;                 // N = rows covered by this launch
  int n0;                      // index of W's first row within the full projection (epilogue indexing)
  const float* x;              // [M, ldx] fp32
  int ldx;
  // LayerNorm prologue (in-proj and logits): act(x) = scale*rstd*(x-mean)+offset
  const float* ln_scale;
  const float* ln_offset;
  const float* stats;          // [M, 2] = (mean, rstd)
  RowMap rows;
  // in-proj epilogue: N = 3*dl + ffl laid out [Q | K | V | FF-in]
  int dl, ffl, d_head, heads, rot;
  const float2* sincos;        // [positions][rot/2] = (sin, cos)
  const float* b_ff;           // [ffl]
  float* q_out;                // [M, dl]
  float* act2;                 // [M, dl + ffl]: attention vector | gelu(ff)
  KvCache kv;
  // out-proj epilogue: out = acc + bias (+ residual); stats of the finished rows
  const float* bias;           // [N]
  const float* residual;       // [M, N] or null
  float* out;                  // [M, N]
  float* stats_out;            // [M, 2] or null
  uint32_t* counters;          // [ceil(M / tile)] zero-initialised, self-resetting
  // logits epilogue: logits[m, n] = acc + bias[n]
  float* logits;
  int ld_logits;
  const int32_t* row_select;   // optional [M]: source row of x / stats for output row m
  int ks_override;             // 0 = pick the K split from the shape; 1/2/4/8 = force it
  uint32_t* dev_err;           // device error word (bounded waits that ran out), may be null
  const uint32_t* slot_sel;    // optional: out += (*slot_sel & 1) * slot_stride (peer all-reduce slots)
  size_t slot_stride;
  int rw_override;             // 0 = default rows per warp group; 8 = eight rows (single-token launches)
};

cudaError_t launch_gemv(GemvEpilogue epi, const GemvArgs& a, cudaStream_t s, bool pdl);

struct EmbedArgs {
  // id of row m = ids[(rows.b0 + m / rows.Tc) * ids_ld + rows.pos0_host + m % rows.Tc]
  const uint32_t* ids;
  int ids_ld;
  RowMap rows;
  int M, d, vocab_local, vocab_start;
  const __nv_bfloat16* table;  // [vocab_local, d]
  const float* bias;           // [d]
  float* x;                    // [M, d]
  float* stats;                // [M, 2] or null
  const uint32_t* slot_sel;    // optional: x += (*slot_sel & 1) * slot_stride (peer all-reduce slots)
  size_t slot_stride;
};
cudaError_t launch_embed(const EmbedArgs& a, cudaStream_t s, bool pdl);

struct DecodeAttnArgs {
  const float* q;              // [B, heads*d_head] rotated, unscaled
  KvCache kv;
  int B, heads, d_head, window;  // window = seq - 1 key slots
  const int32_t* cur_dev;      // absolute position of the query token
  int max_splits;              // stride of the partial buffers
  int grid_splits;             // blocks per (sequence, head) = decode_attn_splits(window)
  int est_pages;               // optional: pages the sequences hold now (sizes the streaming kernel's blocks), 0 = unknown
  int stream_pages;            // set by the launcher: pages one block of the streaming kernel walks
  float* part_o;               // [B, heads, max_splits, d_head]
  float* part_ml;              // [B, heads, max_splits, 2]
  uint32_t* counters;          // [B*heads] zero-initialised, self-resetting
  float* out;                  // act2 base: out[b*ld_out + head*d_head + j] (fp32), or
  __nv_bfloat16* out_bf16;     // the same element in bf16 (operand of the tensor-core out-proj)
  __nv_bfloat16* out_lo;       // optional, with out_bf16: the bf16 rounding error of that element
  int ld_out;
  uint32_t* dev_err;           // may be null
};
int decode_attn_splits(int window);
cudaError_t launch_decode_attn(const DecodeAttnArgs& a, cudaStream_t s, bool pdl);

struct PrefillAttnArgs {
  const float* q;              // [M, heads*d_head] rotated, unscaled
  KvCache kv;
  RowMap rows;
  int M, heads, d_head;
  const int32_t* key_limit;    // optional [batch]: keys with pos > limit are masked (eval ctx mask)
  float* out;                  // fp32 destination, or
  __nv_bfloat16* out_bf16;     // bf16 destination (operand of the tensor-core out-proj); exactly one is set
  int ld_out;
};
cudaError_t launch_prefill_attn(const PrefillAttnArgs& a, cudaStream_t s);

// Tensor-core causal attention for prefill / eval, d_head = 256 (see mtj_attn_tc.cu).
struct PrefillAttnTcArgs {
  KvCache kv;
  RowMap rows;
  int M, heads, d_head;
  const int32_t* key_limit;    // optional [batch]
  __nv_bfloat16* out_bf16;     // [M, ld_out]
  int ld_out;
  uint32_t* dev_err;
};
cudaError_t launch_prefill_attn_tc(const void* map_q, const void* map_k, const void* map_v,
                                   const PrefillAttnTcArgs& a, cudaStream_t s);

// Persistent whole-step decode kernel (mtj_decode_mega.cu), one GPU, 1-4 sequences.
struct MegaLayer {
  const __nv_bfloat16* w_in;
  const float* b_ff;
  const __nv_bfloat16* w_out;
  const float* b_out;
  const float* ln_scale;
  const float* ln_offset;
  __nv_bfloat16* kpool;
  __nv_bfloat16* vpool;
};
constexpr int kMegaPushRows = 4;       // sequences per source rank in the push exchange
struct MegaArgs {
  int L, d, dl, ffl, heads, dh, rot, V, B, window, ring_pages;
  int grid_splits, split_tokens, max_splits;   // attention: splits per (sequence, head), keys per split
  const MegaLayer* layers;     // device array [L]
  const __nv_bfloat16* emb_w;
  const float* emb_b;
  const float* lnf_scale;
  const float* lnf_offset;
  const __nv_bfloat16* proj_w;
  const float* proj_b;
  const float2* sincos;
  const uint32_t* tokens;      // [B]
  const int32_t* cur;
  const int32_t* pad;
  const int32_t* page_table;
  float* x;                    // [B, d]
  float* q;                    // [B, dl]
  float* act2;                 // [B, dl + ffl]
  float* part_o;
  float* part_ml;
  uint32_t* head_counters;     // [B * heads], zero between launches
  float* logits;               // [B, V]
  // greedy token inside the kernel (one GPU): per-row running maximum (zero between launches), the token buffer
  // the last block writes (may be the buffer `tokens` points to) and the position counter it advances; or null
  int ff_row_units;            // 256-thread build: FF-in rows one at a time behind a levelling pair (tensor-parallel slices)
  unsigned long long* amax;    // [4]
  uint32_t* tokens_out;        // [B]
  int32_t* cur_out;
  uint32_t* sync;              // [5 L + 3] phase arrival counters, zero between launches
  // tensor parallel (world > 1): the peer exchange buffers of mtj_p2p.cu
  int rank, world, vocab_start;
  float* slot_base;            // this rank's two data slots
  size_t slot_elems;
  const float* peer_data[8];
  uint32_t* peer_flags[8];
  const uint32_t* local_flags;
  uint32_t* seq;
  // push exchange of the layer all-reduce (null pointers: fall back to the slot protocol): every rank owns
  // recv [2 slots][world sources][kMegaPushRows * d] packets of (value, exchange number + 1)
  uint2* peer_recv[8];
  unsigned long long* trace;   // optional [6 L + 3] phase time stamps of block 0 (ns)
  uint32_t* dev_err;
  int wait_limit;              // spins before a wait on a phase counter, flag or packet gives up
};
cudaError_t launch_decode_mega(const MegaArgs& a, cudaStream_t s, int* grid_out);
// the same kernel built with one 512-thread block per SM (one sequence only); launch_decode_mega picks it on one GPU
cudaError_t launch_decode_mega_wide(const MegaArgs& a, cudaStream_t s, int* grid_out);

struct ArgmaxArgs {
  const float* logits;         // [B, V]
  int B, V;
  uint32_t* tokens;            // [B]
  uint32_t* tokens_copy;       // optional second destination
  int32_t* cur_dev;            // incremented by one after the step (may be null)
};
cudaError_t launch_argmax(const ArgmaxArgs& a, cudaStream_t s, bool pdl);

// Tensor-core GEMM (many token rows): weights bf16 [N, K], activations bf16 [*, K]
// reached through TMA tensor maps; epilogues as in GemvArgs.
struct GemmTcArgs {
  int M, N, K;                 // token rows, weight rows, reduction length (multiple of 64)
  int x_row0;                  // first activation row (TMA row coordinate offset)
  RowMap rows;
  int dl, ffl, d_head, heads, rot;
  const float2* sincos;
  const float* b_ff;
  float* q_out;                // [M, dl] fp32
  __nv_bfloat16* q_bf16;       // optional [M, dl] bf16 copy (operand of the tensor-core attention)
  __nv_bfloat16* act_out;      // [M, dl + ffl] bf16: gelu(ff) goes to columns [dl, dl + ffl)
  __nv_bfloat16* act_lo;       // optional [M, dl + ffl]: bf16 rounding error of act_out (decode epilogue only)
  KvCache kv;
  const float* bias;           // [N] (out-proj, logits)
  const float* residual;       // [M, N] or null
  float* out;                  // out-proj: [M, N]; logits: [M, ld_out]
  int ld_out;
  float* partial;              // split-K: [ksplit, M, N] raw partial sums (out-proj / logits epilogues), or null
  int ksplit;
  // kEpiLogitsCE (ProjectionShard.loss, layers.py:569-593): token row m of this launch is chunk row x_row0 + m
  float* ce_gmax;              // [4 * ceil(N / 128)][ce_ld] max over the group's 32 logits, per token row
  float* ce_gsum;              // same shape: sum of exp(logit - that max)
  int ce_ld;                   // row stride of the two arrays (>= M)
  float* ce_tlogit;            // [M] the target's logit where the target id falls into [ce_vocab_start, + N)
  uint8_t* ce_hit;             // [M] 1 where it does (both zeroed by the caller before the launch)
  const uint32_t* ce_targets;  // [batch, ce_T] target ids; row -> (sequence, position) through `rows`
  int ce_T, ce_vocab_start;
  int cluster_k;               // 2 or 4 (token tiles of at most 64 rows, partial == null): split K over a cluster of
                               // blocks that add their accumulators in shared memory before the fused epilogue
  int pair;                    // wide kernel only: 1 = clusters of 2 blocks on 256 x 256 tiles (tcgen05 cta_group::2)
  uint32_t* dev_err;
};
int gemm_tc_token_tile();                 // widest token tile of launch_gemm_tc (128)
// Token tile launch_gemm_tc uses for M rows (32, 64 or 128): map_x must have been made with this box_rows.
int gemm_tc_token_tile_for(int M);
// Cluster split-K factor (1, 2 or 4) launch_gemm_tc should be given for a decode-size GEMM (GemmTcArgs.cluster_k).
int gemm_tc_decode_cluster_k(int weight_rows, int M, int K);
cudaError_t launch_splitk_reduce(const float* partial, int ksplit, int M, int N, const float* bias,
                                 const float* residual, float* out, int ld_out, const uint32_t* slot_sel,
                                 size_t slot_stride, cudaStream_t s, bool pdl = false);
cudaError_t make_tensor_map_bf16(void* map_out_128B, const void* base, int64_t rows, int64_t K, int box_rows);
// map_x_lo (optional, M <= 64): a second activation view holding the bf16 rounding error of the first
// (x = hi + lo); both are multiplied into the same accumulator.
cudaError_t launch_gemm_tc(GemvEpilogue epi, const void* map_w, const void* map_x, const GemmTcArgs& a,
                           cudaStream_t s, bool pdl, const void* map_x_lo = nullptr);
// Persistent variant for many token rows (tiles of 128 or, as block pairs, 256 weight rows x 256 token rows);
// map_x must have been made with box_rows = gemm_tc_wide_token_tile().  No split-K.
int gemm_tc_wide_token_tile();
cudaError_t launch_gemm_tc_wide(GemvEpilogue epi, const void* map_w, const void* map_x, const GemmTcArgs& a,
                                cudaStream_t s);
cudaError_t launch_ln_rows(const float* x, const float* scale, const float* offset, __nv_bfloat16* out, int rows,
                           int d, cudaStream_t s, bool pdl = false, __nv_bfloat16* out_lo = nullptr);

struct SampleArgs {
  const float* logits;         // [rows, V]
  const float* uniforms;       // [rows, V] in [tiny, 1), or null with rng_seed set
  const uint32_t* rng_seed;    // device, 2 words: key of the counter-based generator (indexed by *cur_dev, row, column)
  const float* top_p;          // [rows]
  const int32_t* top_k;        // [rows] or null (the reference's top_k = None)
  const float* temp;           // [rows]
  int rows, V;
  void* scratch;               // sample_scratch_bytes(rows, V): receives the Gumbel noise of the uniforms
  const float* gumbel;         // set by the launcher
  uint32_t* tokens;            // [rows] (may be null)
  uint32_t* tokens_copy;       // optional second destination
  int32_t* cur_dev;            // incremented by one after the step (may be null)
  float* filtered;             // optional [rows, V]: logits - 1e10 * removed (nucleaus_filter's return value)
};
int64_t sample_scratch_bytes(int rows, int vocab);
// the uniforms that generator yields for (seed, decode position): [rows, V]
cudaError_t launch_rng_uniforms(uint64_t seed, int position, int rows, int V, float* out, cudaStream_t s);
cudaError_t launch_nucleus_filter(const float* logits, const float* top_p, const int32_t* top_k, int rows, int V,
                                  float* filtered, cudaStream_t s);
cudaError_t launch_sample_top_p(const SampleArgs& a, cudaStream_t s, bool pdl);

struct CeArgs {
  const float* logits;         // [rows of this launch, vl] this shard's logits
  int vl, vocab_start;
  RowMap rows;                 // chunk geometry: row m -> (sequence, position)
  int row0;                    // first chunk row covered by `logits`
  int T;                       // targets / outputs are [batch, T]
  const uint32_t* targets;
  float* pmax;                 // [chunk rows] local (then global) max
  float* psum;                 // [chunk rows, 2] sum of exp, target logit
  uint8_t* hit;                // [chunk rows] target id lies in this shard's range
  float* loss_out;             // [batch, T]
  uint8_t* correct_out;        // [batch, T]
};
cudaError_t launch_ce_partial(const CeArgs& a, int rows, cudaStream_t s);
// the same three per-row results from the per-group partials of the fused logits epilogue
// (gmax / gsum [n_groups][ld], tlogit / ghit [rows]) for chunk rows [a.row0, a.row0 + rows)
cudaError_t launch_ce_combine(const CeArgs& a, const float* gmax, const float* gsum, int n_groups, int ld,
                              const float* tlogit, const uint8_t* ghit, int rows, cudaStream_t s);
cudaError_t launch_ce_rescale(const CeArgs& a, const float* lmax, int n, cudaStream_t s);
cudaError_t launch_ce_finalize(const CeArgs& a, int n, cudaStream_t s);

// [K, N] (reference layout, fp32 or bf16) -> bf16 [N, K] at dst + row offset.
cudaError_t launch_pack_transpose(const void* src, int src_is_bf16, int K, int N,
                                  __nv_bfloat16* dst, int ld_dst, int k_offset, cudaStream_t s);
// elementwise copy to fp32 / bf16
cudaError_t launch_to_f32(const void* src, int src_is_bf16, int64_t n, float* dst, cudaStream_t s);
cudaError_t launch_to_bf16(const void* src, int src_is_bf16, int64_t n, __nv_bfloat16* dst,
                           cudaStream_t s);

}  // namespace mtj
