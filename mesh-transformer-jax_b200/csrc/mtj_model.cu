// Model runtime behind the C ABI: weight arena, workspace carving, paged KV
// cache bookkeeping and the per-call kernel sequences (prefill, decode step,
// full-sequence forward).  Host code only; kernels live in the other files.
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../../include/mtj_b200.h"
#include "mtj_comm.h"
#include "mtj_common.cuh"
#include "mtj_kernels.h"

namespace {

thread_local std::string g_last_error;

int32_t fail(int32_t code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

#define MTJ_CUDA(expr)                                                              \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    if (_e != cudaSuccess)                                                          \
      return fail(MTJ_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

constexpr int kTcSplitMax = 8;      // split-K factor limit of the small-M out-projection
constexpr int kTcSplitRows = 128;
constexpr int kHiLoRows = 64;       // decode rows that can carry hi + lo activations
constexpr int kTpPipeMinRows = 128; // a chunk is cut in two for all-reduce overlap only if each half keeps this many rows

struct alignas(64) TensorMap { unsigned char bytes[128]; };   // a CUtensorMap

struct LayerWeights {
  __nv_bfloat16* w_in = nullptr;    // [3*dl + ffl, d]  rows: Q | K | V | FF-in
  float* b_ff = nullptr;            // [ffl]
  __nv_bfloat16* w_out = nullptr;   // [d, dl + ffl]    cols: attn vector | gelu(ff)
  float* b_out = nullptr;           // [d]
  float* ln_scale = nullptr;
  float* ln_offset = nullptr;
  TensorMap map_in, map_out;        // TMA views of w_in / w_out for the tensor-core path
  TensorMap map_k, map_v;           // TMA views of this layer's K / V pools as [pages*heads*64, d_head]
};

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Bump allocator over a caller-provided arena; with base == nullptr it only sizes.
struct Carver {
  char* base;
  int64_t off = 0;
  explicit Carver(void* b) : base(static_cast<char*>(b)) {}
  template <typename T>
  T* take(int64_t count) {
    off = align_up(off, 256);
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * static_cast<int64_t>(sizeof(T));
    return p;
  }
};

}  // namespace

struct mtj_handle {
  mtj_config cfg;
  int L, d, n_heads, heads, dh, rot, V, Vl, seq, W, mp, rank, dl, ffl;
  int max_batch, max_gen, max_rows, ring_pages, n_pages, max_pos, max_splits;

  // weight arena
  __nv_bfloat16* emb_w = nullptr;
  float* emb_b = nullptr;
  std::vector<LayerWeights> layers;
  float* lnf_scale = nullptr;
  float* lnf_offset = nullptr;
  __nv_bfloat16* proj_w = nullptr;
  float* proj_b = nullptr;
  float2* sincos = nullptr;
  std::vector<uint8_t> leaf_loaded;   // one mark per parameter leaf (embedding 2, 10 per layer, projection 4)
  int64_t expected = 0;

  // workspace
  float* x = nullptr;
  float* stats = nullptr;
  float* q = nullptr;
  float* act2 = nullptr;
  float* part_o = nullptr;
  float* part_ml = nullptr;
  uint32_t* counters = nullptr;     // attention + gemv tickets (zeroed at bind)
  uint32_t* gemv_counters = nullptr;
  float* logits = nullptr;          // [max_batch, Vl] this shard's logits
  float* logits_all = nullptr;      // [max_batch, V]  (== logits when mp == 1)
  float* logits_gather = nullptr;   // [mp, max_batch, Vl] all-gather landing zone (mp > 1)
  float* part = nullptr;            // [max_rows, d] this shard's partial sums before the all-reduce (mp > 1)
  void* comm = nullptr;             // ncclComm_t over the "shard" axis
  // peer-memory all-reduce for small messages (decode); buffers are cudaMalloc'ed once at set-up
  // because they have to be exportable to the other ranks' processes
  bool p2p_ready = false;
  int p2p_rows = 0;                 // rows a data slot holds
  char* p2p_local = nullptr;        // [2 slots][p2p_rows * d] floats | flags | seq | ticket
  char* p2p_peer[mtj::kP2pMaxWorld] = {};
  size_t p2p_flag_off = 0;
  size_t p2p_recv_off = 0;          // push exchange of the persistent decode kernel
  size_t p2p_push_off = 0;          // receive area of the per-layer push all-reduce [2][mp][p2p_rows][d] floats
  size_t p2p_pflag_off = 0;         // its row flags [mp][p2p_rows]
  size_t p2p_amax_off = 0;          // greedy-token packets [2][mp][p2p_rows][2] uint2
  bool tp_token = true;             // decode at mp > 1: the greedy token is agreed on by pushing each rank's local
                                    // arg-max to all ranks instead of gathering the logits (MTJ_NO_TP_TOKEN=1: off)
  bool tp_push = false;             // batched decode at mp > 1: push all-reduce fused with the split-K reduction and
                                    // the LayerNorm; default: from 4 shards on (MTJ_TP_PUSH=0 / 1 overrides)
  bool xn_ready = false;            // the bf16 operand of the next projection has already been written
  bool tc_cluster_k = true;         // batched decode: split K over block clusters when tiles are few (MTJ_NO_CLUSTER_K=1: off)
  float* uniforms = nullptr;        // [max_batch, V] sampler inputs of the current step
  float* top_p = nullptr;           // [max_batch]
  float* temp = nullptr;            // [max_batch]
  void* sample_scratch = nullptr;
  // tensor-core path (many token rows): bf16 activation operands and their TMA views
  bool tc_ok = false;
  __nv_bfloat16* xn_bf16 = nullptr;   // [max_rows, d] LayerNorm output
  __nv_bfloat16* act_bf16 = nullptr;  // [max_rows, dl + ffl] attention vector | gelu(ff)
  TensorMap map_xn[3], map_act[3], map_proj, map_q;   // activation views with 32 / 64 / 128-row boxes
  TensorMap map_xn_wide, map_act_wide;   // 256-row boxes for the persistent GEMM
  __nv_bfloat16* q_bf16 = nullptr;    // [max_rows, dl] rotated queries for the tensor-core attention
  bool attn_tc_ok = false;
  // few-sequence decode: the bf16 rounding errors of the two activation operands (x = hi + lo), rows [0, kHiLoRows)
  __nv_bfloat16* xn_lo = nullptr;
  __nv_bfloat16* act_lo = nullptr;
  TensorMap map_xn_lo[2], map_act_lo[2];   // 32 / 64-row boxes
  bool hilo_ok = false;
  int tc_hilo_max_b = kHiLoRows;    // up to this many sequences the activations travel as hi + lo (mtj_config.hilo_max_batch)
  int wait_limit = 1 << 22;         // iteration limit of the bounded device-side waits (mtj_config.wait_limit)
  bool tc_wide_ok = false;   // persistent 128 x 256 GEMM for long chunks
  int tc_pair = 7;           // ... as block pairs on 256 x 256 tiles: bit 0 in-projection, 1 out-projection, 2 logits
                             // (MTJ_TC_PAIR=<mask> overrides, for measurement)
  bool mega_push = true;     // per-block push exchange inside the persistent decode kernel (MTJ_NO_MEGA_PUSH=1: slot protocol)
  float* tc_partial = nullptr;        // [kTcSplitMax, kTcSplitRows, d] split-K partial sums of small-M out-projections
  int eval_rows = 0;                // rows of logits materialised at a time by the loss path
  float* eval_logits = nullptr;     // [eval_rows, Vl]
  // loss path on the persistent GEMM: the logits are never stored, its epilogue leaves per (32-entry vocabulary
  // group, row) the max and the sum of exp, plus the target's logit
  int ce_groups = 0;
  int ce_rows = 0;                  // rows per launch of that GEMM: several 256-row token tiles, so that a block's
                                    // epilogues overlap its next tiles instead of ending the launch
  float* ce_gmax = nullptr;         // [ce_groups, ce_rows]
  float* ce_gsum = nullptr;
  float* ce_tlogit = nullptr;       // [ce_rows]
  uint8_t* ce_ghit = nullptr;       // [ce_rows]
  bool fused_ce = true;             // MTJ_NO_FUSED_CE=1: materialise the logits slice and run ce_partial instead
  float* ce_max = nullptr;          // [max_rows] local max, then global max
  float* ce_lmax = nullptr;         // [max_rows] copy of the local max (mp > 1)
  float* ce_sum = nullptr;          // [max_rows, 2]
  uint8_t* ce_hit = nullptr;        // [max_rows]
  uint32_t* tokens = nullptr;       // [max_batch] next decode input
  int32_t* cur = nullptr;           // absolute position of the next decode token
  int32_t* pad = nullptr;           // [max_batch]
  int32_t* key_limit = nullptr;     // [max_batch]
  int32_t* page_table = nullptr;    // [max_batch, ring_pages]
  int32_t* row_select = nullptr;    // [max_rows]
  uint32_t* dev_err = nullptr;
  uint32_t* rng_seed = nullptr;     // [2] key of the device generator that draws the sampler's uniforms
  int32_t* top_k = nullptr;         // [max_batch] the sampler's top_k, used while has_top_k
  bool has_top_k = false;
  __nv_bfloat16* kpool = nullptr;   // [L][n_pages][heads][kPageTokens][dh]
  __nv_bfloat16* vpool = nullptr;
  int64_t pool_layer_elems = 0;
  bool bound = false;

  // decode state
  int min_pad = 0;                  // smallest first-visible position over the running sequences
  // pages a sequence of the running batch holds at most right now (its window start to the decode position)
  int est_pages() const {
    const int cur = W + steps_done;
    const int start = std::max(min_pad, cur - W + 1);
    return cur / mtj::kPageTokens - start / mtj::kPageTokens + 1;
  }
  int batch = 0;
  bool prefilled = false;
  int steps_done = 0;
  int64_t launches = 0;
  bool use_pdl = true;
  int ks_inproj = 0, ks_out = 0, ks_logits = 0;   // K-split overrides (tuning; 0 = automatic)
  // decode of 1-4 sequences on one GPU: the whole step as one persistent kernel
  bool use_mega = true;
  bool mega_token = true;                  // greedy token picked inside the whole-step kernel (MTJ_NO_MEGA_TOKEN=1: separate kernel)
  mtj::MegaLayer* mega_layers = nullptr;   // device copy of the per-layer pointers
  uint32_t* mega_sync = nullptr;           // [5 L + 3] phase counters
  unsigned long long* mega_amax = nullptr; // [4] running maxima of the in-kernel greedy token
  unsigned long long* mega_trace = nullptr;  // [6 L + 3] phase time stamps (profiling read-out)
  bool mega_trace_on = false;
  // decode: attention runs on a side stream next to the FF half of the in-projection
  bool fork_attn = true;
  int mega_max_b = 1;               // sequences the whole-step decode kernel is used for (mtj_config.mega_max_batch, up to 4)
  int tc_decode_min_b = 2;          // from this many sequences on decode takes the tensor-core GEMM path (mtj_config.tc_decode_min_batch)
  bool tc_pdl = true;               // programmatic dependent launch on the tensor-core decode chain (MTJ_NO_TC_PDL=1: off)
  bool fork_pdl = false;            // let the out-projection start early although it also waits on the side stream
  cudaStream_t side_stream = nullptr;
  // tensor-parallel prefill / eval: two row chunks are in flight, the all-reduce of one (on comm_stream)
  // overlapping the layer of the other.  A view = one half of the row-indexed activation buffers.
  struct ActView {
    float *x, *stats, *part, *q;
    __nv_bfloat16 *xn_bf16, *act_bf16, *q_bf16;
    TensorMap map_xn[3], map_act[3], map_xn_wide, map_act_wide, map_q;
  };
  ActView views[2];
  bool views_ok = false;
  int view_rows[2] = {0, 0};
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ev_layer[2] = {nullptr, nullptr}, ev_reduced[2] = {nullptr, nullptr};
  bool tp_pipe = false;             // overlap the all-reduce of one chunk with the layer of the next; default: from 4
                                    // shards on (MTJ_TP_PIPE=0 / 1 overrides)
  void save_view(int i) {
    ActView& v = views[i];
    v.x = x; v.stats = stats; v.part = part; v.q = q; v.xn_bf16 = xn_bf16; v.act_bf16 = act_bf16; v.q_bf16 = q_bf16;
    for (int k = 0; k < 3; ++k) { v.map_xn[k] = map_xn[k]; v.map_act[k] = map_act[k]; }
    v.map_xn_wide = map_xn_wide; v.map_act_wide = map_act_wide; v.map_q = map_q;
  }
  void use_view(int i) {
    const ActView& v = views[i];
    x = v.x; stats = v.stats; part = v.part; q = v.q; xn_bf16 = v.xn_bf16; act_bf16 = v.act_bf16; q_bf16 = v.q_bf16;
    for (int k = 0; k < 3; ++k) { map_xn[k] = v.map_xn[k]; map_act[k] = v.map_act[k]; }
    map_xn_wide = v.map_xn_wide; map_act_wide = v.map_act_wide; map_q = v.map_q;
  }
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;

  // decode step captured once per batch size and replayed (the step counter,
  // tokens and page table live on the device, so the graph never changes)
  bool use_graph = true;
  cudaStream_t capture_stream = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  int graph_batch = 0;
  int graph_greedy = -1;
  int64_t graph_kernels = 0;

  // optional per-family kernel timing (mtj_profile_*): events around launches
  bool profile = false;
  std::vector<cudaEvent_t> ev_pool;
  size_t ev_used = 0;
  std::vector<std::pair<int, std::pair<size_t, size_t>>> ev_spans;   // (family, (start, stop))

  void prof_begin(int family, cudaStream_t s) {
    if (!profile || ev_used + 2 > ev_pool.size()) return;
    cudaEventRecord(ev_pool[ev_used], s);
    ev_spans.push_back({family, {ev_used, ev_used + 1}});
    ev_used += 2;
  }
  void prof_end(cudaStream_t s) {
    if (!profile || ev_spans.empty()) return;
    cudaEventRecord(ev_pool[ev_spans.back().second.second], s);
  }

  void carve_weights(Carver& c) {
    emb_w = c.take<__nv_bfloat16>(static_cast<int64_t>(Vl) * d);
    emb_b = c.take<float>(d);
    layers.resize(L);
    for (auto& lw : layers) {
      lw.w_in = c.take<__nv_bfloat16>(static_cast<int64_t>(3 * dl + ffl) * d);
      lw.b_ff = c.take<float>(ffl);
      lw.w_out = c.take<__nv_bfloat16>(static_cast<int64_t>(d) * (dl + ffl));
      lw.b_out = c.take<float>(d);
      lw.ln_scale = c.take<float>(d);
      lw.ln_offset = c.take<float>(d);
    }
    lnf_scale = c.take<float>(d);
    lnf_offset = c.take<float>(d);
    proj_w = c.take<__nv_bfloat16>(static_cast<int64_t>(Vl) * d);
    proj_b = c.take<float>(Vl);
    sincos = c.take<float2>(static_cast<int64_t>(max_pos) * (rot / 2));
  }

  void carve_workspace(Carver& c) {
    const int64_t R = max_rows;
    x = c.take<float>(R * d);
    stats = c.take<float>(R * 2);
    q = c.take<float>(R * dl);
    act2 = c.take<float>(R * (dl + ffl));
    part_o = c.take<float>(static_cast<int64_t>(max_batch) * heads * max_splits * dh);
    part_ml = c.take<float>(static_cast<int64_t>(max_batch) * heads * max_splits * 2);
    counters = c.take<uint32_t>(static_cast<int64_t>(max_batch) * heads);
    gemv_counters = c.take<uint32_t>(R);
    logits = c.take<float>(static_cast<int64_t>(std::max(max_batch, 1)) * Vl);
    logits_all = logits;
    if (mp > 1) {
      logits_all = c.take<float>(static_cast<int64_t>(max_batch) * V);
      logits_gather = c.take<float>(static_cast<int64_t>(max_batch) * V);
      part = c.take<float>(R * d);
    }
    uniforms = c.take<float>(static_cast<int64_t>(max_batch) * V);
    top_p = c.take<float>(max_batch);
    temp = c.take<float>(max_batch);
    sample_scratch = c.take<char>(mtj::sample_scratch_bytes(max_batch, V));
    tc_partial = c.take<float>(static_cast<int64_t>(kTcSplitMax) * std::min<int64_t>(R, kTcSplitRows) * d);
    q_bf16 = c.take<__nv_bfloat16>(R * dl);
    xn_bf16 = c.take<__nv_bfloat16>(R * d);
    act_bf16 = c.take<__nv_bfloat16>(R * (dl + ffl));
    xn_lo = c.take<__nv_bfloat16>(std::min<int64_t>(R, kHiLoRows) * d);
    act_lo = c.take<__nv_bfloat16>(std::min<int64_t>(R, kHiLoRows) * (dl + ffl));
    eval_rows = static_cast<int>(std::min<int64_t>(R, 256));
    eval_logits = c.take<float>(static_cast<int64_t>(eval_rows) * Vl);
    ce_groups = 4 * ((Vl + 127) / 128);
    ce_rows = static_cast<int>(std::min<int64_t>(R, 1024));
    ce_gmax = c.take<float>(static_cast<int64_t>(ce_groups) * ce_rows);
    ce_gsum = c.take<float>(static_cast<int64_t>(ce_groups) * ce_rows);
    ce_tlogit = c.take<float>(ce_rows);
    ce_ghit = c.take<uint8_t>(ce_rows);
    ce_max = c.take<float>(R);
    ce_lmax = c.take<float>(R);
    ce_sum = c.take<float>(R * 2);
    ce_hit = c.take<uint8_t>(R);
    mega_layers = c.take<mtj::MegaLayer>(L);
    mega_sync = c.take<uint32_t>(5 * L + 3);
    mega_amax = c.take<unsigned long long>(4);
    mega_trace = c.take<unsigned long long>(6 * L + 3);
    tokens = c.take<uint32_t>(max_batch);
    cur = c.take<int32_t>(4);
    pad = c.take<int32_t>(max_batch);
    key_limit = c.take<int32_t>(max_batch);
    page_table = c.take<int32_t>(static_cast<int64_t>(max_batch) * ring_pages);
    row_select = c.take<int32_t>(R);
    dev_err = c.take<uint32_t>(4);
    rng_seed = c.take<uint32_t>(4);
    top_k = c.take<int32_t>(max_batch);
    pool_layer_elems = static_cast<int64_t>(n_pages) * heads * mtj::kPageTokens * dh;
    kpool = c.take<__nv_bfloat16>(pool_layer_elems * L);
    vpool = c.take<__nv_bfloat16>(pool_layer_elems * L);
  }

  mtj::KvCache kv(int layer) const {
    mtj::KvCache k;
    k.kpool = kpool + pool_layer_elems * layer;
    k.vpool = vpool + pool_layer_elems * layer;
    k.page_table = page_table;
    k.ring_pages = ring_pages;
    k.pad = pad;
    return k;
  }
};

namespace {

using mtj::GemvArgs;

// g_psum of the [M, d] partial sums in h->part, then x (+)= sum and the LN statistics.
bool use_p2p(const mtj_handle* h, int M) { return h->p2p_ready && M <= h->p2p_rows; }
// where the producer of the partial sums writes them: the peer-visible slot or the plain buffer
float* partial_dst(const mtj_handle* h, int M) {
  return use_p2p(h, M) ? reinterpret_cast<float*>(h->p2p_local) : h->part;
}
const uint32_t* partial_slot_sel(const mtj_handle* h, int M) {
  return use_p2p(h, M) ? reinterpret_cast<const uint32_t*>(h->p2p_local + h->p2p_flag_off + 256) : nullptr;
}
size_t partial_slot_stride(const mtj_handle* h) { return static_cast<size_t>(h->p2p_rows) * h->d; }

int32_t reduce_into_x(mtj_handle* h, int M, bool accumulate, bool pdl, cudaStream_t s) {
  if (!h->comm) return fail(MTJ_ERR_STATE, "cores_per_replica > 1 needs mtj_comm_init first");
  if (use_p2p(h, M)) {
    mtj::P2pArgs a = {};
    a.rank = h->rank;
    a.world = h->mp;
    a.d = h->d;
    a.slot_elems = partial_slot_stride(h);
    for (int r = 0; r < h->mp; ++r) {
      a.peer_data[r] = reinterpret_cast<const float*>(h->p2p_peer[r]);
      a.peer_flags[r] = reinterpret_cast<uint32_t*>(h->p2p_peer[r] + h->p2p_flag_off);
    }
    a.local_flags = reinterpret_cast<const uint32_t*>(h->p2p_local + h->p2p_flag_off);
    a.seq = reinterpret_cast<uint32_t*>(h->p2p_local + h->p2p_flag_off + 256);
    a.ticket = a.seq + 1;
    a.x = h->x;
    a.stats = h->stats;
    a.accumulate = accumulate ? 1 : 0;
    a.dev_err = h->dev_err;
    a.wait_limit = h->wait_limit;
    MTJ_CUDA(mtj::launch_p2p_allreduce(a, M, s, pdl));
    h->launches++;
    return MTJ_OK;
  }
  std::string err;
  if (mtj::comm_all_reduce(h->comm, h->part, static_cast<size_t>(M) * h->d, false, s, &err))
    return fail(MTJ_ERR_COMM, err);
  MTJ_CUDA(mtj::launch_residual_stats(h->x, h->part, h->stats, M, h->d, accumulate, s, pdl));
  h->launches += 2;
  return MTJ_OK;
}

// The same g_psum for the batched decode step, push style: split-K partial sums (+ bias) -> every peer's
// receive area -> x (+)= sum, LayerNorm statistics and the normalised bf16 operand of the next projection.
bool use_push(const mtj_handle* h, int M) { return h->tp_push && h->mp > 1 && use_p2p(h, M); }

int32_t push_reduce(mtj_handle* h, int M, const float* partial, int ksplit, const float* bias, bool accumulate,
                    const float* ln_scale, const float* ln_offset, bool hilo, bool pdl, cudaStream_t s) {
  mtj::TpReduceArgs a = {};
  a.rank = h->rank;
  a.world = h->mp;
  a.d = h->d;
  a.rows_cap = h->p2p_rows;
  a.partial = partial;
  a.ksplit = ksplit;
  a.bias = bias;
  for (int r = 0; r < h->mp; ++r) {
    a.peer_recv[r] = reinterpret_cast<float*>(h->p2p_peer[r] + h->p2p_push_off);
    a.peer_flags[r] = reinterpret_cast<uint32_t*>(h->p2p_peer[r] + h->p2p_pflag_off);
  }
  a.seq = reinterpret_cast<uint32_t*>(h->p2p_local + h->p2p_flag_off + 264);
  a.ticket = a.seq + 1;
  a.x = h->x;
  a.stats = h->stats;
  a.accumulate = accumulate ? 1 : 0;
  a.ln_scale = ln_scale;
  a.ln_offset = ln_offset;
  a.xn = ln_scale ? h->xn_bf16 : nullptr;
  a.xn_lo = (ln_scale && hilo) ? h->xn_lo : nullptr;
  a.dev_err = h->dev_err;
  a.wait_limit = h->wait_limit;
  MTJ_CUDA(mtj::launch_tp_push_reduce(a, M, s, pdl));
  h->xn_ready = ln_scale != nullptr;
  h->launches++;
  return MTJ_OK;
}

// One transformer layer over a chunk of rows already in h->x (+ h->stats):
// x <- x + attn(LN(x)) + ff(LN(x))  (layers.py:299-313 / :316-344 / :347-366).
int32_t run_layer(mtj_handle* h, int layer, int M, const mtj::RowMap& rows, bool decode,
                  const int32_t* key_limit, cudaStream_t s, float* detached_out = nullptr) {
  const LayerWeights& lw = h->layers[layer];
  const bool pdl = h->use_pdl && decode;
  GemvArgs a = {};
  a.W = lw.w_in;
  a.N = 3 * h->dl + h->ffl;
  a.K = h->d;
  a.M = M;
  a.x = h->x;
  a.ldx = h->d;
  a.ln_scale = lw.ln_scale;
  a.ln_offset = lw.ln_offset;
  a.stats = h->stats;
  a.rows = rows;
  a.dl = h->dl;
  a.ffl = h->ffl;
  a.d_head = h->dh;
  a.heads = h->heads;
  a.rot = h->rot;
  a.sincos = h->sincos;
  a.b_ff = lw.b_ff;
  a.q_out = h->q;
  a.act2 = h->act2;
  a.kv = h->kv(layer);
  a.dev_err = h->dev_err;
  a.ks_override = decode ? h->ks_inproj : 0;
  // Decode: only the Q/K/V rows have to be finished before attention can start, so the
  // projection is launched in two parts and attention runs beside the FF-in part.
  const bool fork = decode && h->fork_attn;
  if (fork && !h->side_stream) {
    MTJ_CUDA(cudaStreamCreateWithFlags(&h->side_stream, cudaStreamNonBlocking));
    MTJ_CUDA(cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming));
    MTJ_CUDA(cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming));
  }
  cudaStream_t sa = fork ? h->side_stream : s;      // stream of the attention kernel
  h->prof_begin(MTJ_FAMILY_INPROJ, s);
  if (fork) {
    GemvArgs qkv = a;
    qkv.N = 3 * h->dl;
    MTJ_CUDA(mtj::launch_gemv(mtj::kEpiInProj, qkv, s, pdl));
    h->prof_end(s);
    MTJ_CUDA(cudaEventRecord(h->ev_fork, s));
    MTJ_CUDA(cudaStreamWaitEvent(sa, h->ev_fork, 0));
    GemvArgs ffp = a;
    ffp.W = lw.w_in + static_cast<size_t>(3) * h->dl * h->d;
    ffp.N = h->ffl;
    ffp.n0 = 3 * h->dl;
    h->prof_begin(MTJ_FAMILY_FFIN, s);
    MTJ_CUDA(mtj::launch_gemv(mtj::kEpiInProj, ffp, s, pdl));
    h->prof_end(s);
    h->launches++;
  } else {
    MTJ_CUDA(mtj::launch_gemv(mtj::kEpiInProj, a, s, pdl));
    h->prof_end(s);
  }
  h->launches++;

  if (decode) {
    mtj::DecodeAttnArgs d = {};
    d.q = h->q;
    d.kv = h->kv(layer);
    d.B = M;
    d.heads = h->heads;
    d.d_head = h->dh;
    d.window = h->W;
    d.cur_dev = h->cur;
    d.max_splits = h->max_splits;
    d.grid_splits = std::min(mtj::decode_attn_splits(h->W), h->ring_pages);
    d.est_pages = h->est_pages();
    d.dev_err = h->dev_err;
    d.part_o = h->part_o;
    d.part_ml = h->part_ml;
    d.counters = h->counters;
    d.out = h->act2;
    d.ld_out = h->dl + h->ffl;
    h->prof_begin(MTJ_FAMILY_ATTN, sa);
    MTJ_CUDA(mtj::launch_decode_attn(d, sa, pdl && !fork));
    h->prof_end(sa);
    if (fork) {
      MTJ_CUDA(cudaEventRecord(h->ev_join, sa));
      MTJ_CUDA(cudaStreamWaitEvent(s, h->ev_join, 0));
    }
  } else {
    mtj::PrefillAttnArgs p = {};
    p.q = h->q;
    p.kv = h->kv(layer);
    p.rows = rows;
    p.M = M;
    p.heads = h->heads;
    p.d_head = h->dh;
    p.key_limit = key_limit;
    p.out = h->act2;
    p.ld_out = h->dl + h->ffl;
    h->prof_begin(MTJ_FAMILY_ATTN, s);
    MTJ_CUDA(mtj::launch_prefill_attn(p, s));
    h->prof_end(s);
  }
  h->launches++;

  GemvArgs o = {};
  o.W = lw.w_out;
  o.N = h->d;
  o.K = h->dl + h->ffl;
  o.M = M;
  o.x = h->act2;
  o.ldx = h->dl + h->ffl;
  o.rows = rows;
  o.bias = lw.b_out;
  // detached_out: return g_psum(attn + ff) on its own instead of adding it to the residual stream
  o.residual = (h->mp == 1 && !detached_out) ? h->x : nullptr;
  o.out = h->mp == 1 ? (detached_out ? detached_out : h->x) : (detached_out ? h->part : partial_dst(h, M));
  if (h->mp > 1 && !detached_out) {
    o.slot_sel = partial_slot_sel(h, M);
    o.slot_stride = partial_slot_stride(h);
  }
  o.stats_out = (h->mp == 1 && !detached_out) ? h->stats : nullptr;
  o.counters = h->gemv_counters;
  o.dev_err = h->dev_err;
  o.ks_override = decode ? h->ks_out : 0;
  h->prof_begin(MTJ_FAMILY_OUTPROJ, s);
  MTJ_CUDA(mtj::launch_gemv(mtj::kEpiOut, o, s, pdl && (!fork || h->fork_pdl)));
  h->prof_end(s);
  h->launches++;
  if (h->mp > 1 && detached_out) {
    std::string err;
    if (mtj::comm_all_reduce(h->comm, h->part, static_cast<size_t>(M) * h->d, false, s, &err))
      return fail(MTJ_ERR_COMM, err);
    MTJ_CUDA(cudaMemcpyAsync(detached_out, h->part, sizeof(float) * M * h->d, cudaMemcpyDeviceToDevice, s));
    return MTJ_OK;
  }
  if (h->mp > 1) return reduce_into_x(h, M, true, pdl, s);
  return MTJ_OK;
}

int tc_tile_index(int M) { return mtj::gemm_tc_token_tile_for(M) == 32 ? 0 : (mtj::gemm_tc_token_tile_for(M) == 64 ? 1 : 2); }
bool use_tc_wide(const mtj_handle* h, int M) { return h->tc_wide_ok && M > 192; }

// The same layer for many token rows on the tensor cores: LayerNorm to bf16, in-proj GEMM
// (RoPE / KV / GELU epilogue), causal attention, out-proj GEMM (+ bias + residual).
int32_t run_layer_tc(mtj_handle* h, int layer, int M, const mtj::RowMap& rows, const int32_t* key_limit,
                     cudaStream_t s, float* detached_out = nullptr, bool decode = false, bool defer_reduce = false) {
  LayerWeights& lw = h->layers[layer];
  // decode (graph-replayed, launch-latency sensitive): every kernel of the chain waits on its predecessor with
  // griddepcontrol.wait, so each may be scheduled while the previous one drains
  const bool pdl = h->use_pdl && h->tc_pdl && decode;
  // few sequences: activations go through the GEMMs as hi + lo bf16 pairs
  const bool hilo = decode && h->hilo_ok && M <= h->tc_hilo_max_b;
  if (h->xn_ready)
    h->xn_ready = false;            // the previous exchange has already written this layer's operand
  else
    MTJ_CUDA(mtj::launch_ln_rows(h->x, lw.ln_scale, lw.ln_offset, h->xn_bf16, M, h->d, s, pdl, hilo ? h->xn_lo : nullptr));
  mtj::GemmTcArgs a = {};
  a.M = M;
  a.N = 3 * h->dl + h->ffl;
  a.K = h->d;
  a.rows = rows;
  a.dl = h->dl;
  a.ffl = h->ffl;
  a.d_head = h->dh;
  a.heads = h->heads;
  a.rot = h->rot;
  a.sincos = h->sincos;
  a.b_ff = lw.b_ff;
  a.q_out = h->q;
  a.q_bf16 = (h->attn_tc_ok && !decode) ? h->q_bf16 : nullptr;
  a.act_out = h->act_bf16;
  a.act_lo = hilo ? h->act_lo : nullptr;
  a.kv = h->kv(layer);
  a.dev_err = h->dev_err;
  a.cluster_k = (decode && h->tc_cluster_k) ? mtj::gemm_tc_decode_cluster_k(a.N, M, a.K) : 1;
  h->prof_begin(MTJ_FAMILY_INPROJ, s);
  const bool wide = use_tc_wide(h, M) && !decode;
  a.pair = h->tc_pair & 1;
  if (wide)
    MTJ_CUDA(mtj::launch_gemm_tc_wide(mtj::kEpiInProj, &lw.map_in, &h->map_xn_wide, a, s));
  else
    MTJ_CUDA(mtj::launch_gemm_tc(mtj::kEpiInProj, &lw.map_in, &h->map_xn[tc_tile_index(M)], a, s, pdl,
                                 hilo ? &h->map_xn_lo[tc_tile_index(M)] : nullptr));
  h->prof_end(s);

  h->prof_begin(MTJ_FAMILY_ATTN, s);
  if (decode) {
    mtj::DecodeAttnArgs d = {};
    d.q = h->q;
    d.kv = h->kv(layer);
    d.B = M;
    d.heads = h->heads;
    d.d_head = h->dh;
    d.window = h->W;
    d.cur_dev = h->cur;
    d.max_splits = h->max_splits;
    d.grid_splits = std::min(mtj::decode_attn_splits(h->W), h->ring_pages);
    d.est_pages = h->est_pages();
    d.dev_err = h->dev_err;
    d.part_o = h->part_o;
    d.part_ml = h->part_ml;
    d.counters = h->counters;
    d.out_bf16 = h->act_bf16;
    d.out_lo = hilo ? h->act_lo : nullptr;
    d.ld_out = h->dl + h->ffl;
    MTJ_CUDA(mtj::launch_decode_attn(d, s, pdl));
  } else if (h->attn_tc_ok) {
    mtj::PrefillAttnTcArgs p = {};
    p.kv = h->kv(layer);
    p.rows = rows;
    p.M = M;
    p.heads = h->heads;
    p.d_head = h->dh;
    p.key_limit = key_limit;
    p.out_bf16 = h->act_bf16;
    p.ld_out = h->dl + h->ffl;
    p.dev_err = h->dev_err;
    MTJ_CUDA(mtj::launch_prefill_attn_tc(&h->map_q, &lw.map_k, &lw.map_v, p, s));
  } else {
    mtj::PrefillAttnArgs p = {};
    p.q = h->q;
    p.kv = h->kv(layer);
    p.rows = rows;
    p.M = M;
    p.heads = h->heads;
    p.d_head = h->dh;
    p.key_limit = key_limit;
    p.out_bf16 = h->act_bf16;
    p.ld_out = h->dl + h->ffl;
    MTJ_CUDA(mtj::launch_prefill_attn(p, s));
  }
  h->prof_end(s);

  mtj::GemmTcArgs o = {};
  o.M = M;
  o.N = h->d;
  o.K = h->dl + h->ffl;
  o.bias = lw.b_out;
  o.residual = (h->mp == 1 && !detached_out) ? h->x : nullptr;
  const bool to_slot = h->mp > 1 && !detached_out && use_p2p(h, M);
  o.out = h->mp == 1 ? (detached_out ? detached_out : h->x) : (to_slot ? partial_dst(h, M) : h->part);
  o.ld_out = h->d;
  o.dev_err = h->dev_err;
  // Few token rows give only d/128 tiles: split K over blocks so the whole GPU streams the weights.
  const int tiles = ((h->d + 127) / 128) * ((M + mtj::gemm_tc_token_tile() - 1) / mtj::gemm_tc_token_tile());
  int ksplit = 1;
  if (M <= kTcSplitRows && tiles < 148) ksplit = std::max(1, std::min({kTcSplitMax, 296 / tiles, o.K / 64}));
  if (to_slot && ksplit == 1) ksplit = 2;          // the slot is selected by the reduction kernel
  const bool push = decode && !detached_out && !defer_reduce && use_push(h, M) && M <= kTcSplitRows;
  h->prof_begin(MTJ_FAMILY_OUTPROJ, s);
  if (push) {
    // the exchange kernel sums the split-K planes itself, adds the bias, the peers' rows and the residual and
    // writes the next projection's operand (next layer's LayerNorm, or the final one)
    o.partial = h->tc_partial;
    o.ksplit = ksplit;
    MTJ_CUDA(mtj::launch_gemm_tc(mtj::kEpiOut, &lw.map_out, &h->map_act[tc_tile_index(M)], o, s, pdl,
                                 hilo ? &h->map_act_lo[tc_tile_index(M)] : nullptr));
    h->prof_end(s);
    h->launches += 3;
    const bool last = layer + 1 == h->L;
    return push_reduce(h, M, h->tc_partial, ksplit, lw.b_out, true,
                       last ? h->lnf_scale : h->layers[layer + 1].ln_scale,
                       last ? h->lnf_offset : h->layers[layer + 1].ln_offset, hilo, pdl, s);
  }
  if (ksplit > 1) {
    float* dst = o.out;
    const float* res = o.residual;
    o.partial = h->tc_partial;
    o.ksplit = ksplit;
    MTJ_CUDA(mtj::launch_gemm_tc(mtj::kEpiOut, &lw.map_out, &h->map_act[tc_tile_index(M)], o, s, pdl,
                                 hilo ? &h->map_act_lo[tc_tile_index(M)] : nullptr));
    MTJ_CUDA(mtj::launch_splitk_reduce(h->tc_partial, ksplit, M, h->d, lw.b_out, res, dst, h->d,
                                       to_slot ? partial_slot_sel(h, M) : nullptr, partial_slot_stride(h), s, pdl));
    h->launches++;
  } else if (wide) {
    o.pair = (h->tc_pair >> 1) & 1;
    MTJ_CUDA(mtj::launch_gemm_tc_wide(mtj::kEpiOut, &lw.map_out, &h->map_act_wide, o, s));
  } else {
    MTJ_CUDA(mtj::launch_gemm_tc(mtj::kEpiOut, &lw.map_out, &h->map_act[tc_tile_index(M)], o, s, pdl,
                                 hilo ? &h->map_act_lo[tc_tile_index(M)] : nullptr));
  }
  h->prof_end(s);
  h->launches += 4;
  if (h->mp > 1 && detached_out) {
    std::string err;
    if (mtj::comm_all_reduce(h->comm, h->part, static_cast<size_t>(M) * h->d, false, s, &err))
      return fail(MTJ_ERR_COMM, err);
    MTJ_CUDA(cudaMemcpyAsync(detached_out, h->part, sizeof(float) * M * h->d, cudaMemcpyDeviceToDevice, s));
    return MTJ_OK;
  }
  if (h->mp > 1 && !defer_reduce) return reduce_into_x(h, M, true, pdl, s);
  return MTJ_OK;
}

// final LayerNorm + vocab-sharded logits for rows [row0, row0 + M) of h->x on the tensor cores
int32_t run_logits_tc(mtj_handle* h, int M, int row0, float* out, cudaStream_t s, bool pdl = false,
                      bool decode = false) {
  const bool hilo = decode && row0 == 0 && h->hilo_ok && M <= h->tc_hilo_max_b;
  if (h->xn_ready && decode && row0 == 0)
    h->xn_ready = false;            // the last layer's exchange applied the final LayerNorm already
  else
    MTJ_CUDA(mtj::launch_ln_rows(h->x + static_cast<size_t>(row0) * h->d, h->lnf_scale, h->lnf_offset,
                                 h->xn_bf16 + static_cast<size_t>(row0) * h->d, M, h->d, s, pdl,
                                 hilo ? h->xn_lo : nullptr));
  mtj::GemmTcArgs a = {};
  a.M = M;
  a.N = h->Vl;
  a.K = h->d;
  a.x_row0 = row0;
  a.bias = h->proj_b;
  a.out = out;
  a.ld_out = h->Vl;
  a.dev_err = h->dev_err;
  a.cluster_k = (decode && h->tc_cluster_k) ? mtj::gemm_tc_decode_cluster_k(a.N, M, a.K) : 1;
  h->prof_begin(MTJ_FAMILY_LOGITS, s);
  a.pair = (h->tc_pair >> 2) & 1;
  if (use_tc_wide(h, M))
    MTJ_CUDA(mtj::launch_gemm_tc_wide(mtj::kEpiLogits, &h->map_proj, &h->map_xn_wide, a, s));
  else
    MTJ_CUDA(mtj::launch_gemm_tc(mtj::kEpiLogits, &h->map_proj, &h->map_xn[tc_tile_index(M)], a, s, pdl,
                                 hilo ? &h->map_xn_lo[tc_tile_index(M)] : nullptr));
  h->prof_end(s);
  h->launches += 2;
  return MTJ_OK;
}

// ProjectionShard.loss, local part (layers.py:569-585), for rows [row0, row0 + n) of the chunk in h->x: final
// LayerNorm, then the logits GEMM whose epilogue reduces every 32-entry vocabulary group to (max, sum of exp)
// instead of storing logits, then the per-row combination.  Leaves ce.pmax / psum / hit like ce_partial.
int32_t run_loss_rows_fused(mtj_handle* h, int n, int row0, const mtj::CeArgs& ce, cudaStream_t s) {
  MTJ_CUDA(mtj::launch_ln_rows(h->x + static_cast<size_t>(row0) * h->d, h->lnf_scale, h->lnf_offset,
                               h->xn_bf16 + static_cast<size_t>(row0) * h->d, n, h->d, s, false, nullptr));
  MTJ_CUDA(cudaMemsetAsync(h->ce_tlogit, 0, sizeof(float) * n, s));
  MTJ_CUDA(cudaMemsetAsync(h->ce_ghit, 0, n, s));
  mtj::GemmTcArgs a = {};
  a.M = n;
  a.N = h->Vl;
  a.K = h->d;
  a.x_row0 = row0;
  a.rows = ce.rows;
  a.bias = h->proj_b;
  a.ce_gmax = h->ce_gmax;
  a.ce_gsum = h->ce_gsum;
  a.ce_ld = h->ce_rows;
  a.ce_tlogit = h->ce_tlogit;
  a.ce_hit = h->ce_ghit;
  a.ce_targets = ce.targets;
  a.ce_T = ce.T;
  a.ce_vocab_start = ce.vocab_start;
  a.dev_err = h->dev_err;
  h->prof_begin(MTJ_FAMILY_LOGITS, s);
  a.pair = (h->tc_pair >> 2) & 1;
  MTJ_CUDA(mtj::launch_gemm_tc_wide(mtj::kEpiLogitsCE, &h->map_proj, &h->map_xn_wide, a, s));
  h->prof_end(s);
  mtj::CeArgs c2 = ce;
  c2.row0 = row0;
  MTJ_CUDA(mtj::launch_ce_combine(c2, h->ce_gmax, h->ce_gsum, h->ce_groups, h->ce_rows, h->ce_tlogit, h->ce_ghit, n, s));
  h->launches += 3;
  return MTJ_OK;
}

bool use_tc(const mtj_handle* h, int M) { return h->tc_ok && M >= 32; }
// decode: from this many sequences on, one tensor-core pass over the weights beats ceil(B/4) GEMV passes
bool use_tc_decode(const mtj_handle* h, int B) { return h->tc_ok && B >= h->tc_decode_min_b; }

int32_t run_embed(mtj_handle* h, const uint32_t* ids, int ids_ld, int M, const mtj::RowMap& rows,
                  bool decode, cudaStream_t s, bool tc_decode = false) {
  // batched decode at mp > 1: the rows go through the push exchange, which also applies layer 0's LayerNorm
  const bool push = tc_decode && use_push(h, M) && M <= kTcSplitRows;
  mtj::EmbedArgs e = {};
  e.ids = ids;
  e.ids_ld = ids_ld;
  e.rows = rows;
  e.M = M;
  e.d = h->d;
  e.vocab_local = h->Vl;
  e.vocab_start = h->rank * h->Vl;
  e.table = h->emb_w;
  e.bias = h->emb_b;
  e.x = h->mp == 1 ? h->x : (push ? h->tc_partial : partial_dst(h, M));
  if (h->mp > 1 && !push) {
    e.slot_sel = partial_slot_sel(h, M);
    e.slot_stride = partial_slot_stride(h);
  }
  e.stats = h->mp == 1 ? h->stats : nullptr;
  MTJ_CUDA(mtj::launch_embed(e, s, h->use_pdl && decode));
  h->launches++;
  if (push) {
    const bool hilo = h->hilo_ok && M <= h->tc_hilo_max_b;
    return push_reduce(h, M, h->tc_partial, 1, nullptr, false, h->layers[0].ln_scale, h->layers[0].ln_offset, hilo,
                       h->use_pdl && h->tc_pdl, s);
  }
  if (h->mp > 1) return reduce_into_x(h, M, false, h->use_pdl && decode, s);
  return MTJ_OK;
}

// final LayerNorm + vocab-sharded logits for M output rows (layers.py:561-564)
int32_t run_logits(mtj_handle* h, int M, const int32_t* row_select, float* out, bool decode,
                   cudaStream_t s, int row0 = 0) {
  GemvArgs a = {};
  a.W = h->proj_w;
  a.N = h->Vl;
  a.K = h->d;
  a.M = M;
  a.x = h->x + static_cast<size_t>(row0) * h->d;
  a.ldx = h->d;
  a.ln_scale = h->lnf_scale;
  a.ln_offset = h->lnf_offset;
  a.stats = h->stats + 2 * static_cast<size_t>(row0);
  a.bias = h->proj_b;
  a.logits = out;
  a.ld_logits = h->Vl;
  a.row_select = row_select;
  a.dev_err = h->dev_err;
  a.ks_override = decode ? h->ks_logits : 0;
  h->prof_begin(MTJ_FAMILY_LOGITS, s);
  MTJ_CUDA(mtj::launch_gemv(mtj::kEpiLogits, a, s, h->use_pdl && decode));
  h->prof_end(s);
  h->launches++;
  return MTJ_OK;
}

int32_t check_ready(const mtj_handle* h) {
  if (!h) return fail(MTJ_ERR_INVALID, "null handle");
  if (!h->bound) return fail(MTJ_ERR_STATE, "arenas not bound (mtj_bind_arenas)");
  int64_t loaded = 0;
  for (uint8_t m : h->leaf_loaded) loaded += m;
  if (loaded != h->expected)
    return fail(MTJ_ERR_STATE, "parameters missing: loaded " + std::to_string(loaded) + " of " +
                                   std::to_string(h->expected));
  return MTJ_OK;
}

// Sets per-sequence first valid position / key limit and the identity page map.
int32_t setup_sequences(mtj_handle* h, const std::vector<int32_t>& pad,
                        const std::vector<int32_t>& limit, int cur, cudaStream_t s) {
  const int B = static_cast<int>(pad.size());
  std::vector<int32_t> table(static_cast<size_t>(B) * h->ring_pages);
  for (int b = 0; b < B; ++b)
    for (int p = 0; p < h->ring_pages; ++p) table[static_cast<size_t>(b) * h->ring_pages + p] = b * h->ring_pages + p;
  MTJ_CUDA(cudaMemcpyAsync(h->pad, pad.data(), B * sizeof(int32_t), cudaMemcpyHostToDevice, s));
  MTJ_CUDA(cudaMemcpyAsync(h->key_limit, limit.data(), B * sizeof(int32_t), cudaMemcpyHostToDevice, s));
  MTJ_CUDA(cudaMemcpyAsync(h->page_table, table.data(), table.size() * sizeof(int32_t),
                           cudaMemcpyHostToDevice, s));
  const int32_t c = cur;
  MTJ_CUDA(cudaMemcpyAsync(h->cur, &c, sizeof(int32_t), cudaMemcpyHostToDevice, s));
  // the host vectors above are pageable: the copies are staged before returning
  return MTJ_OK;
}

// Runs embed + all layers over [batch, T] ids in chunks of at most max_rows rows.
// After each chunk `after_chunk(b0, nseq, t0, Tc)` may read h->x / h->stats.
template <typename F>
int32_t forward_chunks(mtj_handle* h, const uint32_t* ids, int ids_ld, int batch, int T,
                       const int32_t* key_limit, cudaStream_t s, F&& after_chunk, int t_begin = 0) {
  // positions [0, t_begin) are left padding in every sequence: their rows are never read, so they are not computed
  const int Tv = T - t_begin;
  if (Tv <= 0) return MTJ_OK;
  // Tensor parallel, tensor-core path: pairs of chunks are walked layer by layer together, each in its own
  // half of the activation buffers; while one chunk's partial sums are all-reduced on the communication
  // stream the other chunk's layer runs.  Two position chunks of the same sequences keep their order
  // inside a layer (the later one attends to the keys the earlier one has just written).
  const bool piped = h->mp > 1 && h->tp_pipe && h->views_ok && h->view_rows[1] >= 64;
  const int R = piped ? h->view_rows[1] : h->max_rows;
  int Tc = std::min(Tv, R);
  int nseq = std::max(1, R / Tc);
  if (Tc < Tv) nseq = 1;
  struct Chunk { int b0, ns, t0, tc; };
  std::vector<Chunk> chunks;
  for (int b0 = 0; b0 < batch; b0 += nseq)
    for (int t0 = t_begin; t0 < T; t0 += Tc) chunks.push_back({b0, std::min(nseq, batch - b0), t0, std::min(Tc, T - t0)});
  if (piped && chunks.size() == 1 && chunks[0].ns * chunks[0].tc >= 2 * kTpPipeMinRows) {
    // everything fits one chunk: cut it in two so that there is something to overlap with
    const Chunk c = chunks[0];
    chunks.clear();
    if (c.ns >= 2) {
      chunks.push_back({c.b0, c.ns / 2, c.t0, c.tc});
      chunks.push_back({c.b0 + c.ns / 2, c.ns - c.ns / 2, c.t0, c.tc});
    } else {
      const int half = (c.tc + 1) / 2;
      chunks.push_back({c.b0, 1, c.t0, half});
      chunks.push_back({c.b0, 1, c.t0 + half, c.tc - half});
    }
  }
  if (piped && !h->comm_stream) {
    MTJ_CUDA(cudaStreamCreateWithFlags(&h->comm_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      MTJ_CUDA(cudaEventCreateWithFlags(&h->ev_layer[i], cudaEventDisableTiming));
      MTJ_CUDA(cudaEventCreateWithFlags(&h->ev_reduced[i], cudaEventDisableTiming));
    }
  }
  int32_t rc = MTJ_OK;
  for (size_t i = 0; i < chunks.size() && !rc; i += 2) {
    const int n = (i + 1 < chunks.size()) ? 2 : 1;
    const bool overlap = piped && n == 2 && use_tc(h, chunks[i].ns * chunks[i].tc) &&
                         use_tc(h, chunks[i + 1].ns * chunks[i + 1].tc);
    if (!overlap) {
      for (int k = 0; k < n && !rc; ++k) {
        const Chunk& c = chunks[i + k];
        mtj::RowMap rows = {c.b0, c.tc, c.t0, nullptr};
        const int M = c.ns * c.tc;
        rc = run_embed(h, ids, ids_ld, M, rows, false, s);
        for (int l = 0; l < h->L && !rc; ++l)
          rc = use_tc(h, M) ? run_layer_tc(h, l, M, rows, key_limit, s) : run_layer(h, l, M, rows, false, key_limit, s);
        if (!rc) rc = after_chunk(c.b0, c.ns, c.t0, c.tc);
      }
      continue;
    }
    for (int k = 0; k < 2 && !rc; ++k) {
      const Chunk& c = chunks[i + k];
      mtj::RowMap rows = {c.b0, c.tc, c.t0, nullptr};
      h->use_view(k);
      rc = run_embed(h, ids, ids_ld, c.ns * c.tc, rows, false, s);
    }
    for (int l = 0; l < h->L && !rc; ++l) {
      for (int k = 0; k < 2 && !rc; ++k) {
        const Chunk& c = chunks[i + k];
        mtj::RowMap rows = {c.b0, c.tc, c.t0, nullptr};
        const int M = c.ns * c.tc;
        h->use_view(k);
        if (l > 0) MTJ_CUDA(cudaStreamWaitEvent(s, h->ev_reduced[k], 0));       // x of this chunk is complete
        rc = run_layer_tc(h, l, M, rows, key_limit, s, nullptr, false, /*defer_reduce=*/true);
        if (rc) break;
        MTJ_CUDA(cudaEventRecord(h->ev_layer[k], s));
        MTJ_CUDA(cudaStreamWaitEvent(h->comm_stream, h->ev_layer[k], 0));
        rc = reduce_into_x(h, M, true, false, h->comm_stream);
        if (rc) break;
        MTJ_CUDA(cudaEventRecord(h->ev_reduced[k], h->comm_stream));
      }
    }
    for (int k = 0; k < 2; ++k) MTJ_CUDA(cudaStreamWaitEvent(s, h->ev_reduced[k], 0));
    for (int k = 0; k < 2 && !rc; ++k) {
      const Chunk& c = chunks[i + k];
      h->use_view(k);
      rc = after_chunk(c.b0, c.ns, c.t0, c.tc);
    }
    h->use_view(0);
  }
  if (piped) h->use_view(0);
  return rc;
}

}  // namespace

extern "C" {

const char* mtj_last_error(void) { return g_last_error.c_str(); }
int32_t mtj_set_error(int32_t code, const char* msg) { return fail(code, msg ? msg : ""); }
int32_t mtj_version(void) { return 3; }

int32_t mtj_create(const mtj_config* c, mtj_handle** out) {
  if (!c || !out) return fail(MTJ_ERR_INVALID, "null argument");
  if (c->layers <= 0 || c->d_model <= 0 || c->n_heads <= 0 || c->n_vocab <= 0 || c->seq < 2)
    return fail(MTJ_ERR_INVALID, "non-positive config value");
  const int mp = c->cores_per_replica;
  if (mp <= 0 || c->rank < 0 || c->rank >= mp) return fail(MTJ_ERR_INVALID, "bad rank / cores_per_replica");
  if (c->n_vocab % mp) return fail(MTJ_ERR_INVALID, "n_vocab % cores_per_replica != 0");
  if (c->d_model % c->n_heads) return fail(MTJ_ERR_INVALID, "d_model % n_heads != 0");
  if (c->n_heads % mp) return fail(MTJ_ERR_INVALID, "n_heads % cores_per_replica != 0");
  const int dh = c->d_model / c->n_heads;
  if (dh != 64 && dh != 256) return fail(MTJ_ERR_UNSUPPORTED, "d_head must be 64 or 256");
  const int rot = c->pe_rotary_dims > 0 ? c->pe_rotary_dims : dh;
  if (rot > dh || (rot & 1)) return fail(MTJ_ERR_INVALID, "pe_rotary_dims must be even and <= d_head");
  if (c->d_model % 8 || (c->d_model / mp) % 8) return fail(MTJ_ERR_UNSUPPORTED, "d_model / mp must be a multiple of 8");
  if ((c->n_vocab / mp) % 4) return fail(MTJ_ERR_UNSUPPORTED, "n_vocab / mp must be a multiple of 4");
  if (c->max_batch <= 0 || c->max_gen < 0 || c->max_rows <= 0) return fail(MTJ_ERR_INVALID, "bad capacity");
  if (c->mega_max_batch > 4) return fail(MTJ_ERR_INVALID, "mega_max_batch is at most 4");
  if (mtj::decode_attn_splits(c->seq - 1) > 64)
    return fail(MTJ_ERR_UNSUPPORTED, "seq up to 4032 is supported (64 pages of 64 tokens per sliding window)");

  mtj_handle* h = new mtj_handle();
  h->cfg = *c;
  h->L = c->layers;
  h->d = c->d_model;
  h->n_heads = c->n_heads;
  h->heads = c->n_heads / mp;
  h->dh = dh;
  h->rot = rot;
  h->V = c->n_vocab;
  h->Vl = c->n_vocab / mp;
  h->seq = c->seq;
  h->W = c->seq - 1;
  h->mp = mp;
  h->rank = c->rank;
  h->dl = c->d_model / mp;
  h->ffl = 4 * c->d_model / mp;
  h->max_batch = c->max_batch;
  h->max_gen = c->max_gen;
  h->max_rows = c->max_rows;
  h->max_pos = c->seq + c->max_gen + 1;
  const int need_all = (h->max_pos + mtj::kPageTokens - 1) / mtj::kPageTokens;
  const int need_ring = (c->seq + mtj::kPageTokens - 1) / mtj::kPageTokens + 1;
  h->ring_pages = std::min(need_all, need_ring);
  h->n_pages = h->ring_pages * h->max_batch;
  h->max_splits = mtj::decode_attn_splits(h->W);
  h->expected = 2 + 10LL * h->L + 4;
  const char* e = getenv("MTJ_NO_PDL");
  h->use_pdl = !(e && e[0] == '1');
  e = getenv("MTJ_NO_MEGA");
  h->use_mega = !(e && e[0] == '1');
  h->mega_token = !getenv("MTJ_NO_MEGA_TOKEN");
  if (c->mega_max_batch != 0) h->mega_max_b = std::max(0, c->mega_max_batch);
  if (c->tc_decode_min_batch > 0) h->tc_decode_min_b = c->tc_decode_min_batch;
  if (c->hilo_max_batch != 0) h->tc_hilo_max_b = std::max(0, std::min(kHiLoRows, c->hilo_max_batch));
  if (c->wait_limit > 0) h->wait_limit = c->wait_limit;
  e = getenv("MTJ_NO_TC_PDL");
  h->tc_pdl = !(e && e[0] == '1');
  e = getenv("MTJ_NO_MEGA_PUSH");
  h->mega_push = !(e && e[0] == '1');
  // measured on one box: the fused push exchange loses 6 % of a 32-sequence step at 2 shards and wins 12 % at 4
  // (the pull all-reduce reads every peer's slot, which grows with the shard count; the push does not)
  h->tp_push = mp >= 4;
  e = getenv("MTJ_TP_PUSH");
  if (e) h->tp_push = e[0] == '1';
  e = getenv("MTJ_NO_TP_TOKEN");
  h->tp_token = !(e && e[0] == '1');
  e = getenv("MTJ_NO_CLUSTER_K");
  h->tc_cluster_k = !(e && e[0] == '1');
  e = getenv("MTJ_NO_FUSED_CE");
  h->fused_ce = !(e && e[0] == '1');
  e = getenv("MTJ_NO_FORK");
  h->fork_attn = !(e && e[0] == '1');
  e = getenv("MTJ_FORK_PDL");
  h->fork_pdl = e && e[0] == '1';
  e = getenv("MTJ_KS_INPROJ");
  if (e) h->ks_inproj = atoi(e);
  e = getenv("MTJ_KS_OUT");
  if (e) h->ks_out = atoi(e);
  e = getenv("MTJ_KS_LOGITS");
  if (e) h->ks_logits = atoi(e);
  e = getenv("MTJ_NO_GRAPH");
  h->use_graph = !(e && e[0] == '1');

  *out = h;
  return MTJ_OK;
}

int32_t mtj_destroy(mtj_handle* h) {
  if (h) {
    for (cudaEvent_t e : h->ev_pool) cudaEventDestroy(e);
    if (h->graph_exec) cudaGraphExecDestroy(h->graph_exec);
    if (h->ev_fork) cudaEventDestroy(h->ev_fork);
    if (h->ev_join) cudaEventDestroy(h->ev_join);
    if (h->side_stream) cudaStreamDestroy(h->side_stream);
    if (h->comm_stream) cudaStreamDestroy(h->comm_stream);
    for (int i = 0; i < 2; ++i) {
      if (h->ev_layer[i]) cudaEventDestroy(h->ev_layer[i]);
      if (h->ev_reduced[i]) cudaEventDestroy(h->ev_reduced[i]);
    }
    if (h->comm) mtj::comm_destroy(h->comm);
    for (int r = 0; r < mtj::kP2pMaxWorld; ++r)
      if (h->p2p_peer[r] && h->p2p_peer[r] != h->p2p_local) cudaIpcCloseMemHandle(h->p2p_peer[r]);
    if (h->p2p_local) cudaFree(h->p2p_local);
    if (h->capture_stream) cudaStreamDestroy(h->capture_stream);
  }
  delete h;
  return MTJ_OK;
}

int64_t mtj_weights_bytes(const mtj_handle* h) {
  if (!h) return -1;
  mtj_handle tmp = *h;
  Carver c(nullptr);
  tmp.carve_weights(c);
  return align_up(c.off, 256);
}

int64_t mtj_workspace_bytes(const mtj_handle* h) {
  if (!h) return -1;
  mtj_handle tmp = *h;
  Carver c(nullptr);
  tmp.carve_workspace(c);
  return align_up(c.off, 256);
}

int32_t mtj_bind_arenas(mtj_handle* h, void* wdev, int64_t wbytes, void* sdev, int64_t sbytes,
                        mtj_stream stream) {
  if (!h || !wdev || !sdev) return fail(MTJ_ERR_INVALID, "null argument");
  if ((reinterpret_cast<uintptr_t>(wdev) | reinterpret_cast<uintptr_t>(sdev)) & 255)
    return fail(MTJ_ERR_INVALID, "arenas must be 256-byte aligned");
  if (wbytes < mtj_weights_bytes(h) || sbytes < mtj_workspace_bytes(h))
    return fail(MTJ_ERR_INVALID, "arena too small");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Carver cw(wdev), cs(sdev);
  h->carve_weights(cw);
  h->carve_workspace(cs);
  // RoPE angles in double precision like the reference's NumPy table (layers.py:128-134)
  std::vector<float2> tab(static_cast<size_t>(h->max_pos) * (h->rot / 2));
  for (int p = 0; p < h->max_pos; ++p)
    for (int i = 0; i < h->rot / 2; ++i) {
      const double inv_freq = 1.0 / pow(10000.0, (2.0 * i) / h->rot);
      const double ang = static_cast<double>(p) * inv_freq;
      tab[static_cast<size_t>(p) * (h->rot / 2) + i] = make_float2(static_cast<float>(sin(ang)),
                                                                 static_cast<float>(cos(ang)));
    }
  MTJ_CUDA(cudaMemcpyAsync(h->sincos, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice, s));
  MTJ_CUDA(cudaMemsetAsync(h->counters, 0, sizeof(uint32_t) * h->max_batch * h->heads, s));
  MTJ_CUDA(cudaMemsetAsync(h->gemv_counters, 0, sizeof(uint32_t) * h->max_rows, s));
  MTJ_CUDA(cudaMemsetAsync(h->dev_err, 0, sizeof(uint32_t) * 4, s));
  MTJ_CUDA(cudaMemsetAsync(h->rng_seed, 0, sizeof(uint32_t) * 4, s));
  // The tensor-core attention multiplies masked keys' V rows by exactly zero: slots that were
  // never written must hold finite values, so the pools (and the bf16 operand buffers) start at zero.
  MTJ_CUDA(cudaMemsetAsync(h->kpool, 0, sizeof(__nv_bfloat16) * h->pool_layer_elems * h->L, s));
  MTJ_CUDA(cudaMemsetAsync(h->vpool, 0, sizeof(__nv_bfloat16) * h->pool_layer_elems * h->L, s));
  MTJ_CUDA(cudaMemsetAsync(h->q_bf16, 0, sizeof(__nv_bfloat16) * h->max_rows * h->dl, s));
  MTJ_CUDA(cudaMemsetAsync(h->xn_bf16, 0, sizeof(__nv_bfloat16) * static_cast<size_t>(h->max_rows) * h->d, s));
  MTJ_CUDA(cudaMemsetAsync(h->act_bf16, 0, sizeof(__nv_bfloat16) * static_cast<size_t>(h->max_rows) * (h->dl + h->ffl), s));
  {
    std::vector<mtj::MegaLayer> ml(h->L);
    for (int l = 0; l < h->L; ++l) {
      const LayerWeights& lw = h->layers[l];
      mtj::KvCache kv = h->kv(l);
      ml[l] = {lw.w_in, lw.b_ff, lw.w_out, lw.b_out, lw.ln_scale, lw.ln_offset, kv.kpool, kv.vpool};
    }
    MTJ_CUDA(cudaMemcpyAsync(h->mega_layers, ml.data(), sizeof(mtj::MegaLayer) * h->L, cudaMemcpyHostToDevice, s));
    MTJ_CUDA(cudaMemsetAsync(h->mega_sync, 0, sizeof(uint32_t) * (5 * h->L + 3), s));
    MTJ_CUDA(cudaMemsetAsync(h->mega_amax, 0, sizeof(unsigned long long) * 4, s));
    MTJ_CUDA(cudaStreamSynchronize(s));   // `ml` goes out of scope
  }
  MTJ_CUDA(cudaStreamSynchronize(s));   // `tab` is about to go out of scope
  // TMA views for the tensor-core GEMM (needs K % 64 == 0 on both projections)
  h->tc_ok = false;
  const char* no_tc = getenv("MTJ_NO_TC");
  if (h->d % 64 == 0 && (h->dl + h->ffl) % 64 == 0 && !(no_tc && no_tc[0] == '1')) {
    bool ok = true;
    for (auto& lw : h->layers) {
      ok = ok && mtj::make_tensor_map_bf16(&lw.map_in, lw.w_in, 3 * h->dl + h->ffl, h->d, 128) == cudaSuccess;
      ok = ok && mtj::make_tensor_map_bf16(&lw.map_out, lw.w_out, h->d, h->dl + h->ffl, 128) == cudaSuccess;
    }
    ok = ok && mtj::make_tensor_map_bf16(&h->map_proj, h->proj_w, h->Vl, h->d, 128) == cudaSuccess;
    for (int i = 0; i < 3; ++i) {
      const int box = 32 << i;
      ok = ok && mtj::make_tensor_map_bf16(&h->map_xn[i], h->xn_bf16, h->max_rows, h->d, box) == cudaSuccess;
      ok = ok && mtj::make_tensor_map_bf16(&h->map_act[i], h->act_bf16, h->max_rows, h->dl + h->ffl, box) == cudaSuccess;
    }
    const int bw = mtj::gemm_tc_wide_token_tile();
    ok = ok && mtj::make_tensor_map_bf16(&h->map_xn_wide, h->xn_bf16, h->max_rows, h->d, bw) == cudaSuccess;
    ok = ok && mtj::make_tensor_map_bf16(&h->map_act_wide, h->act_bf16, h->max_rows, h->dl + h->ffl, bw) == cudaSuccess;
    h->tc_wide_ok = ok && !getenv("MTJ_NO_TC_WIDE");
    if (const char* e = getenv("MTJ_TC_PAIR")) h->tc_pair = atoi(e) & 7;
    {
      const int64_t rl = std::min<int64_t>(h->max_rows, kHiLoRows);
      bool okl = ok;
      for (int i = 0; i < 2 && okl; ++i) {
        okl = okl && mtj::make_tensor_map_bf16(&h->map_xn_lo[i], h->xn_lo, rl, h->d, 32 << i) == cudaSuccess;
        okl = okl && mtj::make_tensor_map_bf16(&h->map_act_lo[i], h->act_lo, rl, h->dl + h->ffl, 32 << i) == cudaSuccess;
      }
      h->hilo_ok = okl;
    }
    if (!ok) return fail(MTJ_ERR_CUDA, "cuTensorMapEncodeTiled failed");
    h->tc_ok = true;
    const char* no_atc = getenv("MTJ_NO_ATTN_TC");
    if (h->dh == 256 && !(no_atc && no_atc[0] == '1')) {
      const int64_t pool_rows = static_cast<int64_t>(h->n_pages) * h->heads * mtj::kPageTokens;
      for (int l = 0; l < h->L; ++l) {
        mtj::KvCache kv = h->kv(l);
        ok = ok && mtj::make_tensor_map_bf16(&h->layers[l].map_k, kv.kpool, pool_rows, h->dh, 64) == cudaSuccess;
        ok = ok && mtj::make_tensor_map_bf16(&h->layers[l].map_v, kv.vpool, pool_rows, h->dh, 64) == cudaSuccess;
      }
      ok = ok && mtj::make_tensor_map_bf16(&h->map_q, h->q_bf16, h->max_rows, h->dl, 128) == cudaSuccess;
      if (!ok) return fail(MTJ_ERR_CUDA, "cuTensorMapEncodeTiled failed (attention)");
      h->attn_tc_ok = true;
    }
  }
  // the two halves of the row-indexed activation buffers used by the tensor-parallel chunk pipeline
  h->save_view(0);
  h->views_ok = false;
  if (h->mp > 1 && h->tc_ok) {
    const int64_t r0 = (h->max_rows + 1) / 2, r1 = h->max_rows - r0;
    mtj_handle::ActView& v = h->views[1];
    v = h->views[0];
    v.x = h->x + r0 * h->d;
    v.stats = h->stats + r0 * 2;
    v.part = h->part + r0 * h->d;
    v.q = h->q + r0 * h->dl;
    v.xn_bf16 = h->xn_bf16 + r0 * h->d;
    v.act_bf16 = h->act_bf16 + r0 * (h->dl + h->ffl);
    v.q_bf16 = h->q_bf16 + r0 * h->dl;
    bool ok = r1 >= 1;
    for (int i = 0; i < 3 && ok; ++i) {
      const int box = 32 << i;
      ok = ok && mtj::make_tensor_map_bf16(&v.map_xn[i], v.xn_bf16, r1, h->d, box) == cudaSuccess;
      ok = ok && mtj::make_tensor_map_bf16(&v.map_act[i], v.act_bf16, r1, h->dl + h->ffl, box) == cudaSuccess;
    }
    const int bw = mtj::gemm_tc_wide_token_tile();
    ok = ok && mtj::make_tensor_map_bf16(&v.map_xn_wide, v.xn_bf16, r1, h->d, bw) == cudaSuccess;
    ok = ok && mtj::make_tensor_map_bf16(&v.map_act_wide, v.act_bf16, r1, h->dl + h->ffl, bw) == cudaSuccess;
    if (h->attn_tc_ok) ok = ok && mtj::make_tensor_map_bf16(&v.map_q, v.q_bf16, r1, h->dl, 128) == cudaSuccess;
    h->views_ok = ok;
    h->view_rows[0] = static_cast<int>(r0);
    h->view_rows[1] = static_cast<int>(r1);
    // measured: overlapping one chunk's all-reduce with the other chunk's layer costs 7 % of a 2047-token prefill
    // at 2 shards (the halves quantise worse over the GEMM's blocks) and gains 10 % at 4, where the all-reduce
    // is a larger share
    h->tp_pipe = h->mp >= 4;
    const char* np = getenv("MTJ_TP_PIPE");
    if (np) h->tp_pipe = np[0] == '1';
  }
  h->bound = true;
  h->leaf_loaded.assign(static_cast<size_t>(h->expected), 0);
  return MTJ_OK;
}

int32_t mtj_load_param(mtj_handle* h, const char* name, const void* src, int32_t dtype, int32_t ndim,
                       const int64_t* shape, mtj_stream stream) {
  if (!h || !name || !src || !shape) return fail(MTJ_ERR_INVALID, "null argument");
  if (!h->bound) return fail(MTJ_ERR_STATE, "arenas not bound");
  if (dtype != MTJ_F32 && dtype != MTJ_BF16) return fail(MTJ_ERR_INVALID, "dtype");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // tokens of the Haiku path, "~" and the top-level module name dropped
  std::vector<std::string> tok;
  {
    std::string cur;
    for (const char* p = name;; ++p) {
      if (*p == '/' || *p == 0) {
        if (!cur.empty() && cur != "~" && cur != "causal_transformer_shard") tok.push_back(cur);
        cur.clear();
        if (*p == 0) break;
      } else {
        cur.push_back(*p);
      }
    }
  }
  if (tok.size() != 3) return fail(MTJ_ERR_INVALID, std::string("unrecognised parameter name: ") + name);
  const std::string &mod = tok[0], &lay = tok[1], &leaf = tok[2];
  const int bf = dtype == MTJ_BF16;
  auto want = [&](std::initializer_list<int64_t> dims) {
    if (ndim != static_cast<int32_t>(dims.size())) return false;
    int i = 0;
    for (int64_t v : dims)
      if (shape[i++] != v) return false;
    return true;
  };
  auto bad_shape = [&]() { return fail(MTJ_ERR_INVALID, std::string("shape mismatch for ") + name); };
  const int d = h->d, dl = h->dl, ffl = h->ffl, Vl = h->Vl;
  // which leaf this is: a leaf loaded twice overwrites itself and cannot stand in for a missing one
  int64_t leaf_id = -1;

  if (mod == "embedding_shard" && lay == "linear") {
    leaf_id = leaf == "w" ? 0 : 1;
    if (leaf == "w") {
      if (!want({Vl, d})) return bad_shape();
      MTJ_CUDA(mtj::launch_to_bf16(src, bf, static_cast<int64_t>(Vl) * d, h->emb_w, s));
    } else if (leaf == "b") {
      if (!want({d})) return bad_shape();
      MTJ_CUDA(mtj::launch_to_f32(src, bf, d, h->emb_b, s));
    } else {
      return fail(MTJ_ERR_INVALID, std::string("unknown leaf: ") + name);
    }
  } else if (mod == "projection_shard") {
    const int64_t base = 2 + 10LL * h->L;
    if (lay == "replicated_layer_norm" && (leaf == "scale" || leaf == "offset")) {
      if (!want({d})) return bad_shape();
      leaf_id = base + (leaf == "scale" ? 0 : 1);
      MTJ_CUDA(mtj::launch_to_f32(src, bf, d, leaf == "scale" ? h->lnf_scale : h->lnf_offset, s));
    } else if (lay == "linear" && leaf == "w") {
      leaf_id = base + 2;
      if (!want({d, Vl})) return bad_shape();
      MTJ_CUDA(mtj::launch_pack_transpose(src, bf, d, Vl, h->proj_w, d, 0, s));
    } else if (lay == "linear" && leaf == "b") {
      leaf_id = base + 3;
      if (!want({Vl})) return bad_shape();
      MTJ_CUDA(mtj::launch_to_f32(src, bf, Vl, h->proj_b, s));
    } else {
      return fail(MTJ_ERR_INVALID, std::string("unknown leaf: ") + name);
    }
  } else if (mod.rfind("layer_", 0) == 0) {
    const int li = atoi(mod.c_str() + 6);
    if (li < 0 || li >= h->L) return fail(MTJ_ERR_INVALID, std::string("layer out of range: ") + name);
    LayerWeights& lw = h->layers[li];
    const int kin = dl + ffl;
    const int64_t base = 2 + 10LL * li;
    if (lay == "replicated_layer_norm" && (leaf == "scale" || leaf == "offset")) {
      leaf_id = base + (leaf == "scale" ? 0 : 1);
      if (!want({d})) return bad_shape();
      MTJ_CUDA(mtj::launch_to_f32(src, bf, d, leaf == "scale" ? lw.ln_scale : lw.ln_offset, s));
    } else if (leaf == "w" && (lay == "linear" || lay == "linear_1" || lay == "linear_2")) {
      // q -> rows [0, dl), k (linear_2) -> [dl, 2dl), v (linear_1) -> [2dl, 3dl)
      if (!want({d, dl})) return bad_shape();
      const int region = lay == "linear" ? 0 : (lay == "linear_2" ? 1 : 2);
      leaf_id = base + 2 + region;
      MTJ_CUDA(mtj::launch_pack_transpose(src, bf, d, dl, lw.w_in + static_cast<size_t>(region) * dl * d, d, 0, s));
    } else if (leaf == "w" && lay == "linear_3") {
      if (!want({dl, d})) return bad_shape();
      leaf_id = base + 5;
      MTJ_CUDA(mtj::launch_pack_transpose(src, bf, dl, d, lw.w_out, kin, 0, s));
    } else if (lay == "linear_4") {
      leaf_id = base + (leaf == "w" ? 6 : 7);
      if (leaf == "w") {
        if (!want({d, ffl})) return bad_shape();
        MTJ_CUDA(mtj::launch_pack_transpose(src, bf, d, ffl, lw.w_in + static_cast<size_t>(3) * dl * d, d, 0, s));
      } else if (leaf == "b") {
        if (!want({ffl})) return bad_shape();
        MTJ_CUDA(mtj::launch_to_f32(src, bf, ffl, lw.b_ff, s));
      } else {
        return fail(MTJ_ERR_INVALID, std::string("unknown leaf: ") + name);
      }
    } else if (lay == "linear_5") {
      leaf_id = base + (leaf == "w" ? 8 : 9);
      if (leaf == "w") {
        if (!want({ffl, d})) return bad_shape();
        MTJ_CUDA(mtj::launch_pack_transpose(src, bf, ffl, d, lw.w_out, kin, dl, s));
      } else if (leaf == "b") {
        if (!want({d})) return bad_shape();
        MTJ_CUDA(mtj::launch_to_f32(src, bf, d, lw.b_out, s));
      } else {
        return fail(MTJ_ERR_INVALID, std::string("unknown leaf: ") + name);
      }
    } else {
      return fail(MTJ_ERR_INVALID, std::string("unknown leaf: ") + name);
    }
  } else {
    return fail(MTJ_ERR_INVALID, std::string("unknown module: ") + name);
  }
  if (leaf_id < 0 || leaf_id >= static_cast<int64_t>(h->leaf_loaded.size()))
    return fail(MTJ_ERR_INVALID, std::string("unknown leaf: ") + name);
  h->leaf_loaded[static_cast<size_t>(leaf_id)] = 1;
  return MTJ_OK;
}

int32_t mtj_comm_unique_id(uint8_t* out128) {
  if (!out128) return fail(MTJ_ERR_INVALID, "null argument");
  std::string err;
  if (mtj::comm_unique_id(out128, &err)) return fail(MTJ_ERR_COMM, err);
  return MTJ_OK;
}

int32_t mtj_comm_init(mtj_handle* h, const uint8_t* id128) {
  if (!h || !id128) return fail(MTJ_ERR_INVALID, "null argument");
  if (h->mp == 1) return MTJ_OK;
  if (h->comm) return fail(MTJ_ERR_STATE, "communicator already initialised");
  std::string err;
  if (mtj::comm_init(id128, h->rank, h->mp, &h->comm, &err)) return fail(MTJ_ERR_COMM, err);
  if (h->bound) {
    // first use of each collective sets connections up; do that here, outside any graph capture
    cudaStream_t s = nullptr;
    MTJ_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    MTJ_CUDA(cudaMemsetAsync(h->part, 0, sizeof(float) * h->d, s));
    int32_t rc = mtj::comm_all_reduce(h->comm, h->part, h->d, false, s, &err);
    if (!rc) rc = mtj::comm_all_gather(h->comm, h->logits, h->logits_gather, h->Vl, s, &err);
    cudaError_t ce = cudaStreamSynchronize(s);
    cudaStreamDestroy(s);
    if (rc) return fail(MTJ_ERR_COMM, err);
    if (ce != cudaSuccess) return fail(MTJ_ERR_CUDA, std::string("collective warm-up: ") + cudaGetErrorString(ce));
  }
  return MTJ_OK;
}

int32_t mtj_p2p_export(mtj_handle* h, uint8_t* handle64) {
  if (!h || !handle64) return fail(MTJ_ERR_INVALID, "null argument");
  if (h->mp < 2 || h->mp > mtj::kP2pMaxWorld) return fail(MTJ_ERR_UNSUPPORTED, "peer all-reduce needs 2..8 ranks");
  if (h->p2p_local) return fail(MTJ_ERR_STATE, "already exported");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  h->p2p_rows = std::min(h->max_rows, std::max(h->max_batch, 1));
  const size_t data = 2 * static_cast<size_t>(h->p2p_rows) * h->d * sizeof(float);
  h->p2p_flag_off = (data + 255) / 256 * 256;
  h->p2p_recv_off = h->p2p_flag_off + 512;
  h->p2p_push_off = h->p2p_recv_off + 2 * static_cast<size_t>(h->mp) * mtj::kMegaPushRows * h->d * sizeof(uint2);
  h->p2p_pflag_off = h->p2p_push_off + 2 * static_cast<size_t>(h->mp) * h->p2p_rows * h->d * sizeof(float);
  h->p2p_amax_off = (h->p2p_pflag_off + static_cast<size_t>(h->mp) * h->p2p_rows * sizeof(uint32_t) + 255) / 256 * 256;
  const size_t total = h->p2p_amax_off + 2 * static_cast<size_t>(h->mp) * h->p2p_rows * 2 * sizeof(uint2);
  MTJ_CUDA(cudaMalloc(reinterpret_cast<void**>(&h->p2p_local), total));
  MTJ_CUDA(cudaMemset(h->p2p_local, 0, total));
  cudaIpcMemHandle_t ih;
  MTJ_CUDA(cudaIpcGetMemHandle(&ih, h->p2p_local));
  memcpy(handle64, &ih, 64);
  return MTJ_OK;
}

int32_t mtj_p2p_import(mtj_handle* h, const uint8_t* handles) {
  if (!h || !handles) return fail(MTJ_ERR_INVALID, "null argument");
  if (!h->p2p_local) return fail(MTJ_ERR_STATE, "mtj_p2p_export has not run");
  for (int r = 0; r < h->mp; ++r) {
    if (r == h->rank) {
      h->p2p_peer[r] = h->p2p_local;
      continue;
    }
    cudaIpcMemHandle_t ih;
    memcpy(&ih, handles + 64 * r, 64);
    void* p = nullptr;
    MTJ_CUDA(cudaIpcOpenMemHandle(&p, ih, cudaIpcMemLazyEnablePeerAccess));
    h->p2p_peer[r] = static_cast<char*>(p);
  }
  h->p2p_ready = true;
  return MTJ_OK;
}

int32_t mtj_prefill(mtj_handle* h, const uint32_t* ctx, const uint32_t* ctx_len, int32_t batch,
                    mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (h->mp > 1 && !h->comm) return fail(MTJ_ERR_STATE, "cores_per_replica > 1 needs mtj_comm_init first");
  if (!ctx || !ctx_len || batch <= 0 || batch > h->max_batch) return fail(MTJ_ERR_INVALID, "bad batch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::vector<int32_t> pad(batch), limit(batch, 0x7fffffff);
  for (int b = 0; b < batch; ++b) {
    if (ctx_len[b] < 1 || ctx_len[b] > static_cast<uint32_t>(h->seq))
      return fail(MTJ_ERR_INVALID, "ctx_length must be in [1, seq]");
    pad[b] = h->seq - static_cast<int>(ctx_len[b]);
  }
  rc = setup_sequences(h, pad, limit, h->W, s);
  if (rc) return rc;
  h->min_pad = *std::min_element(pad.begin(), pad.end());
  // held-back last token drives the first decode step (transformer_shard.py:76-77)
  MTJ_CUDA(cudaMemcpy2DAsync(h->tokens, sizeof(uint32_t), ctx + (h->seq - 1), sizeof(uint32_t) * h->seq,
                             sizeof(uint32_t), batch, cudaMemcpyDeviceToDevice, s));
  rc = forward_chunks(h, ctx, h->seq, batch, h->W, nullptr, s,
                      [](int, int, int, int) { return static_cast<int32_t>(MTJ_OK); },
                      *std::min_element(pad.begin(), pad.end()));
  if (rc) return rc;
  h->batch = batch;
  h->prefilled = true;
  h->steps_done = 0;
  return MTJ_OK;
}

int32_t mtj_start_batch(mtj_handle* h, int32_t batch, mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (h->mp > 1 && !h->comm) return fail(MTJ_ERR_STATE, "cores_per_replica > 1 needs mtj_comm_init first");
  if (batch <= 0 || batch > h->max_batch) return fail(MTJ_ERR_INVALID, "bad batch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // every slot idles on a one-key window of its own (zeroed) cache until a sequence is admitted into it
  std::vector<int32_t> pad(batch, h->W), limit(batch, 0x7fffffff);
  rc = setup_sequences(h, pad, limit, h->W, s);
  if (rc) return rc;
  MTJ_CUDA(cudaMemsetAsync(h->tokens, 0, sizeof(uint32_t) * batch, s));
  h->min_pad = h->W;
  h->batch = batch;
  h->prefilled = true;
  h->steps_done = 0;
  return MTJ_OK;
}

int32_t mtj_admit(mtj_handle* h, int32_t slot, const uint32_t* prompt, int32_t len, mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (!h->prefilled) return fail(MTJ_ERR_STATE, "no running batch (mtj_start_batch or mtj_prefill first)");
  if (!prompt || slot < 0 || slot >= h->batch) return fail(MTJ_ERR_INVALID, "bad slot");
  if (len < 1 || len > h->seq) return fail(MTJ_ERR_INVALID, "prompt length must be in [1, seq]");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The batch's next decode position; the prompt's first len - 1 tokens are placed right before it and the last
  // one becomes the slot's next input, exactly what generate_initial does with a left-padded context
  // (transformer_shard.py:76-77) -- in a frame shifted by the steps the batch has already taken.  Keys are
  // cached rotated at absolute positions and attention depends on distances only, so the shift changes nothing.
  const int cur = h->W + h->steps_done;
  const int n = len - 1, pos0 = cur - n;
  if (cur + 1 >= h->max_pos) return fail(MTJ_ERR_STATE, "the batch has used up its positions (max_gen)");
  const int32_t padv = pos0, lim = 0x7fffffff;
  h->min_pad = std::min(h->min_pad, pos0);
  MTJ_CUDA(cudaMemcpyAsync(h->pad + slot, &padv, sizeof(int32_t), cudaMemcpyHostToDevice, s));
  MTJ_CUDA(cudaMemcpyAsync(h->key_limit + slot, &lim, sizeof(int32_t), cudaMemcpyHostToDevice, s));
  MTJ_CUDA(cudaMemcpyAsync(h->tokens + slot, prompt + n, sizeof(uint32_t), cudaMemcpyDeviceToDevice, s));
  h->xn_ready = false;
  for (int t0 = 0; t0 < n && !rc; t0 += h->max_rows) {
    const int M = std::min(h->max_rows, n - t0);
    const mtj::RowMap ids_rows = {0, M, 0, nullptr};                  // the prompt is a flat id array
    const mtj::RowMap rows = {slot, M, pos0 + t0, nullptr};
    rc = run_embed(h, prompt + t0, 0, M, ids_rows, false, s);
    for (int l = 0; l < h->L && !rc; ++l)
      rc = use_tc(h, M) ? run_layer_tc(h, l, M, rows, nullptr, s) : run_layer(h, l, M, rows, false, nullptr, s);
  }
  return rc;
}

int32_t mtj_decode_step(mtj_handle* h, const uint32_t* tokens_in, const float* top_p, const float* temp,
                        const float* uniforms, int32_t greedy, uint32_t* tokens_out, float* logits_out,
                        mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (!h->prefilled) return fail(MTJ_ERR_STATE, "mtj_prefill has not run");
  if (h->steps_done >= h->max_gen) return fail(MTJ_ERR_STATE, "max_gen steps already generated");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int B = h->batch;
  if (!greedy) {
    if (!top_p || !temp) return fail(MTJ_ERR_INVALID, "sampling needs top_p and temp");
    MTJ_CUDA(cudaMemcpyAsync(h->top_p, top_p, sizeof(float) * B, cudaMemcpyDeviceToDevice, s));
    MTJ_CUDA(cudaMemcpyAsync(h->temp, temp, sizeof(float) * B, cudaMemcpyDeviceToDevice, s));
    if (uniforms)      // otherwise the device generator keyed by mtj_set_seed draws them
      MTJ_CUDA(cudaMemcpyAsync(h->uniforms, uniforms, sizeof(float) * B * h->V, cudaMemcpyDeviceToDevice, s));
  }
  if (tokens_in)
    MTJ_CUDA(cudaMemcpyAsync(h->tokens, tokens_in, sizeof(uint32_t) * B, cudaMemcpyDeviceToDevice, s));
  auto enqueue = [&](cudaStream_t st) -> int32_t {
    mtj::RowMap rows = {0, 1, 0, h->cur};
    mtj::RowMap erows = {0, 1, 0, nullptr};
    const bool mega = h->use_mega && (h->mp == 1 || use_p2p(h, B)) && B <= h->mega_max_b && !h->profile && (h->d % 256) == 0;
    const bool tc = use_tc_decode(h, B);
    h->xn_ready = false;
    // one GPU, greedy: the persistent kernel also picks the token and advances the position
    const bool mega_token = mega && greedy && h->mp == 1 && h->mega_token;
    int32_t r = mega ? MTJ_OK : run_embed(h, h->tokens, 1, B, erows, true, st, tc);
    if (r) return r;
    if (mega) {
      mtj::MegaArgs ma = {};
      ma.L = h->L; ma.d = h->d; ma.dl = h->dl; ma.ffl = h->ffl; ma.heads = h->heads; ma.dh = h->dh;
      ma.rot = h->rot; ma.V = h->Vl; ma.B = B; ma.window = h->W; ma.ring_pages = h->ring_pages;
      ma.grid_splits = std::min(mtj::decode_attn_splits(h->W), h->ring_pages);
      ma.max_splits = h->max_splits;
      ma.layers = h->mega_layers;
      ma.emb_w = h->emb_w; ma.emb_b = h->emb_b; ma.lnf_scale = h->lnf_scale; ma.lnf_offset = h->lnf_offset;
      ma.proj_w = h->proj_w; ma.proj_b = h->proj_b; ma.sincos = h->sincos;
      ma.tokens = h->tokens; ma.cur = h->cur; ma.pad = h->pad; ma.page_table = h->page_table;
      ma.x = h->x; ma.q = h->q; ma.act2 = h->act2; ma.part_o = h->part_o; ma.part_ml = h->part_ml;
      ma.head_counters = h->counters; ma.logits = h->logits; ma.sync = h->mega_sync; ma.dev_err = h->dev_err;
      ma.trace = h->mega_trace_on ? h->mega_trace : nullptr;
      ma.wait_limit = h->wait_limit;
      // FF-in rows one at a time from 4 shards on (measured: +4.3 % at 4, -1 % at 2; MTJ_*_ROW_UNITS for measurements)
      ma.ff_row_units = (h->mp >= 4 && !getenv("MTJ_NO_MEGA_ROW_UNITS")) || getenv("MTJ_MEGA_ROW_UNITS") ? 1 : 0;
      if (mega_token) {
        ma.amax = h->mega_amax;
        ma.tokens_out = h->tokens;
        ma.cur_out = h->cur;
      }
      ma.rank = h->rank; ma.world = h->mp; ma.vocab_start = h->rank * h->Vl;
      if (h->mp > 1) {
        ma.slot_base = reinterpret_cast<float*>(h->p2p_local);
        ma.slot_elems = partial_slot_stride(h);
        for (int r = 0; r < h->mp; ++r) {
          ma.peer_data[r] = reinterpret_cast<const float*>(h->p2p_peer[r]);
          ma.peer_flags[r] = reinterpret_cast<uint32_t*>(h->p2p_peer[r] + h->p2p_flag_off);
          if (h->mega_push) {
            ma.peer_recv[r] = reinterpret_cast<uint2*>(h->p2p_peer[r] + h->p2p_recv_off);
          }
        }
        ma.local_flags = reinterpret_cast<const uint32_t*>(h->p2p_local + h->p2p_flag_off);
        ma.seq = reinterpret_cast<uint32_t*>(h->p2p_local + h->p2p_flag_off + 256);
      }
      MTJ_CUDA(mtj::launch_decode_mega(ma, st, nullptr));
      h->launches++;
    }
    for (int l = 0; !mega && l < h->L; ++l) {
      r = tc ? run_layer_tc(h, l, B, rows, nullptr, st, nullptr, true) : run_layer(h, l, B, rows, true, nullptr, st);
      if (r) return r;
    }
    if (!mega) {
      r = tc ? run_logits_tc(h, B, 0, h->logits, st, h->use_pdl && h->tc_pdl, true) : run_logits(h, B, nullptr, h->logits, true, st);
      if (r) return r;
    }
    // greedy and nobody asked for the logits: every rank pushes the arg-max of its vocabulary slice to all ranks
    // and all pick the same winner; the gather of the logits (layers.py:565-567) is not needed for the token
    const bool token_only = greedy && !logits_out && h->tp_token && h->mp > 1 && use_p2p(h, B);
    if (token_only) {
      mtj::TpArgmaxArgs am = {};
      am.logits = h->logits;
      am.Vl = h->Vl;
      am.vocab_start = h->rank * h->Vl;
      am.rank = h->rank;
      am.world = h->mp;
      am.rows_cap = h->p2p_rows;
      for (int q = 0; q < h->mp; ++q) am.peer_amax[q] = reinterpret_cast<uint2*>(h->p2p_peer[q] + h->p2p_amax_off);
      am.seq = reinterpret_cast<uint32_t*>(h->p2p_local + h->p2p_flag_off + 272);
      am.ticket = am.seq + 1;
      am.tokens = h->tokens;
      am.cur_dev = h->cur;
      am.dev_err = h->dev_err;
      am.wait_limit = h->wait_limit;
      MTJ_CUDA(mtj::launch_tp_argmax(am, B, st, h->use_pdl));
      h->launches++;
      return MTJ_OK;
    }
    if (h->mp > 1) {
      // all_gather + transpose + flatten of ProjectionShard.__call__ (layers.py:565-567)
      std::string err;
      if (mtj::comm_all_gather(h->comm, h->logits, h->logits_gather, static_cast<size_t>(B) * h->Vl, st, &err))
        return fail(MTJ_ERR_COMM, err);
      MTJ_CUDA(mtj::launch_gather_rows(h->logits_gather, h->logits_all, h->mp, B, h->Vl, st));
      h->launches += 2;
    }
    if (mega_token) return MTJ_OK;
    if (greedy) {
      mtj::ArgmaxArgs am = {};
      am.logits = h->logits_all;
      am.B = B;
      am.V = h->V;
      am.tokens = h->tokens;
      am.tokens_copy = nullptr;
      am.cur_dev = h->cur;
      MTJ_CUDA(mtj::launch_argmax(am, st, h->use_pdl));
    } else {
      mtj::SampleArgs sa = {};
      sa.logits = h->logits_all;
      sa.uniforms = uniforms ? h->uniforms : nullptr;
      sa.rng_seed = h->rng_seed;
      sa.top_p = h->top_p;
      sa.top_k = h->has_top_k ? h->top_k : nullptr;
      sa.temp = h->temp;
      sa.rows = B;
      sa.V = h->V;
      sa.scratch = h->sample_scratch;
      sa.tokens = h->tokens;
      sa.cur_dev = h->cur;
      MTJ_CUDA(mtj::launch_sample_top_p(sa, st, h->use_pdl));
    }
    h->launches++;
    return MTJ_OK;
  };
  if (h->use_graph && !h->profile && (h->mp == 1 || h->steps_done > 0)) {
    const int graph_kind = (greedy ? 1 : 0) | (logits_out ? 2 : 0) | ((!greedy && !uniforms) ? 4 : 0) |
                           ((!greedy && h->has_top_k) ? 8 : 0);
    if (h->graph_exec == nullptr || h->graph_batch != B || h->graph_greedy != graph_kind) {
      if (h->graph_exec) {
        cudaGraphExecDestroy(h->graph_exec);
        h->graph_exec = nullptr;
      }
      if (!h->capture_stream) MTJ_CUDA(cudaStreamCreateWithFlags(&h->capture_stream, cudaStreamNonBlocking));
      const int64_t before = h->launches;
      MTJ_CUDA(cudaStreamBeginCapture(h->capture_stream, cudaStreamCaptureModeThreadLocal));
      rc = enqueue(h->capture_stream);
      cudaGraph_t graph = nullptr;
      cudaError_t ce = cudaStreamEndCapture(h->capture_stream, &graph);
      h->graph_kernels = h->launches - before;
      h->launches = before;
      if (rc) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
      }
      if (ce != cudaSuccess) return fail(MTJ_ERR_CUDA, std::string("graph capture: ") + cudaGetErrorString(ce));
      ce = cudaGraphInstantiate(&h->graph_exec, graph, 0);
      cudaGraphDestroy(graph);
      if (ce != cudaSuccess) return fail(MTJ_ERR_CUDA, std::string("graph instantiate: ") + cudaGetErrorString(ce));
      h->graph_batch = B;
      h->graph_greedy = graph_kind;
    }
    MTJ_CUDA(cudaGraphLaunch(h->graph_exec, s));
    h->launches += h->graph_kernels;
  } else {
    rc = enqueue(s);
    if (rc) return rc;
  }
  if (tokens_out)
    MTJ_CUDA(cudaMemcpyAsync(tokens_out, h->tokens, sizeof(uint32_t) * B, cudaMemcpyDeviceToDevice, s));
  if (logits_out)
    MTJ_CUDA(cudaMemcpyAsync(logits_out, h->logits_all, sizeof(float) * B * h->V, cudaMemcpyDeviceToDevice, s));
  h->steps_done++;
  return MTJ_OK;
}

int32_t mtj_forward_logits(mtj_handle* h, const uint32_t* obs, const uint32_t* ctx_len, int32_t batch,
                           int32_t T, int32_t n_last, float* logits_out, mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (h->mp > 1 && !h->comm) return fail(MTJ_ERR_STATE, "cores_per_replica > 1 needs mtj_comm_init first");
  if (!obs || !logits_out || batch <= 0 || batch > h->max_batch) return fail(MTJ_ERR_INVALID, "bad batch");
  if (T <= 0 || T > h->ring_pages * mtj::kPageTokens || T > h->max_pos)
    return fail(MTJ_ERR_INVALID, "T exceeds the KV capacity");
  if (n_last <= 0 || n_last > T) return fail(MTJ_ERR_INVALID, "bad n_last");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::vector<int32_t> pad(batch, 0), limit(batch);
  for (int b = 0; b < batch; ++b) limit[b] = ctx_len ? static_cast<int32_t>(std::min<uint32_t>(ctx_len[b], 0x7fffffffu)) : T;
  rc = setup_sequences(h, pad, limit, T, s);
  if (rc) return rc;
  h->prefilled = false;
  const int first = T - n_last;
  rc = forward_chunks(h, obs, T, batch, T, h->key_limit, s, [&](int b0, int ns, int t0, int tc) -> int32_t {
    // rows of this chunk that fall into the last n_last positions
    const int lo = std::max(first, t0), hi = t0 + tc;
    if (lo >= hi) return MTJ_OK;
    const int per = hi - lo;
    if (use_tc(h, ns * tc)) {
      for (int i = 0; i < ns; ++i) {
        float* dst = logits_out + (static_cast<size_t>(b0 + i) * n_last + (lo - first)) * h->Vl;
        int32_t r2 = run_logits_tc(h, per, i * tc + (lo - t0), dst, s);
        if (r2) return r2;
      }
      return MTJ_OK;
    }
    std::vector<int32_t> sel(static_cast<size_t>(ns) * per);
    for (int i = 0; i < ns; ++i)
      for (int t = lo; t < hi; ++t) sel[static_cast<size_t>(i) * per + (t - lo)] = i * tc + (t - t0);
    MTJ_CUDA(cudaMemcpyAsync(h->row_select, sel.data(), sel.size() * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    for (int i = 0; i < ns; ++i) {
      float* dst = logits_out + (static_cast<size_t>(b0 + i) * n_last + (lo - first)) * h->Vl;
      int32_t r2 = run_logits(h, per, h->row_select + static_cast<size_t>(i) * per, dst, false, s);
      if (r2) return r2;
    }
    return MTJ_OK;
  });
  return rc;
}

int32_t mtj_eval_loss(mtj_handle* h, const uint32_t* obs, const uint32_t* target, const uint32_t* ctx_len,
                      int32_t batch, int32_t T, float* all_loss, uint8_t* correct, mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (h->mp > 1 && !h->comm) return fail(MTJ_ERR_STATE, "cores_per_replica > 1 needs mtj_comm_init first");
  if (!obs || !target || !all_loss || !correct || batch <= 0 || batch > h->max_batch)
    return fail(MTJ_ERR_INVALID, "bad argument");
  if (T <= 0 || T > h->ring_pages * mtj::kPageTokens || T > h->max_pos)
    return fail(MTJ_ERR_INVALID, "T exceeds the KV capacity");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::vector<int32_t> pad(batch, 0), limit(batch);
  // mask = (arange(T) > ctx_length) * -1e10 on the keys (transformer_shard.py:130)
  for (int b = 0; b < batch; ++b) limit[b] = ctx_len ? static_cast<int32_t>(std::min<uint32_t>(ctx_len[b], 0x7fffffffu)) : T;
  rc = setup_sequences(h, pad, limit, T, s);
  if (rc) return rc;
  h->prefilled = false;
  rc = forward_chunks(h, obs, T, batch, T, h->key_limit, s, [&](int b0, int ns, int t0, int tc) -> int32_t {
    const int M = ns * tc;
    mtj::CeArgs ce = {};
    ce.vl = h->Vl;
    ce.vocab_start = h->rank * h->Vl;
    ce.rows = {b0, tc, t0, nullptr};
    ce.T = T;
    ce.targets = target;
    ce.pmax = h->ce_max;
    ce.psum = h->ce_sum;
    ce.hit = h->ce_hit;
    ce.loss_out = all_loss;
    ce.correct_out = correct;
    const bool fused = h->fused_ce && use_tc(h, M);
    const int step = fused ? h->ce_rows : h->eval_rows;
    for (int m0 = 0; m0 < M; m0 += step) {
      const int n = std::min(step, M - m0);
      if (fused && use_tc_wide(h, n)) {
        int32_t r3 = run_loss_rows_fused(h, n, m0, ce, s);
        if (r3) return r3;
        continue;
      }
      int32_t r2 = use_tc(h, M) ? run_logits_tc(h, n, m0, h->eval_logits, s)
                                : run_logits(h, n, nullptr, h->eval_logits, false, s, m0);
      if (r2) return r2;
      ce.logits = h->eval_logits;
      ce.row0 = m0;
      MTJ_CUDA(mtj::launch_ce_partial(ce, n, s));
      h->launches++;
    }
    if (h->mp > 1) {
      std::string err;
      MTJ_CUDA(cudaMemcpyAsync(h->ce_lmax, h->ce_max, sizeof(float) * M, cudaMemcpyDeviceToDevice, s));
      if (mtj::comm_all_reduce(h->comm, h->ce_max, M, true, s, &err)) return fail(MTJ_ERR_COMM, err);
    }
    MTJ_CUDA(mtj::launch_ce_rescale(ce, h->mp > 1 ? h->ce_lmax : h->ce_max, M, s));
    if (h->mp > 1) {
      std::string err;
      if (mtj::comm_all_reduce(h->comm, h->ce_sum, 2 * static_cast<size_t>(M), false, s, &err))
        return fail(MTJ_ERR_COMM, err);
    }
    MTJ_CUDA(mtj::launch_ce_finalize(ce, M, s));
    h->launches += 2;
    return MTJ_OK;
  });
  return rc;
}

int32_t mtj_set_seed(mtj_handle* h, uint64_t seed, mtj_stream stream) {
  if (!h || !h->bound) return fail(MTJ_ERR_STATE, "not bound");
  const uint32_t words[2] = {static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MTJ_CUDA(cudaMemcpyAsync(h->rng_seed, words, sizeof(words), cudaMemcpyHostToDevice, s));
  MTJ_CUDA(cudaStreamSynchronize(s));      // `words` lives on this stack frame
  return MTJ_OK;
}

int32_t mtj_generate(mtj_handle* h, int32_t gen_length, int32_t greedy, const float* top_p, const float* temp,
                     const float* uniforms, uint32_t* tokens_out, float* logits_out, mtj_stream stream) {
  if (!h) return fail(MTJ_ERR_INVALID, "null handle");
  if (gen_length <= 0) return fail(MTJ_ERR_INVALID, "gen_length must be positive");
  const size_t B = static_cast<size_t>(h->batch), V = static_cast<size_t>(h->V);
  for (int t = 0; t < gen_length; ++t) {
    const int32_t rc = mtj_decode_step(h, nullptr, top_p, temp, uniforms ? uniforms + t * B * V : nullptr, greedy,
                                       tokens_out ? tokens_out + t * B : nullptr,
                                       logits_out ? logits_out + t * B * V : nullptr, stream);
    if (rc) return rc;
  }
  return MTJ_OK;
}

int64_t mtj_sample_scratch_bytes(int32_t rows, int32_t vocab) {
  if (rows <= 0 || vocab <= 0) return -1;
  return mtj::sample_scratch_bytes(rows, vocab);
}

int32_t mtj_set_top_k(mtj_handle* h, const int32_t* top_k, int32_t batch, mtj_stream stream) {
  if (!h || !h->bound) return fail(MTJ_ERR_STATE, "not bound");
  if (!top_k) {
    h->has_top_k = false;
    return MTJ_OK;
  }
  if (batch < 1 || batch > h->max_batch) return fail(MTJ_ERR_INVALID, "batch outside [1, max_batch]");
  MTJ_CUDA(cudaMemcpyAsync(h->top_k, top_k, sizeof(int32_t) * batch, cudaMemcpyDeviceToDevice,
                           static_cast<cudaStream_t>(stream)));
  h->has_top_k = true;
  return MTJ_OK;
}

int32_t mtj_sample_top_p(const float* logits, const float* uniforms, const float* top_p, const int32_t* top_k,
                         const float* temp, int32_t rows, int32_t vocab, void* scratch, int64_t scratch_bytes,
                         uint32_t* tokens_out, mtj_stream stream) {
  if (!logits || !uniforms || !top_p || !temp || !scratch || !tokens_out)
    return fail(MTJ_ERR_INVALID, "null argument");
  if (rows <= 0 || vocab <= 0) return fail(MTJ_ERR_INVALID, "rows and vocab must be positive");
  if (scratch_bytes < mtj::sample_scratch_bytes(rows, vocab)) return fail(MTJ_ERR_INVALID, "scratch too small");
  mtj::SampleArgs sa = {};
  sa.logits = logits;
  sa.uniforms = uniforms;
  sa.top_p = top_p;
  sa.top_k = top_k;
  sa.temp = temp;
  sa.rows = rows;
  sa.V = vocab;
  sa.scratch = scratch;
  sa.tokens = tokens_out;
  MTJ_CUDA(mtj::launch_sample_top_p(sa, static_cast<cudaStream_t>(stream), false));
  return MTJ_OK;
}

int32_t mtj_mega_trace(mtj_handle* h, int32_t enable, uint64_t* out, int32_t n, mtj_stream stream) {
  if (!h || !h->bound) return fail(MTJ_ERR_STATE, "not bound");
  if (out) {
    if (n > 6 * h->L + 3) n = 6 * h->L + 3;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MTJ_CUDA(cudaMemcpyAsync(out, h->mega_trace, sizeof(uint64_t) * n, cudaMemcpyDeviceToHost, s));
    MTJ_CUDA(cudaStreamSynchronize(s));
  }
  if ((enable != 0) != h->mega_trace_on) {
    h->mega_trace_on = enable != 0;
    if (h->graph_exec) {            // the trace pointer is baked into the captured step
      cudaGraphExecDestroy(h->graph_exec);
      h->graph_exec = nullptr;
    }
  }
  return MTJ_OK;
}

int64_t mtj_launch_count(const mtj_handle* h) { return h ? h->launches : -1; }

int32_t mtj_profile_enable(mtj_handle* h, int32_t on) {
  if (!h) return fail(MTJ_ERR_INVALID, "null handle");
  if (on && h->ev_pool.empty()) {
    h->ev_pool.resize(2 * (4 * static_cast<size_t>(h->L) + 2) * 64);
    for (auto& e : h->ev_pool) MTJ_CUDA(cudaEventCreate(&e));
  }
  h->profile = on != 0;
  h->ev_used = 0;
  h->ev_spans.clear();
  return MTJ_OK;
}

int32_t mtj_profile_read(mtj_handle* h, double* ms_sum, int64_t* count, mtj_stream stream) {
  if (!h || !ms_sum || !count) return fail(MTJ_ERR_INVALID, "null argument");
  MTJ_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  for (int f = 0; f < MTJ_FAMILY_COUNT; ++f) {
    ms_sum[f] = 0.0;
    count[f] = 0;
  }
  for (const auto& sp : h->ev_spans) {
    float ms = 0.f;
    MTJ_CUDA(cudaEventElapsedTime(&ms, h->ev_pool[sp.second.first], h->ev_pool[sp.second.second]));
    ms_sum[sp.first] += ms;
    count[sp.first] += 1;
  }
  h->ev_used = 0;
  h->ev_spans.clear();
  return MTJ_OK;
}

int32_t mtj_check_device_status(mtj_handle* h, mtj_stream stream) {
  if (!h || !h->bound) return fail(MTJ_ERR_STATE, "not bound");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t w = 0;
  MTJ_CUDA(cudaMemcpyAsync(&w, h->dev_err, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
  MTJ_CUDA(cudaStreamSynchronize(s));
  if (w) {
    MTJ_CUDA(cudaMemsetAsync(h->dev_err, 0, sizeof(uint32_t), s));
    if (w & mtj::kDevErrTimeout) return fail(MTJ_ERR_TIMEOUT, "a bounded device-side wait ran out");
    return fail(MTJ_ERR_INVALID, "a kernel rejected an index");
  }
  return MTJ_OK;
}

int32_t mtj_k_layer(mtj_handle* h, int32_t layer, const float* x_in, int32_t batch, int32_t T, int32_t pos0,
                    const int32_t* pad_host, const int32_t* key_limit_host, int32_t decode, float* out,
                    mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (h->mp > 1 && !h->comm) return fail(MTJ_ERR_STATE, "cores_per_replica > 1 needs mtj_comm_init first");
  if (!x_in || !out || layer < 0 || layer >= h->L || batch <= 0 || batch > h->max_batch || T <= 0)
    return fail(MTJ_ERR_INVALID, "bad argument");
  const int64_t M = static_cast<int64_t>(batch) * T;
  if (M > h->max_rows) return fail(MTJ_ERR_INVALID, "batch * T exceeds max_rows");
  if (decode && T != 1) return fail(MTJ_ERR_INVALID, "decode_once takes exactly one token per sequence");   // layers.py:320
  if (pos0 < 0 || pos0 + T > h->max_pos) return fail(MTJ_ERR_INVALID, "position outside the RoPE table");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::vector<int32_t> pad(batch, 0), limit(batch, 0x7fffffff);
  for (int b = 0; b < batch; ++b) {
    if (pad_host) pad[b] = pad_host[b];
    if (key_limit_host) limit[b] = key_limit_host[b];
  }
  rc = setup_sequences(h, pad, limit, pos0, s);
  if (rc) return rc;
  h->prefilled = false;
  // x <- x_in with its LayerNorm statistics
  MTJ_CUDA(mtj::launch_residual_stats(h->x, x_in, h->stats, static_cast<int>(M), h->d, false, s, false));
  h->launches++;
  mtj::RowMap rows = {0, T, pos0, nullptr};
  if (decode) rows = {0, 1, 0, h->cur};
  if (!decode && use_tc(h, static_cast<int>(M)))
    return run_layer_tc(h, layer, static_cast<int>(M), rows, key_limit_host ? h->key_limit : nullptr, s, out);
  return run_layer(h, layer, static_cast<int>(M), rows, decode != 0, key_limit_host ? h->key_limit : nullptr, s, out);
}

int32_t mtj_k_projection(mtj_handle* h, const float* x_in, int32_t rows, float* logits_out, mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (!x_in || !logits_out || rows <= 0 || rows > h->max_rows) return fail(MTJ_ERR_INVALID, "bad argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MTJ_CUDA(mtj::launch_residual_stats(h->x, x_in, h->stats, rows, h->d, false, s, false));
  h->launches++;
  if (use_tc(h, rows)) return run_logits_tc(h, rows, 0, logits_out, s);
  return run_logits(h, rows, nullptr, logits_out, false, s);
}

int32_t mtj_k_projection_loss(mtj_handle* h, const float* x_in, const uint32_t* targets, int32_t rows,
                              float* loss_out, uint8_t* correct_out, mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (h->mp > 1 && !h->comm) return fail(MTJ_ERR_STATE, "cores_per_replica > 1 needs mtj_comm_init first");
  if (!x_in || !targets || !loss_out || !correct_out || rows <= 0 || rows > h->max_rows)
    return fail(MTJ_ERR_INVALID, "bad argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MTJ_CUDA(mtj::launch_residual_stats(h->x, x_in, h->stats, rows, h->d, false, s, false));
  h->launches++;
  mtj::CeArgs ce = {};
  ce.vl = h->Vl;
  ce.vocab_start = h->rank * h->Vl;
  ce.rows = {0, rows, 0, nullptr};
  ce.T = rows;
  ce.targets = targets;
  ce.pmax = h->ce_max;
  ce.psum = h->ce_sum;
  ce.hit = h->ce_hit;
  ce.loss_out = loss_out;
  ce.correct_out = correct_out;
  const bool fused = h->fused_ce && use_tc(h, rows);
  const int step = fused ? h->ce_rows : h->eval_rows;
  for (int m0 = 0; m0 < rows; m0 += step) {
    const int n = std::min(step, rows - m0);
    if (fused && use_tc_wide(h, n)) {
      rc = run_loss_rows_fused(h, n, m0, ce, s);
      if (rc) return rc;
      continue;
    }
    rc = use_tc(h, rows) ? run_logits_tc(h, n, m0, h->eval_logits, s)
                         : run_logits(h, n, nullptr, h->eval_logits, false, s, m0);
    if (rc) return rc;
    ce.logits = h->eval_logits;
    ce.row0 = m0;
    MTJ_CUDA(mtj::launch_ce_partial(ce, n, s));
  }
  std::string err;
  if (h->mp > 1) {
    MTJ_CUDA(cudaMemcpyAsync(h->ce_lmax, h->ce_max, sizeof(float) * rows, cudaMemcpyDeviceToDevice, s));
    if (mtj::comm_all_reduce(h->comm, h->ce_max, rows, true, s, &err)) return fail(MTJ_ERR_COMM, err);
  }
  MTJ_CUDA(mtj::launch_ce_rescale(ce, h->mp > 1 ? h->ce_lmax : h->ce_max, rows, s));
  if (h->mp > 1 && mtj::comm_all_reduce(h->comm, h->ce_sum, 2 * static_cast<size_t>(rows), false, s, &err))
    return fail(MTJ_ERR_COMM, err);
  MTJ_CUDA(mtj::launch_ce_finalize(ce, rows, s));
  return MTJ_OK;
}

int32_t mtj_k_embed(mtj_handle* h, const uint32_t* ids, int32_t rows, float* x_out, float* stats_out,
                    mtj_stream stream) {
  int32_t rc = check_ready(h);
  if (rc) return rc;
  if (!ids || !x_out || rows <= 0) return fail(MTJ_ERR_INVALID, "bad argument");
  mtj::EmbedArgs e = {};
  e.ids = ids;
  e.ids_ld = 0;
  e.rows = {0, rows, 0, nullptr};
  e.M = rows;
  e.d = h->d;
  e.vocab_local = h->Vl;
  e.vocab_start = h->rank * h->Vl;
  e.table = h->emb_w;
  e.bias = h->emb_b;
  e.x = x_out;
  e.stats = stats_out;
  MTJ_CUDA(mtj::launch_embed(e, static_cast<cudaStream_t>(stream), false));
  h->launches++;
  return MTJ_OK;
}

int64_t mtj_k_all_reduce_buffer_bytes(const mtj_handle* h, int32_t rows_cap) {
  if (!h || rows_cap <= 0) return -1;
  const int64_t data = 2LL * rows_cap * h->d * static_cast<int64_t>(sizeof(float));
  return align_up(data, 256) + 512;
}

int32_t mtj_k_all_reduce(mtj_handle* h, void* const* bufs_host, int32_t rank, int32_t world, int32_t rows_cap,
                         int32_t rows, const float* partial, float* x, float* stats, int32_t accumulate,
                         mtj_stream stream) {
  if (!h || !h->bound) return fail(MTJ_ERR_STATE, "not bound");
  if (!bufs_host || !partial || !x || !stats) return fail(MTJ_ERR_INVALID, "null argument");
  if (world < 2 || world > mtj::kP2pMaxWorld || rank < 0 || rank >= world)
    return fail(MTJ_ERR_INVALID, "the peer all-reduce takes 2..8 ranks");
  if (rows <= 0 || rows > rows_cap) return fail(MTJ_ERR_INVALID, "rows must be in [1, rows_cap]");
  for (int r = 0; r < world; ++r)
    if (!bufs_host[r] || (reinterpret_cast<uintptr_t>(bufs_host[r]) & 255))
      return fail(MTJ_ERR_INVALID, "exchange buffers must be 256-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t flag_off = static_cast<size_t>(align_up(2LL * rows_cap * h->d * static_cast<int64_t>(sizeof(float)), 256));
  mtj::P2pArgs a = {};
  a.rank = rank;
  a.world = world;
  a.d = h->d;
  a.slot_elems = static_cast<size_t>(rows_cap) * h->d;
  for (int r = 0; r < world; ++r) {
    a.peer_data[r] = reinterpret_cast<const float*>(bufs_host[r]);
    a.peer_flags[r] = reinterpret_cast<uint32_t*>(static_cast<char*>(bufs_host[r]) + flag_off);
  }
  char* mine = static_cast<char*>(bufs_host[rank]);
  a.local_flags = reinterpret_cast<const uint32_t*>(mine + flag_off);
  a.seq = reinterpret_cast<uint32_t*>(mine + flag_off + 256);
  a.ticket = a.seq + 1;
  a.x = x;
  a.stats = stats;
  a.accumulate = accumulate ? 1 : 0;
  a.dev_err = h->dev_err;
  a.wait_limit = h->wait_limit;
  // this rank's partial sums go into the data slot the exchange counter selects
  MTJ_CUDA(mtj::launch_splitk_reduce(partial, 1, rows, h->d, nullptr, nullptr, reinterpret_cast<float*>(mine), h->d,
                                     a.seq, a.slot_elems, s, false));
  MTJ_CUDA(mtj::launch_p2p_allreduce(a, rows, s, false));
  h->launches += 2;
  return MTJ_OK;
}

}  // extern "C"
