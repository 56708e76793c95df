/*
 * libmtj_b200 -- C ABI of the B200-native GPT-J forward / eval / decode path.
 *
 * The reference (kingoflolz/mesh-transformer-jax) has no FFI boundary: its hot
 * path is Python traced by JAX.  This ABI sits underneath a Python host layer
 * that mirrors the reference classes; each entry point cites the reference
 * code whose work it performs (paths relative to the reference project).
 *
 * Conventions
 *   - every function returns an int32 status (MTJ_OK == 0); nothing aborts,
 *     traps or throws; mtj_last_error() gives a message for the last failure;
 *   - all pointers named *_dev are device pointers owned by the caller; the
 *     library allocates no device memory: weights and workspace are carved
 *     from two caller-provided arenas;
 *   - all kernels are launched on the caller's stream; no entry point
 *     synchronises the device unless its comment says so;
 *   - one handle per GPU / per rank; a handle is used from one thread at a time.
 */
#ifndef MTJ_B200_H_
#define MTJ_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mtj_handle mtj_handle;
typedef void* mtj_stream;              /* a cudaStream_t */

enum {
  MTJ_OK = 0,
  MTJ_ERR_INVALID = 1,        /* bad argument / unsupported shape            */
  MTJ_ERR_STATE = 2,          /* call order (arena not bound, no prefill...) */
  MTJ_ERR_CUDA = 3,           /* a CUDA runtime call failed                  */
  MTJ_ERR_UNSUPPORTED = 4,    /* config outside the GPT-J path               */
  MTJ_ERR_TIMEOUT = 5,        /* a bounded device-side wait ran out          */
  MTJ_ERR_COMM = 6            /* collective / peer set-up failed             */
};

enum { MTJ_F32 = 0, MTJ_BF16 = 1 };

/* Keys of the reference's config JSON that the path reads
 * (configs/6B_roto_256.json:1-12; layers.py:168-170,232-245,548-549;
 * transformer_shard.py:24-26,264-265).  norm must be "layernorm" and pe
 * "rotary"; the host layer rejects anything else before calling in. */
typedef struct mtj_config {
  int32_t layers;
  int32_t d_model;
  int32_t n_heads;
  int32_t n_vocab;
  int32_t pe_rotary_dims;
  int32_t seq;
  int32_t cores_per_replica;   /* tensor-parallel degree (mp)                 */
  int32_t rank;                /* this shard's index on the "shard" axis      */
  int32_t max_batch;           /* sequences resident in the KV cache          */
  int32_t max_gen;             /* generated tokens per generate() call        */
  int32_t max_rows;            /* token rows processed per forward chunk      */
  /* Path selection and limits; 0 selects the default of each.  They are part of
   * the configuration because they change results (summation order, operand
   * precision), not only speed.                                                */
  int32_t hilo_max_batch;      /* decode batches up to this many sequences carry
                                  their activations through the tensor-core GEMMs
                                  as bf16 hi + lo pairs (about 16 mantissa bits;
                                  keeps 32-step greedy ids equal to an fp32 run);
                                  larger batches use plain bf16 activations.
                                  Default 64 (the most the path holds); < 0: never */
  int32_t mega_max_batch;      /* sequences served by the whole-step persistent
                                  decode kernel (fp32 activations); default 1,
                                  at most 4                                      */
  int32_t tc_decode_min_batch; /* from this many sequences on a decode step takes
                                  the tensor-core GEMMs; default 2               */
  int32_t wait_limit;          /* iteration limit of every bounded device-side
                                  wait on a peer or a phase counter; default
                                  1 << 22 (seconds); a wait that runs out sets
                                  the device error word (MTJ_ERR_TIMEOUT)        */
} mtj_config;

const char* mtj_last_error(void);
/* ABI revision: 3 (2: mtj_config with the tuning fields, mtj_generate, mtj_start_batch / mtj_admit;
 * 3: top_k in mtj_sample_top_p / mtj_nucleus_filter, mtj_set_top_k). */
int32_t mtj_version(void);

/* CausalTransformerShard.__init__ (transformer_shard.py:21-45): validates the
 * same divisibility conditions the reference asserts (layers.py:172,238-239,552). */
int32_t mtj_create(const mtj_config* cfg, mtj_handle** out);
int32_t mtj_destroy(mtj_handle* h);

/* Arena sizes for this handle's config, then binding of caller memory. */
int64_t mtj_weights_bytes(const mtj_handle* h);
int64_t mtj_workspace_bytes(const mtj_handle* h);
int32_t mtj_bind_arenas(mtj_handle* h, void* weights_dev, int64_t weights_bytes,
                        void* workspace_dev, int64_t workspace_bytes, mtj_stream s);

/* Loads one per-shard leaf of CausalTransformer.state["params"]
 * (transformer_shard.py:184-188; names and layouts as to_hf_weights.py:160-173:
 * "<module>/<leaf>" with module in {embedding_shard, layer_<i>, projection_shard}
 * and leaf in {linear[_k]/w, linear[_k]/b, replicated_layer_norm/scale|offset}).
 * src_dev holds this shard's slice in the reference layout ([in, out] for w);
 * it is repacked to bf16 into the weight arena (move_xmap's cast,
 * transformer_shard.py:250-253) and may be freed after the stream has run. */
int32_t mtj_load_param(mtj_handle* h, const char* name, const void* src_dev,
                       int32_t dtype, int32_t ndim, const int64_t* shape, mtj_stream s);

/* Tensor-parallel plumbing standing in for jax.lax.psum / pmax / all_gather on
 * the "shard" axis (util.py:134-136; layers.py:193,313,565,575-585): one NCCL
 * communicator over the cores_per_replica ranks.  Rank 0 obtains a 128-byte id
 * with mtj_comm_unique_id, the host distributes it, every rank calls
 * mtj_comm_init (collective; blocks until all ranks have joined).  NCCL is
 * looked up in the process at run time (libnccl.so.2).  Not needed for mp == 1. */
int32_t mtj_comm_unique_id(uint8_t* out128);
int32_t mtj_comm_init(mtj_handle* h, const uint8_t* id128);

/* Optional low-latency form of the same psum for decode-size messages
 * ([batch, d_model] fp32): the ranks read each other's partial sums directly
 * over NVLink peer memory and fuse the residual add and LayerNorm statistics
 * into the same kernel.  mtj_p2p_export allocates this rank's exchange buffer
 * (the one device allocation the library makes itself: it has to be exportable
 * to the other ranks' processes) and returns its 64-byte CUDA IPC handle; the
 * host gathers the handles of all ranks in rank order and passes them to
 * mtj_p2p_import on every rank.  Without these calls all reductions use NCCL. */
int32_t mtj_p2p_export(mtj_handle* h, uint8_t* ipc_handle_out64);
int32_t mtj_p2p_import(mtj_handle* h, const uint8_t* ipc_handles_all_ranks);

/* generate_initial (transformer_shard.py:74-95) for `batch` left-padded
 * contexts: prefills ctx[:, :-1] into the KV cache, keeps ctx[:, -1] as the
 * first decode input.  ctx_dev: [batch, seq] uint32; ctx_length_host: [batch]
 * (number of real tokens, >= 1).  Host-synchronous only in page set-up. */
int32_t mtj_prefill(mtj_handle* h, const uint32_t* ctx_dev, const uint32_t* ctx_length_host,
                    int32_t batch, mtj_stream s);

/* Continuous batching -- the reference's serving loop (device_serve.py:138-194)
 * runs fixed batches: every request waits for a whole generate call.  These two
 * calls let a sequence join a batch that is already decoding.
 * mtj_start_batch opens a running batch of `batch` idle slots (the state
 * mtj_prefill leaves, without any context).  mtj_admit puts a prompt into one
 * slot between two decode steps: its first len - 1 tokens are prefilled at the
 * positions right before the batch's current decode position and its last token
 * becomes the slot's next input -- generate_initial (transformer_shard.py:74-95)
 * in a frame shifted by the steps the batch has taken, which changes nothing
 * because cached keys are rotated at absolute positions and attention depends
 * on distances only.  The slot's earlier contents fall out of its window.
 * prompt_dev: [len] uint32 device, 1 <= len <= seq.  A slot whose sequence has
 * finished simply keeps stepping until the next mtj_admit; the batch can take
 * max_gen steps in total. */
int32_t mtj_start_batch(mtj_handle* h, int32_t batch, mtj_stream s);
int32_t mtj_admit(mtj_handle* h, int32_t slot, const uint32_t* prompt_dev, int32_t len, mtj_stream s);

/* One step of the generate scan (transformer_shard.py:198-210): generate_once
 * then the sampler.  tokens_in_dev may be NULL (use the previous step's
 * sample / the held-back last prompt token).  top_p/temp: [batch] f32 device;
 * uniforms_dev: [batch, n_vocab] f32, or NULL (greedy, or sampling with the
 * device generator of mtj_set_seed).
 * Outputs: tokens_out_dev [batch] uint32 (may be NULL),
 * logits_out_dev [batch, n_vocab] f32 (may be NULL). */
int32_t mtj_decode_step(mtj_handle* h, const uint32_t* tokens_in_dev,
                        const float* top_p_dev, const float* temp_dev,
                        const float* uniforms_dev, int32_t greedy,
                        uint32_t* tokens_out_dev, float* logits_out_dev, mtj_stream s);

/* The PRNG key of the generate scan (transformer_shard.py:327,335:
 * hk.PRNGSequence(random.randint(0, 2**60)), split once per step at :200).
 * When mtj_decode_step / mtj_generate sample (greedy == 0) without supplied
 * uniforms, the uniforms come from a counter-based generator on the device
 * (Philox4x32-10) keyed by this seed and indexed by (decode position,
 * sequence, vocabulary entry): the same seed gives the same tokens, and every
 * shard of a tensor-parallel group must be given the same seed.  Synchronises
 * the stream. */
int32_t mtj_set_seed(mtj_handle* h, uint64_t seed, mtj_stream s);

/* The sampler's top_k option (sampling.py:41 nucleaus_sample(..., top_k)) for
 * the sampled steps of mtj_decode_step / mtj_generate that follow:
 * top_k_dev [batch] int32 is copied; NULL returns to top_k = None. */
int32_t mtj_set_top_k(mtj_handle* h, const int32_t* top_k_dev, int32_t batch, mtj_stream s);

/* The whole scan of generate (transformer_shard.py:198-212) from one call:
 * gen_length decode steps (generate_once + sampler) enqueued back to back on
 * the stream as replays of the captured step, no host round trip in between.
 * tokens_out_dev [gen_length, batch] uint32 (may be NULL), logits_out_dev
 * [gen_length, batch, n_vocab] f32 or NULL, uniforms_dev [gen_length, batch,
 * n_vocab] f32 or NULL (device generator, see mtj_set_seed); top_p/temp as in
 * mtj_decode_step. */
int32_t mtj_generate(mtj_handle* h, int32_t gen_length, int32_t greedy, const float* top_p_dev,
                     const float* temp_dev, const float* uniforms_dev, uint32_t* tokens_out_dev,
                     float* logits_out_dev, mtj_stream s);

/* CausalTransformerShard.loss (transformer_shard.py:47-72, :123-132):
 * obs/target [batch, T] uint32 device, ctx_length_host [batch];
 * all_loss_out_dev [batch, T] f32, correct_out_dev [batch, T] uint8. */
int32_t mtj_eval_loss(mtj_handle* h, const uint32_t* obs_dev, const uint32_t* target_dev,
                      const uint32_t* ctx_length_host, int32_t batch, int32_t T,
                      float* all_loss_out_dev, uint8_t* correct_out_dev, mtj_stream s);

/* Full-sequence logits of the last `n_last` positions (proj(x),
 * transformer_shard.py:95): logits_out_dev [batch, n_last, n_vocab/mp] f32. */
int32_t mtj_forward_logits(mtj_handle* h, const uint32_t* obs_dev, const uint32_t* ctx_length_host,
                           int32_t batch, int32_t T, int32_t n_last,
                           float* logits_out_dev, mtj_stream s);

/* nucleaus_sample (sampling.py:10-44): logits [rows, vocab] f32, uniforms
 * [rows, vocab] f32 in (0,1), top_p/temp [rows], top_k [rows] int32 or NULL
 * (the reference's top_k = None); scratch from
 * mtj_sample_scratch_bytes(rows, vocab).  An entry whose rank in the
 * descending order is >= top_k[r] loses 1e10 * (its own index), as
 * sampling.py:15-26 computes it. */
int64_t mtj_sample_scratch_bytes(int32_t rows, int32_t vocab);
int32_t mtj_sample_top_p(const float* logits_dev, const float* uniforms_dev,
                         const float* top_p_dev, const int32_t* top_k_dev, const float* temp_dev,
                         int32_t rows, int32_t vocab, void* scratch_dev, int64_t scratch_bytes,
                         uint32_t* tokens_out_dev, mtj_stream s);

/* Counters for the benchmark: kernels launched by this handle so far. */
int64_t mtj_launch_count(const mtj_handle* h);

/* Optional kernel-family timing for the benchmark's roofline figure: while
 * enabled, every launch of the dominant kernel families is bracketed by CUDA
 * events on the caller's stream (up to 64 steps' worth between reads).
 * mtj_profile_read synchronises the stream, fills ms_sum[MTJ_FAMILY_COUNT] /
 * count[MTJ_FAMILY_COUNT] and clears the record.  No reference counterpart. */
enum { MTJ_FAMILY_INPROJ = 0,    /* LN + Q/K/V (+ FF-in when launched as one kernel) projection */
       MTJ_FAMILY_ATTN = 1, MTJ_FAMILY_OUTPROJ = 2, MTJ_FAMILY_LOGITS = 3,
       MTJ_FAMILY_FFIN = 4,      /* the FF-in half of the in-projection when it is launched on its own */
       MTJ_FAMILY_COUNT = 5 };
int32_t mtj_profile_enable(mtj_handle* h, int32_t on);
int32_t mtj_profile_read(mtj_handle* h, double* ms_sum, int64_t* count, mtj_stream s);

/* Phase time stamps of the persistent decode kernel (profiling aid, no reference
 * counterpart): enable != 0 makes later steps record, for block 0, the
 * %globaltimer value (ns) at 6 points per layer (before / after the wait for
 * the residual stream, after its in-projection rows, after its attention units,
 * after the wait for all attention + FF-in, after its out-projection rows) and 3
 * at the end; out (host, n entries, may be NULL) receives the last step's record. */
int32_t mtj_mega_trace(mtj_handle* h, int32_t enable, uint64_t* out_host, int32_t n, mtj_stream s);

/* Reads (and clears) the device-side error word of this handle; synchronises
 * the stream.  MTJ_ERR_TIMEOUT if a bounded wait in a kernel ran out. */
int32_t mtj_check_device_status(mtj_handle* h, mtj_stream s);

/* Unit entry points: one per kernel family, for parity tests ---------------- */

/* EmbeddingShard.__call__ (layers.py:187-193), local part: rows of this
 * shard's table for ids in its range (else 0) plus this shard's bias.
 * Also returns LayerNorm statistics (mean, rstd) per row when mp == 1. */
int32_t mtj_k_embed(mtj_handle* h, const uint32_t* ids_dev, int32_t rows,
                    float* x_out_dev, float* stats_out_dev, mtj_stream s);

/* TransformerLayerShard.__call__ (layers.py:299-313), get_init_decode_state
 * (:347-366) and decode_once (:316-344) of layer `layer`: x_dev [batch*T, d] f32
 * is the layer input, out_dev receives g_psum(attn_out + dense_out) -- the
 * residual is NOT added, as in the reference.  Row (b, t) sits at absolute
 * position pos0 + t.  pad_host[b] (or NULL = 0) is the first visible key
 * position (left padding, :353-360); key_limit_host[b] (or NULL) masks keys
 * with position > limit (the eval mask, transformer_shard.py:130).  The
 * layer's K/V for these rows are written to the cache; with decode != 0
 * (T must be 1, :320) attention runs over the sliding window ending at pos0. */
int32_t mtj_k_layer(mtj_handle* h, int32_t layer, const float* x_dev, int32_t batch, int32_t T, int32_t pos0,
                    const int32_t* pad_host, const int32_t* key_limit_host, int32_t decode,
                    float* out_dev, mtj_stream s);

/* ProjectionShard.__call__ before the all-gather (layers.py:561-564):
 * logits_out_dev [rows, n_vocab/mp] of this shard. */
int32_t mtj_k_projection(mtj_handle* h, const float* x_dev, int32_t rows, float* logits_out_dev, mtj_stream s);

/* ProjectionShard.loss with z_loss = 0 (layers.py:569-593): targets_dev [rows]
 * uint32 -> loss_out_dev [rows] f32, correct_out_dev [rows] uint8. */
int32_t mtj_k_projection_loss(mtj_handle* h, const float* x_dev, const uint32_t* targets_dev, int32_t rows,
                              float* loss_out_dev, uint8_t* correct_out_dev, mtj_stream s);

/* Single-query attention of decode_once over the paged bf16 KV cache
 * (layers.py:316-338 with self_attn :260-283, before the output projection):
 * q_dev [batch, heads*d_head] f32 (rotated, unscaled); kpool/vpool
 * [pages][heads][64][d_head] bf16; page_table_dev [batch, ring_pages];
 * pad_dev [batch] first valid position; cur_dev[0] the query position; keys
 * [max(pad, cur-window+1), cur] are visible.  out_dev[b*ld_out + head*d_head + j].
 * scratch_dev (mtj_k_decode_attn_scratch_bytes) holds the per-split partial
 * results; the call clears the part of it that must start at zero. */
int64_t mtj_k_decode_attn_scratch_bytes(int32_t batch, int32_t heads, int32_t d_head, int32_t window,
                                        int32_t split_tokens);
int32_t mtj_k_decode_attn(const float* q_dev, const void* kpool_dev, const void* vpool_dev,
                          const int32_t* page_table_dev, const int32_t* pad_dev, const int32_t* cur_dev,
                          int32_t batch, int32_t heads, int32_t d_head, int32_t window,
                          int32_t ring_pages, int32_t split_tokens,
                          void* scratch_dev, int64_t scratch_bytes,
                          float* out_dev, int32_t ld_out, mtj_stream s);

/* ProjectionShard.__call__ before the all-gather (layers.py:561-564), also the
 * shape of every LayerNorm + Linear pair on the decode path: out[m, n] =
 * sum_k w[n, k] * (scale[k]*rstd[m]*(x[m, k]-mean[m]) + offset[k]) + bias[n].
 * w_dev bf16 [N, K] (the library's packed layout), x_dev f32 [M, K], stats_dev
 * [M, 2] = (mean, rstd).  k_split in {0 (auto),1,2,4,8} and rows_per_group in
 * {0 (default),8} select the launch shape (tuning knobs; results do not depend
 * on them beyond fp32 summation order). */
int32_t mtj_k_ln_gemv(const void* w_dev, const float* x_dev, const float* stats_dev,
                      const float* ln_scale_dev, const float* ln_offset_dev, const float* bias_dev,
                      int32_t M, int32_t N, int32_t K, int32_t k_split, int32_t rows_per_group,
                      float* out_dev, mtj_stream s);

/* The tensor-core form of the same Linear for many token rows (prefill / eval;
 * hk.Linear of layers.py:249-258,559 on [T, d] inputs): out[m, n] =
 * sum_k w[n, k] * x[m, k] + bias[n] with w_dev bf16 [N, K], x_dev bf16 [M, K],
 * fp32 accumulation in tensor memory, out_dev f32 [M, N].  K % 64 == 0. */
int32_t mtj_k_gemm_tc(const void* w_dev, const void* x_dev, const float* bias_dev, int32_t M, int32_t N,
                      int32_t K, float* out_dev, mtj_stream s);

/* The uniforms the device generator yields for (seed, decode position): out_dev
 * [rows, vocab] f32 in [tiny, 1).  The decode position of step t of a generate
 * call is seq - 1 + t.  For tests that replay a sampled step on the host. */
int32_t mtj_k_rng_uniforms(uint64_t seed, int32_t position, int32_t rows, int32_t vocab, float* out_dev,
                           mtj_stream s);

/* nucleaus_filter (sampling.py:10-38; top_k_dev [rows] int32 or NULL) on its own:
 * filtered_out_dev[r, i] = logits[r, i] - 1e10 * removed[r, i], where an entry
 * is removed when the softmax mass of the entries sorted before it (descending,
 * higher index first among equals) exceeds top_p[r]; the first entry stays. */
int32_t mtj_nucleus_filter(const float* logits_dev, const float* top_p_dev, const int32_t* top_k_dev,
                           int32_t rows, int32_t vocab,
                           float* filtered_out_dev, mtj_stream s);

/* The attention of self_attn before the output projection (layers.py:275-283)
 * for the rows of a forward chunk, with the causal mask of :305-308, the
 * left-pad mask of :353-360 and the eval key mask of transformer_shard.py:130:
 * flash-style on the tensor cores, d_head 256.  q_bf16_dev [batch*T, heads*d_head]
 * bf16 (rotated, unscaled), row (b, t) being the query at absolute position
 * pos0 + t of sequence b; the keys and values of positions [pad[b], pos0 + T)
 * must already be in the paged pools (kpool/vpool [n_pages][heads][64][d_head]
 * bf16, keys rotated; page_table_dev [batch, ring_pages]).  A query sees the
 * keys at positions pad[b] <= p <= min(its own, key_limit_dev[b]) (key_limit_dev
 * may be NULL).  out_bf16_dev[(b*T + t)*ld_out + head*d_head + j]; rows that see
 * no key give zeros.  status_dev (may be NULL): a device word that receives bit 0
 * if a bounded wait inside the kernel ran out. */
int32_t mtj_k_prefill_attn(const void* q_bf16_dev, const void* kpool_dev, const void* vpool_dev, int32_t n_pages,
                           const int32_t* page_table_dev, const int32_t* pad_dev, const int32_t* key_limit_dev,
                           int32_t batch, int32_t T, int32_t pos0, int32_t heads, int32_t d_head,
                           int32_t ring_pages, void* out_bf16_dev, int32_t ld_out, uint32_t* status_dev,
                           mtj_stream s);

/* g_psum (util.py:134-136) for decode-size messages over peer memory, fused
 * with the residual add of the caller (transformer_shard.py:60,112) and the
 * LayerNorm statistics of the next layer (layers.py:18-19,32):
 *   x[rows, d_model] (+)= sum over ranks of partial;  stats[rows, 2] = (mean, rstd).
 * Every rank owns one exchange buffer of mtj_k_all_reduce_buffer_bytes bytes,
 * zeroed once and mapped into its peers (CUDA IPC or peer access);
 * bufs_host[r] is rank r's buffer as seen from this process (bufs_host[rank] the
 * rank's own).  All ranks make the same sequence of calls with the same rows_cap;
 * call n of a rank waits -- at most mtj_config.wait_limit polls per peer -- for
 * call n of every peer.  A wait that runs out leaves x unchanged for this call
 * and is reported by mtj_check_device_status as MTJ_ERR_TIMEOUT; the handle and
 * the CUDA context stay usable.  partial_dev [rows, d_model] f32 is read before
 * the call's kernels end; the handle supplies d_model, the wait limit and the
 * error word. */
int64_t mtj_k_all_reduce_buffer_bytes(const mtj_handle* h, int32_t rows_cap);
int32_t mtj_k_all_reduce(mtj_handle* h, void* const* bufs_host, int32_t rank, int32_t world, int32_t rows_cap,
                         int32_t rows, const float* partial_dev, float* x_dev, float* stats_dev,
                         int32_t accumulate, mtj_stream s);

/* No counterpart in the reference.  The same attention as mtj_k_decode_attn
 * for callers that can neither pass scratch memory nor tolerate an allocation
 * inside the library (custom-call handlers with framework-planned buffers,
 * processes whose GPU memory is already reserved by another runtime, loops
 * that cannot afford the device synchronisation an allocation implies).  The
 * scratch is a fixed MTJ_NOALLOC_SCRATCH_BYTES array inside the library image,
 * resident on every GPU that loads the library until the process exits; the
 * call allocates nothing.  Shapes whose scratch need
 * (mtj_k_decode_attn_scratch_bytes) exceeds that size are rejected with
 * MTJ_ERR_INVALID.  The first call on each device looks the array's device
 * address up (with that device current) and should therefore be made before
 * any stream capture begins; the looked-up address is kept until the process
 * exits, so a host that destroys the device's context (cudaDeviceReset) must not
 * use this entry point on that device afterwards.  All calls on a device share
 * the one array: two calls whose kernels can overlap on the GPU (different
 * streams) race; calls on one stream are safe, each call re-initialising what
 * it needs. */
#define MTJ_NOALLOC_SCRATCH_BYTES (4 * 1024 * 1024)
int32_t mtj_k_decode_attn_noalloc(const float* q_dev, const void* kpool_dev, const void* vpool_dev,
                                  const int32_t* page_table_dev, const int32_t* pad_dev,
                                  const int32_t* cur_dev, int32_t batch, int32_t heads, int32_t d_head,
                                  int32_t window, int32_t ring_pages, int32_t split_tokens,
                                  float* out_dev, int32_t ld_out, mtj_stream s);

#ifdef __cplusplus
}
#endif
#endif  /* MTJ_B200_H_ */
