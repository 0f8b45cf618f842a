/*
 * liblcu — C-ABI of the B200 (sm_100a) decode token loop.
 *
 * This is the boundary a host written in any language binds against.  Every entry point
 * names the piece of YdrMaster/llama.cu it stands in for (paths inside that project).
 * Conventions:
 *   - all functions are `extern "C"`, take plain pointers and sizes, never throw;
 *   - unless stated otherwise they return 0 on success and a negative LCU_ERR_* code on
 *     failure, with a human-readable message available from lcu_last_error_string();
 *     the three sampler functions keep the reference's own `cudaError_t` convention;
 *   - operator entry points (lcu_op_*) never allocate, never synchronise and enqueue all
 *     work on the caller's stream, so they may be captured into CUDA graphs — the same
 *     contract as the reference's `Operator::launch` (llama.cu/src/op/mod.rs:29-37);
 *   - the caller owns all device memory handed in; strides are in ELEMENTS.
 * There is no CPU fallback: every compute entry point fails with LCU_ERR_CUDA when no
 * sm_100 device is usable.
 */
#ifndef LCU_H
#define LCU_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LCU_API __attribute__((visibility("default")))
#else
#define LCU_API
#endif

/* `cudaStream_t` without including the CUDA headers */
typedef struct CUstream_st *lcu_stream_t;

enum {
    LCU_OK = 0,
    LCU_ERR_INVALID = -1,   /* bad argument, shape or dtype (the reference panics here) */
    LCU_ERR_CUDA = -2,      /* a CUDA runtime call failed */
    LCU_ERR_OVERFLOW = -3,  /* sequence would exceed nctx (ReturnReason::Overflow, lib.rs:153-158) */
    LCU_ERR_NO_PAGES = -4,  /* KV page pool exhausted */
    LCU_ERR_STATE = -5,     /* call order wrong (weights missing, pool missing ...) */
    LCU_ERR_COMM = -6,      /* collective library unavailable or failed */
    LCU_ERR_TIMEOUT = -7    /* a bounded device- or host-side wait ran out */
};

typedef enum { LCU_F16 = 0, LCU_BF16 = 1, LCU_F32 = 2, LCU_Q8_0 = 3, LCU_U32 = 4 } lcu_dtype;

typedef enum {
    LCU_W_EMBD = 0,      /* token_embd.weight   [vocab, d]                  */
    LCU_W_ATTN_NORM = 1, /* blk.N.attn_norm     [d]                         */
    LCU_W_QKV = 2,       /* blk.N.attn_qkv      [(nh+2*nkvh)*dh, d]  q|k|v  */
    LCU_W_O = 3,         /* blk.N.attn_output   [d, nh*dh]                  */
    LCU_W_FFN_NORM = 4,  /* blk.N.ffn_norm      [d]                         */
    LCU_W_GATE_UP = 5,   /* blk.N.ffn_gate_up   [2*di, d]         gate|up   */
    LCU_W_DOWN = 6,      /* blk.N.ffn_down      [d, di]                     */
    LCU_W_OUT_NORM = 7,  /* output_norm         [d]                         */
    LCU_W_LM_HEAD = 8    /* output.weight       [vocab, d]                  */
} lcu_weight_kind;

/* Model description: the fields llama.cu/src/model/mod.rs:61-78 reads from GGUF metadata.
 * Under tensor parallelism nh, nkvh and di are the WHOLE model's; the context derives the
 * per-rank shapes the way `Distribution{start,len,total}` does (exec/engine.rs:93-97). */
typedef struct {
    int32_t n_layers, d, nh, nkvh, dh, di, vocab, nctx;
    float eps, theta;
    int32_t act_dtype;    /* LCU_F16 or LCU_BF16: activations, KV cache, logits            */
    int32_t weight_dtype; /* dtype of the six linear weights: act_dtype or LCU_Q8_0        */
    int32_t norm_dtype;   /* dtype of the norm weights: act_dtype or LCU_F32               */
    int32_t page_tokens;  /* tokens per KV page, power of two in [8,128]; 0 = reference rule */
    int32_t max_tokens;   /* largest round in tokens; 0 = 1024 (NTOKS, exec/engine.rs:68)  */
    int32_t max_seqs;     /* most requests in one round; 0 = 64                            */
} lcu_model_desc;

/* == `KVPair` (llama.cu/src/op/random_sample/mod.rs:29-36) == cub::KeyValuePair<int,half> */
typedef struct {
    uint32_t idx;
    uint16_t val; /* the winning logit in the activation dtype */
    uint16_t pad;
} lcu_kv_pair;

/* == `SampleArgs` (random_sample/mod.rs:38-83); {0, 1, SIZE_MAX} is ARG_MAX */
typedef struct {
    float temperature;
    float top_p;
    uint64_t top_k;
} lcu_sample_args;

/* One request of a round == `Req{kv_cache,pos,seq}` (exec/group.rs:20-25) */
typedef struct {
    int32_t seq;  /* sequence handle from lcu_seq_create */
    uint32_t pos; /* tokens already in its cache */
    uint32_t len; /* new tokens in this round (prompt length, or 1 when decoding) */
} lcu_req;

typedef struct lcu_ctx lcu_ctx;

/* ------------------------------------------------------------------ errors / info */
LCU_API const char *lcu_last_error_string(void); /* replaces the reference's panics / `check!` asserts */
LCU_API int lcu_version(void);

/* ------------------------------------------------------------------ context
 * == `Handle` + `ModelGroup` + `OutputHead` for one GPU (handle.rs:10-58, exec/group.rs:27-87,
 * exec/output_head.rs:14-52).  `nccl_comm` is an `ncclComm_t` (or NULL when tp_size == 1).
 * The context allocates its activation arena once here; nothing on the step path allocates. */
LCU_API int lcu_ctx_create(const lcu_model_desc *desc, int device, int tp_rank, int tp_size, void *nccl_comm,
                   lcu_ctx **out);
LCU_API int lcu_ctx_destroy(lcu_ctx *ctx);
/* Registers a caller-owned device tensor (weights stay where `load_weight` put them,
 * load/mod.rs:23-67).  `bytes` must equal the per-rank size for that kind.  Q8_0 linear
 * weights are passed in the plane layout produced by lcu_repack_q8_0. */
LCU_API int lcu_set_weight(lcu_ctx *ctx, int layer, int kind, const void *dev_ptr, size_t bytes);
/* Size in bytes of weight `kind` for this rank (after TP slicing and Q8_0 repacking). */
LCU_API size_t lcu_weight_bytes(const lcu_ctx *ctx, int kind);
/* f32 sin/cos tables [nctx, dh/2] on the device == `insert_sin_cos` (model/mod.rs:49-59).
 * Optional: the context builds them itself with lcu_build_sin_cos when never set. */
LCU_API int lcu_set_rope_tables(lcu_ctx *ctx, const float *sin_dev, const float *cos_dev);
/* Host helper == `build_sin_cos` (model/mod.rs:186-220): f32 powf / sin / cos. */
LCU_API int lcu_build_sin_cos(int nctx, int dh, float theta, float *sin_host, float *cos_host);

/* ggml Q8_0 (34-byte blocks) -> planes: int8 quants [rows, cols] then f16 scales
 * [rows, cols/32], 16-byte aligned.  The reference accepts no quantised weights
 * (op/linear.rs:84); this is the loader-side step the quantised path needs. */
LCU_API size_t lcu_q8_0_repacked_bytes(size_t rows, size_t cols);
LCU_API int lcu_repack_q8_0(void *dst_dev, const void *src_blocks_dev, size_t rows, size_t cols, lcu_stream_t s);

/* Tensor-parallel slicing of one weight on the device == `TPAction::move_data`
 * (load/mod.rs:86-99): copies this rank's rows/columns of the full tensor `src` into `dst`. */
LCU_API int lcu_tp_slice_weight(const lcu_ctx *ctx, int kind, void *dst_dev, const void *src_dev, lcu_stream_t s);

/* ------------------------------------------------------------------ KV pages
 * == `MemPages` + `KVCache` (memory.rs:14-53, exec/kv_cache.rs:15-54).  The reference maps
 * 2 MiB VMM pages behind a per-session virtual tensor; here a page is `page_tokens`
 * tokens of every layer, laid out [layer][k|v][kv head][token][dh], taken from one pool
 * and found through a per-sequence page table. */
LCU_API int lcu_kv_pool_create(lcu_ctx *ctx, size_t bytes); /* allocates the pool (set-up time) */
LCU_API int lcu_kv_pool_attach(lcu_ctx *ctx, void *dev_ptr, size_t bytes); /* caller-owned pool */
LCU_API int lcu_kv_page_tokens(const lcu_ctx *ctx);
LCU_API size_t lcu_kv_page_bytes(const lcu_ctx *ctx);
LCU_API int lcu_kv_pages_total(const lcu_ctx *ctx);
LCU_API int lcu_kv_pages_free(const lcu_ctx *ctx);
LCU_API int lcu_seq_create(lcu_ctx *ctx, int *seq_out);          /* == KVCache::new      */
LCU_API int lcu_seq_resize(lcu_ctx *ctx, int seq, uint32_t len); /* == KVCache::update: grows or shrinks */
LCU_API int lcu_seq_len(const lcu_ctx *ctx, int seq);            /* tokens currently backed by pages */
LCU_API int lcu_seq_free(lcu_ctx *ctx, int seq);

/* ------------------------------------------------------------------ one round
 * == the body of `Worker::lead`'s loop from `load_inputs` to `output_head.launch`
 * (exec/engine.rs:251-285): stages the round, runs every layer and the head on `stream`,
 * and leaves one lcu_kv_pair per request in `out_dev` (device memory, n_req entries).
 * Returns without synchronising, so the host can run ahead as the reference does.
 *   tokens      flat host array, sum(len) entries, request after request
 *   args        one per request (NULL = all ARG_MAX); randoms: one f32 in [0,1) per request
 *               (used only by non-argmax requests; the reference draws it with rand::random)
 *   fast_map    n_fast pairs (index into the PREVIOUS round's out pairs, token slot): the
 *               slot's token is replaced on the device == `FastEmbedding` (op/fast_embedding.rs)
 * Decode rounds (one token per request) replay a CUDA graph captured per (n_req, n_fast, sampling or not, out_dev): a
 * host that rotates output buffers holds one graph per buffer; the table is cleared when it reaches 96 entries.
 * Under TP every rank calls this with the same arguments (the reference broadcasts them,
 * exec/group.rs:109-117); only rank 0 writes out_dev (the head itself is sharded over the ranks in
 * arg-max rounds of the peer-memory transport, see lcu_set_head_sharding). */
LCU_API int lcu_step(lcu_ctx *ctx, lcu_stream_t stream, int n_req, const lcu_req *reqs, const uint32_t *tokens,
             const lcu_sample_args *args, const float *randoms, const uint32_t *fast_map, int n_fast,
             lcu_kv_pair *out_dev);
/* Device pointer to the logits of the last round, [n_req, vocab] in the activation dtype. */
LCU_API const void *lcu_logits(const lcu_ctx *ctx);
/* Device pointer to the hidden state (residual stream) of the last round, [n_tok, d]. */
LCU_API const void *lcu_hidden(const lcu_ctx *ctx);
/* Error word written by bounded device-side waits; 0 = none.  Synchronises `stream`.
 * Bits: 4 = a tcgen05 / TMA pipeline wait ran out, 16 = a peer never delivered its part of an all-reduce (or its head
 * candidates), 32 = the token broadcast never arrived.  The word is sticky: once this call has seen one of those bits,
 * every later lcu_step of the context returns LCU_ERR_TIMEOUT (the rank group is out of step) until lcu_reset_status.
 * (The reference has no counterpart: a missing rank blocks its NCCL call for ever, exec/engine.rs:272,339.) */
LCU_API int lcu_device_status(lcu_ctx *ctx, lcu_stream_t stream, uint32_t *status_out);
/* Clears the device status word and the sticky copy (synchronises the device). */
LCU_API int lcu_reset_status(lcu_ctx *ctx);
/* Longest any bounded wait on a peer (all-reduce arrival, token broadcast, head candidates) spins before it gives
 * up and raises its status bit, in microseconds of SM clock at 2 GHz; default about two seconds.  Applies to every
 * context on the device `ctx` lives on.  (No counterpart in the reference.) */
LCU_API int lcu_set_wait_limit_us(lcu_ctx *ctx, long long us);
/* Process-wide tuning values; the defaults are what the committed measurements use.  Keys: "pdl_edges" (bit per
 * layer edge launched as a programmatic dependent: 0 QKV->attention, 1 attention->O, 2 O->gate|up, 3 gate|up->down,
 * 4 down->next QKV, 5 last down->LM head; -1 = default), "gemv_ctas_per_sm" (1, 2; read at a shape's first launch),
 * "q8_rows" (1, 2, 4), "tc" (0: no tcgen05 kernel), "tc_block" (64, 128, 256), "tc_cluster" (0..2),
 * "p2p_scatter_ranks", "p2p_scatter_min", "gemv_lean_norm" (0: general RMSNorm prologue in the one-token GEMV),
 * "rms_pdl" (0: the stand-alone RMSNorm of batched rounds is a plain launch).
 * `ctx` (may be NULL) drops its captured rounds.  A measurement aid without counterpart in the reference. */
LCU_API int lcu_set_tuning(lcu_ctx *ctx, const char *key, long long value);
/* Tensor parallelism over peer memory: 1 (default) = arg-max rounds shard the LM head by vocabulary rows — every rank
 * streams vocab / tp rows and sends one candidate pair per request to the lead rank, which keeps the largest value
 * (lowest index among equals, the reference's tie rule); 0 = the head runs on the lead rank alone, as in the reference
 * (exec/engine.rs:90,201).  With sharding on, lcu_logits of the lead rank holds only its own vocab / tp columns
 * [n_req, vocab / tp].  All ranks must use the same setting. */
LCU_API int lcu_set_head_sharding(lcu_ctx *ctx, int enabled);
/* 1 = replay decode rounds from a captured CUDA graph (default), 0 = launch eagerly
 * == the reference's `--no-cuda-graph` switch (xtask/src/main.rs:45-73). */
LCU_API int lcu_set_cuda_graph(lcu_ctx *ctx, int enabled);
/* Number of kernels of this library launched by the last lcu_step. */
LCU_API int lcu_last_launch_count(const lcu_ctx *ctx);
/* Algorithmic HBM bytes of the last round (weights streamed + KV read), for rooflines. */
LCU_API double lcu_last_step_bytes(const lcu_ctx *ctx);

/* ------------------------------------------------------------------ round builder (host only)
 * == `EngineManager` (exec/engine_manager.rs:15-156): continuous batching — every running session
 * takes part in every round; a new one contributes its whole prompt, a running one a placeholder
 * token that the device replaces with its previous sample (`fast_map`).  Needs no GPU; `ctx` may be
 * NULL when only lcu_engine_prepare is used. */
typedef struct lcu_engine lcu_engine;
typedef struct {
    int32_t n_tok, n_req, n_fast, n_finished, n_overflow;
} lcu_round_info;
LCU_API int lcu_engine_create(lcu_ctx *ctx, uint32_t nctx, lcu_engine **out);
LCU_API int lcu_engine_destroy(lcu_engine *e);
/* == a new `Session{id, sample_args, cache}`; `seq` is its KV handle (lcu_seq_create); args NULL = ARG_MAX */
LCU_API int lcu_engine_session_new(lcu_engine *e, int seq, const lcu_sample_args *args, uint64_t *id_out);
/* == `Terminal::start` / `Command::Insert` (lib.rs:233-243): run `prompt` from the session's position for max_steps rounds */
LCU_API int lcu_engine_start(lcu_engine *e, uint64_t id, const uint32_t *prompt, uint32_t n, int max_steps);
LCU_API int lcu_engine_remove(lcu_engine *e, uint64_t id); /* == `Command::Remove` */
LCU_API int lcu_engine_session_pos(const lcu_engine *e, uint64_t id, uint32_t *pos_out);
LCU_API int lcu_engine_session_set_pos(lcu_engine *e, uint64_t id, uint32_t pos); /* cache.pos rollback (prefix reuse) */
/* == `EngineManager::prepare` (exec/engine_manager.rs:72-130); arrays below stay valid until the next prepare */
LCU_API int lcu_engine_prepare(lcu_engine *e, lcu_round_info *info);
LCU_API const uint32_t *lcu_engine_round_tokens(const lcu_engine *e);            /* n_tok */
LCU_API const lcu_req *lcu_engine_round_reqs(const lcu_engine *e);               /* n_req */
LCU_API const uint32_t *lcu_engine_round_fast_map(const lcu_engine *e);          /* n_fast pairs */
LCU_API const lcu_sample_args *lcu_engine_round_sample_args(const lcu_engine *e); /* n_req */
LCU_API const uint64_t *lcu_engine_round_output(const lcu_engine *e);            /* n_req session ids, output order */
LCU_API const uint64_t *lcu_engine_round_finished(const lcu_engine *e);          /* n_finished */
LCU_API const uint64_t *lcu_engine_round_overflow(const lcu_engine *e);          /* n_overflow */
/* == `pos()` and `out_idx()` (exec/engine.rs:352-371) of the prepared round; either pointer may be NULL */
LCU_API int lcu_engine_round_positions(const lcu_engine *e, uint32_t *pos_out, uint32_t *out_idx_out);
/* One iteration of `Worker::lead`'s loop: prepare + lcu_step.  info->n_tok == 0: nothing to run. */
LCU_API int lcu_engine_step(lcu_engine *e, lcu_stream_t stream, const float *randoms, lcu_kv_pair *out_dev,
                            lcu_round_info *info);
/* Token budget and chunked prefill — what the reference leaves as a TODO (exec/engine_manager.rs:83,100-109: a round
 * takes whole prompts and exec/engine.rs:68 caps it at 1024 tokens).  max_round_tokens > 0: a round holds at most that
 * many tokens — every decoding session always gets its one, prompts share the rest in session order;
 * prefill_chunk > 0: no prompt contributes more than that per round.  A prompt that does not finish in a round
 * contributes a chunk whose entry in lcu_engine_round_output is LCU_ENGINE_NO_OUTPUT (ignore its pair) and which
 * costs no step of max_steps.  0 / 0 (default): whole prompts, as the reference. */
#define LCU_ENGINE_NO_OUTPUT (~0ull)
LCU_API int lcu_engine_set_budget(lcu_engine *e, uint32_t max_round_tokens, uint32_t prefill_chunk);
/* Prefix reuse == `CacheManager` (xtask/src/service/cache_manager.rs:22-66).
 * insert: a finished session's token history and KV sequence are parked (the session id dies).
 * send:   a new session for `tokens` starts from the parked cache sharing the longest prefix with tokens[0 .. n-1)
 *         (the latest parked among equals; with no common prefix a parked cache is still taken and restarted at 0, as
 *         the reference does), rolled back to that length — its pages past it return to the pool like
 *         `KVCache::update` (exec/kv_cache.rs:34-50); without parked caches a fresh sequence.  Only tokens[pos ..] run. */
LCU_API int lcu_engine_cache_insert(lcu_engine *e, uint64_t id, const uint32_t *tokens, uint32_t n);
LCU_API int lcu_engine_cache_send(lcu_engine *e, const uint32_t *tokens, uint32_t n, const lcu_sample_args *args,
                                  int max_steps, uint64_t *id_out, uint32_t *reused_out);
LCU_API int lcu_engine_cache_count(const lcu_engine *e);
/* Seeded sampling: with a seed lcu_engine_step draws the per-request random numbers itself (its `randoms` argument is
 * ignored); the k-th number of a session depends only on (seed, session id, k), so a sampled conversation replays
 * identically whatever it is batched with.  The reference draws rand::random() per row and step
 * (exec/output_head.rs:111) and cannot be replayed.  lcu_engine_round_randoms: the numbers of the last round. */
LCU_API int lcu_engine_set_seed(lcu_engine *e, uint64_t seed);
/* What lcu_engine_step does under a seed, for hosts that call lcu_step themselves: draws the prepared round's numbers
 * (one per request, 0 for arg-max rows and unfinished prefill chunks); call once per prepared round. */
LCU_API int lcu_engine_draw_randoms(lcu_engine *e);
LCU_API const float *lcu_engine_round_randoms(const lcu_engine *e);

/* ------------------------------------------------------------------ GGUF model files
 * == `GGufModel::read` / `merge` (model/gguf.rs:16-72), the metadata -> shape mapping of `GGufModel::llama`
 * (model/mod.rs:61-182) and the weight upload of `load_weight` (load/mod.rs:23-108).  Files use the reference's tensor
 * naming: fused `blk.N.attn_qkv.weight` (rows q|k|v) and `blk.N.ffn_gate_up.weight` (rows gate|up); `output.weight`
 * falls back to `token_embd.weight`.  F16 / BF16 models, F16 / BF16 / F32 norm weights, and Q8_0 linear weights
 * (repacked at load time — the reference itself cannot run them).  Shards: every path is one file of a split model;
 * `general.alignment` and `split.*` keys are per file, any other key may repeat only with the same value. */
typedef struct lcu_gguf lcu_gguf;
LCU_API int lcu_gguf_open(const char *const *paths, int n_paths, lcu_gguf **out);
LCU_API int lcu_gguf_close(lcu_gguf *g); /* also frees the device region lcu_gguf_load filled */
LCU_API int lcu_gguf_n_tensors(const lcu_gguf *g);
/* name (valid until close), lcu_dtype, dims outermost first (the reference reverses ggml's order too, gguf.rs:56-61) */
LCU_API int lcu_gguf_tensor_info(const lcu_gguf *g, int index, const char **name, int *dtype, uint64_t dims4[4], int *n_dims,
                                 size_t *bytes);
LCU_API int lcu_gguf_meta_u64(const lcu_gguf *g, const char *key, uint64_t *out);
LCU_API int lcu_gguf_meta_f32(const lcu_gguf *g, const char *key, float *out);
LCU_API int lcu_gguf_meta_str(const lcu_gguf *g, const char *key, char *buf, size_t cap, size_t *len);
/* Fills the model fields of *desc; nctx, page_tokens, max_tokens, max_seqs are the caller's when non-zero on entry. */
LCU_API int lcu_gguf_model_desc(const lcu_gguf *g, lcu_model_desc *desc);
/* Uploads every weight of `ctx`'s rank into ONE device region owned by the handle (keep it open while the context is
 * in use) through two pinned slabs, cuts linear weights per rank, repacks Q8_0, registers each with lcu_set_weight.
 * Synchronises `stream` as it goes; call with `ctx`'s device current. */
LCU_API int lcu_gguf_load(lcu_gguf *g, lcu_ctx *ctx, lcu_stream_t stream);

/* ------------------------------------------------------------------ operators
 * One entry point per `Operator::launch` implementation so a host can swap them in one
 * at a time behind `launch_nn_exec` (exec/step.rs:101-138).  dt = activation dtype. */

/* == op/embedding.rs + embedding.cuh: out[i,:] = table[index[i],:]  (row_bytes per row) */
LCU_API int lcu_op_embedding(void *out, const void *table, const uint32_t *index, int n, size_t row_bytes,
                     lcu_stream_t s);
/* == op/fast_embedding.rs + .cuh: tokens[map[i][1]] = kv_pairs[map[i][0]].idx */
LCU_API int lcu_op_fast_embedding(uint32_t *tokens, const lcu_kv_pair *kv_pairs, const uint32_t *map_dev, int n_map,
                          lcu_stream_t s);
/* == op/rms_norm.rs + .cuh: y = x * w * rsqrt(mean(x^2) + eps); w_dt = dt or LCU_F32 */
LCU_API int lcu_op_rms_norm(void *y, int stride_y, const void *x, int stride_x, const void *w, int w_dt, float eps,
                    int n, int d, int dt, lcu_stream_t s);
/* == op/linear.rs: y[n,out] = x[n,in] * W[out,in]^T (+ residual[n,out]); f32 accumulation,
 * one rounding.  w_dt = dt, or LCU_Q8_0 with W in the repacked plane layout. */
LCU_API int lcu_op_linear(void *y, int stride_y, const void *x, int stride_x, const void *w, int w_dt,
                  const void *residual, int stride_res, int n, int in, int out, int dt, lcu_stream_t s);
/* == op/rope.rs + rope.cuh: adjacent-pair rotation with f32 tables [nctx, dh/2] */
LCU_API int lcu_op_rope(void *y, int stride_tok_y, int stride_head_y, const void *x, int stride_tok_x,
                int stride_head_x, const uint32_t *pos, const float *sin_t, const float *cos_t, int n, int nh,
                int dh, int dt, lcu_stream_t s);
/* == op/swiglu.rs + swiglu.cuh: out = gate * sigmoid(gate) * up */
LCU_API int lcu_op_swiglu(void *out, int stride_out, const void *gate, int stride_gate, const void *up,
                  int stride_up, int n, int di, int dt, lcu_stream_t s);
/* == op/add.rs + add.cuh: y = k*x + b (k == 0: y = b); strides (row, element) per tensor */
LCU_API int lcu_op_add(void *y, int sny, int sdy, const void *x, int snx, int sdx, const void *b, int snb, int sdb,
               float k, int n, int d, int dt, lcu_stream_t s);
/* == `launch_attn` -> operators::attention_kv_cached for ONE request (exec/step.rs:140-184):
 * writes k,v [seq, nkvh, dh] into the caches at pos.. and computes causal GQA attention of
 * q [seq, nh, dh] over pos+seq cached tokens.  Strides: token, head (elements; dh contiguous). */
LCU_API int lcu_op_attention_kv_cached(void *o, int sto, int sho, const void *q, int stq, int shq, const void *k,
                               int stk, int shk, const void *v, int stv, int shv, void *k_cache, int stkc,
                               int shkc, void *v_cache, int stvc, int shvc, int nh, int nkvh, int dh,
                               int seq, int pos, int dt, lcu_stream_t s);
/* == op/all_reduce.rs: sum over ranks of `count` elements (in place when y == x) */
LCU_API int lcu_op_all_reduce(lcu_ctx *ctx, void *y, const void *x, size_t count, int dt, lcu_stream_t s);

/* Sampler: drop-in for librandom_sample.so — same names' meaning, argument order and
 * `cudaError_t` return as llama.cu/src/op/random_sample/sample.h:15-39.
 * One documented difference in `kv_pair.val` of the STOCHASTIC path: the reference's random_sample_kernel
 * (op/random_sample/sample.cuh:72-87) stores `sorted[i]` after its in-place inclusive scan, i.e. the
 * unnormalised cumulative weight up to the chosen token; lcu_sample_half and the sampling rows of
 * lcu_op_sample_rows store the chosen token's logit, as the arg-max path of both libraries does.  The token
 * index — the only field the token loop consumes (fast_embedding.cuh:7-15, exec/mod.rs:91-115) — is unaffected. */
LCU_API int lcu_calculate_workspace_size_half(size_t *argmax, size_t *random_sample, size_t n);
LCU_API int lcu_argmax_half(void *kv_pair, const void *logits, size_t n, void *workspace_ptr, size_t workspace_len,
                    lcu_stream_t stream);
LCU_API int lcu_sample_half(void *kv_pair, const void *logits, const unsigned int *indices, size_t n, float random,
                    float temperature, float topp, size_t topk, void *workspace_ptr, size_t workspace_len,
                    lcu_stream_t stream);
/* All rows of a round in ONE launch pair (the reference loops over rows on the host,
 * exec/output_head.rs:104-113): logits [rows, n] in dt, args/randoms per row on the device
 * (args NULL = argmax everywhere).  Writes `out` and, when not NULL, a copy in `out_copy`
 * (the `pre_kv_pairs` the next round's fast_embedding reads, exec/engine.rs:285). */
LCU_API size_t lcu_sample_rows_workspace_size(int rows, size_t n);
LCU_API int lcu_op_sample_rows(lcu_kv_pair *out, lcu_kv_pair *out_copy, const void *logits, int rows, size_t n,
                       const lcu_sample_args *args_dev, const float *randoms_dev, int dt, void *workspace,
                       size_t workspace_len, lcu_stream_t s);

/* Arg-max of every row with NO workspace argument and no allocation of any kind.
 * (No counterpart in the reference, whose sampler always takes a caller workspace.)
 * For hosts that can neither pass scratch memory nor let the library allocate it — a serving
 * loop that must keep cudaMalloc (a device-wide synchronisation) off its hot path, a host
 * whose device memory belongs to an external pool, code already inside a stream capture.
 * The partial results live in a fixed 64 KiB array inside the library image (held by every
 * GPU that loads the library until the process exits), which limits the problem to
 * rows * ceil(n / 4096) <= 8192; larger calls fail with LCU_ERR_INVALID and a message.
 * The FIRST call on each device also looks up the array's device address; make that call
 * with the device current and before starting any stream capture.  All calls share the one
 * array: calls that overlap on the GPU (different streams, no ordering) race and give
 * undefined results; nothing in it has to start at zero, so back-to-back calls on one
 * stream need no clearing.  Same result as lcu_op_sample_rows with args_dev == NULL. */
LCU_API int lcu_argmax_rows_noalloc(lcu_kv_pair *out, const void *logits, int rows, size_t n, int dt, lcu_stream_t s);

/* ------------------------------------------------------------------ collectives set-up
 * Thin wrappers over the NCCL library found at run time == `CommunicatorGroup::new`
 * (exec/engine.rs:86), one process per GPU instead of one thread per GPU. */
LCU_API int lcu_comm_unique_id(void *id128);                                   /* rank 0: 128 bytes out */
LCU_API int lcu_comm_init_rank(const void *id128, int rank, int size, void **comm_out);
LCU_API int lcu_comm_destroy(void *comm);

/* Tensor parallelism over NVLink peer memory instead of NCCL, for the two all-reduces of a layer
 * (llama.cu/src/op/all_reduce.rs:36-40) and the token broadcast (exec/engine.rs:264-274).  One
 * process per GPU: every rank calls lcu_p2p_create (allocates its exchange region, returns its
 * 64-byte CUDA IPC handle), the host gathers the tp_size handles in rank order by any means, every
 * rank calls lcu_p2p_attach with all of them.  From then on lcu_step lets the output / down
 * projection kernels store their partials straight into every rank's region and replaces the
 * collective by a small local reduction.  Waits are bounded: a peer that never arrives raises bit
 * 16 (all-reduce) or 32 (broadcast) of lcu_device_status instead of hanging.  All ranks must attach
 * (or none), and all must destroy their contexts only after every rank has finished stepping. */
LCU_API int lcu_p2p_create(lcu_ctx *ctx, void *handle64_out);
LCU_API int lcu_p2p_attach(lcu_ctx *ctx, const void *handles /* tp_size x 64 bytes */);
LCU_API int lcu_p2p_enabled(const lcu_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* LCU_H */
