/*
 * CPU oracle for the decode token loop — TEST INFRASTRUCTURE, not product code.
 *
 * A plain C restatement (f32 arithmetic, optional rounding to the activation
 * dtype at every operator boundary) of the forward pass that
 * YdrMaster/llama.cu runs each round.  Only tests, the smoke check and the
 * CPU-baseline leg of the benchmark may load this library; the CUDA library
 * never links or calls it.
 *
 * PARITY UNPINNED: the reference ships no golden vectors, known-answer tests
 * or fixtures for this path (its whole test suite is one chat-template test
 * and two network client tests), and its Rust host cannot be built without
 * cargo and 21 git dependencies.  What pins this oracle instead:
 *   - the reference's own device kernels (rms_norm, rope, swiglu, embedding,
 *     fast_embedding, argmax/sample), compiled from the reference sources in
 *     place into oracle/_ref and compared op by op on the GPU;
 *   - an independent PyTorch fp32 restatement and gguf's numpy Q8_0 codec.
 * Attention arithmetic (crate `operators` @ed28f2d) and the layer wiring
 * (crate `nn` @1fff7ec) are not in the reference tree; they are restated from
 * the call sites (llama.cu/src/exec/step.rs:140-184, model/mod.rs:90-169).
 */
#ifndef LCU_ORACLE_H
#define LCU_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_F16 = 0, ORC_BF16 = 1, ORC_F32 = 2, ORC_Q8_0 = 3 };

/* weight kinds, same numbering as the CUDA library (include/lcu.h) */
enum {
    ORC_W_EMBD = 0, ORC_W_ATTN_NORM = 1, ORC_W_QKV = 2, ORC_W_O = 3, ORC_W_FFN_NORM = 4,
    ORC_W_GATE_UP = 5, ORC_W_DOWN = 6, ORC_W_OUT_NORM = 7, ORC_W_LM_HEAD = 8
};

typedef struct {
    int32_t n_layers, d, nh, nkvh, dh, di, vocab, nctx;
    float eps, theta;
    int32_t act_dtype; /* ORC_F16 / ORC_BF16: round at every op boundary; ORC_F32: never */
} orc_desc;

typedef struct orc_model orc_model;

/* scalar helpers */
float orc_round(float v, int dtype);
void orc_to_f32(float *dst, const void *src, int dtype, size_t n); /* f16/bf16/f32/q8_0 -> f32 */
void orc_from_f32(void *dst, const float *src, int dtype, size_t n); /* f32 -> f16/bf16 (RNE) */

/* operators (each cites the reference file it follows in the .c file) */
void orc_build_sin_cos(int nctx, int dh, float theta, float *sin_t, float *cos_t);
void orc_embedding(float *out, const float *table, const uint32_t *idx, int n, int d);
void orc_rms_norm(float *y, const float *x, const float *w, int n, int d, float eps, int dt);
void orc_linear(float *y, const float *x, const float *w, const float *residual,
                int n, int in, int out, int dt);
void orc_rope(float *x, int n, int nheads, int dh, int stride_tok, const uint32_t *pos,
              const float *sin_t, const float *cos_t, int dt);
void orc_swiglu(float *out, int stride_out, const float *gate, int stride_gate,
                const float *up, int stride_up, int n, int di, int dt);
/* one request: q [seq, nh*dh] (stride_q), caches [ctx, nkvh*dh] already holding pos+seq tokens */
void orc_attention(float *o, int stride_o, const float *q, int stride_q,
                   const float *kc, const float *vc, int nh, int nkvh, int dh,
                   int pos, int seq, int dt);
void orc_argmax(const float *logits, size_t n, uint32_t *idx, float *val);
uint32_t orc_sample(const float *logits, size_t n, float random, float temperature,
                    float topp, size_t topk, float *val);

/* whole model */
orc_model *orc_model_new(const orc_desc *desc);
void orc_model_free(orc_model *m);
/* data: `count` logical elements of `dtype` (Q8_0: count weights = count/32 blocks of 34 bytes) */
int orc_model_set_weight(orc_model *m, int layer, int kind, const void *data, int dtype, size_t count);
/* timing aid: seeded uniform weights of std 0.02, norm weights 1 (no numpy round trip) */
int orc_model_fill_synthetic(orc_model *m, uint64_t seed);
int orc_seq_new(orc_model *m);          /* returns a sequence slot id */
void orc_seq_free(orc_model *m, int seq);
/* One round: request r owns tokens[off_r .. off_r+seq_len[r]) at positions pos0[r]...
 * Appends K/V to each sequence's cache and returns the logits of each request's last
 * token: logits[n_req, vocab] (f32 holding values already rounded to act_dtype) and the
 * greedy ids (lowest index on ties). Any of logits / ids may be NULL. */
int orc_forward(orc_model *m, int n_req, const int *seqs, const uint32_t *tokens,
                const uint32_t *seq_len, const uint32_t *pos0, float *logits, uint32_t *ids);
/* debugging / per-stage parity: copies of the hidden state after every layer of the last
 * forward, [n_layers+1][n_tok][d]; returns n_tok */
int orc_last_hidden(orc_model *m, float *out, size_t cap);
/* wall-clock seconds the last orc_forward spent in the layers and in the head */
void orc_last_times(orc_model *m, double *t_layers, double *t_head);
int orc_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
