/*
 * CPU oracle for the decode token loop — TEST INFRASTRUCTURE (see lcu_oracle.h).
 * PARITY UNPINNED against the reference binary (no golden vectors exist); pinned op by
 * op against the reference's own kernels compiled into oracle/_ref.
 *
 * Every function names the reference source it restates (paths inside the reference
 * project).  Arithmetic is f32 throughout; with act_dtype f16/bf16 each operator
 * output is rounded once to that type, which is where the reference materialises a
 * tensor in its activation dtype.
 */
#include "lcu_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- rounding */

static inline float round_f16(float v) { return (float)(_Float16)v; }

static inline float round_bf16(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return v; /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);               /* round to nearest even */
    u &= 0xffff0000u;
    memcpy(&v, &u, 4);
    return v;
}

float orc_round(float v, int dt) {
    switch (dt) {
    case ORC_F16: return round_f16(v);
    case ORC_BF16: return round_bf16(v);
    default: return v;
    }
}

void orc_to_f32(float *dst, const void *src, int dt, size_t n) {
    if (dt == ORC_F16) {
        const _Float16 *s = (const _Float16 *)src;
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < n; ++i) dst[i] = (float)s[i];
    } else if (dt == ORC_BF16) {
        const uint16_t *s = (const uint16_t *)src;
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < n; ++i) {
            uint32_t u = (uint32_t)s[i] << 16;
            memcpy(&dst[i], &u, 4);
        }
    } else if (dt == ORC_F32) {
        memcpy(dst, src, n * 4);
    } else if (dt == ORC_Q8_0) {
        /* ggml Q8_0: blocks of {f16 scale; int8 q[32]} = 34 bytes; w = scale * q.
         * (The reference never dequantises: llama.cu/src/op/linear.rs:84 asserts the weight
         * dtype equals the activation dtype.  This is the published ggml definition.) */
        const uint8_t *s = (const uint8_t *)src;
        size_t nb = n / 32;
#pragma omp parallel for schedule(static)
        for (size_t b = 0; b < nb; ++b) {
            _Float16 d;
            memcpy(&d, s + b * 34, 2);
            const int8_t *q = (const int8_t *)(s + b * 34 + 2);
            for (int i = 0; i < 32; ++i) dst[b * 32 + i] = (float)d * (float)q[i];
        }
    }
}

void orc_from_f32(void *dst, const float *src, int dt, size_t n) {
    if (dt == ORC_F16) {
        _Float16 *d = (_Float16 *)dst;
        for (size_t i = 0; i < n; ++i) d[i] = (_Float16)src[i];
    } else if (dt == ORC_BF16) {
        uint16_t *d = (uint16_t *)dst;
        for (size_t i = 0; i < n; ++i) {
            float r = round_bf16(src[i]);
            uint32_t u;
            memcpy(&u, &r, 4);
            d[i] = (uint16_t)(u >> 16);
        }
    } else {
        memcpy(dst, src, n * 4);
    }
}

/* --------------------------------------------------------------- operators */

/* llama.cu/src/model/mod.rs:186-220 (build_sin_cos): f32 powf, f32 product, sin_cos. */
void orc_build_sin_cos(int nctx, int dh, float theta, float *sin_t, float *cos_t) {
    int half = dh / 2;
    for (int pos = 0; pos < nctx; ++pos)
        for (int i = 0; i < half; ++i) {
            float t = powf(theta, -((float)(2 * i) / (float)dh));
            float f = (float)pos * t;
            sin_t[(size_t)pos * half + i] = sinf(f);
            cos_t[(size_t)pos * half + i] = cosf(f);
        }
}

/* llama.cu/src/op/embedding.cuh:1-9: out[i,:] = table[index[i],:] */
void orc_embedding(float *out, const float *table, const uint32_t *idx, int n, int d) {
    for (int i = 0; i < n; ++i) memcpy(out + (size_t)i * d, table + (size_t)idx[i] * d, (size_t)d * 4);
}

/* llama.cu/src/op/rms_norm.cuh:6-81: f32 sum of squares, rms = rsqrt(acc/d + eps),
 * y = Ta(rms * x * w) — a single rounding at the store. */
void orc_rms_norm(float *y, const float *x, const float *w, int n, int d, float eps, int dt) {
    for (int t = 0; t < n; ++t) {
        const float *xr = x + (size_t)t * d;
        float *yr = y + (size_t)t * d;
        float acc[8] = {0};
        int i = 0;
        for (; i + 8 <= d; i += 8)
            for (int j = 0; j < 8; ++j) acc[j] += xr[i + j] * xr[i + j];
        float s = 0;
        for (; i < d; ++i) s += xr[i] * xr[i];
        s += ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
        float rms = 1.0f / sqrtf(s / (float)d + eps);
        for (i = 0; i < d; ++i) yr[i] = orc_round(rms * xr[i] * w[i], dt);
    }
}

static inline float dot_f32(const float *a, const float *b, int n) {
    float acc[16] = {0};
    int i = 0;
    for (; i + 16 <= n; i += 16) {
#pragma omp simd
        for (int j = 0; j < 16; ++j) acc[j] += a[i + j] * b[i + j];
    }
    float s = 0;
    for (; i < n; ++i) s += a[i] * b[i];
    for (int w = 8; w > 0; w >>= 1)
        for (int j = 0; j < w; ++j) acc[j] += acc[j + w];
    return s + acc[0];
}

/* llama.cu/src/op/linear.rs:17-120: y = x·Wᵀ (+ residual), W is [out, in] row-major,
 * f32 accumulation, residual enters as the beta=1 C operand (linear.rs:35-46,62) so the
 * sum acc+residual is rounded once to the activation dtype. */
void orc_linear(float *y, const float *x, const float *w, const float *residual,
                int n, int in, int out, int dt) {
#pragma omp parallel for schedule(static)
    for (int o = 0; o < out; ++o) {
        const float *wr = w + (size_t)o * in;
        for (int t = 0; t < n; ++t) {
            float acc = dot_f32(x + (size_t)t * in, wr, in);
            if (residual) acc += residual[(size_t)t * out + o];
            y[(size_t)t * out + o] = orc_round(acc, dt);
        }
    }
}

/* llama.cu/src/op/rope.cuh:1-35: adjacent pairs (x[2i], x[2i+1]) rotated with the f32
 * tables at row pos[t]; one rounding per output. In place. */
void orc_rope(float *x, int n, int nheads, int dh, int stride_tok, const uint32_t *pos,
              const float *sin_t, const float *cos_t, int dt) {
    int half = dh / 2;
    for (int t = 0; t < n; ++t)
        for (int h = 0; h < nheads; ++h) {
            float *p = x + (size_t)t * stride_tok + (size_t)h * dh;
            for (int i = 0; i < half; ++i) {
                float s = sin_t[(size_t)pos[t] * half + i], c = cos_t[(size_t)pos[t] * half + i];
                float a = p[2 * i], b = p[2 * i + 1];
                p[2 * i] = orc_round(a * c - b * s, dt);
                p[2 * i + 1] = orc_round(a * s + b * c, dt);
            }
        }
}

/* llama.cu/src/op/swiglu.cuh:1-20: out = gate * sigmoid(gate) * up with
 * sigmoid(x) = 1 / (1 + expf(-x)); f32; one rounding. */
void orc_swiglu(float *out, int stride_out, const float *gate, int stride_gate,
                const float *up, int stride_up, int n, int di, int dt) {
    for (int t = 0; t < n; ++t)
        for (int i = 0; i < di; ++i) {
            float g = gate[(size_t)t * stride_gate + i], u = up[(size_t)t * stride_up + i];
            float sg = 1.0f / (1.0f + expf(-g));
            out[(size_t)t * stride_out + i] = orc_round(g * sg * u, dt);
        }
}

/* Call site llama.cu/src/exec/step.rs:140-184 (operator `attention_kv_cached` of crate
 * `operators` @ed28f2d, source not in the reference tree): causal attention of `seq` new
 * queries at positions pos..pos+seq over a cache that already holds pos+seq tokens, with
 * query head h reading KV head h / (nh/nkvh).  ASSUMED (not verifiable from the tree):
 * scale 1/sqrt(dh), f32 scores and softmax, one rounding at the output. */
void orc_attention(float *o, int stride_o, const float *q, int stride_q,
                   const float *kc, const float *vc, int nh, int nkvh, int dh,
                   int pos, int seq, int dt) {
    int g = nh / nkvh, kvd = nkvh * dh;
    float scale = 1.0f / sqrtf((float)dh);
#pragma omp parallel
    {
        float *s = (float *)malloc(sizeof(float) * (size_t)(pos + seq));
        float *acc = (float *)malloc(sizeof(float) * (size_t)dh);
#pragma omp for collapse(2) schedule(static)
        for (int t = 0; t < seq; ++t)
            for (int h = 0; h < nh; ++h) {
                int ctx = pos + t + 1, kvh = h / g;
                const float *qr = q + (size_t)t * stride_q + (size_t)h * dh;
                float mx = -INFINITY;
                for (int j = 0; j < ctx; ++j) {
                    s[j] = dot_f32(qr, kc + (size_t)j * kvd + (size_t)kvh * dh, dh) * scale;
                    if (s[j] > mx) mx = s[j];
                }
                float sum = 0;
                for (int j = 0; j < ctx; ++j) {
                    s[j] = expf(s[j] - mx);
                    sum += s[j];
                }
                for (int i = 0; i < dh; ++i) acc[i] = 0;
                for (int j = 0; j < ctx; ++j) {
                    const float *vr = vc + (size_t)j * kvd + (size_t)kvh * dh;
                    float p = s[j];
                    for (int i = 0; i < dh; ++i) acc[i] += p * vr[i];
                }
                float inv = 1.0f / sum;
                float *orow = o + (size_t)t * stride_o + (size_t)h * dh;
                for (int i = 0; i < dh; ++i) orow[i] = orc_round(acc[i] * inv, dt);
            }
        free(s);
        free(acc);
    }
}

/* llama.cu/src/op/random_sample/sample.cuh:13-25 (cub::DeviceReduce::ArgMax): the largest
 * value, the LOWEST index among equals. */
void orc_argmax(const float *logits, size_t n, uint32_t *idx, float *val) {
    size_t best = 0;
    for (size_t i = 1; i < n; ++i)
        if (logits[i] > logits[best]) best = i;
    if (idx) *idx = (uint32_t)best;
    if (val) *val = logits[best];
}

typedef struct { float v; uint32_t i; } sample_pair;
static int cmp_desc(const void *a, const void *b) {
    const sample_pair *x = (const sample_pair *)a, *y = (const sample_pair *)b;
    if (x->v > y->v) return -1;
    if (x->v < y->v) return 1;
    return (x->i > y->i) - (x->i < y->i); /* stable radix sort keeps index order */
}

/* llama.cu/src/op/random_sample/sample.cuh:156-209: sort descending (stable), weights
 * w[0]=1, w[i]=exp((x[i]-x[0])/T), inclusive prefix sum, threshold
 * p = random * min(topp * total, cum[topk-1]), answer = first i with cum[i] >= p.
 * The reference stores weights and prefix sums in f16 (a CUB scan whose summation order
 * is unspecified); this restatement keeps them in f32. */
uint32_t orc_sample(const float *logits, size_t n, float random, float temperature,
                    float topp, size_t topk, float *val) {
    sample_pair *p = (sample_pair *)malloc(sizeof(sample_pair) * n);
    for (size_t i = 0; i < n; ++i) { p[i].v = logits[i]; p[i].i = (uint32_t)i; }
    qsort(p, n, sizeof(sample_pair), cmp_desc);
    if (topk > n) topk = n;
    float mx = p[0].v;
    double total = 0, cumk = 0;
    for (size_t i = 0; i < n; ++i) {
        float w = i == 0 ? 1.0f : expf((p[i].v - mx) / temperature);
        total += w;
        if (i == topk - 1) cumk = total;
    }
    double lim = (double)topp * total;
    if (cumk < lim) lim = cumk;
    double thr = (double)random * lim, cum = 0;
    uint32_t ans = p[n - 1].i;
    float ansv = p[n - 1].v;
    for (size_t i = 0; i < n; ++i) {
        float w = i == 0 ? 1.0f : expf((p[i].v - mx) / temperature);
        cum += w;
        if (cum >= thr) { ans = p[i].i; ansv = p[i].v; break; }
    }
    if (val) *val = ansv;
    free(p);
    return ans;
}

/* ------------------------------------------------------------- whole model */

#define ORC_MAX_SEQ 256

typedef struct {
    float *attn_norm, *qkv, *o, *ffn_norm, *gate_up, *down;
} orc_layer;

struct orc_model {
    orc_desc c;
    float *embd, *out_norm, *lm_head;
    orc_layer *layers;
    float *sin_t, *cos_t;
    /* per-sequence caches: [n_layers][nctx][nkvh*dh] for k and v */
    float *kc[ORC_MAX_SEQ], *vc[ORC_MAX_SEQ];
    int used[ORC_MAX_SEQ];
    float *hidden; /* [n_layers+1][n_tok][d] of the last forward */
    int hidden_tok;
    double t_layers, t_head; /* wall seconds of the last forward: all layers / the head */
};

orc_model *orc_model_new(const orc_desc *desc) {
    orc_model *m = (orc_model *)calloc(1, sizeof(orc_model));
    m->c = *desc;
    m->layers = (orc_layer *)calloc((size_t)desc->n_layers, sizeof(orc_layer));
    size_t tab = (size_t)desc->nctx * (size_t)(desc->dh / 2);
    m->sin_t = (float *)malloc(tab * 4);
    m->cos_t = (float *)malloc(tab * 4);
    orc_build_sin_cos(desc->nctx, desc->dh, desc->theta, m->sin_t, m->cos_t);
    return m;
}

void orc_model_free(orc_model *m) {
    if (!m) return;
    free(m->embd); free(m->out_norm);
    if (m->lm_head != m->embd) free(m->lm_head);
    for (int l = 0; l < m->c.n_layers; ++l) {
        orc_layer *L = &m->layers[l];
        free(L->attn_norm); free(L->qkv); free(L->o); free(L->ffn_norm); free(L->gate_up); free(L->down);
    }
    for (int s = 0; s < ORC_MAX_SEQ; ++s) { free(m->kc[s]); free(m->vc[s]); }
    free(m->layers); free(m->sin_t); free(m->cos_t); free(m->hidden);
    free(m);
}

/* Tensor names, shapes and fused row orders follow llama.cu/src/model/mod.rs:61-182:
 * attn_qkv [(nh+2*nkvh)*dh, d] rows q|k|v, attn_output [d, nh*dh], ffn_gate_up [2*di, d]
 * rows gate|up, ffn_down [d, di], output [vocab, d] (falls back to token_embd). */
int orc_model_set_weight(orc_model *m, int layer, int kind, const void *data, int dtype, size_t count) {
    const orc_desc *c = &m->c;
    size_t want;
    float **slot;
    switch (kind) {
    case ORC_W_EMBD: want = (size_t)c->vocab * c->d; slot = &m->embd; break;
    case ORC_W_OUT_NORM: want = (size_t)c->d; slot = &m->out_norm; break;
    case ORC_W_LM_HEAD: want = (size_t)c->vocab * c->d; slot = &m->lm_head; break;
    default:
        if (layer < 0 || layer >= c->n_layers) return -1;
        switch (kind) {
        case ORC_W_ATTN_NORM: want = (size_t)c->d; slot = &m->layers[layer].attn_norm; break;
        case ORC_W_QKV: want = (size_t)(c->nh + 2 * c->nkvh) * c->dh * c->d; slot = &m->layers[layer].qkv; break;
        case ORC_W_O: want = (size_t)c->d * c->nh * c->dh; slot = &m->layers[layer].o; break;
        case ORC_W_FFN_NORM: want = (size_t)c->d; slot = &m->layers[layer].ffn_norm; break;
        case ORC_W_GATE_UP: want = (size_t)2 * c->di * c->d; slot = &m->layers[layer].gate_up; break;
        case ORC_W_DOWN: want = (size_t)c->d * c->di; slot = &m->layers[layer].down; break;
        default: return -1;
        }
    }
    if (count != want) return -2;
    free(*slot);
    *slot = (float *)malloc(want * 4);
    orc_to_f32(*slot, data, dtype, want);
    return 0;
}

/* Fills every weight with cheap seeded pseudo-random values of standard deviation 0.02
 * (uniform, not normal) and norm weights of 1: for TIMING the CPU baseline on shapes too
 * large to draw with numpy; parity tests never use it. */
static void fill_uniform(float *w, size_t n, uint64_t seed) {
    const float a = 0.02f * 1.7320508f; /* uniform on [-a, a] has std 0.02 */
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        uint64_t z = (i + seed * 0x9E3779B97F4A7C15ull) + 0x9E3779B97F4A7C15ull; /* splitmix64 */
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        w[i] = ((float)(z >> 40) * (1.0f / 16777216.0f) * 2.0f - 1.0f) * a;
    }
}

int orc_model_fill_synthetic(orc_model *m, uint64_t seed) {
    const orc_desc *c = &m->c;
    for (int kind = 0; kind <= ORC_W_LM_HEAD; ++kind)
        for (int l = 0; l < c->n_layers; ++l) {
            size_t want;
            float **slot;
            switch (kind) {
            case ORC_W_EMBD: want = (size_t)c->vocab * c->d; slot = &m->embd; break;
            case ORC_W_OUT_NORM: want = (size_t)c->d; slot = &m->out_norm; break;
            case ORC_W_LM_HEAD: want = (size_t)c->vocab * c->d; slot = &m->lm_head; break;
            case ORC_W_ATTN_NORM: want = (size_t)c->d; slot = &m->layers[l].attn_norm; break;
            case ORC_W_QKV: want = (size_t)(c->nh + 2 * c->nkvh) * c->dh * c->d; slot = &m->layers[l].qkv; break;
            case ORC_W_O: want = (size_t)c->d * c->nh * c->dh; slot = &m->layers[l].o; break;
            case ORC_W_FFN_NORM: want = (size_t)c->d; slot = &m->layers[l].ffn_norm; break;
            case ORC_W_GATE_UP: want = (size_t)2 * c->di * c->d; slot = &m->layers[l].gate_up; break;
            default: want = (size_t)c->d * c->di; slot = &m->layers[l].down; break;
            }
            int global = kind == ORC_W_EMBD || kind == ORC_W_OUT_NORM || kind == ORC_W_LM_HEAD;
            if (global && l > 0) continue;
            if (kind == ORC_W_EMBD) continue; /* tied to the LM head below: saves a vocab x d fill */
            free(*slot);
            *slot = (float *)malloc(want * 4);
            if (!*slot) return -1;
            if (kind == ORC_W_ATTN_NORM || kind == ORC_W_FFN_NORM || kind == ORC_W_OUT_NORM)
                for (size_t i = 0; i < want; ++i) (*slot)[i] = 1.0f;
            else
                fill_uniform(*slot, want, seed + (uint64_t)kind * 1000 + (uint64_t)l);
        }
    if (m->embd && m->embd != m->lm_head) free(m->embd);
    m->embd = m->lm_head;
    return 0;
}

int orc_seq_new(orc_model *m) {
    for (int s = 0; s < ORC_MAX_SEQ; ++s)
        if (!m->used[s]) {
            size_t n = (size_t)m->c.n_layers * m->c.nctx * m->c.nkvh * m->c.dh;
            m->kc[s] = (float *)calloc(n, 4);
            m->vc[s] = (float *)calloc(n, 4);
            m->used[s] = 1;
            return s;
        }
    return -1;
}

void orc_seq_free(orc_model *m, int s) {
    if (s < 0 || s >= ORC_MAX_SEQ) return;
    free(m->kc[s]); free(m->vc[s]);
    m->kc[s] = m->vc[s] = NULL;
    m->used[s] = 0;
}

/* One round of llama.cu/src/exec/engine.rs:217-295: positions as in engine.rs:352-358,
 * output row = the last token of each request (engine.rs:360-371 with out == 1), layer
 * order as registered in exec/group.rs:183-195 and described in model/mod.rs:90-169,
 * head as in exec/output_head.rs:55-116. */
int orc_forward(orc_model *m, int n_req, const int *seqs, const uint32_t *tokens,
                const uint32_t *seq_len, const uint32_t *pos0, float *logits, uint32_t *ids) {
    const orc_desc *c = &m->c;
    int dt = c->act_dtype, d = c->d, dh = c->dh, nh = c->nh, nkvh = c->nkvh, di = c->di;
    int qd = nh * dh, kvd = nkvh * dh, qkvd = qd + 2 * kvd;
    int n = 0;
    for (int r = 0; r < n_req; ++r) {
        if (pos0[r] + seq_len[r] > (uint32_t)c->nctx) return -3; /* cache overflow */
        n += (int)seq_len[r];
    }
    uint32_t *pos = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)n);
    for (int r = 0, t = 0; r < n_req; ++r)
        for (uint32_t i = 0; i < seq_len[r]; ++i) pos[t++] = pos0[r] + i;

    float *x = (float *)malloc((size_t)n * d * 4), *h = (float *)malloc((size_t)n * d * 4);
    float *qkv = (float *)malloc((size_t)n * qkvd * 4), *att = (float *)malloc((size_t)n * qd * 4);
    float *gu = (float *)malloc((size_t)n * 2 * di * 4), *act = (float *)malloc((size_t)n * di * 4);
    float *x2 = (float *)malloc((size_t)n * d * 4);
    free(m->hidden);
    m->hidden = (float *)malloc((size_t)(c->n_layers + 1) * n * d * 4);
    m->hidden_tok = n;

    struct timespec ts0, ts1, ts2;
    clock_gettime(CLOCK_MONOTONIC, &ts0);
    orc_embedding(x, m->embd, tokens, n, d);
    memcpy(m->hidden, x, (size_t)n * d * 4);
    for (int l = 0; l < c->n_layers; ++l) {
        orc_layer *L = &m->layers[l];
        orc_rms_norm(h, x, L->attn_norm, n, d, c->eps, dt);
        orc_linear(qkv, h, L->qkv, NULL, n, d, qkvd, dt);
        orc_rope(qkv, n, nh, dh, qkvd, pos, m->sin_t, m->cos_t, dt);
        orc_rope(qkv + qd, n, nkvh, dh, qkvd, pos, m->sin_t, m->cos_t, dt);
        for (int r = 0, t0 = 0; r < n_req; t0 += (int)seq_len[r], ++r) {
            size_t lofs = (size_t)l * c->nctx * kvd;
            float *kc = m->kc[seqs[r]] + lofs, *vc = m->vc[seqs[r]] + lofs;
            for (uint32_t i = 0; i < seq_len[r]; ++i) {
                memcpy(kc + (size_t)(pos0[r] + i) * kvd, qkv + (size_t)(t0 + i) * qkvd + qd, (size_t)kvd * 4);
                memcpy(vc + (size_t)(pos0[r] + i) * kvd, qkv + (size_t)(t0 + i) * qkvd + qd + kvd, (size_t)kvd * 4);
            }
            orc_attention(att + (size_t)t0 * qd, qd, qkv + (size_t)t0 * qkvd, qkvd, kc, vc,
                          nh, nkvh, dh, (int)pos0[r], (int)seq_len[r], dt);
        }
        orc_linear(x2, att, L->o, x, n, qd, d, dt);
        orc_rms_norm(h, x2, L->ffn_norm, n, d, c->eps, dt);
        orc_linear(gu, h, L->gate_up, NULL, n, d, 2 * di, dt);
        orc_swiglu(act, di, gu, 2 * di, gu + di, 2 * di, n, di, dt);
        orc_linear(x, act, L->down, x2, n, di, d, dt);
        memcpy(m->hidden + (size_t)(l + 1) * n * d, x, (size_t)n * d * 4);
    }
    clock_gettime(CLOCK_MONOTONIC, &ts1);
    /* head: gather the last token of each request, norm, lm_head, argmax */
    float *xo = (float *)malloc((size_t)n_req * d * 4), *lg = (float *)malloc((size_t)n_req * c->vocab * 4);
    for (int r = 0, t0 = 0; r < n_req; t0 += (int)seq_len[r], ++r)
        memcpy(xo + (size_t)r * d, x + (size_t)(t0 + seq_len[r] - 1) * d, (size_t)d * 4);
    orc_rms_norm(xo, xo, m->out_norm, n_req, d, c->eps, dt);
    orc_linear(lg, xo, m->lm_head ? m->lm_head : m->embd, NULL, n_req, d, c->vocab, dt);
    for (int r = 0; r < n_req; ++r) {
        if (ids) orc_argmax(lg + (size_t)r * c->vocab, (size_t)c->vocab, &ids[r], NULL);
    }
    if (logits) memcpy(logits, lg, (size_t)n_req * c->vocab * 4);
    clock_gettime(CLOCK_MONOTONIC, &ts2);
    m->t_layers = (double)(ts1.tv_sec - ts0.tv_sec) + 1e-9 * (double)(ts1.tv_nsec - ts0.tv_nsec);
    m->t_head = (double)(ts2.tv_sec - ts1.tv_sec) + 1e-9 * (double)(ts2.tv_nsec - ts1.tv_nsec);
    free(pos); free(x); free(h); free(qkv); free(att); free(gu); free(act); free(x2); free(xo); free(lg);
    return 0;
}

/* Worker threads of the parallel loops: launchers such as torchrun export OMP_NUM_THREADS=1, so a
 * caller that wants every host core asks for them here.  Returns the count now in effect. */
int orc_set_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
}

void orc_last_times(orc_model *m, double *t_layers, double *t_head) {
    *t_layers = m->t_layers;
    *t_head = m->t_head;
}

int orc_last_hidden(orc_model *m, float *out, size_t cap) {
    size_t n = (size_t)(m->c.n_layers + 1) * m->hidden_tok * m->c.d;
    if (!m->hidden || cap < n) return -1;
    memcpy(out, m->hidden, n * 4);
    return m->hidden_tok;
}
