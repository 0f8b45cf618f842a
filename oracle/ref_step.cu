// Reference-kernel baseline of the decode step — TEST / MEASUREMENT INFRASTRUCTURE, not product code.
//
// The reference binary (a Rust workspace with un-vendored git dependencies) cannot be built where
// this runs, so this host replays what it would LAUNCH for one round, from the pieces that can be
// built here:
//   * the reference's own kernels (rms_norm, rope, swiglu, embedding, fast_embedding, arg-max),
//     compiled from the reference tree by the Makefile beside this file (ref_shim.cu wraps them
//     with the launch geometry of llama.cu/src/op/*.rs);
//   * `Linear` as the reference issues it: one cublasGemmEx per projection, f16 operands, f32
//     accumulation, the row-major swap trick, and a residual realised as memcpy_d2d(y <- res)
//     followed by beta = 1 (llama.cu/src/op/linear.rs:35-46,85-118,143-198);
//   * the execution plan of llama.cu/src/exec/step.rs:31-98: the non-attention operators of a
//     round captured into L + 1 CUDA graphs cut at every attention node, attention launched
//     eagerly once per request and per layer in between (step.rs:140-184), inputs padded with
//     zeros to the bucket {1, 8, 32, 64, 128, 256, 1024} (exec/group.rs:89-107);
//   * the output head of llama.cu/src/exec/output_head.rs:55-116: stream-ordered allocations,
//     row gather with the embedding kernel, in-place RMSNorm, LM-head GEMM, one arg-max call per
//     row in a host loop;
//   * a KV cache per session laid out [nctx, nblk, 2, nkvh, dh] and viewed per head
//     (exec/kv_cache.rs:15-31); plain device allocations stand in for its virtual-memory pages.
// NOT from the reference: the attention operator.  Its source lives in an external crate
// (operators-rs, pinned ed28f2d) that is absent from the reference tree; it is restated here as
// the composed operator its call site implies — rearrange q, append k and v to the cache, a
// batched GEMM for the scores, a causal softmax kernel, a batched GEMM for the output, rearrange
// back — seven launches per request and layer, f16 storage, f32 accumulation, scale 1/sqrt(dh).
// Single GPU only (the reference's tensor parallelism adds NCCL calls that are not replayed).
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <vector>

// the reference's kernels behind C entry points (ref_shim.cu, random_sample/sample.cu)
extern "C" {
int ref_rms_norm_f16(void *y, int sy, const void *x, int sx, const void *w, int w_is_f32, float eps, int n, int d,
                     cudaStream_t s);
int ref_rope_f16(void *y, int sty, int shy, const void *x, int stx, int shx, const unsigned *pos, const float *sin_t,
                 const float *cos_t, int n, int nh, int dh, cudaStream_t s);
int ref_swiglu_f16(void *out, int so, const void *gate, int sg, const void *up, int su, int n, int di, cudaStream_t s);
int ref_embedding(void *out, const void *table, const unsigned *index, int n, int row_bytes, cudaStream_t s);
int ref_fast_embedding(unsigned *tokens, const void *kv_pairs, const void *map, int n_map, cudaStream_t s);
cudaError_t calculate_workspace_size_half(size_t *argmax, size_t *random_sample, size_t n);
cudaError_t argmax_half(void *kv_pair, void const *logits, size_t n, void *workspace_ptr, size_t workspace_len,
                        cudaStream_t stream);
}

// part of the C interface (a type of an unnamed namespace would give the functions below internal linkage)
struct Desc {
    int32_t n_layers, d, nh, nkvh, dh, di, vocab, nctx;
    float eps, theta;
};
struct Req {
    int32_t seq;
    uint32_t pos, len;
};

namespace {

struct Layer {
    const half *attn_norm = nullptr, *qkv = nullptr, *o = nullptr, *ffn_norm = nullptr, *gate_up = nullptr, *down = nullptr;
};

#define CK(expr)                                                                                  \
    do {                                                                                          \
        cudaError_t e__ = (expr);                                                                 \
        if (e__ != cudaSuccess) {                                                                 \
            snprintf(g_err, sizeof(g_err), "%s: %s", #expr, cudaGetErrorString(e__));             \
            return -2;                                                                            \
        }                                                                                         \
    } while (0)
#define CB(expr)                                                                 \
    do {                                                                         \
        cublasStatus_t s__ = (expr);                                             \
        if (s__ != CUBLAS_STATUS_SUCCESS) {                                      \
            snprintf(g_err, sizeof(g_err), "%s: cuBLAS status %d", #expr, (int)s__); \
            return -3;                                                           \
        }                                                                        \
    } while (0)
#define CR(expr)                                                           \
    do {                                                                   \
        int r__ = (expr);                                                  \
        if (r__ != 0) {                                                    \
            snprintf(g_err, sizeof(g_err), "%s returned %d", #expr, r__);  \
            return -4;                                                     \
        }                                                                  \
    } while (0)
char g_err[512] = "";

struct Model {
    Desc c;
    std::vector<Layer> layers;
    const half *embd = nullptr, *out_norm = nullptr, *lm_head = nullptr;
    float *sin_t = nullptr, *cos_t = nullptr;
    cublasHandle_t blas = nullptr;
    void *blas_ws = nullptr;
    // one workspace for the largest bucket (the reference plans one per bucket and remaps it)
    int max_tok = 1024;
    unsigned *tok = nullptr, *pos = nullptr;
    half *x0 = nullptr, *x1 = nullptr, *h = nullptr, *qkv = nullptr, *att = nullptr, *gu = nullptr, *act = nullptr;
    // restated attention
    half *q_re = nullptr, *o_re = nullptr, *scores = nullptr;
    // head / sampling
    void *argmax_ws = nullptr;
    size_t argmax_ws_len = 0;
    void *pre_pairs = nullptr;  // last round's KVPairs (fast_embedding reads them)
    void *map_dev = nullptr;
    half *last_logits = nullptr;  // copy of the last round's logits for parity checks
    unsigned *host_tok = nullptr, *host_pos = nullptr, *host_idx = nullptr, *host_map = nullptr;  // pinned
    std::vector<half *> caches;  // per session [nctx, L, 2, nkvh, dh]
    std::map<int, std::vector<cudaGraphExec_t>> graphs;  // bucket -> L + 1 segments
    long launches = 0;
};

int bucket_for(int n) {
    const int b[7] = {1, 8, 32, 64, 128, 256, 1024};  // exec/engine.rs:68, group.rs:96-100
    for (int v : b)
        if (v >= n) return v;
    return -1;
}

// y[n, out] = x[n, in] . W^T (+ y): row-major C through the operand swap of linear.rs:162-174
int gemm(Model *m, half *y, int ldy, const half *x, int ldx, const half *w, int n, int in, int out, float beta,
         cudaStream_t s) {
    const float alpha = 1.f;
    CB(cublasSetStream(m->blas, s));
    CB(cublasGemmEx(m->blas, CUBLAS_OP_T, CUBLAS_OP_N, out, n, in, &alpha, w, CUDA_R_16F, in, x, CUDA_R_16F, ldx, &beta, y,
                    CUDA_R_16F, ldy, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT));
    ++m->launches;
    return 0;
}

// ---- restated attention operator (see the header comment)
__global__ void rearrange_heads(half *dst, const half *src, int seq, int nh, int dh, int ld_src, bool to_heads) {
    // to_heads: dst[h][j][e] = src[j][h*dh + e]; else dst[j][h*dh + e] = src[h][j][e] with ld on the token-major side
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= seq * nh * dh) return;
    int e = i % dh, h = (i / dh) % nh, j = i / (dh * nh);
    if (to_heads) dst[((size_t)h * seq + j) * dh + e] = src[(size_t)j * ld_src + h * dh + e];
    else dst[(size_t)j * ld_src + h * dh + e] = src[((size_t)h * seq + j) * dh + e];
}
__global__ void append_cache(half *cache, const half *src, int seq, int nkvh, int dh, int ld_src, size_t tok_stride, int pos) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= seq * nkvh * dh) return;
    int e = i % dh, h = (i / dh) % nkvh, j = i / (dh * nkvh);
    cache[(size_t)(pos + j) * tok_stride + h * dh + e] = src[(size_t)j * ld_src + h * dh + e];
}
// rows = nh * seq, row (h, j) attends positions [0, pos + j]; f32 inside, f16 in place
__global__ void causal_softmax(half *sc, int seq, int ctx, int pos, float scale) {
    int row = blockIdx.x, j = row % seq, lim = pos + j + 1;
    half *p = sc + (size_t)row * ctx;
    __shared__ float red[32];
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < lim; c += blockDim.x) mx = fmaxf(mx, __half2float(p[c]) * scale);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(~0u, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int c = threadIdx.x; c < lim; c += blockDim.x) sum += expf(__half2float(p[c]) * scale - mx);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(~0u, sum, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    sum = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) sum += red[w];
    const float inv = 1.f / sum;
    for (int c = threadIdx.x; c < ctx; c += blockDim.x)
        p[c] = c < lim ? __float2half_rn(expf(__half2float(p[c]) * scale - mx) * inv) : __float2half_rn(0.f);
}

int attention_request(Model *m, int layer, const Req &r, int start, cudaStream_t s) {
    const Desc &c = m->c;
    const int G = c.nh / c.nkvh, seq = (int)r.len, ctx = (int)r.pos + seq;
    const int ldq = (c.nh + 2 * c.nkvh) * c.dh;
    const size_t tok_stride = (size_t)c.n_layers * 2 * c.nkvh * c.dh;
    half *cache = m->caches[r.seq];
    half *kc = cache + ((size_t)layer * 2 + 0) * c.nkvh * c.dh, *vc = cache + ((size_t)layer * 2 + 1) * c.nkvh * c.dh;
    const half *q = m->qkv + (size_t)start * ldq, *k = q + c.nh * c.dh, *v = k + c.nkvh * c.dh;
    const int T = 256;
    rearrange_heads<<<(seq * c.nh * c.dh + T - 1) / T, T, 0, s>>>(m->q_re, q, seq, c.nh, c.dh, ldq, true);
    append_cache<<<(seq * c.nkvh * c.dh + T - 1) / T, T, 0, s>>>(kc, k, seq, c.nkvh, c.dh, ldq, tok_stride, (int)r.pos);
    append_cache<<<(seq * c.nkvh * c.dh + T - 1) / T, T, 0, s>>>(vc, v, seq, c.nkvh, c.dh, ldq, tok_stride, (int)r.pos);
    m->launches += 3;
    // scores[hk][g*seq + j][c] = q_re[hk*G + g][j][:] . K[c][hk][:]     (row-major C = A . B^T)
    const float one = 1.f, zero = 0.f;
    CB(cublasSetStream(m->blas, s));
    CB(cublasGemmStridedBatchedEx(m->blas, CUBLAS_OP_T, CUBLAS_OP_N, ctx, G * seq, c.dh, &one, kc, CUDA_R_16F, (int)tok_stride,
                                  (long long)c.dh, m->q_re, CUDA_R_16F, c.dh, (long long)G * seq * c.dh, &zero, m->scores,
                                  CUDA_R_16F, ctx, (long long)G * seq * ctx, c.nkvh, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT));
    causal_softmax<<<c.nh * seq, 256, 0, s>>>(m->scores, seq, ctx, (int)r.pos, 1.f / sqrtf((float)c.dh));
    // o_re[hk][g*seq + j][:] = P[g*seq + j][:] . V[:][hk][:]
    CB(cublasGemmStridedBatchedEx(m->blas, CUBLAS_OP_N, CUBLAS_OP_N, c.dh, G * seq, ctx, &one, vc, CUDA_R_16F, (int)tok_stride,
                                  (long long)c.dh, m->scores, CUDA_R_16F, ctx, (long long)G * seq * ctx, &zero, m->o_re,
                                  CUDA_R_16F, c.dh, (long long)G * seq * c.dh, c.nkvh, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT));
    rearrange_heads<<<(seq * c.nh * c.dh + T - 1) / T, T, 0, s>>>(m->att + (size_t)start * c.nh * c.dh, m->o_re, seq, c.nh, c.dh,
                                                                  c.nh * c.dh, false);
    m->launches += 4;
    CK(cudaGetLastError());
    return 0;
}

// the operators of one graph segment: seg 0 = embedding .. rope of layer 0; seg l = o-proj of layer l-1 .. rope of
// layer l; seg L = o-proj .. down of the last layer
int enqueue_segment(Model *m, int seg, int N, cudaStream_t s) {
    const Desc &c = m->c;
    const int qd = c.nh * c.dh, kvd = c.nkvh * c.dh, ldq = qd + 2 * kvd;
    if (seg == 0) {
        CR(ref_embedding(m->x0, m->embd, m->tok, N, c.d * 2, s));
        ++m->launches;
    } else {
        const Layer &L = m->layers[seg - 1];
        // linear(o, residual): memcpy_d2d(y <- residual), beta = 1
        CK(cudaMemcpyAsync(m->x1, m->x0, (size_t)N * c.d * 2, cudaMemcpyDeviceToDevice, s));
        if (int rc = gemm(m, m->x1, c.d, m->att, qd, L.o, N, qd, c.d, 1.f, s)) return rc;
        CR(ref_rms_norm_f16(m->h, c.d, m->x1, c.d, L.ffn_norm, 0, c.eps, N, c.d, s));
        if (int rc = gemm(m, m->gu, 2 * c.di, m->h, c.d, L.gate_up, N, c.d, 2 * c.di, 0.f, s)) return rc;
        CR(ref_swiglu_f16(m->act, c.di, m->gu, 2 * c.di, m->gu + c.di, 2 * c.di, N, c.di, s));
        CK(cudaMemcpyAsync(m->x0, m->x1, (size_t)N * c.d * 2, cudaMemcpyDeviceToDevice, s));
        if (int rc = gemm(m, m->x0, c.d, m->act, c.di, L.down, N, c.di, c.d, 1.f, s)) return rc;
        m->launches += 4;
    }
    if (seg < c.n_layers) {
        const Layer &L = m->layers[seg];
        CR(ref_rms_norm_f16(m->h, c.d, m->x0, c.d, L.attn_norm, 0, c.eps, N, c.d, s));
        if (int rc = gemm(m, m->qkv, ldq, m->h, c.d, L.qkv, N, c.d, ldq, 0.f, s)) return rc;
        CR(ref_rope_f16(m->qkv, ldq, c.dh, m->qkv, ldq, c.dh, m->pos, m->sin_t, m->cos_t, N, c.nh, c.dh, s));
        CR(ref_rope_f16(m->qkv + qd, ldq, c.dh, m->qkv + qd, ldq, c.dh, m->pos, m->sin_t, m->cos_t, N, c.nkvh, c.dh, s));
        m->launches += 3;
    }
    return 0;
}

}  // namespace

extern "C" {

const char *refstep_last_error(void) { return g_err; }

int refstep_create(const Desc *desc, void **out) {
    cudaGetLastError();  // a stale error of an earlier, unrelated call must not fail the first check here
    Model *m = new Model();
    m->c = *desc;
    const Desc &c = m->c;
    m->layers.resize(c.n_layers);
    CB(cublasCreate(&m->blas));
    CK(cudaMalloc(&m->blas_ws, (size_t)64 << 20));
    CB(cublasSetWorkspace(m->blas, m->blas_ws, (size_t)64 << 20));
    const int N = m->max_tok, qd = c.nh * c.dh, kvd = c.nkvh * c.dh;
    CK(cudaMalloc(&m->tok, N * 4));
    CK(cudaMalloc(&m->pos, N * 4));
    CK(cudaMalloc(&m->x0, (size_t)N * c.d * 2));
    CK(cudaMalloc(&m->x1, (size_t)N * c.d * 2));
    CK(cudaMalloc(&m->h, (size_t)N * c.d * 2));
    CK(cudaMalloc(&m->qkv, (size_t)N * (qd + 2 * kvd) * 2));
    CK(cudaMalloc(&m->att, (size_t)N * qd * 2));
    CK(cudaMalloc(&m->gu, (size_t)N * 2 * c.di * 2));
    CK(cudaMalloc(&m->act, (size_t)N * c.di * 2));
    CK(cudaMalloc(&m->q_re, (size_t)N * qd * 2));
    CK(cudaMalloc(&m->o_re, (size_t)N * qd * 2));
    CK(cudaMalloc(&m->scores, (size_t)c.nh * N * c.nctx * 2));
    size_t ws_sample = 0;
    CK(calculate_workspace_size_half(&m->argmax_ws_len, &ws_sample, (size_t)c.vocab));
    CK(cudaMalloc(&m->argmax_ws, m->argmax_ws_len));
    CK(cudaMalloc(&m->pre_pairs, (size_t)N * 8));
    CK(cudaMalloc(&m->map_dev, (size_t)N * 8));
    CK(cudaMalloc(&m->last_logits, (size_t)64 * c.vocab * 2));
    CK(cudaMallocHost(&m->host_tok, N * 4));
    CK(cudaMallocHost(&m->host_pos, N * 4));
    CK(cudaMallocHost(&m->host_idx, N * 4));
    CK(cudaMallocHost(&m->host_map, N * 8));
    // sin / cos tables as build_sin_cos makes them (model/mod.rs:186-220): f32 powf, product, sinf / cosf
    const int half_dh = c.dh / 2;
    std::vector<float> tab((size_t)2 * c.nctx * half_dh);
    for (int p = 0; p < c.nctx; ++p)
        for (int i = 0; i < half_dh; ++i) {
            float t = powf(c.theta, -((float)(2 * i) / (float)c.dh)), f = (float)p * t;
            tab[(size_t)p * half_dh + i] = sinf(f);
            tab[(size_t)c.nctx * half_dh + (size_t)p * half_dh + i] = cosf(f);
        }
    CK(cudaMalloc(&m->sin_t, tab.size() * 4));
    CK(cudaMemcpy(m->sin_t, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice));
    m->cos_t = m->sin_t + (size_t)c.nctx * half_dh;
    *out = m;
    return 0;
}

int refstep_destroy(void *mp) {
    Model *m = reinterpret_cast<Model *>(mp);
    if (!m) return 0;
    cudaDeviceSynchronize();
    for (auto &g : m->graphs)
        for (auto e : g.second) cudaGraphExecDestroy(e);
    for (half *p : m->caches) cudaFree(p);
    void *bufs[] = {m->blas_ws, m->tok, m->pos, m->x0, m->x1, m->h, m->qkv, m->att, m->gu, m->act, m->q_re, m->o_re, m->scores,
                    m->argmax_ws, m->pre_pairs, m->map_dev, m->last_logits, m->sin_t};
    for (void *p : bufs) cudaFree(p);
    cudaFreeHost(m->host_tok); cudaFreeHost(m->host_pos); cudaFreeHost(m->host_idx); cudaFreeHost(m->host_map);
    if (m->blas) cublasDestroy(m->blas);
    delete m;
    return 0;
}

// kinds as in include/lcu.h: 0 embd, 1 attn_norm, 2 qkv, 3 o, 4 ffn_norm, 5 gate_up, 6 down, 7 out_norm, 8 lm_head
int refstep_set_weight(void *mp, int layer, int kind, const void *dev) {
    Model *m = reinterpret_cast<Model *>(mp);
    const half *p = reinterpret_cast<const half *>(dev);
    for (auto &g : m->graphs)
        for (auto e : g.second) cudaGraphExecDestroy(e);
    m->graphs.clear();
    switch (kind) {
    case 0: m->embd = p; return 0;
    case 7: m->out_norm = p; return 0;
    case 8: m->lm_head = p; return 0;
    }
    if (layer < 0 || layer >= m->c.n_layers) return -1;
    Layer &L = m->layers[layer];
    switch (kind) {
    case 1: L.attn_norm = p; break;
    case 2: L.qkv = p; break;
    case 3: L.o = p; break;
    case 4: L.ffn_norm = p; break;
    case 5: L.gate_up = p; break;
    case 6: L.down = p; break;
    default: return -1;
    }
    return 0;
}

int refstep_seq_new(void *mp) {
    Model *m = reinterpret_cast<Model *>(mp);
    const Desc &c = m->c;
    half *p = nullptr;
    if (cudaMalloc(&p, (size_t)c.nctx * c.n_layers * 2 * c.nkvh * c.dh * 2) != cudaSuccess) return -1;
    m->caches.push_back(p);
    return (int)m->caches.size() - 1;
}

// One round.  tokens: flat host ids; fast_map: n_fast (pair index, token slot) entries or NULL; out_dev: n_req
// KVPairs.  Returns the launches (kernels, copies, graph launches count as their nodes) through *launches.
int refstep_round(void *mp, cudaStream_t s, int n_req, const Req *reqs, const unsigned *tokens, const unsigned *fast_map,
                  int n_fast, void *out_dev, long *launches) {
    Model *m = reinterpret_cast<Model *>(mp);
    const Desc &c = m->c;
    int n = 0;
    for (int i = 0; i < n_req; ++i) n += (int)reqs[i].len;
    const int N = bucket_for(n);
    if (N < 0 || n_req > 64) { snprintf(g_err, sizeof(g_err), "round of %d tokens / %d requests", n, n_req); return -1; }
    if (s == nullptr || s == cudaStreamLegacy) { snprintf(g_err, sizeof(g_err), "the round captures graphs: pass a created stream"); return -1; }
    m->launches = 0;
    // load_inputs: tokens and positions padded with zeros to the bucket (group.rs:89-107)
    memset(m->host_tok, 0, N * 4);
    memset(m->host_pos, 0, N * 4);
    memcpy(m->host_tok, tokens, n * 4);
    int t = 0;
    for (int i = 0; i < n_req; ++i) {
        for (uint32_t j = 0; j < reqs[i].len; ++j, ++t) m->host_pos[t] = reqs[i].pos + j;
        m->host_idx[i] = (unsigned)(t - 1);
    }
    CK(cudaMemcpyAsync(m->tok, m->host_tok, N * 4, cudaMemcpyHostToDevice, s));
    CK(cudaMemcpyAsync(m->pos, m->host_pos, N * 4, cudaMemcpyHostToDevice, s));
    m->launches += 2;
    if (n_fast > 0) {  // FastEmbedding: H2D of the map, one kernel (fast_embedding.rs:28-44)
        memcpy(m->host_map, fast_map, (size_t)n_fast * 8);
        CK(cudaMemcpyAsync(m->map_dev, m->host_map, (size_t)n_fast * 8, cudaMemcpyHostToDevice, s));
        CR(ref_fast_embedding(m->tok, m->pre_pairs, m->map_dev, n_fast, s));
        m->launches += 2;
    }
    // graph segments of this bucket, captured on first use (step.rs:31-98)
    auto it = m->graphs.find(N);
    if (it == m->graphs.end()) {
        std::vector<cudaGraphExec_t> segs;
        const long keep = m->launches;
        for (int seg = 0; seg <= c.n_layers; ++seg) {
            cudaGraph_t g = nullptr;
            CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            int rc = enqueue_segment(m, seg, N, s);
            cudaError_t e = cudaStreamEndCapture(s, &g);
            if (rc) return rc;
            CK(e);
            cudaGraphExec_t ex = nullptr;
            CK(cudaGraphInstantiate(&ex, g, 0));
            cudaGraphDestroy(g);
            segs.push_back(ex);
        }
        m->launches = keep;
        it = m->graphs.emplace(N, segs).first;
    }
    for (int seg = 0; seg <= c.n_layers; ++seg) {
        CK(cudaGraphLaunch(it->second[seg], s));
        m->launches += seg == 0 ? 4 : (seg < c.n_layers ? 10 : 7);  // nodes of the segment
        if (seg < c.n_layers) {
            int start = 0;
            for (int i = 0; i < n_req; ++i) {  // launch_attn: one operator call per request (step.rs:140-184)
                if (int rc = attention_request(m, seg, reqs[i], start, s)) return rc;
                start += (int)reqs[i].len;
            }
        }
    }
    // output head on stream-ordered allocations (output_head.rs:55-116)
    unsigned *idx_dev = nullptr;
    half *gathered = nullptr, *logits = nullptr;
    CK(cudaMallocAsync(&idx_dev, (size_t)n_req * 4, s));
    CK(cudaMemcpyAsync(idx_dev, m->host_idx, (size_t)n_req * 4, cudaMemcpyHostToDevice, s));
    CK(cudaMallocAsync(&gathered, (size_t)n_req * c.d * 2, s));
    CR(ref_embedding(gathered, m->x0, idx_dev, n_req, c.d * 2, s));
    CK(cudaFreeAsync(idx_dev, s));
    CR(ref_rms_norm_f16(gathered, c.d, gathered, c.d, m->out_norm, 0, c.eps, n_req, c.d, s));
    CK(cudaMallocAsync(&logits, (size_t)n_req * c.vocab * 2, s));
    if (int rc = gemm(m, logits, c.vocab, gathered, c.d, m->lm_head, n_req, c.d, c.vocab, 0.f, s)) return rc;
    CK(cudaFreeAsync(gathered, s));
    for (int i = 0; i < n_req; ++i)  // one arg-max call per row
        CK(argmax_half(reinterpret_cast<unsigned char *>(out_dev) + (size_t)i * 8, logits + (size_t)i * c.vocab, (size_t)c.vocab,
                       m->argmax_ws, m->argmax_ws_len, s));
    m->launches += 3 + 2 * n_req;
    CK(cudaMemcpyAsync(m->last_logits, logits, (size_t)n_req * c.vocab * 2, cudaMemcpyDeviceToDevice, s));  // for the tests only
    CK(cudaFreeAsync(logits, s));
    // kv_pairs -> pre_kv_pairs for the next round's fast_embedding (engine.rs:285)
    CK(cudaMemcpyAsync(m->pre_pairs, out_dev, (size_t)n_req * 8, cudaMemcpyDeviceToDevice, s));
    ++m->launches;
    if (launches) *launches = m->launches;
    return 0;
}

const void *refstep_logits(void *mp) { return reinterpret_cast<Model *>(mp)->last_logits; }

}  // extern "C"
