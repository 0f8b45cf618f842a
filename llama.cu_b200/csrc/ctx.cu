// Context, KV page pool and the per-round step of the decode token loop, plus the
// C-ABI wrappers around them.  Host-side counterpart of llama.cu/src/exec/{group,model,
// step,output_head,kv_cache}.rs and memory.rs for one GPU.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "attention.cuh"
#include "common.cuh"
#include "gemv.cuh"
#include "ops.cuh"
#include "p2p.cuh"
#include "sample.cuh"

namespace lcu {

// ------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return LCU_ERR_CUDA;
}

int sm_count() {
    static std::mutex mu;
    static std::map<int, int> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(dev);
    if (it != cache.end()) return it->second;
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
    return n;
}

Tuning &tuning() {
    static Tuning t;
    return t;
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
static size_t dt_bytes(int dt) { return dt == LCU_F32 || dt == LCU_U32 ? 4 : 2; }

}  // namespace lcu

using namespace lcu;

// ------------------------------------------------------------------ context

struct LayerWeights {
    const void *attn_norm = nullptr, *qkv = nullptr, *o = nullptr, *ffn_norm = nullptr, *gate_up = nullptr,
               *down = nullptr;
};

struct SeqState {
    bool used = false;
    uint32_t len = 0;  // tokens backed by pages
    std::vector<int> pages;
};

struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    int launches = 0;
};

struct lcu_ctx {
    lcu_model_desc desc;
    int device = 0, tp_rank = 0, tp_size = 1;
    void *comm = nullptr;
    int dt = LCU_F16;
    // per-rank shapes
    int nh_l = 0, nkvh_l = 0, di_l = 0, qd = 0, kvd = 0;
    int max_tokens = 0, max_seqs = 0;

    std::vector<LayerWeights> layers;
    const void *embd = nullptr, *out_norm = nullptr, *lm_head = nullptr;
    const float *sin_t = nullptr, *cos_t = nullptr;
    float *own_tables = nullptr;

    // KV pages
    void *pool = nullptr;
    bool own_pool = false;
    KvGeom geom{};
    int n_pages = 0, pt_stride = 0;
    std::vector<int> free_pages;
    std::vector<SeqState> seqs;

    // arena (one allocation)
    void *arena = nullptr;
    void *x = nullptr, *q = nullptr, *att = nullptr, *act = nullptr, *logits = nullptr, *hbuf = nullptr;
    void *sk_ws = nullptr;
    unsigned *sk_tickets = nullptr;
    size_t sk_ws_bytes = 0;
    bool batched_ok = false;  // tensor-core path for rounds of more than 4 tokens
    void *attn_scratch = nullptr, *sample_ws = nullptr;
    size_t sample_ws_bytes = 0;
    lcu_kv_pair *pre_pairs = nullptr;  // copy of the last round's output pairs (token feedback)
    uint32_t *dev_status = nullptr;
    unsigned char *desc_dev = nullptr;  // per-round descriptor
    size_t desc_cap = 0;
    // pinned staging ring for the descriptor
    static constexpr int RING = 4;
    unsigned char *desc_host[RING] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t desc_event[RING] = {nullptr, nullptr, nullptr, nullptr};
    bool desc_used[RING] = {false, false, false, false};
    int ring_idx = 0;

    // tensor parallelism over peer memory (set up by lcu_p2p_create / lcu_p2p_attach)
    P2pState p2p;

    // LM head sharded by vocabulary rows under tensor parallelism (peer-memory transport, arg-max rounds)
    bool head_shard = true;           // lcu_set_head_sharding
    lcu_kv_pair *head_local = nullptr;  // this rank's candidates
    uint32_t sticky_status = 0;       // last value lcu_device_status read

    bool use_graph = true;
    std::map<std::vector<int>, StepGraph> graphs;
    int last_launches = 0;
    double last_bytes = 0;
    int last_n_tok = 0, last_n_req = 0;
};

// offsets of the sections of a round descriptor (all 16-byte aligned)
struct DescLayout {
    size_t tokens, pos, tok_req, out_idx, fast_map, args, randoms, page_table, groups, total;
};
static DescLayout desc_layout(int n_tok, int n_req, int pt_stride) {
    DescLayout L;
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t r = o; o += (bytes + 15) & ~(size_t)15; return r; };
    L.tokens = take((size_t)n_tok * 4);
    L.pos = take((size_t)n_tok * 4);
    L.tok_req = take((size_t)n_tok * 4);
    L.out_idx = take((size_t)n_req * 4);
    L.fast_map = take((size_t)n_req * 8);
    L.args = take((size_t)n_req * sizeof(lcu_sample_args));
    L.randoms = take((size_t)n_req * 4);
    L.page_table = take((size_t)n_req * pt_stride * 4);
    L.groups = take((size_t)n_tok * 8);  // token groups of the prefill form of attention (at most one per token)
    L.total = o;
    return L;
}

// Split-KV plan of the attention launch for a round of n_tok tokens (flash-decoding): every CTA walks
// `tps` 64-position tiles, the grid is deep enough for the longest context the cache allows, and a token
// with a shorter context simply uses fewer of its CTAs.  Fixed per round shape so that a captured graph
// stays valid as contexts grow.  Rounds with enough tokens to fill the GPU on their own (prefill) are
// not split.
// Fewest tokens in a round for which the linear layers run as batched tensor-core kernels instead of
// the register-blocked GEMV (measured on the 8B shapes: the GEMV wins up to 2 tokens).
static int batched_min_tokens() { return 3; }

static void attn_plan(const lcu_ctx *c, int n_tok, int *n_splits, int *tps) {
    const int ctas = c->nkvh_l * n_tok;
    const int max_tiles = (c->desc.nctx + 63) / 64;
    if (ctas >= 8 * sm_count() || max_tiles <= 1) {
        *n_splits = 1;
        *tps = max_tiles;
        return;
    }
    // tiles per CTA: enough CTAs to fill the GPU about four times over when every context is full, at most 4
    int t = (int)(((long)ctas * max_tiles + 4L * sm_count() - 1) / (4L * sm_count()));
    if (t > 4) t = 4;
    if (t < 1) t = 1;
    // a round of a few tokens merges its splits inside one thread-block cluster (at most 8 CTAs): take 2 tiles per
    // CTA when that is what it needs
    if (n_tok < batched_min_tokens() && t == 1 && max_tiles > 8 && max_tiles <= 16) t = 2;
    int z = (max_tiles + t - 1) / t;
    int z_cap = 2048 / n_tok;  // bounds the partial-output scratch
    if (z_cap > 64) z_cap = 64;
    if (z_cap < 1) z_cap = 1;
    if (z > z_cap) {
        z = z_cap;
        t = (max_tiles + z - 1) / z;
    }
    *n_splits = z;
    *tps = t;
}

static int attn_splits(const lcu_ctx *c, int n_tok) {
    int z, t;
    attn_plan(c, n_tok, &z, &t);
    return z;
}

// Rows of the LM head one rank holds when the head is sharded by vocabulary (0: the shape does not allow it).
static int head_rows_per_rank(const lcu_ctx *c) {
    if (c->tp_size <= 1 || c->desc.vocab % c->tp_size) return 0;
    const int v = c->desc.vocab / c->tp_size;
    return v % 2 ? 0 : v;
}

static size_t weight_elems(const lcu_ctx *c, int kind) {
    const lcu_model_desc &d = c->desc;
    switch (kind) {
    case LCU_W_EMBD: return (size_t)d.vocab * d.d;
    case LCU_W_LM_HEAD:  // the lead rank keeps the whole matrix (sampling rounds need every logit), the others their rows
        return (size_t)(c->tp_rank != 0 && head_rows_per_rank(c) ? head_rows_per_rank(c) : d.vocab) * d.d;
    case LCU_W_ATTN_NORM: case LCU_W_FFN_NORM: case LCU_W_OUT_NORM: return (size_t)d.d;
    case LCU_W_QKV: return (size_t)(c->qd + 2 * c->kvd) * d.d;
    case LCU_W_O: return (size_t)d.d * c->qd;
    case LCU_W_GATE_UP: return (size_t)2 * c->di_l * d.d;
    case LCU_W_DOWN: return (size_t)d.d * c->di_l;
    default: return 0;
    }
}
static bool is_linear_kind(int kind) {
    return kind == LCU_W_QKV || kind == LCU_W_O || kind == LCU_W_GATE_UP || kind == LCU_W_DOWN;
}

// captured graphs hold weight pointers: any change of registered memory drops them
static void drop_graphs(lcu_ctx *c) {
    for (auto &g : c->graphs)
        if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    c->graphs.clear();
}

static void p2p_release(lcu_ctx *c) {
    P2pState &st = c->p2p;
    for (int r = 0; r < st.n; ++r)
        if (r != st.rank && st.base[r]) cudaIpcCloseMemHandle(st.base[r]);
    if (st.own) cudaFree(st.own);
    st = P2pState();
}

extern "C" {

const char *lcu_last_error_string(void) { return g_err; }
int lcu_version(void) { return 100; }

size_t lcu_weight_bytes(const lcu_ctx *c, int kind) {
    if (!c) return 0;
    size_t n = weight_elems(c, kind);
    if (kind == LCU_W_ATTN_NORM || kind == LCU_W_FFN_NORM || kind == LCU_W_OUT_NORM)
        return n * dt_bytes(c->desc.norm_dtype);
    if (is_linear_kind(kind) && c->desc.weight_dtype == LCU_Q8_0) return n + n / 32 * 2;
    return n * 2;
}

int lcu_build_sin_cos(int nctx, int dh, float theta, float *sin_host, float *cos_host) {
    LCU_REQUIRE(nctx > 0 && dh > 0 && dh % 2 == 0 && sin_host && cos_host, "build_sin_cos: bad arguments");
    int half = dh / 2;
    // f32 powf, f32 product, f32 sin/cos — as build_sin_cos does (model/mod.rs:202-210)
    for (int pos = 0; pos < nctx; ++pos)
        for (int i = 0; i < half; ++i) {
            float t = powf(theta, -((float)(2 * i) / (float)dh));
            float f = (float)pos * t;
            sin_host[(size_t)pos * half + i] = sinf(f);
            cos_host[(size_t)pos * half + i] = cosf(f);
        }
    return LCU_OK;
}

int lcu_ctx_create(const lcu_model_desc *desc, int device, int tp_rank, int tp_size, void *nccl_comm, lcu_ctx **out) {
    LCU_REQUIRE(desc && out, "ctx_create: null argument");
    const lcu_model_desc &d = *desc;
    LCU_REQUIRE(d.n_layers > 0 && d.d > 0 && d.nh > 0 && d.nkvh > 0 && d.dh > 0 && d.di > 0 && d.vocab > 0 && d.nctx > 0,
                "ctx_create: non-positive model dimension");
    LCU_REQUIRE(d.act_dtype == LCU_F16 || d.act_dtype == LCU_BF16, "ctx_create: activation dtype %d (f16 or bf16)", d.act_dtype);
    LCU_REQUIRE(d.weight_dtype == d.act_dtype || (d.weight_dtype == LCU_Q8_0 && d.act_dtype == LCU_F16),
                "ctx_create: weight dtype %d must equal the activation dtype, or be Q8_0 with f16 activations", d.weight_dtype);
    LCU_REQUIRE(d.norm_dtype == d.act_dtype || d.norm_dtype == LCU_F32, "ctx_create: norm dtype %d", d.norm_dtype);
    LCU_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, "ctx_create: rank %d of %d", tp_rank, tp_size);
    LCU_REQUIRE(d.nh % d.nkvh == 0, "ctx_create: nh %d is not a multiple of nkvh %d", d.nh, d.nkvh);
    LCU_REQUIRE(d.nkvh % tp_size == 0 && d.di % tp_size == 0, "ctx_create: nkvh %d and di %d must divide by tp %d", d.nkvh, d.di, tp_size);
    LCU_REQUIRE(d.dh == 64 || d.dh == 128, "ctx_create: dh %d (64 or 128)", d.dh);
    LCU_REQUIRE(d.d % 8 == 0 && (d.di / tp_size) % 8 == 0, "ctx_create: d and di/tp must be multiples of 8");
    LCU_REQUIRE(tp_size == 1 || nccl_comm, "ctx_create: tensor parallelism needs a communicator");
    int g = d.nh / d.nkvh;
    LCU_REQUIRE(g == 1 || g == 2 || g == 4 || g == 8, "ctx_create: nh/nkvh = %d (1, 2, 4, 8)", g);

    int ndev = 0;
    LCU_CHECK_CUDA(cudaGetDeviceCount(&ndev));
    LCU_REQUIRE(device >= 0 && device < ndev, "ctx_create: device %d of %d", device, ndev);
    LCU_CHECK_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    LCU_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("ctx_create: device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return LCU_ERR_CUDA;
    }

    lcu_ctx *c = new lcu_ctx();
    c->desc = d;
    c->device = device;
    c->tp_rank = tp_rank;
    c->tp_size = tp_size;
    c->comm = nccl_comm;
    c->dt = d.act_dtype;
    c->nh_l = d.nh / tp_size;
    c->nkvh_l = d.nkvh / tp_size;
    c->di_l = d.di / tp_size;
    c->qd = c->nh_l * d.dh;
    c->kvd = c->nkvh_l * d.dh;
    c->max_tokens = d.max_tokens > 0 ? d.max_tokens : 1024;
    c->max_seqs = d.max_seqs > 0 ? d.max_seqs : 64;
    if (c->max_seqs > c->max_tokens) c->max_seqs = c->max_tokens;
    c->layers.resize(d.n_layers);

    // page geometry: the reference maps 2 MiB pages (memory.rs:14-19); keep a power of two
    int pt = d.page_tokens;
    if (pt <= 0) {
        size_t per_tok = (size_t)d.n_layers * 2 * c->kvd * 2;
        pt = 16;
        while (pt < 64 && (size_t)pt * 2 * per_tok <= ((size_t)2 << 20)) pt *= 2;
    }
    if (pt < 8 || pt > 128 || (pt & (pt - 1))) {
        set_error("ctx_create: page_tokens %d must be a power of two in [8,128]", pt);
        delete c;
        return LCU_ERR_INVALID;
    }
    c->geom.n_layers = d.n_layers;
    c->geom.nkvh = c->nkvh_l;
    c->geom.dh = d.dh;
    c->geom.page_tokens = pt;
    c->geom.page_shift = 0;
    while ((1 << c->geom.page_shift) < pt) ++c->geom.page_shift;
    c->geom.page_elems = (size_t)d.n_layers * 2 * c->nkvh_l * pt * d.dh;
    c->pt_stride = (d.nctx + pt - 1) / pt;
    c->seqs.resize(1024);

    // arena
    size_t eb = 2;
    size_t sz_x = align256((size_t)c->max_tokens * d.d * eb);
    size_t sz_q = align256((size_t)c->max_tokens * c->qd * eb);
    size_t sz_act = align256((size_t)c->max_tokens * c->di_l * eb);
    size_t sz_logits = align256((size_t)c->max_seqs * d.vocab * eb);
    size_t sz_attn = 0;
    for (int n = 1; n <= c->max_tokens; ++n) {
        int sp = attn_splits(c, n);
        if (sp > 1) {
            size_t b = attn_scratch_bytes(n, c->nh_l, c->nkvh_l, d.dh, sp, c->max_tokens);
            if (b > sz_attn) sz_attn = b;
        }
    }
    sz_attn = align256(sz_attn + 256);
    c->sample_ws_bytes = align256(sample_workspace_bytes(c->max_seqs, (size_t)d.vocab));
    size_t sz_pairs = align256((size_t)c->max_tokens * sizeof(lcu_kv_pair));
    size_t sz_head_local = align256((size_t)c->max_seqs * sizeof(lcu_kv_pair));
    c->desc_cap = align256(desc_layout(c->max_tokens, c->max_seqs, c->pt_stride).total);
    const size_t sz_sk_ws = (size_t)16 << 20, sz_sk_tickets = (size_t)16 << 10;
    size_t total = sz_x + 2 * sz_q + sz_act + sz_logits + sz_attn + c->sample_ws_bytes + sz_pairs + 512 + c->desc_cap +
                   sz_x + sz_sk_ws + sz_sk_tickets + sz_head_local;
    cudaError_t e = cudaMalloc(&c->arena, total);
    if (e != cudaSuccess) {
        delete c;
        return cuda_fail(e, "cudaMalloc(arena)");
    }
    cudaMemset(c->arena, 0, total);
    unsigned char *p = reinterpret_cast<unsigned char *>(c->arena);
    c->x = p; p += sz_x;
    c->q = p; p += sz_q;
    c->att = p; p += sz_q;
    c->act = p; p += sz_act;
    c->logits = p; p += sz_logits;
    c->attn_scratch = p; p += sz_attn;
    c->sample_ws = p; p += c->sample_ws_bytes;
    c->pre_pairs = reinterpret_cast<lcu_kv_pair *>(p); p += sz_pairs;
    c->dev_status = reinterpret_cast<uint32_t *>(p);
    p += 512;
    c->desc_dev = p; p += c->desc_cap;
    c->hbuf = p; p += sz_x;
    c->sk_ws = p; p += sz_sk_ws;
    c->sk_tickets = reinterpret_cast<unsigned *>(p); p += sz_sk_tickets;
    c->head_local = reinterpret_cast<lcu_kv_pair *>(p);
    c->sk_ws_bytes = sz_sk_ws;
    for (int i = 0; i < lcu_ctx::RING; ++i) {
        e = cudaMallocHost(reinterpret_cast<void **>(&c->desc_host[i]), c->desc_cap);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->desc_event[i], cudaEventDisableTiming);
        if (e != cudaSuccess) {
            lcu_ctx_destroy(c);
            return cuda_fail(e, "descriptor staging");
        }
    }
    // prepare every kernel variant now: nothing but launches may happen inside a capture
    {
        bool q8 = d.weight_dtype == LCU_Q8_0;
        int rc = gemv_warm(d.d, c->qd + 2 * c->kvd, q8, c->dt);
        if (!rc) rc = gemv_warm(c->qd, d.d, q8, c->dt);
        if (!rc) rc = gemv_warm(c->di_l, d.d, q8, c->dt);
        if (!rc) rc = gemv_warm(d.d, d.vocab & ~1, false, c->dt);
        if (!rc) {
            AttnArgs a{};
            a.n_tok = 1; a.nh = c->nh_l; a.nkvh = c->nkvh_l; a.dh = d.dh; a.n_splits = 1;
            rc = attn_launch(a, c->dt, nullptr, false, true);
            if (!rc) rc = attn_prefill_launch(a, nullptr, 0, c->dt, nullptr, true);
        }
        if (rc) {
            lcu_ctx_destroy(c);
            return rc;
        }
        // the batched (tensor-core) form of the linear layers
        c->batched_ok = gemm_skinny_supported(d.d, q8) && gemm_skinny_supported(c->qd, q8) && gemm_skinny_supported(c->di_l, q8);
        if (c->batched_ok) {
            rc = gemm_skinny_warm(d.d, c->qd + 2 * c->kvd, c->dt, q8);
            if (!rc) rc = gemm_skinny_warm(c->qd, d.d, c->dt, q8);
            if (!rc) rc = gemm_skinny_warm(c->di_l, d.d, c->dt, q8);
            if (!rc) rc = gemm_skinny_warm(d.d, d.vocab & ~1, c->dt);
            if (!rc && gemm_tc_supported(d.d, q8)) rc = gemm_tc_warm(c->dt);
            if (rc) {
                lcu_ctx_destroy(c);
                return rc;
            }
        }
    }
    *out = c;
    return LCU_OK;
}

int lcu_ctx_destroy(lcu_ctx *c) {
    if (!c) return LCU_OK;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (auto &g : c->graphs)
        if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    for (int i = 0; i < lcu_ctx::RING; ++i) {
        if (c->desc_host[i]) cudaFreeHost(c->desc_host[i]);
        if (c->desc_event[i]) cudaEventDestroy(c->desc_event[i]);
    }
    if (c->own_pool && c->pool) cudaFree(c->pool);
    if (c->own_tables) cudaFree(c->own_tables);
    p2p_release(c);
    if (c->arena) cudaFree(c->arena);
    delete c;
    return LCU_OK;
}

int lcu_set_weight(lcu_ctx *c, int layer, int kind, const void *dev_ptr, size_t bytes) {
    LCU_REQUIRE(c && dev_ptr, "set_weight: null argument");
    size_t want = lcu_weight_bytes(c, kind);
    LCU_REQUIRE(want > 0, "set_weight: unknown kind %d", kind);
    LCU_REQUIRE(bytes == want, "set_weight: kind %d expects %zu bytes on this rank, got %zu", kind, want, bytes);
    LCU_REQUIRE(((uintptr_t)dev_ptr % 16) == 0, "set_weight: pointer must be 16-byte aligned");
    switch (kind) {
    case LCU_W_EMBD: c->embd = dev_ptr; drop_graphs(c); return LCU_OK;
    case LCU_W_OUT_NORM: c->out_norm = dev_ptr; drop_graphs(c); return LCU_OK;
    case LCU_W_LM_HEAD: c->lm_head = dev_ptr; drop_graphs(c); return LCU_OK;
    default: break;
    }
    LCU_REQUIRE(layer >= 0 && layer < c->desc.n_layers, "set_weight: layer %d of %d", layer, c->desc.n_layers);
    LayerWeights &L = c->layers[layer];
    switch (kind) {
    case LCU_W_ATTN_NORM: L.attn_norm = dev_ptr; break;
    case LCU_W_QKV: L.qkv = dev_ptr; break;
    case LCU_W_O: L.o = dev_ptr; break;
    case LCU_W_FFN_NORM: L.ffn_norm = dev_ptr; break;
    case LCU_W_GATE_UP: L.gate_up = dev_ptr; break;
    case LCU_W_DOWN: L.down = dev_ptr; break;
    }
    drop_graphs(c);
    return LCU_OK;
}

int lcu_set_rope_tables(lcu_ctx *c, const float *sin_dev, const float *cos_dev) {
    LCU_REQUIRE(c && sin_dev && cos_dev, "set_rope_tables: null argument");
    c->sin_t = sin_dev;
    c->cos_t = cos_dev;
    drop_graphs(c);
    return LCU_OK;
}

static int ensure_tables(lcu_ctx *c) {
    if (c->sin_t && c->cos_t) return LCU_OK;
    size_t n = (size_t)c->desc.nctx * (c->desc.dh / 2);
    std::vector<float> host(2 * n);
    int rc = lcu_build_sin_cos(c->desc.nctx, c->desc.dh, c->desc.theta, host.data(), host.data() + n);
    if (rc) return rc;
    LCU_CHECK_CUDA(cudaMalloc(reinterpret_cast<void **>(&c->own_tables), 2 * n * 4));
    LCU_CHECK_CUDA(cudaMemcpy(c->own_tables, host.data(), 2 * n * 4, cudaMemcpyHostToDevice));
    c->sin_t = c->own_tables;
    c->cos_t = c->own_tables + n;
    return LCU_OK;
}

// ------------------------------------------------------------------ KV pages

int lcu_kv_pool_attach(lcu_ctx *c, void *dev_ptr, size_t bytes) {
    LCU_REQUIRE(c && dev_ptr, "kv_pool_attach: null argument");
    LCU_REQUIRE(!c->pool, "kv_pool_attach: a pool is already attached");
    LCU_REQUIRE(((uintptr_t)dev_ptr % 256) == 0, "kv_pool_attach: pool must be 256-byte aligned");
    size_t page_bytes = c->geom.page_elems * 2;
    int n = (int)(bytes / page_bytes);
    LCU_REQUIRE(n >= 1, "kv_pool_attach: %zu bytes hold no page of %zu bytes", bytes, page_bytes);
    c->pool = dev_ptr;
    c->n_pages = n;
    c->free_pages.clear();
    for (int i = n - 1; i >= 0; --i) c->free_pages.push_back(i);
    return LCU_OK;
}

int lcu_kv_pool_create(lcu_ctx *c, size_t bytes) {
    LCU_REQUIRE(c, "kv_pool_create: null context");
    LCU_REQUIRE(!c->pool, "kv_pool_create: a pool already exists");
    size_t page_bytes = c->geom.page_elems * 2;
    size_t n = bytes / page_bytes;
    LCU_REQUIRE(n >= 1, "kv_pool_create: %zu bytes hold no page of %zu bytes", bytes, page_bytes);
    void *p = nullptr;
    LCU_CHECK_CUDA(cudaSetDevice(c->device));
    LCU_CHECK_CUDA(cudaMalloc(&p, n * page_bytes));
    int rc = lcu_kv_pool_attach(c, p, n * page_bytes);
    if (rc) {
        cudaFree(p);
        return rc;
    }
    c->own_pool = true;
    return LCU_OK;
}

int lcu_kv_page_tokens(const lcu_ctx *c) { return c ? c->geom.page_tokens : 0; }
size_t lcu_kv_page_bytes(const lcu_ctx *c) { return c ? c->geom.page_elems * 2 : 0; }
int lcu_kv_pages_total(const lcu_ctx *c) { return c ? c->n_pages : 0; }
int lcu_kv_pages_free(const lcu_ctx *c) { return c ? (int)c->free_pages.size() : 0; }

int lcu_seq_create(lcu_ctx *c, int *seq_out) {
    LCU_REQUIRE(c && seq_out, "seq_create: null argument");
    for (size_t i = 0; i < c->seqs.size(); ++i)
        if (!c->seqs[i].used) {
            c->seqs[i].used = true;
            c->seqs[i].len = 0;
            c->seqs[i].pages.clear();
            *seq_out = (int)i;
            return LCU_OK;
        }
    set_error("seq_create: all %zu sequence slots are in use", c->seqs.size());
    return LCU_ERR_STATE;
}

int lcu_seq_resize(lcu_ctx *c, int seq, uint32_t len) {
    LCU_REQUIRE(c && seq >= 0 && seq < (int)c->seqs.size() && c->seqs[seq].used, "seq_resize: bad sequence %d", seq);
    if (len > (uint32_t)c->desc.nctx) {
        set_error("seq_resize: %u tokens exceed the context length %d", len, c->desc.nctx);
        return LCU_ERR_OVERFLOW;
    }
    if (!c->pool) {
        set_error("seq_resize: no KV pool");
        return LCU_ERR_STATE;
    }
    SeqState &s = c->seqs[seq];
    size_t target = ((size_t)len + c->geom.page_tokens - 1) / c->geom.page_tokens;
    if (target > s.pages.size() && target - s.pages.size() > c->free_pages.size()) {
        set_error("seq_resize: %zu pages needed, %zu free", target - s.pages.size(), c->free_pages.size());
        return LCU_ERR_NO_PAGES;
    }
    while (s.pages.size() < target) {  // grow
        s.pages.push_back(c->free_pages.back());
        c->free_pages.pop_back();
    }
    while (s.pages.size() > target) {  // shrink, as KVCache::update does on a rollback
        c->free_pages.push_back(s.pages.back());
        s.pages.pop_back();
    }
    s.len = len;
    return LCU_OK;
}

int lcu_seq_len(const lcu_ctx *c, int seq) {
    if (!c || seq < 0 || seq >= (int)c->seqs.size() || !c->seqs[seq].used) return -1;
    return (int)c->seqs[seq].len;
}

int lcu_seq_free(lcu_ctx *c, int seq) {
    LCU_REQUIRE(c && seq >= 0 && seq < (int)c->seqs.size() && c->seqs[seq].used, "seq_free: bad sequence %d", seq);
    SeqState &s = c->seqs[seq];
    for (int p : s.pages) c->free_pages.push_back(p);
    s.pages.clear();
    s.len = 0;
    s.used = false;
    return LCU_OK;
}

int lcu_set_cuda_graph(lcu_ctx *c, int enabled) {
    LCU_REQUIRE(c, "set_cuda_graph: null context");
    c->use_graph = enabled != 0;
    return LCU_OK;
}
int lcu_set_tuning(lcu_ctx *c, const char *key, long long value) {
    LCU_REQUIRE(key, "set_tuning: null key");
    Tuning &t = tuning();
    const std::string k(key);
    if (k == "pdl_edges") t.pdl_edges = (int)value;
    else if (k == "gemv_ctas_per_sm") { LCU_REQUIRE(value >= 1 && value <= 2, "set_tuning: gemv_ctas_per_sm = %lld (1, 2)", value); t.gemv_ctas_per_sm = (int)value; }
    else if (k == "q8_rows") { LCU_REQUIRE(value == 1 || value == 2 || value == 4, "set_tuning: q8_rows = %lld (1, 2, 4)", value); t.q8_rows = (int)value; }
    else if (k == "gemv_lean_norm") t.gemv_lean_norm = value != 0;
    else if (k == "rms_pdl") t.rms_pdl = value != 0;
    else if (k == "tc") t.tc = value != 0;
    else if (k == "tc_block") { LCU_REQUIRE(value == 64 || value == 128 || value == 256, "set_tuning: tc_block = %lld (64, 128, 256)", value); t.tc_block = (int)value; }
    else if (k == "tc_cluster") { LCU_REQUIRE(value >= 0 && value <= 2, "set_tuning: tc_cluster = %lld (0..2)", value); t.tc_cluster = (int)value; }
    else if (k == "p2p_scatter_ranks") t.p2p_scatter_ranks = (int)value;
    else if (k == "p2p_scatter_min") t.p2p_scatter_min = (long)value;
    else {
        set_error("set_tuning: unknown key '%s'", key);
        return LCU_ERR_INVALID;
    }
    if (c) drop_graphs(c);  // captured rounds hold the old choice
    return LCU_OK;
}
int lcu_set_head_sharding(lcu_ctx *c, int enabled) {
    LCU_REQUIRE(c, "set_head_sharding: null context");
    if (c->head_shard != (enabled != 0)) drop_graphs(c);
    c->head_shard = enabled != 0;
    return LCU_OK;
}
int lcu_set_wait_limit_us(lcu_ctx *c, long long us) {
    LCU_REQUIRE(c, "set_wait_limit_us: null context");
    LCU_CHECK_CUDA(cudaSetDevice(c->device));
    return p2p_set_wait_limit_us(us);
}
int lcu_reset_status(lcu_ctx *c) {
    LCU_REQUIRE(c, "reset_status: null context");
    LCU_CHECK_CUDA(cudaSetDevice(c->device));
    LCU_CHECK_CUDA(cudaDeviceSynchronize());
    LCU_CHECK_CUDA(cudaMemset(c->dev_status, 0, 4));
    c->sticky_status = 0;
    return LCU_OK;
}
int lcu_last_launch_count(const lcu_ctx *c) { return c ? c->last_launches : 0; }
double lcu_last_step_bytes(const lcu_ctx *c) { return c ? c->last_bytes : 0.0; }
const void *lcu_logits(const lcu_ctx *c) { return c ? c->logits : nullptr; }
const void *lcu_hidden(const lcu_ctx *c) { return c ? c->x : nullptr; }

int lcu_device_status(lcu_ctx *c, lcu_stream_t stream, uint32_t *status_out) {
    LCU_REQUIRE(c && status_out, "device_status: null argument");
    LCU_CHECK_CUDA(cudaMemcpyAsync(status_out, c->dev_status, 4, cudaMemcpyDeviceToHost, as_stream(stream)));
    LCU_CHECK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    c->sticky_status = *status_out;
    return LCU_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ the round

namespace {

struct Round {
    int n_tok, n_req, n_fast;
    int n_groups;  // token groups for the prefill form of attention (0: decode form)
    bool any_sampling;
    bool decode_only;  // one new token per sequence
    DescLayout L;
};

// Enqueues every kernel of one round on `s`; returns the number of launches through *count.
int enqueue_round(lcu_ctx *c, const Round &r, lcu_kv_pair *out_dev, cudaStream_t s, int *count) {
    const lcu_model_desc &d = c->desc;
    const int dt = c->dt;
    // Programmatic dependent launch, edge by edge (bit 0: QKV -> attention, 1: attention -> O, 2: O -> gate|up,
    // 3: gate|up -> down, 4: down -> next QKV, 5: last down -> LM head): the successor is launched with the attribute
    // and the predecessor releases it as soon as all its CTAs are running.  Putting the attribute on EVERY launch
    // measured slower than plain graph edges (3.8 ms against 3.3 ms per 8B step) and is not offered.
    const bool pdl = false;
    const int pdl_trigger = 2;     // a kernel without a dependent edge releases nothing before it exits
    const int pdl_edges_env = tuning().pdl_edges;
    const int early_prefetch = 1;  // GEMV request order: activations, then weights (weights first when launched early)
    int launches = 0;
    unsigned char *D = c->desc_dev;
    uint32_t *tokens = reinterpret_cast<uint32_t *>(D + r.L.tokens);
    const uint32_t *pos = reinterpret_cast<const uint32_t *>(D + r.L.pos);
    const int32_t *tok_req = reinterpret_cast<const int32_t *>(D + r.L.tok_req);
    const uint32_t *out_idx = reinterpret_cast<const uint32_t *>(D + r.L.out_idx);
    const uint32_t *fast_map = reinterpret_cast<const uint32_t *>(D + r.L.fast_map);
    const lcu_sample_args *args = reinterpret_cast<const lcu_sample_args *>(D + r.L.args);
    const float *randoms = reinterpret_cast<const float *>(D + r.L.randoms);
    const int32_t *page_table = reinterpret_cast<const int32_t *>(D + r.L.page_table);
    const bool q8 = d.weight_dtype == LCU_Q8_0;
    int rc;

    // token feedback, then the embedding gather
    if (r.n_fast > 0) {
        // the sampled ids live on the lead rank only: it patches the token buffer and, under
        // tensor parallelism, broadcasts it (FastEmbedding then share_inputs, exec/engine.rs:258-274)
        if (c->tp_rank == 0) {
            rc = op_fast_embedding(tokens, c->pre_pairs, fast_map, r.n_fast, s, false);
            if (rc) return rc;
            ++launches;
        }
        if (c->tp_size > 1) {
            rc = c->p2p.ready ? p2p_broadcast_launch(c->p2p, tokens, (size_t)r.n_tok * 4, 0, c->dev_status, s)
                              : comm_broadcast(c->comm, tokens, (size_t)r.n_tok * 4, 0, s);
            if (rc) return rc;
            ++launches;
        }
    }
    rc = op_embedding(c->x, c->embd, tokens, r.n_tok, (size_t)d.d * 2, s, r.n_fast > 0);
    if (rc) return rc;
    ++launches;

    auto w_scales = [&](const void *w, size_t rows, size_t cols) -> const void * {
        return q8 ? reinterpret_cast<const unsigned char *>(w) + rows * cols : nullptr;
    };
    const size_t eb = 2;
    auto row = [&](void *base, size_t stride_elems, int t) -> void * {
        return reinterpret_cast<unsigned char *>(base) + (size_t)t * stride_elems * eb;
    };

    int n_splits, attn_tps;
    attn_plan(c, r.n_tok, &n_splits, &attn_tps);
    const bool batched = c->batched_ok && r.n_tok >= batched_min_tokens();
    // GEMV rounds: the three GEMV -> GEMV edges (the edges around attention lose there); batched rounds: also attention -> O
    const int pdl_edges = pdl_edges_env >= 0 ? pdl_edges_env : (batched ? 30 : 28);
    gemm_skinny_set_scratch(c->sk_ws, c->sk_ws_bytes, c->sk_tickets, 4096);
    gemm_tc_set_scratch(c->sk_ws, c->sk_ws_bytes, c->sk_tickets, 4096, c->dev_status);
    const bool tc_on = tuning().tc != 0;
    const int norm_dt = d.norm_dtype;
    // One linear layer over `n` rows: token groups of <= 4 through the GEMV (RMSNorm fused as its
    // prologue), or blocks of <= 64 through the tensor-core kernel (activations normalised before).
    const bool p2p = c->tp_size > 1 && c->p2p.ready;
    // large rounds reduce-scatter + all-gather through the column owners instead of pushing everything to everyone:
    // 2 (n - 1) / n of the message per rank instead of (n - 1), for one more hop.  Measured on the 70B shape with 64
    // tokens per round (1 MiB messages): 17.5 ms per step against 16.9 ms for the push form on 4 ranks, 12.5 against
    // 15.0 ms on 8 — so from 8 ranks on (tuning: p2p_scatter_ranks) for rounds of 128 KB and more (p2p_scatter_min).
    const long scatter_min = tuning().p2p_scatter_min;
    const int scatter_ranks = tuning().p2p_scatter_ranks;
    const int scatter_cols = (p2p && c->tp_size >= scatter_ranks && (long)r.n_tok * d.d * 2 >= scatter_min &&
                              d.d % (c->tp_size * 8) == 0) ? d.d / c->tp_size : 0;
    c->p2p.parity = 0;  // every step holds an even number of all-reduces, so captured graphs agree on it
    const bool reduce_pdl = true;  // the reduction kernel is a programmatic dependent of the producing projection
    int linear_ctas = 0;  // CTAs of the launches of the last `linear` call
    auto linear = [&](GemvArgs proto, int n, const void *xin, int stride_in, void *yout, int stride_out, bool norm,
                      const void *norm_w, bool push = false, int edge_in = -1, int edge_out = -1) -> int {
        const bool pdl_in = pdl || (edge_in >= 0 && ((pdl_edges >> edge_in) & 1));
        const int trig = (edge_out >= 0 && ((pdl_edges >> edge_out) & 1)) ? 0 : pdl_trigger;
        linear_ctas = 0;
        const void *src = xin;
        int src_stride = stride_in;
        if (batched && norm) {
            // launched as a programmatic dependent where the tcgen05 kernels follow (8B batch 32: 4.94 -> 4.85 ms, 70B per-rank
            // step: 8.35 -> 8.23 ms); ahead of the mma.sync kernels of Q8_0 rounds it costs (batch 16: 4.90 -> 5.34 ms)
            const bool rms_pdl = tuning().rms_pdl && tc_on && n > 8 && gemm_tc_supported(proto.in, proto.w_q8);
            int rc2 = op_rms_norm(c->hbuf, d.d, xin, stride_in, norm_w, norm_dt, d.eps, n, d.d, dt, s, pdl || rms_pdl);
            if (rc2) return rc2;
            ++launches;
            src = c->hbuf;
            src_stride = d.d;
        }
        for (int t0 = 0; t0 < n;) {
            int nt;
            // token blocks of up to 256 on the tcgen05 path (a weight tile is then streamed once per 256 tokens), 64 otherwise
            const int blk = (tc_on && gemm_tc_supported(proto.in, proto.w_q8)) ? tuning().tc_block : 64;
            if (batched) nt = n - t0 < blk ? n - t0 : blk;
            else {
                nt = gemv_max_tokens(proto.in);
                if (nt > n - t0) nt = n - t0;
                if (nt == 3) nt = 2;
            }
            GemvArgs a = proto;
            a.x = reinterpret_cast<const unsigned char *>(src) + (size_t)t0 * src_stride * eb;
            a.stride_x = src_stride;
            a.n_tok = nt;
            a.y = reinterpret_cast<unsigned char *>(yout) + (size_t)t0 * stride_out * eb;
            a.stride_y = stride_out;
            if (a.res) { a.res = a.y; a.stride_res = stride_out; }
            if (a.pos) { a.pos += t0; a.tok_seq += t0; }
            if (!batched && norm) { a.prologue = PRO_RMSNORM; a.norm_w = norm_w; a.norm_f32 = norm_dt == LCU_F32; a.eps = d.eps; }
            else a.prologue = PRO_NONE;
            a.pdl_trigger = trig;
            // launched early: the first weights are requested before waiting for the predecessor, then the activations
            a.early_prefetch = (pdl_in && early_prefetch == 1) ? 3 : early_prefetch;
            if (push) p2p_make_push(c->p2p, (size_t)t0 * stride_out * eb, &a.push, scatter_cols);
            // more than 8 tokens: tcgen05 / TMEM kernel; 5..8: mma.sync kernel; up to 4: GEMV
            const bool tc = batched && tc_on && nt > 8 && gemm_tc_supported(a.in, a.w_q8);
            int rc2 = tc ? gemm_tc_launch(a, dt, s, pdl_in) : (batched ? gemm_skinny_launch(a, dt, s, pdl_in) : gemv_launch(a, dt, s, pdl_in));
            if (rc2) return rc2;
            ++launches;
            linear_ctas += g_linear_last_ctas;
            t0 += nt;
        }
        return LCU_OK;
    };
    // sum of every rank's partial of the residual stream: fused peer-memory form, or ncclAllReduce
    // edge_out: the layer edge the producing projection releases its dependents on (the reduction then starts as
    // their programmatic dependent, spinning on the arrival counter while the producers drain)
    auto all_reduce_x = [&](int edge_out) -> int {
        if (c->tp_size == 1) return LCU_OK;
        ++launches;
        if (p2p)
            return p2p_reduce_launch(c->p2p, c->x, r.n_tok, d.d, dt, (unsigned)(c->tp_size * linear_ctas), scatter_cols, c->dev_status, s,
                                     reduce_pdl && (pdl || ((pdl_edges >> edge_out) & 1)));
        return lcu_op_all_reduce(c, c->x, c->x, (size_t)r.n_tok * d.d, dt, reinterpret_cast<lcu_stream_t>(s));
    };
    for (int l = 0; l < d.n_layers; ++l) {
        const LayerWeights &W = c->layers[l];
        // --- RMSNorm + QKV projection + RoPE + KV append
        {
            GemvArgs a{};
            a.w = W.qkv; a.w_q8 = q8; a.w_scales = w_scales(W.qkv, (size_t)c->qd + 2 * c->kvd, d.d);
            a.in = d.d; a.out = c->qd + 2 * c->kvd;
            a.epilogue = EPI_ROPE_KV;
            a.qd = c->qd; a.kvd = c->kvd; a.dh = d.dh; a.pos = pos; a.sin_t = c->sin_t; a.cos_t = c->cos_t;
            a.kv_pool = c->pool; a.geom = c->geom; a.layer = l; a.tok_seq = tok_req; a.page_table = page_table;
            a.pt_stride = c->pt_stride;
            rc = linear(a, r.n_tok, c->x, d.d, c->q, c->qd, true, W.attn_norm, false, 4, 0);
            if (rc) return rc;
        }
        // --- attention over the paged cache
        {
            AttnArgs a{};
            a.q = c->q; a.stride_q = c->qd; a.o = c->att; a.stride_o = c->qd;
            a.n_tok = r.n_tok; a.nh = c->nh_l; a.nkvh = c->nkvh_l; a.dh = d.dh;
            a.kv_pool = c->pool; a.geom = c->geom; a.layer = l; a.tok_seq = tok_req; a.tok_pos = pos;
            a.page_table = page_table; a.pt_stride = c->pt_stride; a.n_splits = n_splits; a.tiles_per_split = attn_tps;
            if (n_splits > 1) attn_bind_scratch(a, c->attn_scratch, c->max_tokens);
            // GEMV rounds: the splits of a (token, KV head) merge through distributed shared memory (one cluster of up
            // to 8 CTAs) instead of scratch + ticket: 2.89 -> 2.83 ms per 8B batch-1 step.  Batched rounds keep the
            // scratch merge (many CTAs without work would sit in cluster barriers: 4.77 -> 5.75 ms at batch 32).
            a.cluster_z = (!batched && n_splits >= 2 && n_splits <= 8) ? n_splits : 0;
            // launched as a programmatic dependent of the QKV projection (edge 0, off by default: it measured no
            // gain, the GEMV's CTAs fill every register file until they leave) a decode round fetches the cached
            // rows of earlier rounds before it waits; its own dependents start once its first tile has landed
            const bool attn_pdl = pdl || (!batched && (pdl_edges & 1));
            a.early_kv = (attn_pdl && r.decode_only) ? 1 : 0;
            a.pdl_trigger = 1;
            // rounds that hold prompts: 64 query rows per CTA share every K/V tile (prefill form)
            if (r.n_groups > 0) rc = attn_prefill_launch(a, D + r.L.groups, r.n_groups, dt, s);
            else rc = attn_launch(a, dt, s, attn_pdl);
            if (rc) return rc;
            ++launches;
        }
        // --- output projection + residual (rank 0 adds the residual under TP)
        {
            GemvArgs a{};
            a.w = W.o; a.w_q8 = q8; a.w_scales = w_scales(W.o, d.d, c->qd);
            a.in = c->qd; a.out = d.d;
            a.epilogue = c->tp_rank == 0 ? EPI_RESIDUAL : EPI_STORE;
            a.res = c->tp_rank == 0 ? c->x : nullptr;
            rc = linear(a, r.n_tok, c->att, c->qd, c->x, d.d, false, nullptr, p2p, 1, 2);
            if (rc) return rc;
        }
        rc = all_reduce_x(2);
        if (rc) return rc;
        // --- RMSNorm + gate|up projection + SwiGLU
        {
            GemvArgs a{};
            a.w = W.gate_up; a.w_q8 = q8; a.w_scales = w_scales(W.gate_up, (size_t)2 * c->di_l, d.d);
            a.in = d.d; a.out = 2 * c->di_l;
            a.epilogue = EPI_SWIGLU; a.di = c->di_l;
            rc = linear(a, r.n_tok, c->x, d.d, c->act, c->di_l, true, W.ffn_norm, false, 2, 3);
            if (rc) return rc;
        }
        // --- down projection + residual
        {
            GemvArgs a{};
            a.w = W.down; a.w_q8 = q8; a.w_scales = w_scales(W.down, d.d, c->di_l);
            a.in = c->di_l; a.out = d.d;
            a.epilogue = c->tp_rank == 0 ? EPI_RESIDUAL : EPI_STORE;
            a.res = c->tp_rank == 0 ? c->x : nullptr;
            rc = linear(a, r.n_tok, c->act, c->di_l, c->x, d.d, false, nullptr, p2p, 3, l + 1 < d.n_layers ? 4 : 5);
            if (rc) return rc;
        }
        rc = all_reduce_x(l + 1 < d.n_layers ? 4 : 5);
        if (rc) return rc;
    }

    // --- head (exec/engine.rs:90,201): gather + RMSNorm + LM head + sampling.  The reference runs it on the lead rank
    // alone; with the peer-memory transport an arg-max round shards it by vocabulary rows instead: every rank streams
    // vocab / tp rows, arg-maxes them, the lead rank keeps the best candidate per row (lowest index among equals).
    const int v_rows = head_rows_per_rank(c);
    const bool head_sharded = p2p && c->head_shard && v_rows > 0 && !r.any_sampling;
    if (c->tp_rank == 0 || head_sharded) {
        const int vocab_l = head_sharded ? v_rows : d.vocab;  // the lead rank's slice is the first rows of its full matrix
        const bool head_batched = c->batched_ok && r.n_req >= batched_min_tokens();
        if (head_batched) {
            // gather the output rows (Embedding reused as a row gather, exec/output_head.rs:75-77), norm, LM head
            rc = op_embedding(c->hbuf, c->x, out_idx, r.n_req, (size_t)d.d * 2, s, pdl);
            if (!rc) rc = op_rms_norm(c->hbuf, d.d, c->hbuf, d.d, c->out_norm, norm_dt, d.eps, r.n_req, d.d, dt, s, pdl);
            if (rc) return rc;
            launches += 2;
            for (int r0 = 0; r0 < r.n_req; r0 += 64) {
                GemvArgs a{};
                a.w = c->lm_head; a.w_q8 = 0;
                a.x = row(c->hbuf, d.d, r0); a.stride_x = d.d; a.n_tok = r.n_req - r0 < 64 ? r.n_req - r0 : 64;
                a.in = d.d; a.out = vocab_l; a.prologue = PRO_NONE; a.epilogue = EPI_STORE;
                a.y = row(c->logits, vocab_l, r0); a.stride_y = vocab_l;
                const bool tc = tc_on && a.n_tok > 8 && gemm_tc_supported(a.in, 0);
                rc = tc ? gemm_tc_launch(a, dt, s, pdl) : gemm_skinny_launch(a, dt, s, pdl);
                if (rc) return rc;
                ++launches;
            }
        }
        for (int r0 = 0; r0 < r.n_req && !head_batched;) {
            int nt = gemv_max_tokens(d.d);
            if (nt > r.n_req - r0) nt = r.n_req - r0;
            if (nt == 3) nt = 2;
            GemvArgs a{};
            a.w = c->lm_head; a.w_q8 = 0;
            a.x = c->x; a.stride_x = d.d; a.x_rows = out_idx + r0; a.n_tok = nt; a.in = d.d; a.out = vocab_l;
            a.prologue = PRO_RMSNORM; a.norm_w = c->out_norm; a.norm_f32 = d.norm_dtype == LCU_F32; a.eps = d.eps;
            a.epilogue = EPI_STORE; a.y = row(c->logits, vocab_l, r0); a.stride_y = vocab_l;
            // after the last layer's reduction (tensor parallelism) or its down projection
            const bool head_pdl = pdl || (((pdl_edges >> 5) & 1) && (c->tp_size == 1 || (p2p && reduce_pdl)));
            a.pdl_trigger = pdl_trigger; a.early_prefetch = (head_pdl && early_prefetch == 1) ? 3 : early_prefetch;
            rc = gemv_launch(a, dt, s, head_pdl);
            if (rc) return rc;
            ++launches;
            r0 += nt;
        }
        lcu_kv_pair *pairs_out = head_sharded ? c->head_local : out_dev;
        rc = sample_rows(pairs_out, head_sharded ? nullptr : c->pre_pairs, c->logits, r.n_req, (size_t)vocab_l,
                         r.any_sampling ? args : nullptr, randoms, dt, c->sample_ws, c->sample_ws_bytes, s, pdl, r.any_sampling);
        if (rc) return rc;
        launches += r.any_sampling ? 3 : 2;
        if (head_sharded) {
            rc = c->tp_rank == 0 ? p2p_head_pick_launch(c->p2p, c->head_local, r.n_req, dt, out_dev, c->pre_pairs, c->dev_status, s)
                                 : p2p_head_push_launch(c->p2p, c->head_local, r.n_req, (uint32_t)(c->tp_rank * v_rows), s);
            if (rc) return rc;
            ++launches;
        }
    }
    *count = launches;
    return LCU_OK;
}

}  // namespace

// ------------------------------------------------------------------ tensor parallelism over peer memory

extern "C" int lcu_p2p_create(lcu_ctx *c, void *handle64_out) {
    LCU_REQUIRE(c && handle64_out, "p2p_create: null argument");
    LCU_REQUIRE(c->tp_size > 1 && c->tp_size <= P2P_MAX_RANKS, "p2p_create: tp_size = %d (2..%d)", c->tp_size, P2P_MAX_RANKS);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    LCU_CHECK_CUDA(cudaSetDevice(c->device));
    drop_graphs(c);
    p2p_release(c);
    P2pState &st = c->p2p;
    st.rank = c->tp_rank;
    st.n = c->tp_size;
    st.slot_bytes = ((size_t)c->max_tokens * c->desc.d * 2 + 255) / 256 * 256;
    const size_t bcast = (((size_t)c->max_tokens * 4 + 15) / 16) * 16;
    const size_t cand = (size_t)P2P_MAX_RANKS * c->max_seqs * sizeof(lcu_kv_pair);
    st.hdr_bytes = p2p_header_bytes(bcast, cand);
    st.cand_off = 256 + bcast;
    st.max_seqs = c->max_seqs;
    const size_t bytes = p2p_region_bytes(st.n, st.slot_bytes, bcast, cand);
    LCU_CHECK_CUDA(cudaMalloc(&st.own, bytes));
    LCU_CHECK_CUDA(cudaMemset(st.own, 0, bytes));
    LCU_CHECK_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    LCU_CHECK_CUDA(cudaIpcGetMemHandle(&h, st.own));
    memcpy(handle64_out, &h, 64);
    return LCU_OK;
}

extern "C" int lcu_p2p_attach(lcu_ctx *c, const void *handles) {
    LCU_REQUIRE(c && handles, "p2p_attach: null argument");
    P2pState &st = c->p2p;
    LCU_REQUIRE(st.own && !st.ready, "p2p_attach: call lcu_p2p_create first (once)");
    LCU_CHECK_CUDA(cudaSetDevice(c->device));
    for (int r = 0; r < st.n; ++r) {
        if (r == st.rank) {
            st.base[r] = st.own;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, reinterpret_cast<const unsigned char *>(handles) + (size_t)r * 64, 64);
        LCU_CHECK_CUDA(cudaIpcOpenMemHandle(&st.base[r], h, cudaIpcMemLazyEnablePeerAccess));
    }
    drop_graphs(c);
    st.ready = true;
    return LCU_OK;
}

extern "C" int lcu_p2p_enabled(const lcu_ctx *c) { return c && c->p2p.ready ? 1 : 0; }

extern "C" int lcu_step(lcu_ctx *c, lcu_stream_t stream, int n_req, const lcu_req *reqs, const uint32_t *tokens,
                        const lcu_sample_args *args, const float *randoms, const uint32_t *fast_map, int n_fast,
                        lcu_kv_pair *out_dev) {
    LCU_REQUIRE(c && reqs && tokens, "step: null argument");
    LCU_REQUIRE(n_req >= 1 && n_req <= c->max_seqs, "step: %d requests (1..%d)", n_req, c->max_seqs);
    LCU_REQUIRE(c->tp_rank != 0 || out_dev, "step: the lead rank needs an output buffer");
    LCU_REQUIRE(n_fast >= 0 && n_fast <= n_req && (n_fast == 0 || fast_map), "step: bad fast_map");
    const lcu_model_desc &d = c->desc;
    LCU_REQUIRE(d.vocab % 2 == 0, "step: vocab %d must be even", d.vocab);
    if (!c->pool) { set_error("step: no KV pool"); return LCU_ERR_STATE; }
    const bool head_everywhere = c->p2p.ready && c->head_shard && head_rows_per_rank(c) > 0;
    if (!c->embd || ((c->tp_rank == 0 || head_everywhere) && (!c->out_norm || !c->lm_head))) { set_error("step: embedding / output weights missing"); return LCU_ERR_STATE; }
    if (c->sticky_status & (4u | 16u | 32u)) {
        set_error("step: a bounded device-side wait ran out earlier (status %u); the group is broken until lcu_reset_status", c->sticky_status);
        return LCU_ERR_TIMEOUT;
    }
    for (int l = 0; l < d.n_layers; ++l) {
        const LayerWeights &W = c->layers[l];
        if (!W.attn_norm || !W.qkv || !W.o || !W.ffn_norm || !W.gate_up || !W.down) {
            set_error("step: weights of layer %d missing", l);
            return LCU_ERR_STATE;
        }
    }
    LCU_CHECK_CUDA(cudaSetDevice(c->device));
    int rc = ensure_tables(c);
    if (rc) return rc;

    // validate, then back every sequence with pages (KVCache::update, exec/group.rs:134-144)
    int n_tok = 0;
    bool decode_only = true, any_sampling = false;
    for (int i = 0; i < n_req; ++i) {
        const lcu_req &q = reqs[i];
        LCU_REQUIRE(q.seq >= 0 && q.seq < (int)c->seqs.size() && c->seqs[q.seq].used, "step: request %d names sequence %d", i, q.seq);
        LCU_REQUIRE(q.len >= 1, "step: request %d has no tokens", i);
        for (int j = 0; j < i; ++j) LCU_REQUIRE(reqs[j].seq != q.seq, "step: sequence %d appears twice", q.seq);
        if ((uint64_t)q.pos + q.len > (uint64_t)d.nctx) {
            set_error("step: request %d overflows the context (%u + %u > %d)", i, q.pos, q.len, d.nctx);
            return LCU_ERR_OVERFLOW;
        }
        if (q.len != 1) decode_only = false;
        n_tok += (int)q.len;
        if (args && !(args[i].temperature == 0.f || args[i].top_k == 1)) {
            LCU_REQUIRE(args[i].temperature > 0.f && args[i].top_p > 0.f && args[i].top_k >= 1, "step: bad sample args for request %d", i);
            LCU_REQUIRE(randoms, "step: sampling requests need random numbers");
            any_sampling = true;
        }
    }
    LCU_REQUIRE(n_tok <= c->max_tokens, "step: %d tokens exceed max_tokens %d", n_tok, c->max_tokens);
    for (int i = 0; i < n_fast; ++i)
        LCU_REQUIRE(fast_map[2 * i] < (uint32_t)c->max_tokens && fast_map[2 * i + 1] < (uint32_t)n_tok, "step: fast_map entry %d out of range", i);
    size_t pages_needed = 0;
    for (int i = 0; i < n_req; ++i) {
        size_t target = ((size_t)reqs[i].pos + reqs[i].len + c->geom.page_tokens - 1) / c->geom.page_tokens;
        size_t have = c->seqs[reqs[i].seq].pages.size();
        if (target > have) pages_needed += target - have;
    }
    if (pages_needed > c->free_pages.size()) {
        set_error("step: %zu KV pages needed, %zu free", pages_needed, c->free_pages.size());
        return LCU_ERR_NO_PAGES;
    }
    for (int i = 0; i < n_req; ++i) {
        rc = lcu_seq_resize(c, reqs[i].seq, reqs[i].pos + reqs[i].len);
        if (rc) return rc;
    }

    // stage the round descriptor in the next pinned buffer (BufN, exec/engine.rs:373-429)
    Round r;
    r.n_tok = n_tok; r.n_req = n_req; r.n_fast = n_fast; r.any_sampling = any_sampling; r.decode_only = decode_only;
    r.L = desc_layout(n_tok, n_req, c->pt_stride);
    cudaStream_t s = as_stream(stream);
    int slot = c->ring_idx;
    c->ring_idx = (c->ring_idx + 1) % lcu_ctx::RING;
    if (c->desc_used[slot]) LCU_CHECK_CUDA(cudaEventSynchronize(c->desc_event[slot]));
    unsigned char *H = c->desc_host[slot];
    memset(H, 0, r.L.total);
    memcpy(H + r.L.tokens, tokens, (size_t)n_tok * 4);
    {
        uint32_t *hp = reinterpret_cast<uint32_t *>(H + r.L.pos);
        int32_t *hr = reinterpret_cast<int32_t *>(H + r.L.tok_req);
        uint32_t *ho = reinterpret_cast<uint32_t *>(H + r.L.out_idx);
        int32_t *ht = reinterpret_cast<int32_t *>(H + r.L.page_table);
        int t = 0;
        for (int i = 0; i < n_req; ++i) {
            for (uint32_t j = 0; j < reqs[i].len; ++j, ++t) {  // pos(), exec/engine.rs:352-358
                hp[t] = reqs[i].pos + j;
                hr[t] = i;
            }
            ho[i] = (uint32_t)(t - 1);  // out_idx() with out == 1, exec/engine.rs:360-371
            const SeqState &sq = c->seqs[reqs[i].seq];
            for (size_t pg = 0; pg < sq.pages.size(); ++pg) ht[(size_t)i * c->pt_stride + pg] = sq.pages[pg];
        }
        // prompts in the round: consecutive tokens of a request are grouped for the prefill form of attention
        r.n_groups = 0;
        if (!decode_only && attn_prefill_supported(c->pt_stride)) {
            int32_t *hg = reinterpret_cast<int32_t *>(H + r.L.groups);
            const int gt = attn_prefill_group_tokens(c->nh_l, c->nkvh_l);
            int t0 = 0;
            for (int i = 0; i < n_req; ++i) {
                for (uint32_t j = 0; j < reqs[i].len; j += gt) {
                    hg[2 * r.n_groups] = t0 + (int)j;
                    hg[2 * r.n_groups + 1] = (int)(reqs[i].len - j < (uint32_t)gt ? reqs[i].len - j : gt);
                    ++r.n_groups;
                }
                t0 += (int)reqs[i].len;
            }
        }
        if (n_fast) memcpy(H + r.L.fast_map, fast_map, (size_t)n_fast * 8);
        lcu_sample_args *ha = reinterpret_cast<lcu_sample_args *>(H + r.L.args);
        for (int i = 0; i < n_req; ++i) {
            if (args) ha[i] = args[i];
            else { ha[i].temperature = 0.f; ha[i].top_p = 1.f; ha[i].top_k = ~0ull; }
        }
        if (randoms) memcpy(H + r.L.randoms, randoms, (size_t)n_req * 4);
    }
    LCU_CHECK_CUDA(cudaMemcpyAsync(c->desc_dev, H, r.L.total, cudaMemcpyHostToDevice, s));
    LCU_CHECK_CUDA(cudaEventRecord(c->desc_event[slot], s));
    c->desc_used[slot] = true;

    // algorithmic bytes of the round: every linear weight once, the LM head, the cached K/V
    {
        double wb = d.weight_dtype == LCU_Q8_0 ? 34.0 / 32.0 : 2.0;
        double per_layer = ((double)(c->qd + 2 * c->kvd) * d.d + (double)d.d * c->qd + 2.0 * c->di_l * d.d + (double)d.d * c->di_l) * wb;
        const bool sharded = head_everywhere && !any_sampling;
        double bytes = per_layer * d.n_layers + (sharded ? (double)head_rows_per_rank(c) * d.d * 2.0
                                                         : (c->tp_rank == 0 ? (double)d.vocab * d.d * 2.0 : 0.0));
        for (int i = 0; i < n_req; ++i)
            for (uint32_t j = 0; j < reqs[i].len; ++j)
                bytes += (double)(reqs[i].pos + j + 1) * 2.0 * c->kvd * d.n_layers * 2.0;
        c->last_bytes = bytes;
    }
    c->last_n_tok = n_tok;
    c->last_n_req = n_req;

    // decode rounds replay a captured graph; everything else (and stream 0) runs eagerly.
    // NCCL collectives are captured like any other node (exec/step.rs:82-86).
    bool graph_ok = c->use_graph && decode_only && s != nullptr;
    if (!graph_ok) {
        int count = 0;
        rc = enqueue_round(c, r, out_dev, s, &count);
        c->last_launches = count;
        return rc;
    }
    std::vector<int> key = {n_req, n_tok, n_fast, any_sampling ? 1 : 0, (int)((uintptr_t)out_dev & 0x7fffffff),
                            (int)((uintptr_t)out_dev >> 31), c->head_shard ? 1 : 0};
    auto it = c->graphs.find(key);
    if (it == c->graphs.end()) {
        // A captured round is keyed by its shape AND by the output buffer (a host that rotates output buffers, as the
        // reference's triple-buffered loop does, holds one graph per buffer): keep the table bounded
        if (c->graphs.size() >= 96) drop_graphs(c);
        cudaGraph_t graph = nullptr;
        LCU_CHECK_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        int count = 0;
        rc = enqueue_round(c, r, out_dev, s, &count);
        cudaError_t e = cudaStreamEndCapture(s, &graph);
        if (rc) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
        StepGraph g;
        e = cudaGraphInstantiate(&g.exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
        g.launches = count;
        it = c->graphs.emplace(key, g).first;
    }
    LCU_CHECK_CUDA(cudaGraphLaunch(it->second.exec, s));
    c->last_launches = it->second.launches;
    return LCU_OK;
}

namespace lcu {
struct CtxShape {
    int d, nh, nkvh, dh, di, vocab, tp_rank, tp_size, act_dtype, weight_dtype, norm_dtype;
    void *comm;
};
// the few context fields the operator wrappers in api.cu need
CtxShape ctx_shape(const lcu_ctx *c) {
    const lcu_model_desc &d = c->desc;
    return CtxShape{d.d, d.nh, d.nkvh, d.dh, d.di, d.vocab, c->tp_rank, c->tp_size, d.act_dtype, d.weight_dtype,
                    d.norm_dtype, c->comm};
}
}  // namespace lcu
