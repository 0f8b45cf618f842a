// GGUF model files -> model description and device weights of a context.  The C++ counterpart of the
// reference's load path: `GGufModel::read` / `merge` (llama.cu/src/model/gguf.rs:16-72: every shard is mapped and
// parsed, metadata and tensors are merged, `general.alignment` and `split.*` keys are dropped), the metadata ->
// shape mapping of `GGufModel::llama` (model/mod.rs:61-182: fused `attn_qkv` and `ffn_gate_up` tensors, `output.weight`
// falling back to `token_embd.weight`) and the upload with tensor-parallel slicing of `load_weight`
// (load/mod.rs:23-108, load/loader.rs: pinned slabs, one device region for all weights).
// Differences, on purpose: Q8_0 linear weights are accepted and repacked into the plane layout at load time (the
// reference cannot run quantised weights, op/linear.rs:92-97); bf16 is accepted; a metadata key that repeats in
// another shard WITH THE SAME VALUE is tolerated (the reference rejects any repeat).
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/lcu.h"

namespace lcu {
void set_error(const char *fmt, ...);
}

namespace {

enum GType { T_U8 = 0, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 };
// ggml tensor types this loader understands
enum { GGML_F32 = 0, GGML_F16 = 1, GGML_Q8_0 = 8, GGML_BF16 = 30 };

struct Meta {
    uint32_t type = 0;
    const unsigned char *value = nullptr;  // first byte of the value inside the mapping
    size_t bytes = 0;                      // length of the value's encoding
    uint32_t arr_type = 0;
    uint64_t arr_len = 0;
};
struct TensorInfo {
    std::string name;
    uint32_t ggml_type = 0;
    int n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};  // ggml order: dims[0] is the innermost (contiguous) extent
    const unsigned char *data = nullptr;
    size_t bytes = 0;
};
struct Mapping {
    void *base = nullptr;
    size_t len = 0;
};

size_t scalar_size(uint32_t t) {
    switch (t) {
    case T_U8: case T_I8: case T_BOOL: return 1;
    case T_U16: case T_I16: return 2;
    case T_U32: case T_I32: case T_F32: return 4;
    case T_U64: case T_I64: case T_F64: return 8;
    default: return 0;
    }
}

size_t tensor_bytes(uint32_t ggml_type, uint64_t elems) {
    switch (ggml_type) {
    case GGML_F32: return elems * 4;
    case GGML_F16: case GGML_BF16: return elems * 2;
    case GGML_Q8_0: return elems / 32 * 34;
    default: return 0;
    }
}

struct Reader {
    const unsigned char *p, *end;
    bool ok = true;
    template <class T> T get() {
        T v{};
        if ((size_t)(end - p) < sizeof(T)) { ok = false; return v; }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        uint64_t n = get<uint64_t>();
        if (!ok || (uint64_t)(end - p) < n) { ok = false; return std::string(); }
        std::string s(reinterpret_cast<const char *>(p), (size_t)n);
        p += n;
        return s;
    }
    // skips one value of type t; returns false on a malformed file
    bool skip(uint32_t t) {
        if (t == T_STR) { str(); return ok; }
        if (t == T_ARR) {
            uint32_t et = get<uint32_t>();
            uint64_t n = get<uint64_t>();
            if (!ok || et == T_ARR) return ok = false;
            if (et == T_STR) {
                for (uint64_t i = 0; i < n && ok; ++i) str();
                return ok;
            }
            size_t sz = scalar_size(et);
            if (!sz || (uint64_t)(end - p) / sz < n) return ok = false;
            p += n * sz;
            return true;
        }
        size_t sz = scalar_size(t);
        if (!sz || (size_t)(end - p) < sz) return ok = false;
        p += sz;
        return true;
    }
};

}  // namespace

struct lcu_gguf {
    std::vector<Mapping> maps;
    std::map<std::string, Meta> meta;
    std::map<std::string, TensorInfo> tensors;
    std::vector<std::string> order;  // tensor names in file order
    void *dev_weights = nullptr;     // the one device region lcu_gguf_load fills
    int device = -1;
};

#define GG_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) {                   \
            lcu::set_error(__VA_ARGS__); \
            return LCU_ERR_INVALID;      \
        }                                \
    } while (0)

namespace {

int parse_shard(lcu_gguf *g, const Mapping &m, const char *path) {
    Reader r{reinterpret_cast<const unsigned char *>(m.base), reinterpret_cast<const unsigned char *>(m.base) + m.len};
    const uint32_t magic = r.get<uint32_t>(), version = r.get<uint32_t>();
    GG_REQUIRE(r.ok && magic == 0x46554747u, "gguf: %s is not a GGUF file", path);
    GG_REQUIRE(version == 2 || version == 3, "gguf: %s has version %u (2 and 3 are supported)", path, version);
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    uint64_t alignment = 32;
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = r.str();
        Meta kv;
        kv.type = r.get<uint32_t>();
        kv.value = r.p;
        if (kv.type == T_ARR && (size_t)(r.end - r.p) >= 12) {
            memcpy(&kv.arr_type, r.p, 4);
            memcpy(&kv.arr_len, r.p + 4, 8);
        }
        GG_REQUIRE(r.skip(kv.type), "gguf: %s: malformed metadata value of key %zu", path, (size_t)i);
        kv.bytes = (size_t)(r.p - kv.value);
        if (key == "general.alignment") {  // per file, not merged (gguf.rs:41-43)
            if (kv.type == T_U32) { uint32_t a; memcpy(&a, kv.value, 4); alignment = a; }
            continue;
        }
        if (key.rfind("split.", 0) == 0) continue;
        auto it = g->meta.find(key);
        if (it != g->meta.end()) {
            GG_REQUIRE(it->second.type == kv.type && it->second.bytes == kv.bytes && !memcmp(it->second.value, kv.value, kv.bytes),
                       "gguf: metadata key '%s' repeats with another value in %s", key.c_str(), path);
            continue;
        }
        g->meta[key] = kv;
    }
    GG_REQUIRE(alignment > 0 && (alignment & (alignment - 1)) == 0, "gguf: %s: alignment %llu", path, (unsigned long long)alignment);
    std::vector<std::pair<std::string, uint64_t>> offsets;
    for (uint64_t i = 0; i < n_tensors; ++i) {
        TensorInfo t;
        t.name = r.str();
        t.n_dims = (int)r.get<uint32_t>();
        GG_REQUIRE(r.ok && t.n_dims >= 1 && t.n_dims <= 4, "gguf: %s: tensor %zu has %d dimensions", path, (size_t)i, t.n_dims);
        uint64_t elems = 1;
        for (int d = 0; d < t.n_dims; ++d) {
            t.dims[d] = r.get<uint64_t>();
            elems *= t.dims[d];
        }
        t.ggml_type = r.get<uint32_t>();
        const uint64_t off = r.get<uint64_t>();
        GG_REQUIRE(r.ok, "gguf: %s: truncated tensor table", path);
        t.bytes = tensor_bytes(t.ggml_type, elems);
        GG_REQUIRE(t.bytes > 0, "gguf: tensor '%s' has ggml type %u (F32, F16, BF16 and Q8_0 are supported)", t.name.c_str(), t.ggml_type);
        GG_REQUIRE(t.ggml_type != GGML_Q8_0 || t.dims[0] % 32 == 0, "gguf: Q8_0 tensor '%s' has rows of %llu", t.name.c_str(),
                   (unsigned long long)t.dims[0]);
        GG_REQUIRE(!g->tensors.count(t.name), "gguf: tensor '%s' appears twice (%s)", t.name.c_str(), path);
        g->tensors[t.name] = t;
        g->order.push_back(t.name);
        offsets.emplace_back(t.name, off);
    }
    const size_t header = (size_t)(r.p - reinterpret_cast<const unsigned char *>(m.base));
    const size_t data0 = (header + alignment - 1) / alignment * alignment;
    for (auto &o : offsets) {
        TensorInfo &t = g->tensors[o.first];
        GG_REQUIRE(data0 + o.second + t.bytes <= m.len, "gguf: tensor '%s' reaches past the end of %s", t.name.c_str(), path);
        t.data = reinterpret_cast<const unsigned char *>(m.base) + data0 + o.second;
    }
    return LCU_OK;
}

bool meta_u64(const lcu_gguf *g, const std::string &key, uint64_t *out) {
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return false;
    const Meta &m = it->second;
    switch (m.type) {
    case T_U8: { uint8_t v; memcpy(&v, m.value, 1); *out = v; return true; }
    case T_U16: { uint16_t v; memcpy(&v, m.value, 2); *out = v; return true; }
    case T_U32: { uint32_t v; memcpy(&v, m.value, 4); *out = v; return true; }
    case T_U64: { uint64_t v; memcpy(&v, m.value, 8); *out = v; return true; }
    case T_I32: { int32_t v; memcpy(&v, m.value, 4); *out = (uint64_t)v; return v >= 0; }
    case T_I64: { int64_t v; memcpy(&v, m.value, 8); *out = (uint64_t)v; return v >= 0; }
    default: return false;
    }
}
bool meta_f32(const lcu_gguf *g, const std::string &key, float *out) {
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return false;
    if (it->second.type == T_F32) { memcpy(out, it->second.value, 4); return true; }
    if (it->second.type == T_F64) { double v; memcpy(&v, it->second.value, 8); *out = (float)v; return true; }
    return false;
}
std::string meta_str(const lcu_gguf *g, const std::string &key) {
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != T_STR) return std::string();
    uint64_t n;
    memcpy(&n, it->second.value, 8);
    return std::string(reinterpret_cast<const char *>(it->second.value + 8), (size_t)n);
}

int dtype_of(uint32_t ggml_type) {
    switch (ggml_type) {
    case GGML_F32: return LCU_F32;
    case GGML_F16: return LCU_F16;
    case GGML_BF16: return LCU_BF16;
    case GGML_Q8_0: return LCU_Q8_0;
    default: return -1;
    }
}

const TensorInfo *find(const lcu_gguf *g, const std::string &name) {
    auto it = g->tensors.find(name);
    return it == g->tensors.end() ? nullptr : &it->second;
}

}  // namespace

extern "C" {

// == GGufModel::read: maps and parses every shard, merges them
int lcu_gguf_open(const char *const *paths, int n_paths, lcu_gguf **out) {
    GG_REQUIRE(paths && n_paths >= 1 && out, "gguf_open: bad arguments");
    lcu_gguf *g = new lcu_gguf();
    for (int i = 0; i < n_paths; ++i) {
        int fd = open(paths[i], O_RDONLY);
        struct stat st;
        if (fd < 0 || fstat(fd, &st) != 0 || st.st_size < 24) {
            if (fd >= 0) close(fd);
            lcu::set_error("gguf_open: cannot read %s", paths[i]);
            lcu_gguf_close(g);
            return LCU_ERR_INVALID;
        }
        void *base = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
        close(fd);
        if (base == MAP_FAILED) {
            lcu::set_error("gguf_open: mmap of %s failed", paths[i]);
            lcu_gguf_close(g);
            return LCU_ERR_INVALID;
        }
        g->maps.push_back(Mapping{base, (size_t)st.st_size});
        int rc = parse_shard(g, g->maps.back(), paths[i]);
        if (rc) {
            lcu_gguf_close(g);
            return rc;
        }
    }
    *out = g;
    return LCU_OK;
}

int lcu_gguf_close(lcu_gguf *g) {
    if (!g) return LCU_OK;
    if (g->dev_weights) {
        if (g->device >= 0) cudaSetDevice(g->device);
        cudaFree(g->dev_weights);
    }
    for (Mapping &m : g->maps) munmap(m.base, m.len);
    delete g;
    return LCU_OK;
}

int lcu_gguf_n_tensors(const lcu_gguf *g) { return g ? (int)g->order.size() : 0; }

// name (valid until close), dtype (lcu_dtype), dims in ROW-MAJOR order (outermost first, like the reference's reversed
// shape, gguf.rs:56-61), byte length
int lcu_gguf_tensor_info(const lcu_gguf *g, int index, const char **name, int *dtype, uint64_t dims4[4], int *n_dims,
                         size_t *bytes) {
    GG_REQUIRE(g && index >= 0 && index < (int)g->order.size(), "gguf_tensor_info: index %d", index);
    const TensorInfo &t = g->tensors.at(g->order[index]);
    if (name) *name = t.name.c_str();
    if (dtype) *dtype = dtype_of(t.ggml_type);
    if (n_dims) *n_dims = t.n_dims;
    if (dims4)
        for (int d = 0; d < 4; ++d) dims4[d] = d < t.n_dims ? t.dims[t.n_dims - 1 - d] : 1;
    if (bytes) *bytes = t.bytes;
    return LCU_OK;
}

int lcu_gguf_meta_u64(const lcu_gguf *g, const char *key, uint64_t *out) {
    GG_REQUIRE(g && key && out, "gguf_meta_u64: null argument");
    GG_REQUIRE(meta_u64(g, key, out), "gguf: no unsigned metadata value '%s'", key);
    return LCU_OK;
}
int lcu_gguf_meta_f32(const lcu_gguf *g, const char *key, float *out) {
    GG_REQUIRE(g && key && out, "gguf_meta_f32: null argument");
    GG_REQUIRE(meta_f32(g, key, out), "gguf: no float metadata value '%s'", key);
    return LCU_OK;
}
// copies at most cap - 1 characters; returns the string's length through *len
int lcu_gguf_meta_str(const lcu_gguf *g, const char *key, char *buf, size_t cap, size_t *len) {
    GG_REQUIRE(g && key, "gguf_meta_str: null argument");
    auto it = g->meta.find(key);
    GG_REQUIRE(it != g->meta.end() && it->second.type == T_STR, "gguf: no string metadata value '%s'", key);
    const std::string s = meta_str(g, key);
    if (len) *len = s.size();
    if (buf && cap) {
        size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return LCU_OK;
}

// == the metadata half of GGufModel::llama (model/mod.rs:61-78).  nctx, page_tokens, max_tokens, max_seqs of *desc
// are left to the caller when they are non-zero on entry (nctx: the file's context length otherwise).
int lcu_gguf_model_desc(const lcu_gguf *g, lcu_model_desc *desc) {
    GG_REQUIRE(g && desc, "gguf_model_desc: null argument");
    const std::string arch = meta_str(g, "general.architecture");
    GG_REQUIRE(arch == "llama", "gguf: architecture '%s' (only 'llama' is supported; qwen2 needs the bias path)", arch.c_str());
    uint64_t nblk, d, nh, nkvh, dh, di, nctx;
    GG_REQUIRE(meta_u64(g, arch + ".block_count", &nblk), "gguf: %s.block_count missing", arch.c_str());
    GG_REQUIRE(meta_u64(g, arch + ".embedding_length", &d), "gguf: %s.embedding_length missing", arch.c_str());
    GG_REQUIRE(meta_u64(g, arch + ".attention.head_count", &nh), "gguf: %s.attention.head_count missing", arch.c_str());
    if (!meta_u64(g, arch + ".attention.head_count_kv", &nkvh)) nkvh = nh;
    if (!meta_u64(g, arch + ".rope.dimension_count", &dh)) dh = d / nh;
    GG_REQUIRE(meta_u64(g, arch + ".feed_forward_length", &di), "gguf: %s.feed_forward_length missing", arch.c_str());
    GG_REQUIRE(meta_u64(g, arch + ".context_length", &nctx), "gguf: %s.context_length missing", arch.c_str());
    float eps = 1e-5f, theta = 1e4f;
    meta_f32(g, arch + ".attention.layer_norm_rms_epsilon", &eps);
    meta_f32(g, arch + ".rope.freq_base", &theta);
    const TensorInfo *embd = find(g, "token_embd.weight"), *qkv = find(g, "blk.0.attn_qkv.weight"), *norm = find(g, "output_norm.weight");
    GG_REQUIRE(embd && qkv && norm, "gguf: token_embd.weight, blk.0.attn_qkv.weight (fused q|k|v) or output_norm.weight missing");
    uint64_t nvoc = 0;
    auto tk = g->meta.find("tokenizer.ggml.tokens");
    if (tk != g->meta.end() && tk->second.type == T_ARR) nvoc = tk->second.arr_len;  // meta![tokenizer_ggml_tokens].len()
    if (!nvoc) nvoc = embd->dims[1];
    GG_REQUIRE(embd->dims[0] == d && embd->dims[1] == nvoc, "gguf: token_embd.weight is [%llu, %llu], expected [%llu, %llu]",
               (unsigned long long)embd->dims[1], (unsigned long long)embd->dims[0], (unsigned long long)nvoc, (unsigned long long)d);
    const int act = dtype_of(embd->ggml_type), wdt = dtype_of(qkv->ggml_type), ndt = dtype_of(norm->ggml_type);
    GG_REQUIRE(act == LCU_F16 || act == LCU_BF16, "gguf: token_embd.weight must be F16 or BF16");
    desc->n_layers = (int32_t)nblk; desc->d = (int32_t)d; desc->nh = (int32_t)nh; desc->nkvh = (int32_t)nkvh;
    desc->dh = (int32_t)dh; desc->di = (int32_t)di; desc->vocab = (int32_t)nvoc;
    if (desc->nctx <= 0) desc->nctx = (int32_t)nctx;
    desc->eps = eps; desc->theta = theta;
    desc->act_dtype = act; desc->weight_dtype = wdt; desc->norm_dtype = ndt;
    return LCU_OK;
}

// == load_weight (load/mod.rs:23-108): every weight of `ctx`'s rank goes into ONE device region owned by the handle
// (keep it open while the context is in use), staged through two pinned slabs; linear weights are cut per rank and
// Q8_0 blocks are repacked into planes on the device; each tensor is then registered with lcu_set_weight.
int lcu_gguf_load(lcu_gguf *g, lcu_ctx *ctx, lcu_stream_t stream) {
    GG_REQUIRE(g && ctx, "gguf_load: null argument");
    GG_REQUIRE(!g->dev_weights, "gguf_load: this handle has already loaded a context");
    lcu_model_desc d{};
    int rc = lcu_gguf_model_desc(g, &d);
    if (rc) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    struct Item {
        int layer, kind;
        const TensorInfo *t;
        size_t off, bytes;
    };
    std::vector<Item> items;
    size_t total = 0, largest_src = 0, largest_dst = 0;
    auto add = [&](int layer, int kind, const std::string &name, const std::string &fallback) -> int {
        const TensorInfo *t = find(g, name);
        if (!t && !fallback.empty()) t = find(g, fallback);
        GG_REQUIRE(t, "gguf: tensor '%s' missing", name.c_str());
        const size_t bytes = lcu_weight_bytes(ctx, kind);
        GG_REQUIRE(bytes > 0, "gguf_load: the context has no weight of kind %d", kind);
        const bool lin = kind == LCU_W_QKV || kind == LCU_W_O || kind == LCU_W_GATE_UP || kind == LCU_W_DOWN;
        const int want = (kind == LCU_W_ATTN_NORM || kind == LCU_W_FFN_NORM || kind == LCU_W_OUT_NORM) ? d.norm_dtype
                         : (lin ? d.weight_dtype : d.act_dtype);
        GG_REQUIRE(dtype_of(t->ggml_type) == want, "gguf: '%s' has dtype %d, the model uses %d for this kind", t->name.c_str(),
                   dtype_of(t->ggml_type), want);
        items.push_back(Item{layer, kind, t, total, bytes});
        total += (bytes + 255) / 256 * 256;
        if (t->bytes > largest_src) largest_src = t->bytes;
        if (bytes > largest_dst) largest_dst = bytes;
        return LCU_OK;
    };
    if ((rc = add(0, LCU_W_EMBD, "token_embd.weight", ""))) return rc;
    for (int l = 0; l < d.n_layers; ++l) {
        const std::string b = "blk." + std::to_string(l) + ".";
        if ((rc = add(l, LCU_W_ATTN_NORM, b + "attn_norm.weight", ""))) return rc;
        if ((rc = add(l, LCU_W_QKV, b + "attn_qkv.weight", ""))) return rc;
        if ((rc = add(l, LCU_W_O, b + "attn_output.weight", ""))) return rc;
        if ((rc = add(l, LCU_W_FFN_NORM, b + "ffn_norm.weight", ""))) return rc;
        if ((rc = add(l, LCU_W_GATE_UP, b + "ffn_gate_up.weight", ""))) return rc;
        if ((rc = add(l, LCU_W_DOWN, b + "ffn_down.weight", ""))) return rc;
    }
    if ((rc = add(0, LCU_W_OUT_NORM, "output_norm.weight", ""))) return rc;
    if ((rc = add(0, LCU_W_LM_HEAD, "output.weight", "token_embd.weight"))) return rc;  // tied embeddings (mod.rs:83-87)

    cudaGetDevice(&g->device);
    unsigned char *region = nullptr, *tmp_a = nullptr, *tmp_b = nullptr, *slab[2] = {nullptr, nullptr};
    cudaEvent_t ev[2] = {nullptr, nullptr};
    const size_t SLAB = (size_t)32 << 20;
    auto cleanup = [&](bool keep_region) {
        if (!keep_region) cudaFree(region);
        cudaFree(tmp_a); cudaFree(tmp_b);
        for (int i = 0; i < 2; ++i) { if (slab[i]) cudaFreeHost(slab[i]); if (ev[i]) cudaEventDestroy(ev[i]); }
    };
    auto fail = [&](cudaError_t e, const char *what) {
        lcu::set_error("gguf_load: %s: %s", what, cudaGetErrorString(e));
        cleanup(false);
        return LCU_ERR_CUDA;
    };
    cudaError_t e;
    if ((e = cudaMalloc(reinterpret_cast<void **>(&region), total)) != cudaSuccess) return fail(e, "cudaMalloc(weights)");
    if ((e = cudaMalloc(reinterpret_cast<void **>(&tmp_a), largest_src)) != cudaSuccess) return fail(e, "cudaMalloc(staging)");
    if ((e = cudaMalloc(reinterpret_cast<void **>(&tmp_b), largest_src)) != cudaSuccess) return fail(e, "cudaMalloc(staging)");
    for (int i = 0; i < 2; ++i) {
        if ((e = cudaMallocHost(reinterpret_cast<void **>(&slab[i]), SLAB)) != cudaSuccess) return fail(e, "cudaMallocHost");
        if ((e = cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming)) != cudaSuccess) return fail(e, "cudaEventCreate");
    }
    int which = 0;
    bool used[2] = {false, false};
    for (const Item &it : items) {
        const TensorInfo &t = *it.t;
        // file -> device through the pinned slabs (the copy of chunk i overlaps the host read of chunk i + 1)
        for (size_t off = 0; off < t.bytes; off += SLAB, which ^= 1) {
            const size_t n = t.bytes - off < SLAB ? t.bytes - off : SLAB;
            if (used[which] && (e = cudaEventSynchronize(ev[which])) != cudaSuccess) return fail(e, "cudaEventSynchronize");
            memcpy(slab[which], t.data + off, n);
            if ((e = cudaMemcpyAsync(tmp_a + off, slab[which], n, cudaMemcpyHostToDevice, s)) != cudaSuccess) return fail(e, "H2D");
            cudaEventRecord(ev[which], s);
            used[which] = true;
        }
        const bool linear = it.kind == LCU_W_QKV || it.kind == LCU_W_O || it.kind == LCU_W_GATE_UP || it.kind == LCU_W_DOWN;
        const unsigned char *full = tmp_a;
        if (linear && t.ggml_type == GGML_Q8_0) {  // ggml blocks -> planes (rows = dims[1], columns = dims[0]); same byte count
            if ((rc = lcu_repack_q8_0(tmp_b, tmp_a, t.dims[1], t.dims[0], stream))) { cleanup(false); return rc; }
            full = tmp_b;
        }
        if ((rc = lcu_tp_slice_weight(ctx, it.kind, region + it.off, full, stream))) { cleanup(false); return rc; }
        if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return fail(e, "cudaStreamSynchronize");  // tmp_a / tmp_b are reused
        if ((rc = lcu_set_weight(ctx, it.layer, it.kind, region + it.off, it.bytes))) { cleanup(false); return rc; }
    }
    cleanup(true);
    g->dev_weights = region;
    return LCU_OK;
}

}  // extern "C"
