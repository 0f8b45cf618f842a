// C-ABI wrappers of the stand-alone operators, the sampler entry points that replace
// librandom_sample.so, the Q8_0 repacker and the tensor-parallel weight slicer.
#include <cstdlib>
#include <cstring>

#include "attention.cuh"
#include "common.cuh"
#include "gemv.cuh"
#include "ops.cuh"
#include "sample.cuh"

using namespace lcu;

namespace {

// ggml Q8_0 block: f16 scale followed by 32 int8 quants (34 bytes, 2-byte aligned)
__global__ void repack_q8_0_kernel(int8_t *__restrict__ q, uint16_t *__restrict__ scales,
                                   const unsigned char *__restrict__ blocks, size_t n_blocks) {
    size_t b = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    int lane = threadIdx.x & 31;
    if (b >= n_blocks) return;
    const unsigned char *src = blocks + b * 34;
    if (lane == 0) scales[b] = (uint16_t)src[0] | ((uint16_t)src[1] << 8);
    q[b * 32 + lane] = (int8_t)src[2 + lane];
}

// copies rows [r0, r0+nr) x byte columns [c0, c0+cb) of a row-major matrix
int copy_block(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t r0, size_t nr, size_t c0, size_t cb,
               cudaStream_t s) {
    LCU_CHECK_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, reinterpret_cast<const unsigned char *>(src) + r0 * src_pitch + c0,
                                     src_pitch, cb, nr, cudaMemcpyDeviceToDevice, s));
    return LCU_OK;
}

}  // namespace

struct lcu_ctx;
extern "C" size_t lcu_weight_bytes(const lcu_ctx *ctx, int kind);
// accessors implemented next to the context definition
namespace lcu {
struct CtxShape {
    int d, nh, nkvh, dh, di, vocab, tp_rank, tp_size, act_dtype, weight_dtype, norm_dtype;
    void *comm;
};
CtxShape ctx_shape(const lcu_ctx *c);
}  // namespace lcu

extern "C" {

size_t lcu_q8_0_repacked_bytes(size_t rows, size_t cols) { return rows * cols + rows * cols / 32 * 2; }

int lcu_repack_q8_0(void *dst_dev, const void *src_blocks_dev, size_t rows, size_t cols, lcu_stream_t s) {
    LCU_REQUIRE(dst_dev && src_blocks_dev, "repack_q8_0: null argument");
    LCU_REQUIRE(cols % 32 == 0 && rows > 0, "repack_q8_0: %zu columns are not a multiple of 32", cols);
    size_t nb = rows * cols / 32;
    int8_t *q = reinterpret_cast<int8_t *>(dst_dev);
    uint16_t *sc = reinterpret_cast<uint16_t *>(q + rows * cols);
    unsigned grid = (unsigned)((nb + 7) / 8);
    repack_q8_0_kernel<<<grid, 256, 0, as_stream(s)>>>(q, sc, reinterpret_cast<const unsigned char *>(src_blocks_dev), nb);
    LCU_CHECK_CUDA(cudaGetLastError());
    return LCU_OK;
}

int lcu_tp_slice_weight(const lcu_ctx *ctx, int kind, void *dst, const void *src, lcu_stream_t stream) {
    LCU_REQUIRE(ctx && dst && src, "tp_slice_weight: null argument");
    CtxShape c = ctx_shape(ctx);
    cudaStream_t s = as_stream(stream);
    const bool linear = kind == LCU_W_QKV || kind == LCU_W_O || kind == LCU_W_GATE_UP || kind == LCU_W_DOWN;
    if (kind == LCU_W_LM_HEAD && c.tp_size > 1 && c.tp_rank != 0) {
        // rows [rank * vocab / tp, (rank + 1) * vocab / tp) when the head can be sharded (lcu_weight_bytes says so)
        const size_t bytes = lcu_weight_bytes(ctx, kind), full = (size_t)c.vocab * c.d * 2;
        const size_t off = bytes < full ? (size_t)c.tp_rank * bytes : 0;
        LCU_CHECK_CUDA(cudaMemcpyAsync(dst, reinterpret_cast<const unsigned char *>(src) + off, bytes, cudaMemcpyDeviceToDevice, s));
        return LCU_OK;
    }
    if (!linear || c.tp_size == 1) {
        LCU_CHECK_CUDA(cudaMemcpyAsync(dst, src, lcu_weight_bytes(ctx, kind), cudaMemcpyDeviceToDevice, s));
        return LCU_OK;
    }
    // The cut `TPAction::move_data` makes with Distribution{start = rank, len = 1, total = tp} (load/mod.rs:86-99):
    // up to three row segments of the full matrix and one column range, in elements.
    const int tp = c.tp_size, r = c.tp_rank;
    const size_t nh_l = c.nh / tp, nkvh_l = c.nkvh / tp, di_l = c.di / tp, dh = c.dh, d = c.d;
    struct Seg { size_t r0, nr; } seg[3];
    int n_seg = 0;
    size_t full_cols = 0, c0 = 0, nc = 0;
    switch (kind) {
    case LCU_W_QKV:  // rows q | k | v, each split by heads
        seg[0] = {r * nh_l * dh, nh_l * dh};
        seg[1] = {(size_t)c.nh * dh + r * nkvh_l * dh, nkvh_l * dh};
        seg[2] = {(size_t)(c.nh + c.nkvh) * dh + r * nkvh_l * dh, nkvh_l * dh};
        n_seg = 3; full_cols = d; c0 = 0; nc = d;
        break;
    case LCU_W_O:  // input columns split by heads
        seg[0] = {0, d};
        n_seg = 1; full_cols = (size_t)c.nh * dh; c0 = r * nh_l * dh; nc = nh_l * dh;
        break;
    case LCU_W_GATE_UP:  // rows gate | up, each split
        seg[0] = {r * di_l, di_l};
        seg[1] = {(size_t)c.di + r * di_l, di_l};
        n_seg = 2; full_cols = d; c0 = 0; nc = d;
        break;
    default:  // LCU_W_DOWN: input columns split
        seg[0] = {0, d};
        n_seg = 1; full_cols = (size_t)c.di; c0 = r * di_l; nc = di_l;
        break;
    }
    size_t full_rows = kind == LCU_W_QKV ? (size_t)(c.nh + 2 * c.nkvh) * dh : (kind == LCU_W_GATE_UP ? (size_t)2 * c.di : d);
    // one plane of `eb`-byte elements whose columns are the matrix columns divided by `per`
    auto plane = [&](unsigned char *out, const unsigned char *in, size_t eb, size_t per) -> int {
        const size_t src_pitch = full_cols / per * eb, dst_pitch = nc / per * eb;
        for (int i = 0; i < n_seg; ++i) {
            int rc = copy_block(out, dst_pitch, in, src_pitch, seg[i].r0, seg[i].nr, c0 / per * eb, dst_pitch, s);
            if (rc) return rc;
            out += seg[i].nr * dst_pitch;
        }
        return LCU_OK;
    };
    unsigned char *out = reinterpret_cast<unsigned char *>(dst);
    const unsigned char *in = reinterpret_cast<const unsigned char *>(src);
    if (c.weight_dtype != LCU_Q8_0) return plane(out, in, 2, 1);
    // Q8_0 in the plane layout (lcu_repack_q8_0): int8 [rows, cols] followed by f16 scales [rows, cols / 32]
    LCU_REQUIRE(c0 % 32 == 0 && nc % 32 == 0, "tp_slice_weight: Q8_0 column range [%zu, +%zu) is not a multiple of 32", c0, nc);
    size_t my_rows = 0;
    for (int i = 0; i < n_seg; ++i) my_rows += seg[i].nr;
    int rc = plane(out, in, 1, 1);
    if (rc) return rc;
    return plane(out + my_rows * nc, in + full_rows * full_cols, 2, 32);
}

// ------------------------------------------------------------------ operators

int lcu_op_embedding(void *out, const void *table, const uint32_t *index, int n, size_t row_bytes, lcu_stream_t s) {
    LCU_REQUIRE(out && table && index && n >= 0, "embedding: bad arguments");
    return op_embedding(out, table, index, n, row_bytes, as_stream(s), false);
}

int lcu_op_fast_embedding(uint32_t *tokens, const lcu_kv_pair *kv_pairs, const uint32_t *map_dev, int n_map,
                          lcu_stream_t s) {
    LCU_REQUIRE(n_map >= 0 && n_map <= 1024, "fast_embedding: %d entries (0..1024)", n_map);
    LCU_REQUIRE(n_map == 0 || (tokens && kv_pairs && map_dev), "fast_embedding: null argument");
    return op_fast_embedding(tokens, kv_pairs, map_dev, n_map, as_stream(s), false);
}

int lcu_op_rms_norm(void *y, int stride_y, const void *x, int stride_x, const void *w, int w_dt, float eps, int n,
                    int d, int dt, lcu_stream_t s) {
    LCU_REQUIRE(y && x && w && n >= 0, "rms_norm: bad arguments");
    return op_rms_norm(y, stride_y, x, stride_x, w, w_dt, eps, n, d, dt, as_stream(s), false);
}

int lcu_op_linear(void *y, int stride_y, const void *x, int stride_x, const void *w, int w_dt, const void *residual,
                  int stride_res, int n, int in, int out, int dt, lcu_stream_t s) {
    LCU_REQUIRE(y && x && w && n >= 0 && in > 0 && out > 0, "linear: bad arguments");
    LCU_REQUIRE(w_dt == dt || (w_dt == LCU_Q8_0 && dt == LCU_F16), "linear: weight dtype %d with activation dtype %d", w_dt, dt);
    const size_t eb = 2;
    const bool batched = n > 4 && gemm_skinny_supported(in, w_dt == LCU_Q8_0) && out % 2 == 0;
    if (batched) gemm_skinny_set_scratch(nullptr, 0, nullptr, 0);  // the stand-alone operator owns no scratch: no K split
    const bool tc_on = tuning().tc != 0;
    const bool tc = batched && tc_on && n > 8 && gemm_tc_supported(in, w_dt == LCU_Q8_0);
    if (tc) gemm_tc_set_scratch(nullptr, 0, nullptr, 0, nullptr);
    for (int t0 = 0; t0 < n;) {
        int nt = batched ? 64 : gemv_max_tokens(in);
        if (nt > n - t0) nt = n - t0;
        if (nt == 3 && !batched) nt = 2;
        GemvArgs a{};
        a.w = w;
        a.w_q8 = w_dt == LCU_Q8_0;
        a.w_scales = a.w_q8 ? reinterpret_cast<const unsigned char *>(w) + (size_t)out * in : nullptr;
        a.x = reinterpret_cast<const unsigned char *>(x) + (size_t)t0 * stride_x * eb;
        a.stride_x = stride_x;
        a.n_tok = nt;
        a.in = in;
        a.out = out;
        a.prologue = PRO_NONE;
        a.epilogue = residual ? EPI_RESIDUAL : EPI_STORE;
        a.y = reinterpret_cast<unsigned char *>(y) + (size_t)t0 * stride_y * eb;
        a.stride_y = stride_y;
        a.res = residual ? reinterpret_cast<const unsigned char *>(residual) + (size_t)t0 * stride_res * eb : nullptr;
        a.stride_res = stride_res;
        a.early_prefetch = 1;
        int rc = tc ? gemm_tc_launch(a, dt, as_stream(s), false)
                    : (batched ? gemm_skinny_launch(a, dt, as_stream(s), false) : gemv_launch(a, dt, as_stream(s), false));
        if (rc) return rc;
        t0 += nt;
    }
    return LCU_OK;
}

int lcu_op_rope(void *y, int sty, int shy, const void *x, int stx, int shx, const uint32_t *pos, const float *sin_t,
                const float *cos_t, int n, int nh, int dh, int dt, lcu_stream_t s) {
    LCU_REQUIRE(y && x && pos && sin_t && cos_t && n >= 0, "rope: bad arguments");
    return op_rope(y, sty, shy, x, stx, shx, pos, sin_t, cos_t, n, nh, dh, dt, as_stream(s), false);
}

int lcu_op_swiglu(void *out, int so, const void *gate, int sg, const void *up, int su, int n, int di, int dt,
                  lcu_stream_t s) {
    LCU_REQUIRE(out && gate && up && n >= 0 && di > 0, "swiglu: bad arguments");
    return op_swiglu(out, so, gate, sg, up, su, n, di, dt, as_stream(s), false);
}

int lcu_op_add(void *y, int sny, int sdy, const void *x, int snx, int sdx, const void *b, int snb, int sdb, float k,
               int n, int d, int dt, lcu_stream_t s) {
    LCU_REQUIRE(y && b && (x || k == 0.f) && n >= 0 && d > 0, "add: bad arguments");
    return op_add(y, sny, sdy, x ? x : b, snx, sdx, b, snb, sdb, k, n, d, dt, as_stream(s));
}

int lcu_op_attention_kv_cached(void *o, int sto, int sho, const void *q, int stq, int shq, const void *k, int stk,
                               int shk, const void *v, int stv, int shv, void *k_cache, int stkc, int shkc,
                               void *v_cache, int stvc, int shvc, int nh, int nkvh, int dh, int seq, int pos, int dt,
                               lcu_stream_t s) {
    LCU_REQUIRE(o && q && k && v && k_cache && v_cache, "attention: null argument");
    LCU_REQUIRE(seq >= 1 && pos >= 0 && nh > 0 && nkvh > 0, "attention: bad shape");
    LCU_REQUIRE(shq == dh && sho == dh, "attention: q and o heads must be contiguous (head stride == dh)");
    int rc = kv_append_linear(k_cache, stkc, shkc, v_cache, stvc, shvc, k, stk, shk, v, stv, shv, nkvh, dh, seq, pos, dt,
                              as_stream(s));
    if (rc) return rc;
    AttnArgs a{};
    a.q = q; a.stride_q = stq; a.o = o; a.stride_o = sto;
    a.n_tok = seq; a.nh = nh; a.nkvh = nkvh; a.dh = dh;
    a.kv_pool = nullptr;
    a.k_lin = k_cache; a.v_lin = v_cache; a.stk = stkc; a.shk = shkc; a.stv = stvc; a.shv = shvc; a.pos0 = pos;
    a.n_splits = 1;  // no caller workspace, as in the reference's call (`&mut []`, exec/step.rs:179)
    return attn_launch(a, dt, as_stream(s), false);
}

int lcu_op_all_reduce(lcu_ctx *ctx, void *y, const void *x, size_t count, int dt, lcu_stream_t s) {
    LCU_REQUIRE(ctx && y && x, "all_reduce: null argument");
    CtxShape c = ctx_shape(ctx);
    if (c.tp_size == 1) {
        if (y != x) LCU_CHECK_CUDA(cudaMemcpyAsync(y, x, count * (dt == LCU_F32 ? 4 : 2), cudaMemcpyDeviceToDevice, as_stream(s)));
        return LCU_OK;
    }
    return comm_all_reduce(c.comm, y, x, count, dt, as_stream(s));
}

// ------------------------------------------------------------------ sampler (sample.h drop-in)

int lcu_calculate_workspace_size_half(size_t *argmax, size_t *random_sample, size_t n) {
    if (!argmax || !random_sample) return (int)cudaErrorInvalidValue;
    *argmax = argmax_workspace_bytes(1, n) + 256;
    *random_sample = sample_workspace_bytes(1, n) + 256 + sizeof(lcu_sample_args) + 16;
    return (int)cudaSuccess;
}

int lcu_argmax_half(void *kv_pair, const void *logits, size_t n, void *workspace_ptr, size_t workspace_len,
                    lcu_stream_t stream) {
    if (!kv_pair || !logits || !workspace_ptr) return (int)cudaErrorInvalidValue;
    uintptr_t p = ((uintptr_t)workspace_ptr + 255) & ~(uintptr_t)255;
    size_t skip = p - (uintptr_t)workspace_ptr;
    if (workspace_len < skip + argmax_workspace_bytes(1, n)) return (int)cudaErrorInvalidValue;
    int rc = sample_rows(reinterpret_cast<lcu_kv_pair *>(kv_pair), nullptr, logits, 1, n, nullptr, nullptr, LCU_F16,
                         reinterpret_cast<void *>(p), workspace_len - skip, as_stream(stream), false, false);
    return rc == LCU_OK ? (int)cudaSuccess : (int)cudaErrorUnknown;
}

int lcu_sample_half(void *kv_pair, const void *logits, const unsigned int *indices, size_t n, float random,
                    float temperature, float topp, size_t topk, void *workspace_ptr, size_t workspace_len,
                    lcu_stream_t stream) {
    (void)indices;  // the reference needs an iota array for its sort; the histogram sampler does not
    if (!kv_pair || !logits || !workspace_ptr) return (int)cudaErrorInvalidValue;
    uintptr_t p = ((uintptr_t)workspace_ptr + 255) & ~(uintptr_t)255;
    size_t skip = p - (uintptr_t)workspace_ptr;
    size_t ws = sample_workspace_bytes(1, n);
    if (workspace_len < skip + ws + sizeof(lcu_sample_args) + 16) return (int)cudaErrorInvalidValue;
    // the arguments travel to the device in the tail of the workspace
    struct { lcu_sample_args a; float r; } host;
    host.a.temperature = temperature;
    host.a.top_p = topp;
    host.a.top_k = topk;
    host.r = random;
    unsigned char *tail = reinterpret_cast<unsigned char *>(p) + ws;
    cudaError_t e = cudaMemcpyAsync(tail, &host, sizeof(host), cudaMemcpyHostToDevice, as_stream(stream));
    if (e != cudaSuccess) return (int)e;
    int rc = sample_rows(reinterpret_cast<lcu_kv_pair *>(kv_pair), nullptr, logits, 1, n,
                         reinterpret_cast<const lcu_sample_args *>(tail),
                         reinterpret_cast<const float *>(tail + sizeof(lcu_sample_args)), LCU_F16,
                         reinterpret_cast<void *>(p), ws, as_stream(stream), false, true);
    return rc == LCU_OK ? (int)cudaSuccess : (int)cudaErrorUnknown;
}

size_t lcu_sample_rows_workspace_size(int rows, size_t n) { return sample_workspace_bytes(rows, n); }

int lcu_op_sample_rows(lcu_kv_pair *out, lcu_kv_pair *out_copy, const void *logits, int rows, size_t n,
                       const lcu_sample_args *args_dev, const float *randoms_dev, int dt, void *workspace,
                       size_t workspace_len, lcu_stream_t s) {
    LCU_REQUIRE(out && logits && workspace, "sample_rows: null argument");
    return sample_rows(out, out_copy, logits, rows, n, args_dev, randoms_dev, dt, workspace, workspace_len, as_stream(s),
                       false, args_dev != nullptr);
}

}  // extern "C"
