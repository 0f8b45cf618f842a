// Weight-streaming GEMV family: the `Linear` operator of the decode step for 1..4 tokens
// with the neighbouring small operators fused in.  Interface only; kernels in gemv.cu.
#pragma once
#include "common.cuh"
#include "p2p.cuh"

namespace lcu {

enum GemvPrologue { PRO_NONE = 0, PRO_RMSNORM = 1 };
enum GemvEpilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_ROPE_KV = 2, EPI_SWIGLU = 3 };

struct GemvArgs {
    // weights [out, in] row-major in the activation dtype, or Q8_0 planes
    const void *w;
    const void *w_scales;  // Q8_0 only: f16 [out, in/32]
    int w_q8;
    // activations: token t reads row x_rows ? x_rows[t] : t of x
    const void *x;
    int stride_x;
    const uint32_t *x_rows;
    int n_tok;  // 1..4
    int in, out;
    // prologue
    int prologue;
    const void *norm_w;
    int norm_f32;
    float eps;
    // epilogue
    int epilogue;
    void *y;
    int stride_y;
    const void *res;
    int stride_res;
    // EPI_ROPE_KV: rows [0,qd) are q heads, [qd,qd+kvd) k heads, then v heads
    int qd, kvd, dh;
    const uint32_t *pos;      // [n_tok]
    const float *sin_t, *cos_t;
    void *kv_pool;
    KvGeom geom;
    int layer;
    const int32_t *tok_seq;     // [n_tok] sequence slot of each token
    const int32_t *page_table;  // [slots, pt_stride]
    int pt_stride;
    // EPI_SWIGLU: rows [0,di) gate, [di,2di) up; y gets [n_tok, di]
    int di;
    // tuning: 0 = trigger dependents at kernel start, 1 = after the main loop, 2 = never (implicit at exit)
    int pdl_trigger;
    int early_prefetch;  // 1 = first weight loads before griddepcontrol.wait
    int lean_norm;       // one token: RMSNorm prologue from registers (norm weights fetched before the wait)
    // tensor parallelism: EPI_STORE / EPI_RESIDUAL outputs go to every rank's all-reduce slot instead of y
    P2pPush push;
};

#ifdef __CUDACC__
// ---- fused epilogue of one row pair for one token, shared by the GEMV and the batched kernel
__device__ __forceinline__ float swiglu_act(float gate, float up) {
    return gate * __fdividef(1.f, 1.f + expf(-gate)) * up;
}

// Values an epilogue would otherwise fetch from global memory behind the weight stream: the per-token constants of the
// RoPE / KV-append epilogue (position, cache page, sin and cos rows; head sizes up to 128), staged in shared memory
// before the main loop, and the residual pair of this output, loaded before the group's arithmetic.
struct RopeStage {
    uint32_t pos[4];
    int page[4];
    float sn[4][64], cs[4][64];
};
struct EpiPre {
    const RopeStage *rope = nullptr;  // EPI_ROPE_KV
    uint32_t res = 0;                 // EPI_RESIDUAL: the packed residual pair
    bool has_res = false;
};

template <class T>
__device__ void gemv_epilogue(const GemvArgs &a, int pair, int t, float va, float vb, const EpiPre &pre = EpiPre()) {
    T *y = reinterpret_cast<T *>(a.y);
    switch (a.epilogue) {
    case EPI_STORE: {
        size_t r = (size_t)pair * 2;
        if (a.push.n) {
            const uint32_t packed = Act<T>::pack(va, vb);
            if (a.push.scatter_cols) {
                *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.push.slot[r / a.push.scatter_cols]) + (size_t)t * a.stride_y + r) = packed;
                break;
            }
            for (int k = 0; k < a.push.n; ++k)
                *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.push.slot[k]) + (size_t)t * a.stride_y + r) = packed;
            break;
        }
        y[(size_t)t * a.stride_y + r] = Act<T>::from_f(va);
        y[(size_t)t * a.stride_y + r + 1] = Act<T>::from_f(vb);
        break;
    }
    case EPI_RESIDUAL: {
        size_t r = (size_t)pair * 2;
        const T *res = reinterpret_cast<const T *>(a.res) + (size_t)t * a.stride_res + r;
        // residual enters as the beta = 1 operand of the GEMM: one rounding of acc + res
        uint32_t rr = pre.has_res ? pre.res : *reinterpret_cast<const uint32_t *>(res);
        float2 rf = Act<T>::to_f2(rr);
        const uint32_t packed = Act<T>::pack(va + rf.x, vb + rf.y);
        if (a.push.n) {
            if (a.push.scatter_cols) {
                *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.push.slot[r / a.push.scatter_cols]) + (size_t)t * a.stride_y + r) = packed;
                break;
            }
            for (int k = 0; k < a.push.n; ++k)
                *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.push.slot[k]) + (size_t)t * a.stride_y + r) = packed;
            break;
        }
        *reinterpret_cast<uint32_t *>(&y[(size_t)t * a.stride_y + r]) = packed;
        break;
    }
    case EPI_ROPE_KV: {
        int r = pair * 2;
        // the qkv projection is materialised in the activation dtype before rope reads it
        float xa = round_act<T>(va), xb = round_act<T>(vb);
        int sect = r < a.qd ? 0 : (r < a.qd + a.kvd ? 1 : 2);
        int rr = r - (sect == 0 ? 0 : (sect == 1 ? a.qd : a.qd + a.kvd));
        int head = rr / a.dh, e = rr - head * a.dh;
        uint32_t p = pre.rope ? pre.rope->pos[t] : a.pos[t];
        if (sect < 2) {
            int half_dh = a.dh >> 1;
            float sn = pre.rope ? pre.rope->sn[t][e >> 1] : a.sin_t[(size_t)p * half_dh + (e >> 1)];
            float cs = pre.rope ? pre.rope->cs[t][e >> 1] : a.cos_t[(size_t)p * half_dh + (e >> 1)];
            float ya = xa * cs - xb * sn, yb = xa * sn + xb * cs;
            xa = ya;
            xb = yb;
        }
        uint32_t packed = Act<T>::pack(xa, xb);
        if (sect == 0) {
            *reinterpret_cast<uint32_t *>(&y[(size_t)t * a.stride_y + r]) = packed;
        } else {
            int page = pre.rope ? pre.rope->page[t] : a.page_table[(size_t)a.tok_seq[t] * a.pt_stride + (p >> a.geom.page_shift)];
            int slot = p & (a.geom.page_tokens - 1);
            size_t off = a.geom.block_off(page, a.layer, sect - 1, head) + (size_t)slot * a.dh + e;
            *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.kv_pool) + off) = packed;
        }
        break;
    }
    case EPI_SWIGLU: {
        // gate = row pair, up = row pair + di, both materialised before swiglu reads them
        float g = round_act<T>(va), u = round_act<T>(vb);
        y[(size_t)t * a.stride_y + pair] = Act<T>::from_f(swiglu_act(g, u));
        break;
    }
    }
}

#endif  // __CUDACC__

// Enqueues one GEMV; dt = LCU_F16 / LCU_BF16.  pdl: launch with programmatic serialisation.
int gemv_launch(const GemvArgs &a, int dt, cudaStream_t s, bool pdl, bool dry = false);
// Prepares (attributes, occupancy) every variant used for this shape without launching.
int gemv_warm(int in, int out, bool q8, int dt);
// Batched form for up to 64 tokens per launch (gemm_skinny.cu): same arguments and epilogues, but the
// activations must be prepared (no RMSNorm prologue, no row gather).
bool gemm_skinny_supported(int in, int w_q8);
int gemm_skinny_launch(const GemvArgs &a, int dt, cudaStream_t s, bool pdl, bool dry = false);
int gemm_skinny_warm(int in, int out, int dt, int w_q8 = 0);
// Split-K scratch (f32 partial sums) and zeroed tickets (one per 128-row block) for the calling thread.
void gemm_skinny_set_scratch(void *ws, size_t ws_bytes, unsigned *tickets, int n_tickets);
// tcgen05 / TMEM / TMA form of the batched kernel (gemm_tc.cu): same arguments.
bool gemm_tc_supported(int in, int w_q8);
int gemm_tc_launch(const GemvArgs &a, int dt, cudaStream_t s, bool pdl, bool dry = false);
int gemm_tc_warm(int dt);
void gemm_tc_set_scratch(void *ws, size_t ws_bytes, unsigned *tickets, int n_tickets, uint32_t *status);
// CTAs of the calling thread's most recent linear-layer launch (GEMV or batched): the peer all-reduce
// counts one arrival per producing CTA.
extern thread_local int g_linear_last_ctas;
// Most tokens one launch can take for this input width (activations live in shared memory).
int gemv_max_tokens(int in);

}  // namespace lcu
