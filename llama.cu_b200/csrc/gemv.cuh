// Weight-streaming GEMV family: the `Linear` operator of the decode step for 1..4 tokens
// with the neighbouring small operators fused in.  Interface only; kernels in gemv.cu.
#pragma once
#include "common.cuh"

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
};

// Enqueues one GEMV; dt = LCU_F16 / LCU_BF16.  pdl: launch with programmatic serialisation.
int gemv_launch(const GemvArgs &a, int dt, cudaStream_t s, bool pdl, bool dry = false);
// Prepares (attributes, occupancy) every variant used for this shape without launching.
int gemv_warm(int in, int out, bool q8, int dt);
// Most tokens one launch can take for this input width (activations live in shared memory).
int gemv_max_tokens(int in);

}  // namespace lcu
