// Persistent whole-step decode kernel for 1..4 sequences (one token each).  Interface only.
#pragma once
#include "common.cuh"

namespace lcu {

enum MkPhaseKind { MK_QKV = 0, MK_ATTN = 1, MK_O = 2, MK_GATE_UP = 3, MK_DOWN = 4, MK_HEAD = 5 };

// One phase of the step.  Weight phases stream `w` [out, in] row-major as tiles of R rows x KC
// columns; rows are taken in PAIRS (adjacent rows, or row p with row p + di for gate|up).
struct MkPhase {
    const void *w;
    const void *norm_w;  // RMSNorm weights of the prologue (QKV, gate|up, head)
    int kind, layer;
    int in, n_pairs;
    int R, KC, n_kc;     // tile geometry: R rows (even) x KC columns, n_kc chunks per row
    int swiglu_di;       // > 0: pair p joins rows p and p + di
};

struct MkArgs {
    const MkPhase *phases;
    int n_phases;
    int n_tok;           // sequences in the round (1..4), one token each
    int d, qd, kvd, dh, nh, nkvh, di, vocab;
    float eps;
    int norm_f32;
    // round descriptor (device)
    uint32_t *tokens;
    const uint32_t *pos;
    const uint32_t *fast_map;
    int n_fast;
    const lcu_kv_pair *pre_pairs_in;
    const int32_t *page_table;
    int pt_stride;
    // model state
    const void *embd;
    const float *sin_t, *cos_t;
    void *kv_pool;
    KvGeom geom;
    // activations (global)
    void *x;        // residual stream [n_tok, d]
    void *q;        // [n_tok, qd]
    void *act;      // [n_tok, di]
    void *logits;   // [n_tok, vocab]
    float *attn_part;   // [n_tok, nh, s_max, dh + 2]  (o[dh], m, l)
    int s_max;          // splits per (token, kv head)
    float *head_best_v; // [grid, n_tok]
    uint32_t *head_best_i;
    lcu_kv_pair *out, *out_copy;
    // synchronisation / status
    unsigned *grid_bar;   // zeroed before every launch
    long long *prof;      // optional: 16 cycle counters filled by CTA 0 (nullptr = off)
    uint32_t *status;     // error word: bit 0 = barrier wait ran out, bit 1 = pipeline wait ran out
    int n_stages;
    int l2_ahead;         // tiles the L2 prefetch runs ahead of the shared-memory copies (0 = off)
    int smem_x_bytes;     // activation / attention scratch region
    int smem_part_bytes;  // partial-sum buffers (2 per ring stage), also the attention-merge weights
};

// Shared memory the kernel needs for this model and batch; 0 when it does not fit.
size_t mk_smem_bytes(int n_tok, int max_in, int nh, int nkvh, int dh, int *n_stages, int *x_bytes, int *part_bytes);
// Tile geometry for an input width (elements): fills R, KC, n_kc.  false when unsupported.
bool mk_plan_tiles(int in, int *R, int *KC, int *n_kc);
// Upper bound of per-(token,kv head) context splits for a grid of `grid` CTAs.
int mk_splits(int grid, int n_tok, int nkvh);
int mk_prepare(int dt, int n_tok, size_t smem);  // attributes + occupancy check; returns LCU_* status
int mk_launch(const MkArgs &a, int dt, size_t smem, cudaStream_t s);

}  // namespace lcu
