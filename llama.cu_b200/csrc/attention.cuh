// Causal GQA attention over the KV cache for the tokens of one round.  Interface only.
#pragma once
#include "common.cuh"

namespace lcu {

struct AttnArgs {
    const void *q;  // [n_tok, nh*dh], row stride stride_q (elements)
    int stride_q;
    void *o;  // [n_tok, nh*dh]
    int stride_o;
    int n_tok, nh, nkvh, dh;
    // paged cache (kv_pool != nullptr): token t attends positions [0, tok_pos[t]] of sequence tok_seq[t]
    const void *kv_pool;
    KvGeom geom;
    int layer;
    const int32_t *tok_seq;
    const uint32_t *tok_pos;
    const int32_t *page_table;
    int pt_stride;
    // linear cache (kv_pool == nullptr): one request; token t attends [0, pos0 + t]
    const void *k_lin, *v_lin;
    int stk, shk, stv, shv;  // token / head strides of the caches (elements)
    int pos0;
    // split-KV scratch: partial outputs, (max, sum) pairs and arrival counters
    int n_splits;          // grid depth = most splits any token of the round can need
    int tiles_per_split;   // 64-position tiles one CTA walks (0: context / n_splits); a token with a short
                           // context uses fewer splits and the CTAs beyond them exit at once
    int cluster_z;         // > 0 (== n_splits, <= 8): the splits form a thread-block cluster; each stores its partial into
                           // the first split's shared memory, which merges after one cluster barrier (no scratch)
    // Programmatic dependent launch.  early_kv: the round holds ONE new token per sequence, so every cached row below
    // a token's own position was written by an earlier round and may be fetched before the wait on the predecessor
    // (which writes only the new row).  pdl_trigger: 0 = dependents may start as soon as this grid is resident,
    // 1 = once a CTA's first K/V tile has landed (its remaining traffic is on chip).
    int early_kv;
    int pdl_trigger;
    float *part_o;        // [n_tok, nh, n_splits, dh]
    float *part_ml;       // [n_tok, nh, n_splits, 2]
    unsigned *counters;   // [n_tok, nkvh], zero before the first launch; the kernel re-zeroes them
};

// Bytes of split-KV scratch for a round of n_tok tokens when the largest round has max_tok.
size_t attn_scratch_bytes(int n_tok, int nh, int nkvh, int dh, int n_splits, int max_tok);
// Carves counters / part_ml / part_o out of `scratch`; the counters sit first, at a place that
// does not depend on the round's shape, and must have been zeroed once.
void attn_bind_scratch(AttnArgs &a, void *scratch, int max_tok);
// dry: only prepare the kernel variant (shared-memory attribute), launch nothing.
int attn_launch(const AttnArgs &a, int dt, cudaStream_t s, bool pdl, bool dry = false);

// Prefill form: one CTA per (KV head, group of up to attn_prefill_group_tokens consecutive tokens of ONE sequence);
// groups_dev: n_groups pairs (index of the first token in the round, tokens in the group).  Paged cache only, no
// split-KV; needs pt_stride <= 512 (attn_prefill_supported).
int attn_prefill_group_tokens(int nh, int nkvh);
bool attn_prefill_supported(int pt_stride);
int attn_prefill_launch(const AttnArgs &a, const void *groups_dev, int n_groups, int dt, cudaStream_t s, bool dry = false);

// Appends k, v [seq, nkvh, dh] (strided) to linear caches at pos.. (the write half of
// operators::attention_kv_cached as called from llama.cu/src/exec/step.rs:162-182).
int kv_append_linear(void *k_cache, int stkc, int shkc, void *v_cache, int stvc, int shvc, const void *k, int stk,
                     int shk, const void *v, int stv, int shv, int nkvh, int dh, int seq, int pos, int dt,
                     cudaStream_t s);

}  // namespace lcu
