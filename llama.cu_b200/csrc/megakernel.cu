// Persistent whole-step decode kernel: ONE cooperative launch runs every layer and the head
// of a decode round for 1..4 sequences (f16 / bf16 weights).
//
// Why: at batch 1 the step is a chain of ~160 short weight-streaming phases (QKV 50 MB,
// O 34 MB, gate|up 235 MB, down 117 MB per layer for the 8B shape).  As separate launches
// each phase pays launch latency, an activation prologue and a drain tail during which HBM
// idles — measured 5-8 us per launch, a third of the step.  Here the weight stream never
// stops:
//   - one CTA per SM, 16 consumer warps + 1 producer warp;
//   - the producer walks the static list of (phase, tile) work items of its CTA for the
//     WHOLE step and copies weight tiles global -> shared with cp.async.bulk into a ring of
//     32 KB stages (mbarrier full/empty pairs).  Weights never change, so the producer runs
//     ahead of the consumers across phase boundaries and grid barriers: while the consumers
//     wait at a barrier, normalise activations or do attention, the next phase's weights
//     are already landing in shared memory and HBM stays busy;
//   - consumers multiply tiles from shared memory against activations held in shared memory
//     (f32 accumulate), reduce across the CTA and run the fused epilogues (RoPE + KV append,
//     residual add, SwiGLU, logits + arg-max) with the same rounding points as the separate
//     kernels;
//   - phases are separated by a grid barrier (arrive counter + acquire poll).  Activations
//     written by other CTAs are read with ld.global.cg because L1 is not invalidated inside
//     one launch;
//   - attention runs as a phase: (token, KV head, split) units over the CTAs, one warp per
//     cached position, partial (o, max, sum) per split to global scratch; the O-projection
//     phase's prologue merges the splits, so attention costs one barrier, not two.
// Every wait (mbarrier, grid barrier) is bounded by a wall-clock limit; on expiry the kernel
// records a status bit, stops issuing work, drains its own copies and returns.
#include "megakernel.cuh"

#include <map>
#include <mutex>

namespace lcu {

constexpr int MK_CONSUMERS = 512;
constexpr int MK_WARPS = MK_CONSUMERS / 32;
constexpr int MK_THREADS = MK_CONSUMERS + 32;
constexpr int MK_GROUP_WARPS = 4;                     // consumer warps that share one weight tile
constexpr int MK_GROUP_THREADS = MK_GROUP_WARPS * 32;
constexpr int MK_GROUPS = MK_WARPS / MK_GROUP_WARPS;  // tiles in flight per CTA
constexpr int MK_STAGE_BYTES = 32768;
constexpr int MK_MAX_R = 8;
constexpr int MK_MAX_NT = 4;
constexpr unsigned long long MK_WAIT_NS = 2000000000ull;  // 2 s per wait

// ------------------------------------------------------------------ small PTX helpers
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(MK_CONSUMERS) : "memory"); }
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the limit ran out or another thread of the CTA gave up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try(bar, parity)) return true;
    unsigned long long t0 = global_ns();
    for (unsigned it = 1;; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 255u) == 0 && (*abort_flag || global_ns() - t0 > MK_WAIT_NS)) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 ldcg128(const void *p) { return __ldcg(reinterpret_cast<const uint4 *>(p)); }

template <class T>
__device__ __forceinline__ void v8_to_f32(const uint4 &v, float f[8]) {
    float2 a = Act<T>::to_f2(v.x), b = Act<T>::to_f2(v.y), c = Act<T>::to_f2(v.z), d = Act<T>::to_f2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <class T> __device__ __forceinline__ float mk_bits_to_f(unsigned short b);
template <> __device__ __forceinline__ float mk_bits_to_f<__half>(unsigned short b) { return __half2float(__ushort_as_half(b)); }
template <> __device__ __forceinline__ float mk_bits_to_f<__nv_bfloat16>(unsigned short b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ float mk_swiglu(float gate, float up) { return gate * __fdividef(1.f, 1.f + expf(-gate)) * up; }

struct MkShared {
    unsigned long long full[8], empty[8];
    int abort_flag;
    int issued, consumed;          // tiles issued by the producer (set when it stops)
    float red[MK_MAX_NT * MK_WARPS];
    float rms[MK_MAX_NT];
    float fin_v[MK_WARPS * 16];
    uint32_t fin_i[MK_WARPS * 16];
    uint32_t tok[MK_MAX_NT];
    int cnt[16];                   // arrival counters of the partial-sum buffers
    int rel[8];                    // per ring slot: releases so far (4 per lap)
};

// context splits of one token: identical on the writer (attention phase) and the reader (O prologue)
__device__ __forceinline__ int mk_token_splits(int ctx, int s_max) {
    int s = (ctx + 31) / 32;
    return s < 1 ? 1 : (s > s_max ? s_max : s);
}

__device__ __forceinline__ void mk_pair_range(int n_pairs, int &p_begin, int &p_end) {
    p_begin = (int)((long long)n_pairs * blockIdx.x / gridDim.x);
    p_end = (int)((long long)n_pairs * (blockIdx.x + 1) / gridDim.x);
}

// ------------------------------------------------------------------ grid barrier
__device__ __forceinline__ void mk_grid_barrier(const MkArgs &a, unsigned &target, MkShared *sh) {
    consumer_sync();
    if (threadIdx.x == 0) {
        target += gridDim.x;
        __threadfence();
        atomicAdd(a.grid_bar, 1u);
        unsigned long long t0 = global_ns();
        for (unsigned it = 0;; ++it) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.grid_bar) : "memory");
            if (v >= target) break;
            if ((it & 63u) == 63u && (sh->abort_flag || global_ns() - t0 > MK_WAIT_NS)) {
                atomicOr(a.status, 1u);
                sh->abort_flag = 1;
                break;
            }
        }
        __threadfence();
    }
    consumer_sync();
}

// ------------------------------------------------------------------ producer
// Walks the (phase, row group, K chunk) tiles of this CTA in the order they are consumed.
struct MkTileCursor {
    int pi, p0, kc, p_begin, p_end;
    MkPhase ph;
    bool valid;
    __device__ void seek_phase(const MkArgs &a) {
        valid = false;
        for (; pi < a.n_phases; ++pi) {
            ph = a.phases[pi];
            if (ph.kind == MK_ATTN) continue;
            mk_pair_range(ph.n_pairs, p_begin, p_end);
            if (p_begin < p_end) { p0 = p_begin; kc = 0; valid = true; return; }
        }
    }
    __device__ void init(const MkArgs &a) { pi = 0; seek_phase(a); }
    __device__ void next(const MkArgs &a) {
        if (++kc < ph.n_kc) return;
        kc = 0;
        p0 += ph.R >> 1;
        if (p0 < p_end) return;
        ++pi;
        seek_phase(a);
    }
};

__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Issues the copies of one tile: into shared memory (bar != 0) or as L2 prefetches (bar == 0).
__device__ __forceinline__ uint32_t mk_issue_tile(const MkTileCursor &c, uint32_t dst, uint32_t bar) {
    const MkPhase &ph = c.ph;
    const int RP = ph.R >> 1;
    const int rv = min(RP, c.p_end - c.p0);
    const size_t row_bytes = (size_t)ph.in * 2;
    const uint32_t kc_bytes = (uint32_t)ph.KC * 2;
    const unsigned char *w = reinterpret_cast<const unsigned char *>(ph.w);
    if (bar) mbar_expect_tx(bar, (uint32_t)(2 * rv) * kc_bytes);
    if (ph.swiglu_di > 0) {
        const unsigned char *g = w + (size_t)c.p0 * row_bytes + (size_t)c.kc * kc_bytes;
        const unsigned char *u = g + (size_t)ph.swiglu_di * row_bytes;
        if (ph.n_kc == 1) {
            if (bar) {
                bulk_g2s(dst, g, (uint32_t)rv * kc_bytes, bar);
                bulk_g2s(dst + (uint32_t)RP * kc_bytes, u, (uint32_t)rv * kc_bytes, bar);
            } else {
                l2_prefetch(g, (uint32_t)rv * kc_bytes);
                l2_prefetch(u, (uint32_t)rv * kc_bytes);
            }
        } else {
            for (int r = 0; r < rv; ++r) {
                if (bar) {
                    bulk_g2s(dst + (uint32_t)r * kc_bytes, g + (size_t)r * row_bytes, kc_bytes, bar);
                    bulk_g2s(dst + (uint32_t)(RP + r) * kc_bytes, u + (size_t)r * row_bytes, kc_bytes, bar);
                } else {
                    l2_prefetch(g + (size_t)r * row_bytes, kc_bytes);
                    l2_prefetch(u + (size_t)r * row_bytes, kc_bytes);
                }
            }
        }
    } else {
        const unsigned char *src = w + (size_t)(2 * c.p0) * row_bytes + (size_t)c.kc * kc_bytes;
        if (ph.n_kc == 1) {
            if (bar) bulk_g2s(dst, src, (uint32_t)(2 * rv) * kc_bytes, bar);
            else l2_prefetch(src, (uint32_t)(2 * rv) * kc_bytes);
        } else {
            for (int r = 0; r < 2 * rv; ++r) {
                if (bar) bulk_g2s(dst + (uint32_t)r * kc_bytes, src + (size_t)r * row_bytes, kc_bytes, bar);
                else l2_prefetch(src + (size_t)r * row_bytes, kc_bytes);
            }
        }
    }
    return 0;
}

__device__ void mk_producer(const MkArgs &a, MkShared *sh, unsigned char *ring) {
    const int S = a.n_stages;
    int slot = 0;
    uint32_t parity = 0;  // parity of the `empty` phase to wait for; fresh barriers pass parity 1
    int issued = 0;
    MkTileCursor cur, ahead;
    cur.init(a);
    ahead.init(a);
    // L2 prefetches run `l2_ahead` tiles in front of the shared-memory copies: HBM keeps streaming
    // into the (large) L2 while the ring is full and the consumers sit in a barrier or prologue
    for (int i = 0; i < a.l2_ahead && ahead.valid; ++i) {
        mk_issue_tile(ahead, 0, 0);
        ahead.next(a);
    }
    while (cur.valid) {
        if (a.l2_ahead > 0 && ahead.valid) {
            mk_issue_tile(ahead, 0, 0);
            ahead.next(a);
        }
        if (!mbar_wait(smem_u32(&sh->empty[slot]), parity ^ 1u, &sh->abort_flag)) {
            atomicOr(a.status, 2u);
            sh->abort_flag = 1;
            break;
        }
        mk_issue_tile(cur, smem_u32(ring + (size_t)slot * MK_STAGE_BYTES), smem_u32(&sh->full[slot]));
        cur.next(a);
        ++issued;
        if (++slot == S) { slot = 0; parity ^= 1u; }
    }
    sh->issued = issued;
}

// ------------------------------------------------------------------ consumer prologues
// xs[t][0..in) = RMSNorm(source row t) * norm_w, rounded to T (op/rms_norm.cuh arithmetic)
template <class T, int NT>
__device__ void mk_prologue_rmsnorm(const MkArgs &a, const MkPhase &ph, MkShared *sh, T *xs, bool from_embedding,
                                    bool head) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nv8 = ph.in / 8;
    const T *xg = reinterpret_cast<const T *>(a.x);
    const T *embd = reinterpret_cast<const T *>(a.embd);
    (void)head;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        uint4 *dst = reinterpret_cast<uint4 *>(xs + (size_t)t * ph.in);
        if (t < a.n_tok) {
            const T *src = from_embedding ? embd + (size_t)sh->tok[t] * a.d : xg + (size_t)t * a.d;
            for (int i = tid; i < nv8; i += MK_CONSUMERS) {
                uint4 v = from_embedding ? __ldg(reinterpret_cast<const uint4 *>(src) + i) : ldcg128(reinterpret_cast<const uint4 *>(src) + i);
                dst[i] = v;
                // the embedding row is the residual stream of layer 0: one CTA materialises it
                if (from_embedding && blockIdx.x == 0) reinterpret_cast<uint4 *>(const_cast<T *>(xg) + (size_t)t * a.d)[i] = v;
            }
        } else {
            for (int i = tid; i < nv8; i += MK_CONSUMERS) dst[i] = make_uint4(0, 0, 0, 0);
        }
    }
    consumer_sync();
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        float ss = 0.f;
        const uint4 *src = reinterpret_cast<const uint4 *>(xs + (size_t)t * ph.in);
        for (int i = tid; i < nv8; i += MK_CONSUMERS) {
            float f[8];
            v8_to_f32<T>(src[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
        }
        ss = warp_sum(ss);
        if (lane == 0) sh->red[t * MK_WARPS + warp] = ss;
    }
    consumer_sync();
    if (tid < NT) {
        float v = 0.f;
        for (int w = 0; w < MK_WARPS; ++w) v += sh->red[tid * MK_WARPS + w];
        sh->rms[tid] = rsqrtf(v / (float)ph.in + a.eps);
    }
    consumer_sync();
    for (int i = tid; i < nv8; i += MK_CONSUMERS) {
        float wf[8];
        if (a.norm_f32) {
            const float4 *nw = reinterpret_cast<const float4 *>(ph.norm_w);
            float4 w0 = nw[2 * i], w1 = nw[2 * i + 1];
            wf[0] = w0.x; wf[1] = w0.y; wf[2] = w0.z; wf[3] = w0.w; wf[4] = w1.x; wf[5] = w1.y; wf[6] = w1.z; wf[7] = w1.w;
        } else {
            v8_to_f32<T>(reinterpret_cast<const uint4 *>(ph.norm_w)[i], wf);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            uint4 *row = reinterpret_cast<uint4 *>(xs + (size_t)t * ph.in);
            float f[8];
            v8_to_f32<T>(row[i], f);
            const float r = sh->rms[t];
            uint4 o;
            o.x = Act<T>::pack(r * f[0] * wf[0], r * f[1] * wf[1]);
            o.y = Act<T>::pack(r * f[2] * wf[2], r * f[3] * wf[3]);
            o.z = Act<T>::pack(r * f[4] * wf[4], r * f[5] * wf[5]);
            o.w = Act<T>::pack(r * f[6] * wf[6], r * f[7] * wf[7]);
            row[i] = o;
        }
    }
    consumer_sync();
}

// xs[t][0..in) = rows of a global activation buffer written by other CTAs
template <class T, int NT>
__device__ void mk_prologue_copy(const MkArgs &a, const MkPhase &ph, T *xs, const void *src_base, int src_stride) {
    const int nv8 = ph.in / 8;
    const T *src = reinterpret_cast<const T *>(src_base);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        uint4 *dst = reinterpret_cast<uint4 *>(xs + (size_t)t * ph.in);
        for (int i = threadIdx.x; i < nv8; i += MK_CONSUMERS)
            dst[i] = t < a.n_tok ? ldcg128(reinterpret_cast<const uint4 *>(src + (size_t)t * src_stride) + i) : make_uint4(0, 0, 0, 0);
    }
    consumer_sync();
}

// xs[t][head*dh + d] = merged attention output of every head (splits combined, normalised, rounded).
// Two passes so that each costs one L2 round trip: per-(token, head) split weights into shared
// memory first, then every thread folds its output elements with independent loads.
template <class T, int NT>
__device__ void mk_prologue_attn_merge(const MkArgs &a, const MkPhase &ph, T *xs, float *wts) {
    const int DHP = a.dh + 2;
    for (int idx = threadIdx.x; idx < a.n_tok * a.nh; idx += MK_CONSUMERS) {
        int t = idx / a.nh;
        int ns = mk_token_splits((int)a.pos[t] + 1, a.s_max);
        const float *base = a.attn_part + (size_t)idx * a.s_max * DHP;
        float mv[16], lv[16];
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            mv[s] = s < ns ? __ldcg(base + (size_t)s * DHP + a.dh) : -INFINITY;
            lv[s] = s < ns ? __ldcg(base + (size_t)s * DHP + a.dh + 1) : 0.f;
        }
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < 16; ++s) M = fmaxf(M, mv[s]);
        float L = 0.f;
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            mv[s] = mv[s] == -INFINITY ? 0.f : expf(mv[s] - M);
            L = fmaf(lv[s], mv[s], L);
        }
        // the reference normalises after the weighted sum: keep O / L as the last operation
        wts[idx * 17 + 16] = L;
#pragma unroll
        for (int s = 0; s < 16; ++s) wts[idx * 17 + s] = mv[s];
    }
    consumer_sync();
    for (int idx = threadIdx.x; idx < NT * a.qd; idx += MK_CONSUMERS) {
        int t = idx / a.qd, rem = idx - t * a.qd;
        float out = 0.f;
        if (t < a.n_tok) {
            int head = rem / a.dh, d = rem - head * a.dh;
            int ns = mk_token_splits((int)a.pos[t] + 1, a.s_max);
            const float *base = a.attn_part + ((size_t)(t * a.nh + head) * a.s_max) * DHP + d;
            const float *w = wts + (size_t)(t * a.nh + head) * 17;
            float ov[16];
#pragma unroll
            for (int s = 0; s < 16; ++s) ov[s] = s < ns ? __ldcg(base + (size_t)s * DHP) : 0.f;
            float O = 0.f;
#pragma unroll
            for (int s = 0; s < 16; ++s) O = fmaf(ov[s], w[s], O);
            out = O / w[16];
        }
        xs[(size_t)t * ph.in + rem] = Act<T>::from_f(out);
    }
    consumer_sync();
}

// ------------------------------------------------------------------ attention phase
template <class T, int DH>
__device__ void mk_attention(const MkArgs &a, const MkPhase &ph, float *scratch) {
    constexpr int EPL = DH / 32;  // elements per lane
    constexpr int MAXG = 8;
    const int G = a.nh / a.nkvh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int units = a.n_tok * a.nkvh * a.s_max;
    const int u = blockIdx.x;
    if (u >= units) return;
    const int t = u / (a.nkvh * a.s_max), h = (u / a.s_max) % a.nkvh, s = u % a.s_max;
    const int ctx = (int)a.pos[t] + 1;
    const int ns = mk_token_splits(ctx, a.s_max);
    if (s >= ns) return;
    const int tps = (ctx + ns - 1) / ns;
    const int j0 = s * tps, j1 = min(ctx, j0 + tps);
    if (j0 >= j1) {  // an empty split still has to leave a neutral partial for the merge
        for (int i = tid; i < G; i += MK_CONSUMERS) {
            float *dst = a.attn_part + ((size_t)(t * a.nh + h * G + i) * a.s_max + s) * (DH + 2);
            dst[DH] = -INFINITY;
            dst[DH + 1] = 0.f;
        }
        return;
    }
    const T *kv_pool = reinterpret_cast<const T *>(a.kv_pool);
    const float scale = 1.0f / sqrtf((float)DH);

    float qf[MAXG][EPL], of[MAXG][EPL], m[MAXG], l[MAXG];
    {
        const T *qg = reinterpret_cast<const T *>(a.q) + (size_t)t * a.qd + (size_t)h * G * DH;
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                of[g][e] = 0.f;
                unsigned short bits = g < G ? __ldcg(reinterpret_cast<const unsigned short *>(qg) + g * DH + lane * EPL + e)
                                            : (unsigned short)0;
                qf[g][e] = mk_bits_to_f<T>(bits);
            }
        }
    }
    for (int jb = j0 + warp; jb < j1; jb += 2 * MK_WARPS) {
        float kf[2][EPL], vf[2][EPL];
        bool have[2];
#pragma unroll
        for (int u2 = 0; u2 < 2; ++u2) {
            const int j = jb + u2 * MK_WARPS;
            have[u2] = j < j1;
            const int jj = have[u2] ? j : jb;
            int page = a.page_table[(size_t)t * a.pt_stride + (jj >> a.geom.page_shift)];
            int slot = jj & (a.geom.page_tokens - 1);
            size_t off = a.geom.block_off(page, ph.layer, 0, h) + (size_t)slot * DH + lane * EPL;
            if constexpr (EPL == 4) {
                uint2 kk = __ldcg(reinterpret_cast<const uint2 *>(kv_pool + off));
                uint2 vv = __ldcg(reinterpret_cast<const uint2 *>(kv_pool + off + (size_t)a.geom.nkvh * a.geom.page_tokens * DH));
                float2 k0 = Act<T>::to_f2(kk.x), k1 = Act<T>::to_f2(kk.y), v0 = Act<T>::to_f2(vv.x), v1 = Act<T>::to_f2(vv.y);
                kf[u2][0] = k0.x; kf[u2][1] = k0.y; kf[u2][2] = k1.x; kf[u2][3] = k1.y;
                vf[u2][0] = v0.x; vf[u2][1] = v0.y; vf[u2][2] = v1.x; vf[u2][3] = v1.y;
            } else {
                uint32_t kk = __ldcg(reinterpret_cast<const uint32_t *>(kv_pool + off));
                uint32_t vv = __ldcg(reinterpret_cast<const uint32_t *>(kv_pool + off + (size_t)a.geom.nkvh * a.geom.page_tokens * DH));
                float2 k0 = Act<T>::to_f2(kk), v0 = Act<T>::to_f2(vv);
                kf[u2][0] = k0.x; kf[u2][1] = k0.y;
                vf[u2][0] = v0.x; vf[u2][1] = v0.y;
            }
        }
#pragma unroll
        for (int u2 = 0; u2 < 2; ++u2) {
            if (!have[u2]) continue;
#pragma unroll
            for (int g = 0; g < MAXG; ++g) {
                if (g < G) {
                    float d = 0.f;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) d = fmaf(qf[g][e], kf[u2][e], d);
                    float sc = warp_sum(d) * scale;
                    float mn = fmaxf(m[g], sc);
                    float c = m[g] == -INFINITY ? 0.f : expf(m[g] - mn);
                    float p = expf(sc - mn);
                    l[g] = l[g] * c + p;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) of[g][e] = of[g][e] * c + p * vf[u2][e];
                    m[g] = mn;
                }
            }
        }
    }
    // per-warp partials -> shared scratch [warp][g][DH + 2]
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
        if (g < G) {
            float *dst = scratch + ((size_t)warp * G + g) * (DH + 2);
#pragma unroll
            for (int e = 0; e < EPL; ++e) dst[lane * EPL + e] = of[g][e];
            if (lane == 0) {
                dst[DH] = m[g];
                dst[DH + 1] = l[g];
            }
        }
    }
    consumer_sync();
    for (int idx = tid; idx < G * DH; idx += MK_CONSUMERS) {
        int g = idx / DH, d = idx - g * DH;
        float M = -INFINITY;
        for (int w = 0; w < MK_WARPS; ++w) M = fmaxf(M, scratch[((size_t)w * G + g) * (DH + 2) + DH]);
        float L = 0.f, O = 0.f;
        for (int w = 0; w < MK_WARPS; ++w) {
            const float *src = scratch + ((size_t)w * G + g) * (DH + 2);
            float wt = src[DH] == -INFINITY ? 0.f : expf(src[DH] - M);
            L = fmaf(src[DH + 1], wt, L);
            O = fmaf(src[d], wt, O);
        }
        float *dst = a.attn_part + ((size_t)(t * a.nh + h * G + g) * a.s_max + s) * (DH + 2);
        dst[d] = O;
        if (d == 0) {
            dst[DH] = M;
            dst[DH + 1] = L;
        }
    }
}

// ------------------------------------------------------------------ epilogues (one pair of rows, one token)
template <class T>
__device__ __forceinline__ void mk_epilogue(const MkArgs &a, const MkPhase &ph, int pair, int t, float va, float vb,
                                            float &best_v, uint32_t &best_i) {
    switch (ph.kind) {
    case MK_QKV: {
        int r = pair * 2;
        float xa = round_act<T>(va), xb = round_act<T>(vb);
        int sect = r < a.qd ? 0 : (r < a.qd + a.kvd ? 1 : 2);
        int rr = r - (sect == 0 ? 0 : (sect == 1 ? a.qd : a.qd + a.kvd));
        int head = rr / a.dh, e = rr - head * a.dh;
        uint32_t p = a.pos[t];
        if (sect < 2) {
            int half_dh = a.dh >> 1;
            float sn = a.sin_t[(size_t)p * half_dh + (e >> 1)], cs = a.cos_t[(size_t)p * half_dh + (e >> 1)];
            float ya = xa * cs - xb * sn, yb = xa * sn + xb * cs;
            xa = ya;
            xb = yb;
        }
        uint32_t packed = Act<T>::pack(xa, xb);
        if (sect == 0) {
            *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.q) + (size_t)t * a.qd + r) = packed;
        } else {
            int page = a.page_table[(size_t)t * a.pt_stride + (p >> a.geom.page_shift)];
            int slot = p & (a.geom.page_tokens - 1);
            size_t off = a.geom.block_off(page, ph.layer, sect - 1, head) + (size_t)slot * a.dh + e;
            *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.kv_pool) + off) = packed;
        }
        break;
    }
    case MK_O:
    case MK_DOWN: {
        int r = pair * 2;
        uint32_t *px = reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.x) + (size_t)t * a.d + r);
        float2 rf = Act<T>::to_f2(__ldcg(px));
        *px = Act<T>::pack(va + rf.x, vb + rf.y);
        break;
    }
    case MK_GATE_UP: {
        float g = round_act<T>(va), u = round_act<T>(vb);
        reinterpret_cast<T *>(a.act)[(size_t)t * a.di + pair] = Act<T>::from_f(mk_swiglu(g, u));
        break;
    }
    case MK_HEAD: {
        int r = pair * 2;
        uint32_t packed = Act<T>::pack(va, vb);
        *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.logits) + (size_t)t * a.vocab + r) = packed;
        float2 lf = Act<T>::to_f2(packed);  // compare the ROUNDED logits, lowest index wins ties
        if (best_i == 0xffffffffu || lf.x > best_v) { best_v = lf.x; best_i = (uint32_t)r; }
        if (lf.y > best_v) { best_v = lf.y; best_i = (uint32_t)r + 1; }
        break;
    }
    }
}

// ------------------------------------------------------------------ the kernel
template <class T, int NT>
__global__ void __launch_bounds__(MK_THREADS, 1) decode_step_kernel(const MkArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: [ring: n_stages x 32 KB][x / attention scratch][partials][control]
    unsigned char *ring = smem;
    T *xs = reinterpret_cast<T *>(smem + (size_t)a.n_stages * MK_STAGE_BYTES);
    float *part = reinterpret_cast<float *>(smem + (size_t)a.n_stages * MK_STAGE_BYTES + a.smem_x_bytes);  // [2*stages][16][MAX_R*NT]
    MkShared *sh = reinterpret_cast<MkShared *>(reinterpret_cast<unsigned char *>(part) + a.smem_part_bytes);

    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int i = 0; i < a.n_stages; ++i) {
            mbar_init(smem_u32(&sh->full[i]), 1);
            mbar_init(smem_u32(&sh->empty[i]), MK_GROUP_WARPS);
        }
        sh->abort_flag = 0;
        for (int i = 0; i < 16; ++i) sh->cnt[i] = 0;
        for (int i = 0; i < 8; ++i) sh->rel[i] = 0;
        sh->issued = -1;
        sh->consumed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (tid >= MK_CONSUMERS) {
        // ---------------- producer warp: one elected lane streams every weight tile of this CTA
        if (tid == MK_CONSUMERS) mk_producer(a, sh, ring);
    } else {
        // ---------------- consumers
        const int lane = tid & 31, warp = tid >> 5;
        // token ids of the round, with the device-side feedback of the previous round applied
        if (tid < MK_MAX_NT) {
            uint32_t tok = 0;
            if (tid < a.n_tok) {
                tok = a.tokens[tid];
                for (int i = 0; i < a.n_fast; ++i)
                    if (a.fast_map[2 * i + 1] == (uint32_t)tid) tok = a.pre_pairs_in[a.fast_map[2 * i]].idx;
            }
            sh->tok[tid] = tok;
        }
        consumer_sync();

        unsigned bar_target = 0;
        int gcount = 0, tidx = 0;           // row groups / weight tiles consumed so far by the whole CTA
        const int wg = warp / MK_GROUP_WARPS, wl = warp % MK_GROUP_WARPS, gtid = tid % MK_GROUP_THREADS;
        const int nbuf = 2 * a.n_stages;  // partial-sum buffers: no warp runs more than a ring ahead
        bool dead = false;

        // optional cycle counters (thread 0 of CTA 0): [kind] tile loops, [8] barriers, [9] prologues, [10] pipeline waits
        const bool prof = a.prof && blockIdx.x == 0 && tid == 0;
        long long t_wait = 0;
        for (int pi = 0; pi < a.n_phases && !dead; ++pi) {
            const MkPhase ph = a.phases[pi];
            long long c0 = clock64();
            if (ph.kind == MK_ATTN) {
                if (a.dh == 128) mk_attention<T, 128>(a, ph, reinterpret_cast<float *>(xs));
                else mk_attention<T, 64>(a, ph, reinterpret_cast<float *>(xs));
                long long c1 = clock64();
                mk_grid_barrier(a, bar_target, sh);
                if (prof) { a.prof[MK_ATTN] += c1 - c0; a.prof[8] += clock64() - c1; }
                dead = sh->abort_flag != 0;
                continue;
            }
            // ---- prologue: activations of this phase into shared memory
            switch (ph.kind) {
            case MK_QKV: mk_prologue_rmsnorm<T, NT>(a, ph, sh, xs, ph.layer == 0, false); break;
            case MK_GATE_UP: mk_prologue_rmsnorm<T, NT>(a, ph, sh, xs, false, false); break;
            case MK_HEAD: mk_prologue_rmsnorm<T, NT>(a, ph, sh, xs, false, true); break;
            case MK_O: mk_prologue_attn_merge<T, NT>(a, ph, xs, part); break;
            default: mk_prologue_copy<T, NT>(a, ph, xs, a.act, a.di); break;
            }
            long long c1 = clock64();
            // ---- tiles.  The 16 consumer warps form 4 groups of 4; group k takes every 4th row
            // group of the phase, so four row groups are in flight per CTA and each warp does
            // enough work per tile to cover the fixed latency of a wait / reduce / epilogue.
            // There is no CTA-wide synchronisation in this loop: the warps of a group leave
            // partial sums in a buffer of the row group and the LAST one to arrive (shared-memory
            // counter) adds them in a fixed order and runs the epilogue.
            int p_begin, p_end;
            mk_pair_range(ph.n_pairs, p_begin, p_end);
            const int R = ph.R, RP = R >> 1;
            const int nv = ph.KC / 8;
            // narrow rows: split the rows of a tile over thread sub-groups so that no thread idles
            int cpp = (nv + 31) & ~31;
            if (cpp > MK_GROUP_THREADS || MK_GROUP_THREADS % cpp) cpp = MK_GROUP_THREADS;
            const int rsplit = MK_GROUP_THREADS / cpp, col0 = gtid % cpp, rpart = gtid / cpp;
            float best_v = -INFINITY;
            uint32_t best_i = 0xffffffffu;
            for (int p0 = p_begin; p0 < p_end && !dead; p0 += RP, ++gcount, tidx += ph.n_kc) {
                if ((gcount & (MK_GROUPS - 1)) != wg) continue;
                float acc[MK_MAX_R][NT];
#pragma unroll
                for (int r = 0; r < MK_MAX_R; ++r)
#pragma unroll
                    for (int t = 0; t < NT; ++t) acc[r][t] = 0.f;
                for (int kc = 0; kc < ph.n_kc; ++kc) {
                    const int ti = tidx + kc;
                    const int slot = ti % a.n_stages;
                    const int lap = ti / a.n_stages;
                    const uint32_t parity = (uint32_t)lap & 1u;
                    long long w0 = prof ? clock64() : 0;
                    // A parity wait can only tell one ring lap from the next.  Only this group waits
                    // for this tile, so it must first know that the slot's previous lap is over
                    // (released by its owners): then the barrier can only be in this lap.
                    bool ok = true;
                    if (lap > 0) {
                        const volatile int *rel = &sh->rel[slot];
                        if (*rel < MK_GROUP_WARPS * lap) {
                            unsigned long long t0 = global_ns();
                            for (unsigned it = 1; *rel < MK_GROUP_WARPS * lap; ++it)
                                if ((it & 255u) == 0 && (sh->abort_flag || global_ns() - t0 > MK_WAIT_NS)) { ok = false; break; }
                        }
                    }
                    if (!ok || !mbar_wait(smem_u32(&sh->full[slot]), parity, &sh->abort_flag)) {
                        atomicOr(a.status, 2u);
                        sh->abort_flag = 1;
                        dead = true;
                        break;
                    }
                    if (prof) t_wait += clock64() - w0;
                    const uint4 *tile = reinterpret_cast<const uint4 *>(ring + (size_t)slot * MK_STAGE_BYTES);
                    for (int col = col0; col < nv; col += cpp) {
                        uint4 xv[NT];
#pragma unroll
                        for (int t = 0; t < NT; ++t) xv[t] = reinterpret_cast<const uint4 *>(xs + (size_t)t * ph.in)[kc * nv + col];
#pragma unroll
                        for (int r = 0; r < MK_MAX_R; ++r) {
                            if (r < R && (r & (rsplit - 1)) == (rpart & (rsplit - 1))) {
                                const uint4 wv = tile[(size_t)r * nv + col];
#pragma unroll
                                for (int t = 0; t < NT; ++t) acc[r][t] = dot8_mixed<T>(wv, xv[t], acc[r][t]);
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(smem_u32(&sh->empty[slot]));
                        atomicAdd(&sh->rel[slot], 1);
                    }
                }
                if (dead) break;
                const int gb = gcount % nbuf;
                float *pbuf = part + (size_t)gb * MK_GROUP_WARPS * (MK_MAX_R * NT);
#pragma unroll
                for (int r = 0; r < MK_MAX_R; ++r) {
                    if (r < R) {
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            float v = warp_sum(acc[r][t]);
                            if (lane == 0) pbuf[wl * (MK_MAX_R * NT) + r * NT + t] = v;
                        }
                    }
                }
                int last = 0;
                if (lane == 0) {
                    __threadfence_block();
                    last = atomicAdd(&sh->cnt[gb], 1) == MK_GROUP_WARPS - 1;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence_block();
                    if (lane == 0) sh->cnt[gb] = 0;
                    if (lane < RP * NT) {
                        int i = lane / NT, t = lane - i * NT;
                        int p = p0 + i;
                        if (p < p_end && t < a.n_tok) {
                            int ra = ph.swiglu_di > 0 ? i : 2 * i, rb = ph.swiglu_di > 0 ? RP + i : 2 * i + 1;
                            const volatile float *pv = pbuf;
                            float va = 0.f, vb = 0.f;
#pragma unroll
                            for (int w = 0; w < MK_GROUP_WARPS; ++w) {
                                va += pv[w * (MK_MAX_R * NT) + ra * NT + t];
                                vb += pv[w * (MK_MAX_R * NT) + rb * NT + t];
                            }
                            mk_epilogue<T>(a, ph, p, t, va, vb, best_v, best_i);
                        }
                    }
                }
            }
            if (ph.kind == MK_HEAD && !dead) {
                // per-CTA arg-max: every warp may have finalised some groups
                if (lane < 16) {
                    sh->fin_v[warp * 16 + lane] = best_v;
                    sh->fin_i[warp * 16 + lane] = best_i;
                }
                consumer_sync();
                if (tid < a.n_tok) {
                    float bv = -INFINITY;
                    uint32_t bi = 0xffffffffu;
                    for (int w = 0; w < MK_WARPS; ++w)
                        for (int i = 0; i < RP; ++i) {
                            float v = sh->fin_v[w * 16 + i * NT + tid];
                            uint32_t ix = sh->fin_i[w * 16 + i * NT + tid];
                            if (ix != 0xffffffffu && (bi == 0xffffffffu || v > bv || (v == bv && ix < bi))) { bv = v; bi = ix; }
                        }
                    a.head_best_v[(size_t)blockIdx.x * NT + tid] = bv;
                    a.head_best_i[(size_t)blockIdx.x * NT + tid] = bi;
                }
            }
            long long c2 = clock64();
            mk_grid_barrier(a, bar_target, sh);
            if (prof) { a.prof[9] += c1 - c0; a.prof[ph.kind] += c2 - c1; a.prof[8] += clock64() - c2; }
            dead = dead || sh->abort_flag != 0;
        }
        if (prof) { a.prof[10] += t_wait; a.prof[11] += 1; }
        // ---- final: CTA 0 folds the per-CTA winners into one pair per token
        if (!dead && blockIdx.x == 0 && warp < a.n_tok) {
            const int t = warp;
            float bv = -INFINITY;
            uint32_t bi = 0xffffffffu;
            for (int b = lane; b < (int)gridDim.x; b += 32) {
                float v = __ldcg(a.head_best_v + (size_t)b * NT + t);
                uint32_t ix = __ldcg(a.head_best_i + (size_t)b * NT + t);
                if (ix != 0xffffffffu && (bi == 0xffffffffu || v > bv || (v == bv && ix < bi))) { bv = v; bi = ix; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0xffffffffu && (bi == 0xffffffffu || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
            }
            if (lane == 0) {
                lcu_kv_pair r;
                r.idx = bi;
                r.val = __ldcg(reinterpret_cast<const unsigned short *>(a.logits) + (size_t)t * a.vocab + bi);
                r.pad = 0;
                a.out[t] = r;
                if (a.out_copy) a.out_copy[t] = r;
            }
        }
    }
    // ---- drain: never leave with bulk copies still in flight into this CTA's shared memory
    __syncthreads();
    if (tid == 0 && sh->abort_flag) {
        const int issued = sh->issued;
        int dummy = 0;
        for (int i = issued > a.n_stages ? issued - a.n_stages : 0; i < issued; ++i)
            mbar_wait(smem_u32(&sh->full[i % a.n_stages]), (uint32_t)(i / a.n_stages) & 1u, &dummy);
    }
}

// ------------------------------------------------------------------ host side

bool mk_plan_tiles(int in, int *R, int *KC, int *n_kc) {
    if (in <= 0 || in % 8) return false;
    const int cap = MK_STAGE_BYTES / 2;  // elements per stage
    if (2 * in <= cap) {
        int r = cap / in;
        r = r >= 8 ? 8 : (r >= 4 ? 4 : 2);
        *R = r; *KC = in; *n_kc = 1;
        return true;
    }
    for (int n = 2; n <= 64; ++n) {
        if (in % n) continue;
        int kc = in / n;
        if (kc % 8) continue;
        if (2 * kc <= cap) {
            *R = 2; *KC = kc; *n_kc = n;
            return true;
        }
    }
    return false;
}

int mk_splits(int grid, int n_tok, int nkvh) {
    int s = grid / (n_tok * nkvh);
    if (s > 16) s = 16;
    if (s < 1) s = 1;
    return s;
}

size_t mk_smem_bytes(int n_tok, int max_in, int nh, int nkvh, int dh, int *n_stages, int *x_bytes, int *part_bytes) {
    int nt = n_tok <= 1 ? 1 : (n_tok == 2 ? 2 : 4);
    size_t x = (size_t)nt * max_in * 2;
    size_t attn = (size_t)MK_WARPS * (nh / nkvh) * (dh + 2) * 4;
    if (attn > x) x = attn;
    x = (x + 127) & ~(size_t)127;
    const size_t limit = 227 * 1024;
    const size_t ctl = sizeof(MkShared) + 256;
    const size_t merge = (size_t)nt * nh * 17 * 4;               // split weights of the attention merge
    const size_t per_stage_part = (size_t)2 * MK_GROUP_WARPS * MK_MAX_R * nt * 4;  // two partial buffers per stage
    for (int stages = 8; stages >= 2; --stages) {
        size_t part = stages * per_stage_part;
        if (part < merge) part = merge;
        part = (part + 127) & ~(size_t)127;
        size_t total = (size_t)stages * MK_STAGE_BYTES + x + part + ctl;
        if (total <= limit) {
            *n_stages = stages;
            *x_bytes = (int)x;
            *part_bytes = (int)part;
            return total;
        }
    }
    return 0;
}

template <class T, int NT>
static int mk_prepare_inst(size_t smem) {
    auto kernel = decode_step_kernel<T, NT>;
    LCU_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int occ = 0;
    LCU_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, MK_THREADS, smem));
    if (occ < 1) {
        set_error("decode_step_kernel does not fit on an SM with %zu bytes of shared memory", smem);
        return LCU_ERR_INVALID;
    }
    return LCU_OK;
}

int mk_prepare(int dt, int n_tok, size_t smem) {
    int dev = 0, coop = 0;
    LCU_CHECK_CUDA(cudaGetDevice(&dev));
    LCU_CHECK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) {
        set_error("device does not support cooperative launches");
        return LCU_ERR_INVALID;
    }
    int nt = n_tok <= 1 ? 1 : (n_tok == 2 ? 2 : 4);
    if (dt == LCU_F16) return nt == 1 ? mk_prepare_inst<__half, 1>(smem) : (nt == 2 ? mk_prepare_inst<__half, 2>(smem) : mk_prepare_inst<__half, 4>(smem));
    if (dt == LCU_BF16) return nt == 1 ? mk_prepare_inst<__nv_bfloat16, 1>(smem) : (nt == 2 ? mk_prepare_inst<__nv_bfloat16, 2>(smem) : mk_prepare_inst<__nv_bfloat16, 4>(smem));
    set_error("decode_step_kernel: dtype %d unsupported", dt);
    return LCU_ERR_INVALID;
}

template <class T, int NT>
static int mk_launch_inst(const MkArgs &a, size_t smem, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(MK_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LCU_CHECK_CUDA(cudaLaunchKernelEx(&cfg, decode_step_kernel<T, NT>, a));
    return LCU_OK;
}

int mk_launch(const MkArgs &a, int dt, size_t smem, cudaStream_t s) {
    int nt = a.n_tok <= 1 ? 1 : (a.n_tok == 2 ? 2 : 4);
    if (dt == LCU_F16) return nt == 1 ? mk_launch_inst<__half, 1>(a, smem, s) : (nt == 2 ? mk_launch_inst<__half, 2>(a, smem, s) : mk_launch_inst<__half, 4>(a, smem, s));
    if (dt == LCU_BF16) return nt == 1 ? mk_launch_inst<__nv_bfloat16, 1>(a, smem, s) : (nt == 2 ? mk_launch_inst<__nv_bfloat16, 2>(a, smem, s) : mk_launch_inst<__nv_bfloat16, 4>(a, smem, s));
    set_error("decode_step_kernel: dtype %d unsupported", dt);
    return LCU_ERR_INVALID;
}

}  // namespace lcu
