// Causal GQA attention over the KV cache — the sm_100a counterpart of
// `operators::attention_kv_cached`, which the reference launches once per request and per
// layer outside its CUDA graphs (llama.cu/src/exec/step.rs:140-184).  Here ONE launch per
// layer covers every token of the round, inside the step's graph.
//
// Arithmetic (the external operator's source is not part of the reference tree, so this
// is the stated contract rather than a transcription): score = (q·k) / sqrt(dh) in f32,
// softmax in f32 over positions [0, pos], output = sum p·v in f32, one rounding to the
// activation dtype.  Query head h reads KV head h / (nh/nkvh).
//
// Shape of the kernel: a CTA owns (token, KV head, split) and serves all G = nh/nkvh
// query heads of that KV head from one pass over the keys/values (GQA packing: KV bytes
// are read once per group, not once per query head).  KV rows are gathered page by page
// through the page table into a double-buffered shared-memory tile with 16-byte
// cp.async copies (rows past the context are zero-filled), scores/softmax/PV run out of
// shared memory with an online (running max / running sum) softmax.  The context is cut
// into `n_splits` ranges (flash-decoding); each split leaves an unnormalised partial and
// its (max, sum) in scratch memory and the last split to arrive — found with an atomic
// ticket — merges them, so no second launch is needed.
#include "attention.cuh"

#include <map>
#include <mutex>

namespace lcu {

constexpr int ATT_TILE = 64;
constexpr int ATT_THREADS = 128;

__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gsrc, bool valid) {
    unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <class T, int DH, int G>
__global__ void __launch_bounds__(ATT_THREADS) attn_kernel(const AttnArgs a) {
    constexpr int ROW = DH + 8;        // padded row (elements): 16 extra bytes break bank conflicts
    constexpr int CH = DH / 8;         // 16-byte chunks per row
    constexpr int NP = DH / 2;         // dimension pairs of a head
    constexpr int NGRP = ATT_THREADS / NP;           // thread groups in the P·V phase
    constexpr int HG = (G + NGRP - 1) / NGRP;        // heads per group
    extern __shared__ __align__(16) unsigned char smem[];
    T *Ks = reinterpret_cast<T *>(smem);                 // [TILE][ROW]
    T *Vs = Ks + ATT_TILE * ROW;                         // [TILE][ROW]
    T *qs = Vs + ATT_TILE * ROW;                         // [G][DH] in the activation dtype
    float *S = reinterpret_cast<float *>(qs + G * DH);   // [G][TILE] scores, then probabilities
    float *Sp = S + G * ATT_TILE;                        // [2][G][TILE] half-row partial dots
    float *corr = Sp + 2 * G * ATT_TILE;                 // [G]
    float *m_run = corr + G;                             // [G]
    float *l_run = m_run + G;                            // [G]
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hkv = blockIdx.x, t = blockIdx.y, sp = blockIdx.z;
    const T *kv_pool = reinterpret_cast<const T *>(a.kv_pool);
    const bool paged = kv_pool != nullptr;

    grid_dep_launch();
    grid_dep_wait();

    const int ctx = paged ? (int)a.tok_pos[t] + 1 : a.pos0 + t + 1;
    const int seq = paged ? a.tok_seq[t] : 0;
    const int n_tiles = (ctx + ATT_TILE - 1) / ATT_TILE;
    // splits of THIS token: fixed work per CTA, so short and long contexts of one round balance
    int tps = (n_tiles + a.n_splits - 1) / a.n_splits;
    if (a.tiles_per_split > tps) tps = a.tiles_per_split;
    const int my_splits = (n_tiles + tps - 1) / tps;
    if (sp >= my_splits) return;
    const int tile0 = sp * tps;
    const int tile1 = min(n_tiles, tile0 + tps);
    const float scale = 1.0f / sqrtf((float)DH);

    {
        const T *qg = reinterpret_cast<const T *>(a.q) + (size_t)t * a.stride_q + (size_t)hkv * G * DH;
        for (int i = tid; i < G * DH; i += ATT_THREADS) qs[i] = qg[i];
        if (tid < G) {
            m_run[tid] = -INFINITY;
            l_run[tid] = 0.f;
            corr[tid] = 1.f;
        }
    }

    auto load_tile = [&](int tile) {
        T *kd = Ks, *vd = Vs;
#pragma unroll
        for (int i = 0; i < (ATT_TILE * CH) / ATT_THREADS; ++i) {
            int c = tid + ATT_THREADS * i;
            int j = c / CH, col = c - j * CH;
            int pos = tile * ATT_TILE + j;
            bool valid = pos < ctx;
            const T *ksrc, *vsrc;
            if (paged) {
                int page = valid ? a.page_table[(size_t)seq * a.pt_stride + (pos >> a.geom.page_shift)] : 0;
                int slot = pos & (a.geom.page_tokens - 1);
                size_t off = a.geom.block_off(page, a.layer, 0, hkv) + (size_t)slot * DH + col * 8;
                ksrc = kv_pool + (valid ? off : 0);
                vsrc = kv_pool + (valid ? off + (size_t)a.geom.nkvh * a.geom.page_tokens * DH : 0);
            } else {
                const T *kl = reinterpret_cast<const T *>(a.k_lin), *vl = reinterpret_cast<const T *>(a.v_lin);
                ksrc = valid ? kl + (size_t)pos * a.stk + (size_t)hkv * a.shk + col * 8 : kl;
                vsrc = valid ? vl + (size_t)pos * a.stv + (size_t)hkv * a.shv + col * 8 : vl;
            }
            cp_async_16(kd + j * ROW + col * 8, ksrc, valid);
            cp_async_16(vd + j * ROW + col * 8, vsrc, valid);
        }
    };

    // P·V ownership: thread = (dimension pair dp, head group gh)
    const int dp = tid % NP, gh = tid / NP;
    float acc[HG][2];
#pragma unroll
    for (int i = 0; i < HG; ++i) acc[i][0] = acc[i][1] = 0.f;
    // score ownership: thread = (position j, half of the head dimension hf)
    const int sj = tid & (ATT_TILE - 1), hf = tid / ATT_TILE;

    // One tile buffer per CTA: several CTAs share an SM (shared memory allows 5), so the loads of one
    // overlap the arithmetic of the others.
    for (int tile = tile0; tile < tile1; ++tile) {
        load_tile(tile);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        const T *kt = Ks, *vt = Vs;

        // scores: a thread reads half of one K row ONCE and dots it with all G query heads
        // (q is broadcast from shared memory; mixed-precision FMA, no conversions)
        {
            const uint4 *kr = reinterpret_cast<const uint4 *>(kt + sj * ROW) + hf * (CH / 2);
            float d[G];
#pragma unroll
            for (int g = 0; g < G; ++g) d[g] = 0.f;
#pragma unroll
            for (int c = 0; c < CH / 2; ++c) {
                const uint4 kv = kr[c];
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const uint4 qv = reinterpret_cast<const uint4 *>(qs + g * DH)[hf * (CH / 2) + c];
                    d[g] = dot8_mixed<T>(kv, qv, d[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) Sp[(hf * G + g) * ATT_TILE + sj] = d[g];
        }
        __syncthreads();

        // online softmax, one warp per head
        for (int g = warp; g < G; g += ATT_THREADS / 32) {
            const int p0 = tile * ATT_TILE + lane, p1 = p0 + 32;
            float s0 = p0 < ctx ? (Sp[g * ATT_TILE + lane] + Sp[(G + g) * ATT_TILE + lane]) * scale : -INFINITY;
            float s1 = p1 < ctx ? (Sp[g * ATT_TILE + lane + 32] + Sp[(G + g) * ATT_TILE + lane + 32]) * scale : -INFINITY;
            float mt = warp_max(fmaxf(s0, s1));
            float mo = m_run[g];
            float mn = fmaxf(mo, mt);
            float pa = s0 == -INFINITY ? 0.f : expf(s0 - mn);
            float pb = s1 == -INFINITY ? 0.f : expf(s1 - mn);
            float sum = warp_sum(pa + pb);
            S[g * ATT_TILE + lane] = pa;
            S[g * ATT_TILE + lane + 32] = pb;
            if (lane == 0) {
                float c = mo == -INFINITY ? 0.f : expf(mo - mn);
                corr[g] = c;
                l_run[g] = l_run[g] * c + sum;
                m_run[g] = mn;
            }
        }
        __syncthreads();

        // P·V: a thread owns two adjacent dimensions of HG heads; V is read as packed pairs
#pragma unroll
        for (int i = 0; i < HG; ++i) {
            const int g = gh * HG + i;
            if (g < G) {
                float c = corr[g];
                float o0 = acc[i][0] * c, o1 = acc[i][1] * c;
                const float *pr = S + g * ATT_TILE;
                const T *vcol = vt + 2 * dp;
#pragma unroll 8
                for (int j = 0; j < ATT_TILE; ++j) {
                    float2 v = Act<T>::to_f2(*reinterpret_cast<const uint32_t *>(vcol + j * ROW));
                    float pj = pr[j];
                    o0 = fmaf(pj, v.x, o0);
                    o1 = fmaf(pj, v.y, o1);
                }
                acc[i][0] = o0;
                acc[i][1] = o1;
            }
        }
        __syncthreads();
    }

    T *og = reinterpret_cast<T *>(a.o) + (size_t)t * a.stride_o + (size_t)hkv * G * DH;
    if (my_splits == 1) {
#pragma unroll
        for (int i = 0; i < HG; ++i) {
            const int g = gh * HG + i;
            if (g < G) {
                *reinterpret_cast<uint32_t *>(og + g * DH + 2 * dp) = Act<T>::pack(acc[i][0] / l_run[g], acc[i][1] / l_run[g]);
            }
        }
        return;
    }

    // leave the unnormalised partial and (max, sum); the last split to arrive merges
    const size_t head0 = (size_t)t * a.nh + (size_t)hkv * G;
#pragma unroll
    for (int i = 0; i < HG; ++i) {
        const int g = gh * HG + i;
        if (g < G) {
            float *dst = a.part_o + ((head0 + g) * a.n_splits + sp) * DH + 2 * dp;
            dst[0] = acc[i][0];
            dst[1] = acc[i][1];
        }
    }
    if (tid < G) {
        a.part_ml[((head0 + tid) * a.n_splits + sp) * 2] = m_run[tid];
        a.part_ml[((head0 + tid) * a.n_splits + sp) * 2 + 1] = l_run[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned ticket = atomicAdd(&a.counters[(size_t)t * a.nkvh + hkv], 1u);
        is_last = ticket == (unsigned)my_splits - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
#pragma unroll
    for (int i = 0; i < HG; ++i) {
        const int g = gh * HG + i;
        if (g < G) {
            const float *ml = a.part_ml + (head0 + g) * a.n_splits * 2;
            float M = -INFINITY;
            for (int s2 = 0; s2 < my_splits; ++s2) M = fmaxf(M, __ldcg(ml + 2 * s2));
            float L = 0.f, O0 = 0.f, O1 = 0.f;
            for (int s2 = 0; s2 < my_splits; ++s2) {
                float ms = __ldcg(ml + 2 * s2), ls = __ldcg(ml + 2 * s2 + 1);
                float w = ms == -INFINITY ? 0.f : expf(ms - M);
                L = fmaf(ls, w, L);
                float2 o = __ldcg(reinterpret_cast<const float2 *>(a.part_o + ((head0 + g) * a.n_splits + s2) * DH + 2 * dp));
                O0 = fmaf(o.x, w, O0);
                O1 = fmaf(o.y, w, O1);
            }
            *reinterpret_cast<uint32_t *>(og + g * DH + 2 * dp) = Act<T>::pack(O0 / L, O1 / L);
        }
    }
    if (tid == 0) a.counters[(size_t)t * a.nkvh + hkv] = 0;  // ready for the next launch
}

// ------------------------------------------------------------------ host side

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Scratch layout: arrival counters FIRST, at a fixed place and sized for the largest round,
// so that partial outputs of a round with another (tokens, splits) shape can never land on
// them — the counters must read zero whenever a launch starts.
size_t attn_scratch_bytes(int n_tok, int nh, int nkvh, int dh, int n_splits, int max_tok) {
    return align256((size_t)max_tok * nkvh * 4) + align256((size_t)n_tok * nh * n_splits * 2 * 4) +
           align256((size_t)n_tok * nh * n_splits * dh * 4);
}

void attn_bind_scratch(AttnArgs &a, void *scratch, int max_tok) {
    unsigned char *p = reinterpret_cast<unsigned char *>(scratch);
    a.counters = reinterpret_cast<unsigned *>(p);
    p += align256((size_t)max_tok * a.nkvh * 4);
    a.part_ml = reinterpret_cast<float *>(p);
    p += align256((size_t)a.n_tok * a.nh * a.n_splits * 2 * 4);
    a.part_o = reinterpret_cast<float *>(p);
}

template <class T, int DH, int G>
static int attn_inst(const AttnArgs &a, cudaStream_t s, bool pdl, bool dry) {
    auto kernel = attn_kernel<T, DH, G>;
    size_t smem = (size_t)2 * ATT_TILE * (DH + 8) * sizeof(T) + (size_t)G * DH * sizeof(T) +
                  (size_t)(3 * G * ATT_TILE + 3 * G) * sizeof(float);
    static std::mutex mu;
    static std::map<int, bool> done;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!done[dev]) {
            if (smem > 48 * 1024) LCU_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            done[dev] = true;
        }
    }
    if (dry) return LCU_OK;
    dim3 grid(a.nkvh, a.n_tok, a.n_splits);
    LCU_CHECK_CUDA(launch_kernel(kernel, grid, dim3(ATT_THREADS), smem, s, pdl, a));
    return LCU_OK;
}

template <class T, int DH>
static int attn_dh(const AttnArgs &a, cudaStream_t s, bool pdl, bool dry) {
    switch (a.nh / a.nkvh) {
    case 1: return attn_inst<T, DH, 1>(a, s, pdl, dry);
    case 2: return attn_inst<T, DH, 2>(a, s, pdl, dry);
    case 4: return attn_inst<T, DH, 4>(a, s, pdl, dry);
    case 8: return attn_inst<T, DH, 8>(a, s, pdl, dry);
    default: set_error("attention: nh/nkvh = %d unsupported (1, 2, 4, 8)", a.nh / a.nkvh); return LCU_ERR_INVALID;
    }
}

int attn_launch(const AttnArgs &a, int dt, cudaStream_t s, bool pdl, bool dry) {
    if (a.n_tok <= 0) return LCU_OK;
    LCU_REQUIRE(a.nkvh > 0 && a.nh % a.nkvh == 0, "attention: nh = %d is not a multiple of nkvh = %d", a.nh, a.nkvh);
    LCU_REQUIRE(a.dh == 64 || a.dh == 128, "attention: dh = %d unsupported (64, 128)", a.dh);
    LCU_REQUIRE(a.n_splits >= 1 && a.n_splits <= 65535 && a.n_tok <= 65535, "attention: grid out of range");
    LCU_REQUIRE(dry || a.n_splits == 1 || (a.part_o && a.part_ml && a.counters), "attention: split-KV needs scratch");
    if (!a.kv_pool && !dry) {
        LCU_REQUIRE(a.k_lin && a.v_lin, "attention: no cache given");
        LCU_REQUIRE(a.stk % 8 == 0 && a.shk % 8 == 0 && a.stv % 8 == 0 && a.shv % 8 == 0 &&
                        ((uintptr_t)a.k_lin % 16) == 0 && ((uintptr_t)a.v_lin % 16) == 0,
                    "attention: cache rows must be 16-byte aligned");
    }
    if (dt == LCU_F16) return a.dh == 64 ? attn_dh<__half, 64>(a, s, pdl, dry) : attn_dh<__half, 128>(a, s, pdl, dry);
    if (dt == LCU_BF16)
        return a.dh == 64 ? attn_dh<__nv_bfloat16, 64>(a, s, pdl, dry) : attn_dh<__nv_bfloat16, 128>(a, s, pdl, dry);
    set_error("attention: activation dtype %d unsupported", dt);
    return LCU_ERR_INVALID;
}

// ------------------------------------------------------------------ linear-cache append
template <class T>
__global__ void kv_append_kernel(T *kc, int stkc, int shkc, T *vc, int stvc, int shvc, const T *k, int stk, int shk,
                                 const T *v, int stv, int shv, int nkvh, int dh, int pos) {
    int t = blockIdx.y;
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nkvh * dh) return;
    int h = i / dh, e = i - h * dh;
    kc[(size_t)(pos + t) * stkc + (size_t)h * shkc + e] = k[(size_t)t * stk + (size_t)h * shk + e];
    vc[(size_t)(pos + t) * stvc + (size_t)h * shvc + e] = v[(size_t)t * stv + (size_t)h * shv + e];
}

int kv_append_linear(void *k_cache, int stkc, int shkc, void *v_cache, int stvc, int shvc, const void *k, int stk,
                     int shk, const void *v, int stv, int shv, int nkvh, int dh, int seq, int pos, int dt,
                     cudaStream_t s) {
    if (seq <= 0) return LCU_OK;
    dim3 grid((nkvh * dh + 255) / 256, seq), block(256);
    // f16 and bf16 are both 2-byte copies
    (void)dt;
    kv_append_kernel<uint16_t><<<grid, block, 0, s>>>((uint16_t *)k_cache, stkc, shkc, (uint16_t *)v_cache, stvc, shvc,
                                                      (const uint16_t *)k, stk, shk, (const uint16_t *)v, stv, shv,
                                                      nkvh, dh, pos);
    LCU_CHECK_CUDA(cudaGetLastError());
    return LCU_OK;
}

}  // namespace lcu
