// Causal GQA attention over the KV cache — the sm_100a counterpart of
// `operators::attention_kv_cached`, which the reference launches once per request and per
// layer outside its CUDA graphs (llama.cu/src/exec/step.rs:140-184).  Here ONE launch per
// layer covers every token of the round, inside the step's graph.
//
// Arithmetic (the external operator's source is not part of the reference tree, so this
// is the stated contract rather than a transcription): score = (q·k) / sqrt(dh) in f32,
// softmax in f32 over positions [0, pos], probabilities rounded to the activation dtype,
// output = sum p·v in f32, one rounding to the activation dtype.  Query head h reads KV
// head h / (nh/nkvh).
//
// Shape of the kernel: a CTA (4 warps) owns (KV head, token, split) and serves all
// G = nh/nkvh query heads of that KV head from one pass over the keys/values (GQA packing:
// KV bytes are read once per group, not once per query head).  K/V rows are gathered page
// by page through the page table into one K and one V shared-memory tile with 16-byte
// cp.async copies (rows past the context are zero-filled); both products run on tensor
// cores (mma.sync m16n8k16) with an online (running max / running sum) softmax between
// them.  The context is cut into splits (flash-decoding); the splits of a (token, KV head)
// merge either through distributed shared memory inside one thread-block cluster or
// through scratch memory where the last split to arrive — found with an atomic ticket —
// sums the partials, so no second launch is needed.
//
// Under programmatic dependent launch everything that depends only on the round
// descriptor (context length, page numbers, cached rows of earlier rounds) is done BEFORE
// the wait on the predecessor (the QKV projection, which writes q and the new K/V row).
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

__device__ __forceinline__ void ldmatrix_x4(uint32_t r[4], const void *smem_row) {
    unsigned a = (unsigned)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t r[4], const void *smem_row) {
    unsigned a = (unsigned)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// thread-block cluster helpers for the split-KV merge through distributed shared memory
__device__ __forceinline__ void att_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t att_map_peer(const void *local, uint32_t cta) {
    uint32_t la = (uint32_t)__cvta_generic_to_shared(local), ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(cta));
    return ra;
}
__device__ __forceinline__ void att_st_peer2(uint32_t ra, float x, float y) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1,%2};" ::"r"(ra), "f"(x), "f"(y) : "memory");
}
// Bytes of the decode kernel's shared memory in front of the cluster-merge region (K, V, probabilities, scores and
// the running softmax state), rounded up to 16.
template <class T, int DH, int G>
__host__ __device__ constexpr size_t att_merge_offset() {
    return ((size_t)2 * ATT_TILE * (DH + 8) * sizeof(T) + (size_t)16 * (ATT_TILE + 8) * sizeof(T) +
            (size_t)(G * ATT_TILE + 3 * G) * sizeof(float) + 15) / 16 * 16;
}
// Both products run on tensor cores (mma.sync m16n8k16, f32 accumulation):
//   scores  S[pos][head] = K[pos][:] . q[head][:]   M = 16 positions per warp, N = 8 head slots (G used), K = dh
//   output  O[head][d]   = P[head][:] . V[:][d]     M = 16 head slots (G used), N = dh / 4 per warp, K = 64 positions
// K and V fragments come from the shared-memory tile with ldmatrix (V transposed on the way), the query
// fragments stay in registers for the whole kernel, probabilities are rounded to the activation dtype
// before the second product and the row sum is taken over the rounded values.
template <class T, int DH, int G>
__global__ void __launch_bounds__(ATT_THREADS) attn_kernel(const AttnArgs a) {
    constexpr int ROW = DH + 8;        // padded K/V row (elements): 16 extra bytes keep ldmatrix conflict-free
    constexpr int PROW = ATT_TILE + 8; // padded probability row
    constexpr int CH = DH / 8;         // 16-byte chunks per row
    constexpr int KSTEPS = DH / 16;    // k-steps of the score product
    constexpr int DW = DH / 4;         // output dimensions per warp
    constexpr int NT = DW / 8;         // 8-wide output tiles per warp
    extern __shared__ __align__(16) unsigned char smem[];
    T *Ks = reinterpret_cast<T *>(smem);                 // [TILE][ROW]
    T *Vs = Ks + ATT_TILE * ROW;                         // [TILE][ROW]
    T *Ps = Vs + ATT_TILE * ROW;                         // [16][PROW] probabilities, rows >= G stay zero
    float *S = reinterpret_cast<float *>(Ps + 16 * PROW);  // [G][TILE] raw scores
    float *corr = S + G * ATT_TILE;                      // [G]
    float *m_run = corr + G;                             // [G]
    float *l_run = m_run + G;                            // [G]
    // cluster merge only: every split's unnormalised partial [z][G][DH] and (max, sum) [z][G][2], filled in the FIRST
    // split's shared memory by its peers
    float *mrg_o = reinterpret_cast<float *>(smem + att_merge_offset<T, DH, G>());
    float *mrg_ml = mrg_o + (size_t)a.cluster_z * G * DH;
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, t4 = lane & 3;
    const int hkv = blockIdx.x, t = blockIdx.y, sp = blockIdx.z;
    const T *kv_pool = reinterpret_cast<const T *>(a.kv_pool);
    const bool paged = kv_pool != nullptr;

    const int ctx = paged ? (int)a.tok_pos[t] + 1 : a.pos0 + t + 1;
    const int seq = paged ? a.tok_seq[t] : 0;
    const int n_tiles = (ctx + ATT_TILE - 1) / ATT_TILE;
    // splits of THIS token: fixed work per CTA, so short and long contexts of one round balance
    int tps = (n_tiles + a.n_splits - 1) / a.n_splits;
    if (a.tiles_per_split > tps) tps = a.tiles_per_split;
    const int my_splits = (n_tiles + tps - 1) / tps;
    // cluster_z > 0: the splits of a (token, KV head) are one thread-block cluster and merge through distributed
    // shared memory; CTAs without work still take part in its barrier
    const bool clus = a.cluster_z > 0;
    if (sp >= my_splits) {
        if (clus) att_cluster_sync();
        return;  // leaving counts as releasing the dependents
    }
    if (a.pdl_trigger == 0) grid_dep_launch();
    const int tile0 = sp * tps;
    const int tile1 = min(n_tiles, tile0 + tps);
    const float scale = 1.0f / sqrtf((float)DH);

    // Page numbers are fetched into shared memory a window of tiles at a time (128 pages: 32 to 128 tiles),
    // so the gathers below have no dependent global load in front of their copies.
    __shared__ int pg[128];
    const int ppt = paged ? (ATT_TILE >> a.geom.page_shift > 1 ? ATT_TILE >> a.geom.page_shift : 1) : 1;  // pages per tile
    const int WT = 128 / ppt;                                                                          // tiles per window
    auto fetch_window = [&](int tile_first) {
        if (!paged) return;
        for (int i = tid; i < 128; i += ATT_THREADS) {
            const long long first = (long long)tile_first * ATT_TILE + (long long)i * a.geom.page_tokens;
            pg[i] = first < ctx ? a.page_table[(size_t)seq * a.pt_stride + (int)(first >> a.geom.page_shift)] : 0;
        }
    };
    const size_t blk = paged ? (size_t)a.geom.page_tokens * DH : 0;
    const size_t kbase = paged ? ((size_t)(a.layer * 2) * a.geom.nkvh + hkv) * blk : 0;
    const size_t voff = paged ? (size_t)a.geom.nkvh * blk : 0;
    const int lcol8 = (tid % CH) * 8, j0 = tid / CH;  // this thread's 16-byte column and first row of a tile

    // gathers the K (which = 0) or V (which = 1) rows of a tile; rows past the context are zero-filled.
    // rows: 0 = every row, 1 = all but the token's own row (position ctx - 1), 2 = only that row
    auto load_rows = [&](int tile, int which, int rows) {
        T *dst = which ? Vs : Ks;
        const int w0 = ((tile - tile0) % WT) * ppt;
#pragma unroll
        for (int i = 0; i < (ATT_TILE * CH) / ATT_THREADS; ++i) {
            const int j = j0 + (ATT_THREADS / CH) * i;
            const int pos = tile * ATT_TILE + j;
            const bool valid = pos < ctx;
            if (rows == 1 && pos == ctx - 1) continue;
            if (rows == 2 && pos != ctx - 1) continue;
            const T *src;
            if (paged) {
                const int page = pg[w0 + (j >> a.geom.page_shift)];
                const int slot = pos & (a.geom.page_tokens - 1);
                src = kv_pool + (valid ? (size_t)page * a.geom.page_elems + kbase + (which ? voff : 0) + (size_t)slot * DH + lcol8 : 0);
            } else if (which) {
                const T *vl = reinterpret_cast<const T *>(a.v_lin);
                src = valid ? vl + (size_t)pos * a.stv + (size_t)hkv * a.shv + lcol8 : vl;
            } else {
                const T *kl = reinterpret_cast<const T *>(a.k_lin);
                src = valid ? kl + (size_t)pos * a.stk + (size_t)hkv * a.shk + lcol8 : kl;
            }
            cp_async_16(dst + j * ROW + lcol8, src, valid);
        }
    };
    fetch_window(tile0);
    for (int i = tid; i < 16 * PROW / 2; i += ATT_THREADS) reinterpret_cast<uint32_t *>(Ps)[i] = 0u;
    if (tid < G) {
        m_run[tid] = -INFINITY;
        l_run[tid] = 0.f;
        corr[tid] = 1.f;
    }
    __syncthreads();

    // One K and one V buffer per CTA, software-pipelined with two cp.async groups per tile: V(t) lands while
    // the scores and the softmax of tile t run, K(t+1) while the softmax and P.V of tile t run.  Several CTAs
    // share an SM (shared memory allows 5), which hides what is left.
    const bool early = paged && a.early_kv;
    if (early) {  // rows of earlier rounds: in flight while the predecessor drains
        load_rows(tile0, 0, 1);
        cp_async_commit();
        load_rows(tile0, 1, 1);
        cp_async_commit();
    }
    grid_dep_wait();

    // query fragments (B operand of the score product): head slot gid, k = 16 ks + 2 t4 (+8)
    uint32_t qb[KSTEPS][2];
    {
        const T *qg = reinterpret_cast<const T *>(a.q) + (size_t)t * a.stride_q + (size_t)hkv * G * DH + (size_t)gid * DH;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            qb[ks][0] = gid < G ? *reinterpret_cast<const uint32_t *>(qg + ks * 16 + 2 * t4) : 0u;
            qb[ks][1] = gid < G ? *reinterpret_cast<const uint32_t *>(qg + ks * 16 + 8 + 2 * t4) : 0u;
        }
    }
    if (early) {  // the row the predecessor has just written (if this split holds it)
        load_rows(tile0, 0, 2);
        load_rows(tile0, 1, 2);
        cp_async_commit();
    } else {
        load_rows(tile0, 0, 0);
        cp_async_commit();
        load_rows(tile0, 1, 0);
        cp_async_commit();
    }

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int lrow = lane & 15, lcol = (lane >> 4) * 8;  // ldmatrix.x4 address pattern of this lane

    for (int tile = tile0; tile < tile1; ++tile) {
        if (paged && tile + 1 < tile1 && (tile + 1 - tile0) % WT == 0) {
            __syncthreads();  // every copy that reads the old window has been issued
            fetch_window(tile + 1);
        }
        if (early && tile == tile0) cp_async_wait<0>();  // old rows and the new row of K and V
        else cp_async_wait<1>();                         // K(tile) has landed; V(tile) may still be in flight
        __syncthreads();
        if (a.pdl_trigger == 1 && tile == tile0) grid_dep_launch();

        // scores of positions [16 warp, 16 warp + 16) for every head slot
        {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const T *krow = Ks + (warp * 16 + lrow) * ROW + lcol;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t af[4];
                ldmatrix_x4(af, krow + ks * 16);
                mma16816<T>(c, af[0], af[1], af[2], af[3], qb[ks][0], qb[ks][1]);
            }
            const int h0 = 2 * t4, p0 = warp * 16 + gid;
            if (h0 < G) {
                S[h0 * ATT_TILE + p0] = c[0];
                S[h0 * ATT_TILE + p0 + 8] = c[2];
            }
            if (h0 + 1 < G) {
                S[(h0 + 1) * ATT_TILE + p0] = c[1];
                S[(h0 + 1) * ATT_TILE + p0 + 8] = c[3];
            }
        }
        __syncthreads();  // scores complete, K buffer free
        if (tile + 1 < tile1) load_rows(tile + 1, 0, 0);
        cp_async_commit();

        // online softmax, one warp per head
        for (int g = warp; g < G; g += ATT_THREADS / 32) {
            const int p0 = tile * ATT_TILE + lane, p1 = p0 + 32;
            float s0 = p0 < ctx ? S[g * ATT_TILE + lane] * scale : -INFINITY;
            float s1 = p1 < ctx ? S[g * ATT_TILE + lane + 32] * scale : -INFINITY;
            float mt = warp_max(fmaxf(s0, s1));
            float mo = m_run[g];
            float mn = fmaxf(mo, mt);
            const T pa = Act<T>::from_f(s0 == -INFINITY ? 0.f : expf(s0 - mn));
            const T pb = Act<T>::from_f(s1 == -INFINITY ? 0.f : expf(s1 - mn));
            float sum = warp_sum(Act<T>::to_f(pa) + Act<T>::to_f(pb));
            Ps[g * PROW + lane] = pa;
            Ps[g * PROW + lane + 32] = pb;
            if (lane == 0) {
                float c = mo == -INFINITY ? 0.f : expf(mo - mn);
                corr[g] = c;
                l_run[g] = l_run[g] * c + sum;
                m_run[g] = mn;
            }
        }
        cp_async_wait<1>();  // V(tile) has landed; K(tile + 1) may still be in flight
        __syncthreads();

        // O += P . V for output dimensions [DW warp, DW warp + DW)
        {
            const float cr = gid < G ? corr[gid] : 0.f;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                acc[i][0] *= cr;
                acc[i][1] *= cr;
            }
#pragma unroll
            for (int ks = 0; ks < ATT_TILE / 16; ++ks) {
                uint32_t pf[4];
                ldmatrix_x4(pf, Ps + lrow * PROW + ks * 16 + lcol);
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, Vs + (ks * 16 + lrow) * ROW + warp * DW + np * 16 + lcol);
                    mma16816<T>(acc[2 * np], pf[0], pf[1], pf[2], pf[3], vf[0], vf[1]);
                    mma16816<T>(acc[2 * np + 1], pf[0], pf[1], pf[2], pf[3], vf[2], vf[3]);
                }
            }
        }
        __syncthreads();  // V buffer and probabilities free
        if (tile + 1 < tile1) load_rows(tile + 1, 1, 0);
        cp_async_commit();
    }
    cp_async_wait<0>();

    // this thread holds head slot gid, dimensions warp*DW + 8 i + 2 t4 (+1) in acc[i][0..1]
    const int d0 = warp * DW + 2 * t4;
    T *og = reinterpret_cast<T *>(a.o) + (size_t)t * a.stride_o + (size_t)hkv * G * DH;
    if (clus) {
        // every split stores its unnormalised partial and (max, sum) into the FIRST split's shared memory (remote
        // stores through the cluster's distributed shared memory), one barrier publishes them, and the first split
        // merges from its own shared memory; nobody reads a peer's memory, so the peers leave after the barrier
        if (my_splits > 1) {
            if (gid < G) {
                const uint32_t ob = att_map_peer(mrg_o + ((size_t)sp * G + gid) * DH + d0, 0u);
#pragma unroll
                for (int i = 0; i < NT; ++i) att_st_peer2(ob + 32 * i, acc[i][0], acc[i][1]);
            }
            if (tid < G) att_st_peer2(att_map_peer(mrg_ml + ((size_t)sp * G + tid) * 2, 0u), m_run[tid], l_run[tid]);
        }
        att_cluster_sync();
        if (sp != 0 || gid >= G) return;
        if (my_splits == 1) {
            const float inv = 1.f / l_run[gid];
#pragma unroll
            for (int i = 0; i < NT; ++i)
                *reinterpret_cast<uint32_t *>(og + gid * DH + d0 + 8 * i) = Act<T>::pack(acc[i][0] * inv, acc[i][1] * inv);
            return;
        }
        float M = -INFINITY;
        for (int s2 = 0; s2 < my_splits; ++s2) M = fmaxf(M, mrg_ml[((size_t)s2 * G + gid) * 2]);
        float L = 0.f, O[NT][2];
#pragma unroll
        for (int i = 0; i < NT; ++i) O[i][0] = O[i][1] = 0.f;
        for (int s2 = 0; s2 < my_splits; ++s2) {
            const float ms = mrg_ml[((size_t)s2 * G + gid) * 2], ls = mrg_ml[((size_t)s2 * G + gid) * 2 + 1];
            const float w = ms == -INFINITY ? 0.f : expf(ms - M);
            L = fmaf(ls, w, L);
            const float *ob = mrg_o + ((size_t)s2 * G + gid) * DH + d0;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const float2 o = *reinterpret_cast<const float2 *>(ob + 8 * i);
                O[i][0] = fmaf(o.x, w, O[i][0]);
                O[i][1] = fmaf(o.y, w, O[i][1]);
            }
        }
        const float inv = 1.f / L;
#pragma unroll
        for (int i = 0; i < NT; ++i)
            *reinterpret_cast<uint32_t *>(og + gid * DH + d0 + 8 * i) = Act<T>::pack(O[i][0] * inv, O[i][1] * inv);
        return;
    }
    if (my_splits == 1) {
        if (gid < G) {
            const float inv = 1.f / l_run[gid];
#pragma unroll
            for (int i = 0; i < NT; ++i)
                *reinterpret_cast<uint32_t *>(og + gid * DH + d0 + 8 * i) = Act<T>::pack(acc[i][0] * inv, acc[i][1] * inv);
        }
        return;
    }

    // leave the unnormalised partial and (max, sum); the last split to arrive merges
    const size_t head0 = (size_t)t * a.nh + (size_t)hkv * G;
    if (gid < G) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
            *reinterpret_cast<float2 *>(a.part_o + ((head0 + gid) * a.n_splits + sp) * DH + d0 + 8 * i) =
                make_float2(acc[i][0], acc[i][1]);
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
    if (gid < G) {
        const float *ml = a.part_ml + (head0 + gid) * a.n_splits * 2;
        float M = -INFINITY;
        for (int s2 = 0; s2 < my_splits; ++s2) M = fmaxf(M, __ldcg(ml + 2 * s2));
        float L = 0.f, O[NT][2];
#pragma unroll
        for (int i = 0; i < NT; ++i) O[i][0] = O[i][1] = 0.f;
        for (int s2 = 0; s2 < my_splits; ++s2) {
            float ms = __ldcg(ml + 2 * s2), ls = __ldcg(ml + 2 * s2 + 1);
            float w = ms == -INFINITY ? 0.f : expf(ms - M);
            L = fmaf(ls, w, L);
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                float2 o = __ldcg(reinterpret_cast<const float2 *>(a.part_o + ((head0 + gid) * a.n_splits + s2) * DH + d0 + 8 * i));
                O[i][0] = fmaf(o.x, w, O[i][0]);
                O[i][1] = fmaf(o.y, w, O[i][1]);
            }
        }
        const float inv = 1.f / L;
#pragma unroll
        for (int i = 0; i < NT; ++i)
            *reinterpret_cast<uint32_t *>(og + gid * DH + d0 + 8 * i) = Act<T>::pack(O[i][0] * inv, O[i][1] * inv);
    }
    if (tid == 0) a.counters[(size_t)t * a.nkvh + hkv] = 0;  // ready for the next launch
}

// ------------------------------------------------------------------ prefill form
// Rounds that hold prompts (several tokens of one sequence): a CTA owns a KV head and a GROUP of up to 64 / G
// consecutive tokens of one sequence, i.e. 64 query rows (token, head) that all attend the same cached rows — the K/V
// tile is gathered once per 64 queries instead of once per token.  Queries are the M side of both products (16 rows
// per warp): S = Q.K^T with the query fragments held in registers for the whole kernel and K from the shared-memory
// tile (ldmatrix), online softmax per row in registers (row maximum and sum across the four lanes of a quad),
// probabilities rounded to the activation dtype and fed straight back as the A operand of P.V (no trip through shared
// memory), V transposed by ldmatrix.  K and V tiles are double-buffered: the gather of tile t + 1 is in flight while
// tile t is multiplied.  The causal limit is per row: a query at position p attends positions [0, p].  Same
// arithmetic contract as the decode form (f32 scores and softmax, rounded probabilities, row sum over the rounded
// values, one rounding of the output); no split-KV — a prefill round has CTAs to spare.
struct AttnGroup {
    int first, count;  // index of the group's first token in the round, tokens in the group (<= 64 / G)
};
constexpr int ATT_MAX_PAGES = 512;  // page ids of one sequence held in shared memory

template <class T, int DH, int G>
__global__ void __launch_bounds__(ATT_THREADS) attn_prefill_kernel(const AttnArgs a, const AttnGroup *__restrict__ groups) {
    constexpr int ROW = DH + 8;      // padded K/V row (elements)
    constexpr int CH = DH / 8;       // 16-byte chunks per row
    constexpr int KSTEPS = DH / 16;  // k-steps of the score product
    constexpr int NTS = ATT_TILE / 8;  // 8-wide score tiles per K tile
    constexpr int NTO = DH / 8;        // 8-wide output tiles
    extern __shared__ __align__(16) unsigned char smem[];
    T *Ks = reinterpret_cast<T *>(smem);      // [2][TILE][ROW]
    T *Vs = Ks + 2 * ATT_TILE * ROW;          // [2][TILE][ROW]
    __shared__ int pg[ATT_MAX_PAGES];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, t4 = lane & 3;
    const int hkv = blockIdx.x;
    const AttnGroup grp = groups[blockIdx.y];
    const T *kv_pool = reinterpret_cast<const T *>(a.kv_pool);

    const int pos0 = (int)a.tok_pos[grp.first];           // position of the group's first token
    const int ctx = pos0 + grp.count;                     // rows the group's last token attends
    const int seq = a.tok_seq[grp.first];
    const int n_tiles = (ctx + ATT_TILE - 1) / ATT_TILE;
    const int n_pages = (ctx + a.geom.page_tokens - 1) >> a.geom.page_shift;
    for (int i = tid; i < n_pages; i += ATT_THREADS) pg[i] = a.page_table[(size_t)seq * a.pt_stride + i];
    grid_dep_wait();

    // this thread's two query rows: r0 = 16 warp + gid, r1 = r0 + 8; row r = (token r / G, head r % G)
    const int r0 = warp * 16 + gid, r1 = r0 + 8;
    const int tt0 = r0 / G, tt1 = r1 / G;
    const bool v0 = tt0 < grp.count, v1 = tt1 < grp.count;
    const int lim0 = v0 ? pos0 + tt0 : -1, lim1 = v1 ? pos0 + tt1 : -1;  // last position each row attends
    uint32_t qa[KSTEPS][4];
    {
        const T *q0 = reinterpret_cast<const T *>(a.q) + (size_t)(grp.first + (v0 ? tt0 : 0)) * a.stride_q + (size_t)(hkv * G + r0 % G) * DH;
        const T *q1 = reinterpret_cast<const T *>(a.q) + (size_t)(grp.first + (v1 ? tt1 : 0)) * a.stride_q + (size_t)(hkv * G + r1 % G) * DH;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t *>(q0 + ks * 16 + 2 * t4) : 0u;
            qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t *>(q1 + ks * 16 + 2 * t4) : 0u;
            qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t *>(q0 + ks * 16 + 8 + 2 * t4) : 0u;
            qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t *>(q1 + ks * 16 + 8 + 2 * t4) : 0u;
        }
    }
    const size_t blk = (size_t)a.geom.page_tokens * DH;
    const size_t kbase = ((size_t)(a.layer * 2) * a.geom.nkvh + hkv) * blk;
    const size_t voff = (size_t)a.geom.nkvh * blk;
    const int lcol8 = (tid % CH) * 8, j0 = tid / CH;
    auto load_tile = [&](int tile, int buf) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            T *dst = (which ? Vs : Ks) + (size_t)buf * ATT_TILE * ROW;
#pragma unroll
            for (int i = 0; i < (ATT_TILE * CH) / ATT_THREADS; ++i) {
                const int j = j0 + (ATT_THREADS / CH) * i;
                const int pos = tile * ATT_TILE + j;
                const bool valid = pos < ctx;
                const int page = valid ? pg[pos >> a.geom.page_shift] : 0;
                const int slot = pos & (a.geom.page_tokens - 1);
                const T *src = kv_pool + (valid ? (size_t)page * a.geom.page_elems + kbase + (which ? voff : 0) + (size_t)slot * DH + lcol8 : 0);
                cp_async_16(dst + j * ROW + lcol8, src, valid);
            }
        }
    };
    __syncthreads();  // page ids staged
    load_tile(0, 0);
    cp_async_commit();

    const float scale = 1.0f / sqrtf((float)DH);
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[NTO][4];
#pragma unroll
    for (int i = 0; i < NTO; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int tile = 0; tile < n_tiles; ++tile) {
        const int buf = tile & 1;
        if (tile + 1 < n_tiles) load_tile(tile + 1, buf ^ 1);  // the other buffer was released by the barrier below
        cp_async_commit();
        cp_async_wait<1>();  // tile `tile` has landed
        __syncthreads();
        const T *Kt = Ks + (size_t)buf * ATT_TILE * ROW, *Vt = Vs + (size_t)buf * ATT_TILE * ROW;

        // ---- scores of this warp's 16 query rows against the 64 positions of the tile
        float sc[NTS][4];
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int np = 0; np < NTS / 2; ++np) {
                uint32_t kb[4];  // K fragments of score tiles 2 np and 2 np + 1
                ldmatrix_x4(kb, Kt + (size_t)(np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * ROW + ks * 16 + ((lane >> 3) & 1) * 8);
                mma16816<T>(sc[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[0], kb[1]);
                mma16816<T>(sc[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[2], kb[3]);
            }
        }
        // ---- causal mask, online softmax per row
        float mt0 = -INFINITY, mt1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt) {
            const int p = tile * ATT_TILE + nt * 8 + 2 * t4;
            sc[nt][0] = p <= lim0 ? sc[nt][0] * scale : -INFINITY;
            sc[nt][1] = p + 1 <= lim0 ? sc[nt][1] * scale : -INFINITY;
            sc[nt][2] = p <= lim1 ? sc[nt][2] * scale : -INFINITY;
            sc[nt][3] = p + 1 <= lim1 ? sc[nt][3] * scale : -INFINITY;
            mt0 = fmaxf(mt0, fmaxf(sc[nt][0], sc[nt][1]));
            mt1 = fmaxf(mt1, fmaxf(sc[nt][2], sc[nt][3]));
        }
        mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 1));
        mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 2));
        mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 1));
        mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 2));
        const float mn0 = fmaxf(m0, mt0), mn1 = fmaxf(m1, mt1);
        const float c0 = m0 == -INFINITY ? 0.f : expf(m0 - mn0), c1 = m1 == -INFINITY ? 0.f : expf(m1 - mn1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;  // a fully masked row stays at zero
        m0 = mn0;
        m1 = mn1;
        uint32_t pa[NTS][2];  // probabilities rounded to the activation dtype: rows r0 (pa[.][0]) and r1 (pa[.][1])
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt) {
            const T p00 = Act<T>::from_f(expf(sc[nt][0] - mu0)), p01 = Act<T>::from_f(expf(sc[nt][1] - mu0));
            const T p10 = Act<T>::from_f(expf(sc[nt][2] - mu1)), p11 = Act<T>::from_f(expf(sc[nt][3] - mu1));
            s0 += Act<T>::to_f(p00) + Act<T>::to_f(p01);
            s1 += Act<T>::to_f(p10) + Act<T>::to_f(p11);
            pa[nt][0] = Act<T>::pack(Act<T>::to_f(p00), Act<T>::to_f(p01));
            pa[nt][1] = Act<T>::pack(Act<T>::to_f(p10), Act<T>::to_f(p11));
        }
        l0 = l0 * c0 + s0;  // per-thread partial sums: the four lanes of a quad are added at the end
        l1 = l1 * c1 + s1;
#pragma unroll
        for (int i = 0; i < NTO; ++i) {
            o[i][0] *= c0; o[i][1] *= c0;
            o[i][2] *= c1; o[i][3] *= c1;
        }
        // ---- O += P . V: k-step kk covers positions [16 kk, 16 kk + 16) = score tiles 2 kk, 2 kk + 1
#pragma unroll
        for (int kk = 0; kk < ATT_TILE / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < NTO / 2; ++dp) {
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, Vt + (size_t)(kk * 16 + (lane & 15)) * ROW + dp * 16 + (lane >> 4) * 8);
                mma16816<T>(o[2 * dp], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1], vb[0], vb[1]);
                mma16816<T>(o[2 * dp + 1], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1], vb[2], vb[3]);
            }
        }
        __syncthreads();  // everyone is done with buffer `buf`: the next iteration's gather may overwrite it
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    T *out = reinterpret_cast<T *>(a.o);
    if (v0) {
        const float inv = 1.f / l0;
        T *dst = out + (size_t)(grp.first + tt0) * a.stride_o + (size_t)(hkv * G + r0 % G) * DH + 2 * t4;
#pragma unroll
        for (int i = 0; i < NTO; ++i) *reinterpret_cast<uint32_t *>(dst + 8 * i) = Act<T>::pack(o[i][0] * inv, o[i][1] * inv);
    }
    if (v1) {
        const float inv = 1.f / l1;
        T *dst = out + (size_t)(grp.first + tt1) * a.stride_o + (size_t)(hkv * G + r1 % G) * DH + 2 * t4;
#pragma unroll
        for (int i = 0; i < NTO; ++i) *reinterpret_cast<uint32_t *>(dst + 8 * i) = Act<T>::pack(o[i][2] * inv, o[i][3] * inv);
    }
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
    // a cluster launch adds the merge region: [z][G][DH] partials and [z][G][2] (max, sum)
    const size_t smem_max = att_merge_offset<T, DH, G>() + (size_t)8 * G * (DH + 2) * sizeof(float);
    size_t smem = att_merge_offset<T, DH, G>() + (size_t)(a.cluster_z > 0 ? a.cluster_z : 0) * G * (DH + 2) * sizeof(float);
    static std::mutex mu;
    static std::map<int, bool> done;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!done[dev]) {
            if (smem_max > 48 * 1024) LCU_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
            done[dev] = true;
        }
    }
    if (dry) return LCU_OK;
    dim3 grid(a.nkvh, a.n_tok, a.n_splits);
    if (a.cluster_z > 0) {
        LCU_REQUIRE(a.cluster_z == a.n_splits && a.cluster_z <= 8, "attention: cluster of %d splits (grid depth %d, at most 8)", a.cluster_z, a.n_splits);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(ATT_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = (unsigned)a.cluster_z;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 2 : 1;
        LCU_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, a));
        return LCU_OK;
    }
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
    LCU_REQUIRE(dry || a.n_splits == 1 || a.cluster_z > 0 || (a.part_o && a.part_ml && a.counters), "attention: split-KV needs scratch");
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


// ---- prefill form
template <class T, int DH, int G>
static int attn_prefill_inst(const AttnArgs &a, const void *groups, int n_groups, cudaStream_t s, bool dry) {
    auto kernel = attn_prefill_kernel<T, DH, G>;
    const size_t smem = (size_t)4 * ATT_TILE * (DH + 8) * sizeof(T);
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
    LCU_CHECK_CUDA(launch_kernel(kernel, dim3(a.nkvh, n_groups), dim3(ATT_THREADS), smem, s, false, a,
                                 reinterpret_cast<const AttnGroup *>(groups)));
    return LCU_OK;
}

template <class T, int DH>
static int attn_prefill_dh(const AttnArgs &a, const void *groups, int n_groups, cudaStream_t s, bool dry) {
    switch (a.nh / a.nkvh) {
    case 1: return attn_prefill_inst<T, DH, 1>(a, groups, n_groups, s, dry);
    case 2: return attn_prefill_inst<T, DH, 2>(a, groups, n_groups, s, dry);
    case 4: return attn_prefill_inst<T, DH, 4>(a, groups, n_groups, s, dry);
    case 8: return attn_prefill_inst<T, DH, 8>(a, groups, n_groups, s, dry);
    default: set_error("attention: nh/nkvh = %d unsupported (1, 2, 4, 8)", a.nh / a.nkvh); return LCU_ERR_INVALID;
    }
}

int attn_prefill_group_tokens(int nh, int nkvh) { return ATT_TILE / (nh / nkvh); }
bool attn_prefill_supported(int pt_stride) { return pt_stride <= ATT_MAX_PAGES; }

int attn_prefill_launch(const AttnArgs &a, const void *groups_dev, int n_groups, int dt, cudaStream_t s, bool dry) {
    if (n_groups <= 0 && !dry) return LCU_OK;
    LCU_REQUIRE(a.nkvh > 0 && a.nh % a.nkvh == 0, "attention: nh = %d is not a multiple of nkvh = %d", a.nh, a.nkvh);
    LCU_REQUIRE(a.dh == 64 || a.dh == 128, "attention: dh = %d unsupported (64, 128)", a.dh);
    LCU_REQUIRE(dry || (a.kv_pool && groups_dev && a.pt_stride <= ATT_MAX_PAGES), "attention (prefill form): needs the paged cache, groups and at most %d pages per sequence", ATT_MAX_PAGES);
    if (dt == LCU_F16) return a.dh == 64 ? attn_prefill_dh<__half, 64>(a, groups_dev, n_groups, s, dry) : attn_prefill_dh<__half, 128>(a, groups_dev, n_groups, s, dry);
    if (dt == LCU_BF16)
        return a.dh == 64 ? attn_prefill_dh<__nv_bfloat16, 64>(a, groups_dev, n_groups, s, dry)
                          : attn_prefill_dh<__nv_bfloat16, 128>(a, groups_dev, n_groups, s, dry);
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
