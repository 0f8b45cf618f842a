// Batched `Linear` on the 5th-generation tensor cores: tcgen05.mma with TMA-fed shared-memory
// operands and the accumulator in tensor memory (TMEM) — for 9..64 tokens per pass (batched decode
// rounds and prefill chunks).  Same operator as llama.cu/src/op/linear.rs:17-120 (the reference
// calls cuBLAS GemmEx with m = out, n = bucketed token count, k = in).
//
// The GEMM is computed "swapped": D[128 weight rows x N tokens] += W_tile[128 x 64] · X[N x 64]^T,
// so the weight dimension fills the 128-row MMA and the small token block is N (16, 32 or 64).
//   - warp 0 (one lane): TMA producer — cp.async.bulk.tensor.2d loads of the weight tile (two
//     64-row boxes) and of the activation tile into a ring of stages, 128-byte swizzle,
//     completion on mbarriers.  Each weight byte is read once from HBM;
//   - warp 1 (one lane): MMA issuer — four tcgen05.mma (K = 16 each) per stage, accumulating into
//     TMEM; tcgen05.commit frees the stage and, after the last one, signals the epilogue;
//   - warps 2..5: epilogue — tcgen05.ld of the 128 x N f32 accumulator into registers, staging
//     through shared memory, then the same fused epilogues as the GEMV (gemv_epilogue: store,
//     residual, RoPE + KV append, SwiGLU).  The two rows of a pair sit in one tile (adjacent rows,
//     or 64 gate rows followed by their 64 up rows);
//   - matrices with few rows are split along K across CTAs (grid.y); partial sums go through
//     scratch memory and the last CTA of a row block to arrive adds them in split order.
// Every mbarrier wait is bounded by a wall-clock limit: on expiry the kernel records a status bit,
// skips the remaining work, frees its TMEM and returns.
#include <cuda.h>

#include <cstdlib>
#include <map>
#include <mutex>

#include "gemv.cuh"

namespace lcu {

constexpr int TC_THREADS = 192;
constexpr int TC_BM = 128;         // weight rows per CTA tile
constexpr int TC_BK = 64;          // K elements per stage (128 bytes: one swizzle row)
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;
constexpr unsigned long long TC_WAIT_NS = 2000000000ull;

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ unsigned long long tc_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t tc_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (tc_mbar_try(bar, parity)) return true;
    unsigned long long t0 = tc_ns();
    for (unsigned it = 1;; ++it) {
        if (tc_mbar_try(bar, parity)) return true;
        if ((it & 255u) == 0 && (*abort_flag || tc_ns() - t0 > TC_WAIT_NS)) return false;
    }
}
__device__ __forceinline__ void tc_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// shared-memory operand descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t r[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t r[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}

constexpr int TC_MAX_STAGES = 12;

struct TcShared {
    unsigned long long full[TC_MAX_STAGES], empty[TC_MAX_STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int last;
};

// Vector form of the fused epilogues for one token and 8 consecutive outputs.  Everything a thread reads
// from global memory for its items (residual, rotation table, page number) is fetched by tc_prefetch
// before tc_finish stores anything: outputs may alias inputs (the residual is updated in place), so the
// compiler cannot hoist those loads itself, and a chain of dependent round trips per item is what made
// the scalar form slow.  Every access is 16 bytes.
//   STORE / RESIDUAL / ROPE_KV: v[0..7] = 8 consecutive rows;  SWIGLU: v = gate, u = up of 8 pairs
struct TcPre {
    uint4 res;
    float4 sn, cs;
    uint32_t p;
    int page;
};

template <class T>
__device__ __forceinline__ void tc_prefetch(const GemvArgs &a, int n, int first, TcPre &pre) {
    if (a.epilogue == EPI_RESIDUAL) {
        pre.res = *reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.res) + (size_t)n * a.stride_res + first);
    } else if (a.epilogue == EPI_ROPE_KV) {
        const int sect = first < a.qd ? 0 : (first < a.qd + a.kvd ? 1 : 2);
        const int rr = first - (sect == 0 ? 0 : (sect == 1 ? a.qd : a.qd + a.kvd));
        const int e = rr % a.dh;
        pre.p = a.pos[n];
        if (sect < 2) {
            const size_t ti = (size_t)pre.p * (a.dh >> 1) + (e >> 1);
            pre.sn = *reinterpret_cast<const float4 *>(a.sin_t + ti);
            pre.cs = *reinterpret_cast<const float4 *>(a.cos_t + ti);
        }
        if (sect > 0) pre.page = a.page_table[(size_t)a.tok_seq[n] * a.pt_stride + (pre.p >> a.geom.page_shift)];
    }
}

template <class T>
__device__ __forceinline__ void tc_finish(const GemvArgs &a, int n, int first, float v[8], const float u[8], const TcPre &pre) {
    T *dst = reinterpret_cast<T *>(a.y) + (size_t)n * a.stride_y + first;
    if (a.epilogue == EPI_SWIGLU) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = swiglu_act(round_act<T>(v[i]), round_act<T>(u[i]));
    } else if (a.epilogue == EPI_RESIDUAL) {
        const uint32_t rw[4] = {pre.res.x, pre.res.y, pre.res.z, pre.res.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 rf = Act<T>::to_f2(rw[i]);
            v[2 * i] += rf.x;
            v[2 * i + 1] += rf.y;
        }
    } else if (a.epilogue == EPI_ROPE_KV) {
        const int sect = first < a.qd ? 0 : (first < a.qd + a.kvd ? 1 : 2);
        const int rr = first - (sect == 0 ? 0 : (sect == 1 ? a.qd : a.qd + a.kvd));
        const int head = rr / a.dh, e = rr - head * a.dh;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = round_act<T>(v[i]);  // the projection is materialised before rope
        if (sect < 2) {
            const float sn[4] = {pre.sn.x, pre.sn.y, pre.sn.z, pre.sn.w}, cs[4] = {pre.cs.x, pre.cs.y, pre.cs.z, pre.cs.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float xa = v[2 * i], xb = v[2 * i + 1];
                v[2 * i] = xa * cs[i] - xb * sn[i];
                v[2 * i + 1] = xa * sn[i] + xb * cs[i];
            }
        }
        if (sect > 0) {
            const int slot = pre.p & (a.geom.page_tokens - 1);
            dst = reinterpret_cast<T *>(a.kv_pool) + a.geom.block_off(pre.page, a.layer, sect - 1, head) + (size_t)slot * a.dh + e;
        }
    }
    uint4 o;
    o.x = Act<T>::pack(v[0], v[1]); o.y = Act<T>::pack(v[2], v[3]); o.z = Act<T>::pack(v[4], v[5]); o.w = Act<T>::pack(v[6], v[7]);
    if (a.push.n && (a.epilogue == EPI_STORE || a.epilogue == EPI_RESIDUAL)) {
        // tensor parallelism: the partial goes to the owner's (scatter form) or every rank's all-reduce slot over peer memory
        if (a.push.scatter_cols) {
            *reinterpret_cast<uint4 *>(reinterpret_cast<T *>(a.push.slot[first / a.push.scatter_cols]) + (size_t)n * a.stride_y + first) = o;
            return;
        }
        for (int k = 0; k < a.push.n; ++k)
            *reinterpret_cast<uint4 *>(reinterpret_cast<T *>(a.push.slot[k]) + (size_t)n * a.stride_y + first) = o;
        return;
    }
    *reinterpret_cast<uint4 *>(dst) = o;
}

// Persistent: grid = min(tiles, SMs); a tile is (row block of 128 rows = 64 pairs, K split); CTA c takes
// tiles c, c + grid, ...  The shared-memory ring keeps running across tiles and the accumulator is
// double-buffered in TMEM, so the epilogue of one tile overlaps the loads and MMAs of the next.
// block = 6 warps: TMA producer, MMA issuer, 4 epilogue warps.
template <class T>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const GemvArgs a, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               int n_pairs, int N, int n_stages, int units_per_cta, int max_seg, int vec, uint32_t idesc, float *ws,
               unsigned *tickets, uint32_t *status) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows = 1024 bytes
    unsigned char *smem = smem_raw + ((1024u - (tc_smem(smem_raw) & 1023u)) & 1023u);
    const int stage_bytes = TC_A_BYTES + N * 128;
    float *stg = reinterpret_cast<float *>(smem + (size_t)n_stages * stage_bytes);  // [128][N + 1]
    TcShared *sh = reinterpret_cast<TcShared *>(reinterpret_cast<unsigned char *>(stg) + (size_t)TC_BM * (N + 1) * 4);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (a.pdl_trigger == 0) grid_dep_launch();
    const int nkb = a.in / TC_BK;  // K blocks of a whole row block
    const bool swiglu = a.epilogue == EPI_SWIGLU;
    const int acc_cols = N < 32 ? 32 : N;      // TMEM columns of one accumulator
    const int tm_cols = 2 * acc_cols;          // two accumulators
    const int n_rb = (n_pairs + 63) / 64;
    // work units = (row block, K block) pairs in row-block-major order; this CTA owns a contiguous range and
    // walks it as segments that end at row-block boundaries (stream-K)
    const int total_units = n_rb * nkb;
    const int u_begin = min(total_units, (int)blockIdx.x * units_per_cta);
    const int u_end = min(total_units, u_begin + units_per_cta);

    if (tid == 0) {
        for (int i = 0; i < n_stages; ++i) {
            tc_mbar_init(tc_smem(&sh->full[i]), 1);
            tc_mbar_init(tc_smem(&sh->empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(tc_smem(&sh->tmem_full[i]), 1);
            tc_mbar_init(tc_smem(&sh->tmem_empty[i]), 1);
        }
        sh->abort_flag = 0;
        sh->last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation is a warp-wide operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&sh->tmem_base)), "r"(tm_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer: unit j of this CTA is (row block, K block) = divmod(u_begin + j, nkb)
        const int n_units = u_end - u_begin;
        auto issue = [&](int j, bool weights, bool acts) {
            const int u = u_begin + j, rb = u / nkb, kb = u - rb * nkb;
            const int slot = j % n_stages;
            const uint32_t bar = tc_smem(&sh->full[slot]);
            const uint32_t dst = tc_smem(smem + (size_t)slot * stage_bytes);
            const int kx = kb * TC_BK;
            if (weights) {
                tc_mbar_expect_tx(bar, (uint32_t)stage_bytes);
                tc_tma_2d(dst, &map_w, kx, swiglu ? rb * 64 : rb * TC_BM, bar);
                tc_tma_2d(dst + TC_A_BYTES / 2, &map_w, kx, swiglu ? a.di + rb * 64 : rb * TC_BM + 64, bar);
            }
            if (acts) tc_tma_2d(dst + TC_A_BYTES, &map_x, kx, 0, bar);
        };
        // The weights do not depend on the previous kernel: when this launch was allowed to start early
        // (programmatic dependent launch) the first ring of weight tiles is already streaming while the predecessor
        // finishes; the activation tiles of those stages follow once it has.
        const int first = n_units < n_stages ? n_units : n_stages;
        for (int j = 0; j < first; ++j) issue(j, true, false);
        grid_dep_wait();
        for (int j = 0; j < first; ++j) issue(j, false, true);
        for (int j = first; j < n_units && !sh->abort_flag; ++j) {
            const int slot = j % n_stages;
            const uint32_t parity = (uint32_t)(j / n_stages) & 1u;
            if (!tc_mbar_wait(tc_smem(&sh->empty[slot]), parity ^ 1u, &sh->abort_flag)) {
                atomicOr(status, 4u);
                sh->abort_flag = 1;
                break;
            }
            issue(j, true, true);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        int it = 0, ti = 0;
        for (int u = u_begin; u < u_end && !sh->abort_flag; ++ti) {
            const int rb = u / nkb, kb0 = u - rb * nkb;
            const int kb1 = min(nkb, kb0 + (u_end - u));
            u += kb1 - kb0;
            const int ab = ti & 1;
            // the epilogue must have drained this accumulator (two tiles ago)
            if (!tc_mbar_wait(tc_smem(&sh->tmem_empty[ab]), ((uint32_t)(ti >> 1) & 1u) ^ 1u, &sh->abort_flag)) {
                atomicOr(status, 4u);
                sh->abort_flag = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t d_tmem = tmem + (uint32_t)(ab * acc_cols);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const int slot = it % n_stages;
                const uint32_t parity = (uint32_t)(it / n_stages) & 1u;
                if (!tc_mbar_wait(tc_smem(&sh->full[slot]), parity, &sh->abort_flag)) {
                    atomicOr(status, 4u);
                    sh->abort_flag = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = tc_smem(smem + (size_t)slot * stage_bytes), sb = sa + TC_A_BYTES;
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)
                    tc_mma_f16(d_tmem, tc_desc(sa + k * 32), tc_desc(sb + k * 32), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                tc_commit(tc_smem(&sh->empty[slot]));  // the stage is free once these MMAs have read it
            }
            tc_commit(tc_smem(&sh->tmem_full[ab]));     // accumulator complete
        }
    } else if (warp >= 2) {
        // ---------------- epilogue warps: TMEM -> registers -> shared staging -> fused epilogue
        const int et = tid - 64;
        const int q = warp & 3;                      // a warp may only touch TMEM lanes [32q, 32q + 32)
        const int row = q * 32 + lane;
        int ti = 0;
        for (int u = u_begin; u < u_end; ++ti) {
            const int rb = u / nkb, kb0 = u - rb * nkb;
            const int kb1 = min(nkb, kb0 + (u_end - u));
            u += kb1 - kb0;
            const bool whole = kb0 == 0 && kb1 == nkb;  // this CTA holds the complete sum of the row block
            // otherwise: CTAs first_cta .. last_cta share the row block, in K order
            const int first_cta = (rb * nkb) / units_per_cta, last_cta = (rb * nkb + nkb - 1) / units_per_cta;
            const int n_seg = last_cta - first_cta + 1, seg = (int)blockIdx.x - first_cta;
            const int ab = ti & 1;
            bool ok = tc_mbar_wait(tc_smem(&sh->tmem_full[ab]), (uint32_t)(ti >> 1) & 1u, &sh->abort_flag);
            if (!ok) {
                atomicOr(status, 4u);
                sh->abort_flag = 1;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (ok) {
                for (int c0 = 0; c0 < N; c0 += 16) {
                    uint32_t r[16];
                    tc_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(ab * acc_cols + c0), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; ++i) stg[row * (N + 1) + c0 + i] = __uint_as_float(r[i]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            // the barrier also ANDs every thread's `ok`: the 128 epilogue threads leave the loop together or not at
            // all (a thread whose wait ran out must not strand the others at the next barrier)
            uint32_t all_ok;
            asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 p, %1, 0;\n bar.red.and.pred q, 2, 128, p;\n selp.u32 %0, 1, 0, q;\n}"
                         : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
            if (et == 0) {  // the accumulator may be overwritten from here on
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&sh->tmem_empty[ab])) : "memory");
            }
            if (!all_ok) break;
            const int items = 64 * N;
            if (whole && vec) {
                // (token, 8 outputs) items; residual vectors are fetched first, then everything is stored
                const int chunks = swiglu ? 8 : 16;
                TcPre pre[8];
                int cnt = 0;
                for (int idx = et; idx < chunks * N; idx += 128, ++cnt) {
                    int c = idx % chunks, n = idx / chunks;
                    int first = swiglu ? rb * 64 + 8 * c : rb * TC_BM + 8 * c;
                    if (n < a.n_tok && first + 8 <= (swiglu ? a.di : a.out)) tc_prefetch<T>(a, n, first, pre[cnt]);
                }
                cnt = 0;
                for (int idx = et; idx < chunks * N; idx += 128, ++cnt) {
                    int c = idx % chunks, n = idx / chunks;
                    int first = swiglu ? rb * 64 + 8 * c : rb * TC_BM + 8 * c;
                    if (!(n < a.n_tok && first + 8 <= (swiglu ? a.di : a.out))) continue;
                    float v[8], u[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[i] = stg[(8 * c + i) * (N + 1) + n];
                        u[i] = swiglu ? stg[(64 + 8 * c + i) * (N + 1) + n] : 0.f;
                    }
                    tc_finish<T>(a, n, first, v, u, pre[cnt]);
                }
            } else if (whole) {
                for (int idx = et; idx < items; idx += 128) {
                    int j = idx / N, n = idx - j * N;
                    int p = rb * 64 + j;
                    if (p >= n_pairs || n >= a.n_tok) continue;
                    int ra = swiglu ? j : 2 * j, rb2 = swiglu ? 64 + j : 2 * j + 1;
                    gemv_epilogue<T>(a, p, n, stg[ra * (N + 1) + n], stg[rb2 * (N + 1) + n]);
                }
            } else {
                // the row block is shared (the host only cuts row blocks when the vector epilogue applies).  Partial
                // tiles go to scratch token-major, 128 floats per (row block, segment, token); the CTA that takes
                // the last ticket sums them in K order and finishes.
                for (int idx = et; idx < 16 * N; idx += 128) {
                    int c = idx & 15, n = idx >> 4;
                    if (n >= a.n_tok) continue;
                    float4 lo, hi;
                    lo.x = stg[(8 * c + 0) * (N + 1) + n]; lo.y = stg[(8 * c + 1) * (N + 1) + n];
                    lo.z = stg[(8 * c + 2) * (N + 1) + n]; lo.w = stg[(8 * c + 3) * (N + 1) + n];
                    hi.x = stg[(8 * c + 4) * (N + 1) + n]; hi.y = stg[(8 * c + 5) * (N + 1) + n];
                    hi.z = stg[(8 * c + 6) * (N + 1) + n]; hi.w = stg[(8 * c + 7) * (N + 1) + n];
                    float *dst = ws + (((size_t)rb * max_seg + seg) * N + n) * TC_BM + 8 * c;
                    __stcg(reinterpret_cast<float4 *>(dst), lo);
                    __stcg(reinterpret_cast<float4 *>(dst + 4), hi);
                }
                __threadfence();
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (et == 0) {
                    unsigned ticket = atomicAdd(&tickets[rb], 1u);
                    sh->last = ticket == (unsigned)n_seg - 1;
                    if (sh->last) tickets[rb] = 0;
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (sh->last) {
                    __threadfence();
                    // Merge of the segments' partial sums.  A partial row lives in the L2 slice of whichever SM wrote
                    // it and one dependent round trip costs more than a microsecond here, so the loads of up to 6
                    // segments for TWO rows of 8 floats are all issued before the first add (96 registers of loads in
                    // flight per thread; the epilogue warps have registers to spare), the adds then run in K order.
                    // Measured on a 6-segment merge of a 128 x 32 tile: 11 us with one segment after the other.
                    const size_t seg_stride = (size_t)N * TC_BM;
                    auto merge2 = [&](const float *r0, const float *r1, float o0[8], float o1[8]) {
                        float4 b0[12], b1[12];
#pragma unroll
                        for (int s2 = 0; s2 < 6; ++s2) {
                            if (s2 < n_seg) {
                                b0[2 * s2] = __ldcg(reinterpret_cast<const float4 *>(r0 + s2 * seg_stride));
                                b0[2 * s2 + 1] = __ldcg(reinterpret_cast<const float4 *>(r0 + s2 * seg_stride + 4));
                                b1[2 * s2] = __ldcg(reinterpret_cast<const float4 *>(r1 + s2 * seg_stride));
                                b1[2 * s2 + 1] = __ldcg(reinterpret_cast<const float4 *>(r1 + s2 * seg_stride + 4));
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) o0[i] = o1[i] = 0.f;
#pragma unroll
                        for (int s2 = 0; s2 < 6; ++s2) {
                            if (s2 < n_seg) {
                                o0[0] += b0[2 * s2].x; o0[1] += b0[2 * s2].y; o0[2] += b0[2 * s2].z; o0[3] += b0[2 * s2].w;
                                o0[4] += b0[2 * s2 + 1].x; o0[5] += b0[2 * s2 + 1].y; o0[6] += b0[2 * s2 + 1].z; o0[7] += b0[2 * s2 + 1].w;
                                o1[0] += b1[2 * s2].x; o1[1] += b1[2 * s2].y; o1[2] += b1[2 * s2].z; o1[3] += b1[2 * s2].w;
                                o1[4] += b1[2 * s2 + 1].x; o1[5] += b1[2 * s2 + 1].y; o1[6] += b1[2 * s2 + 1].z; o1[7] += b1[2 * s2 + 1].w;
                            }
                        }
                        for (int s2 = 6; s2 < n_seg; ++s2) {  // more than 6 CTAs on one row block: small launches only
                            const float4 a0 = __ldcg(reinterpret_cast<const float4 *>(r0 + s2 * seg_stride));
                            const float4 a1 = __ldcg(reinterpret_cast<const float4 *>(r0 + s2 * seg_stride + 4));
                            const float4 c0 = __ldcg(reinterpret_cast<const float4 *>(r1 + s2 * seg_stride));
                            const float4 c1 = __ldcg(reinterpret_cast<const float4 *>(r1 + s2 * seg_stride + 4));
                            o0[0] += a0.x; o0[1] += a0.y; o0[2] += a0.z; o0[3] += a0.w; o0[4] += a1.x; o0[5] += a1.y; o0[6] += a1.z; o0[7] += a1.w;
                            o1[0] += c0.x; o1[1] += c0.y; o1[2] += c0.z; o1[3] += c0.w; o1[4] += c1.x; o1[5] += c1.y; o1[6] += c1.z; o1[7] += c1.w;
                        }
                    };
                    const float *tile0 = ws + (size_t)rb * max_seg * seg_stride;
                    const float zero8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    if (swiglu) {
                        // one item (8 pairs of one token) per pass: its gate row and its up row
                        for (int idx = et; idx < 8 * N; idx += 128) {
                            const int c = idx & 7, n = idx >> 3;
                            const int first = rb * 64 + 8 * c;
                            if (!(n < a.n_tok && first + 8 <= a.di)) continue;
                            float g8[8], u8[8];
                            const float *r = tile0 + (size_t)n * TC_BM + 8 * c;
                            merge2(r, r + 64, g8, u8);
                            TcPre pre;
                            tc_finish<T>(a, n, first, g8, u8, pre);
                        }
                    } else {
                        // two items per pass: 8 consecutive rows of token n and of token n + 8 (idx and idx + 128)
                        for (int idx = et; idx < 16 * N; idx += 256) {
                            const int c = idx & 15, n0 = idx >> 4, n1 = n0 + 8;
                            const int first = rb * TC_BM + 8 * c;
                            const bool rows_ok = first + 8 <= a.out;
                            const bool v0 = rows_ok && n0 < a.n_tok, v1 = rows_ok && n1 < a.n_tok && idx + 128 < 16 * N;
                            if (!v0 && !v1) continue;
                            TcPre pre0, pre1;
                            if (v0) tc_prefetch<T>(a, n0, first, pre0);
                            if (v1) tc_prefetch<T>(a, n1, first, pre1);
                            float o0[8], o1[8];
                            const float *r0 = tile0 + (size_t)(v0 ? n0 : n1) * TC_BM + 8 * c;
                            const float *r1 = tile0 + (size_t)(v1 ? n1 : n0) * TC_BM + 8 * c;
                            merge2(r0, r1, o0, o1);
                            if (v0) tc_finish<T>(a, n0, first, o0, zero8, pre0);
                            if (v1) tc_finish<T>(a, n1, first, o1, zero8, pre1);
                        }
                    }
                }
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");  // staging buffer is reused by the next tile
        }
    }
    // ---------------- tail: everyone meets, then the allocating warp returns the TMEM columns
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    p2p_signal(a.push);  // no-op without tensor parallelism
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tm_cols) : "memory");
    }
}

// ------------------------------------------------------------------ cluster split-K form
// For matrices with fewer row blocks than SMs.  The KS CTAs that share a row block form a thread-block cluster
// (consecutive blockIdx.x): each accumulates its K range in TMEM, stages the partial tile token-major in its own
// shared memory, and after a cluster barrier every CTA sums ITS share of the (token, 8 rows) items over all peers'
// tiles through distributed shared memory (peers in K order, so the result does not depend on timing) and runs the
// fused epilogue for them.  No scratch in global memory, no fence / ticket / reload chain: the hand-over costs two
// cluster barriers and one round of DSMEM loads.  A second cluster barrier keeps every tile alive until all peers
// have read it.  All threads of all CTAs reach both barriers on every path (a timed-out wait only skips work).
constexpr int TCK_LD = TC_BM + 4;  // floats per token row of the staged tile (16-byte aligned, bank-skewed)

__device__ __forceinline__ uint32_t tc_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void tc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 tc_ld_dsmem4(uint32_t local_saddr, uint32_t cta) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_saddr), "r"(cta));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra) : "memory");
    return v;
}

// Token blocks of 128 and 256 (prefill): the MMA takes all N tokens at once (tcgen05 allows N up to 256 columns of
// TMEM per accumulator), so a weight tile is streamed once per 256 tokens instead of once per 64; the epilogue then
// walks the accumulator in passes of NS = 64 tokens through the same staging tile and the same two cluster barriers.
template <class T>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tck_kernel(const GemvArgs a, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                int N, int n_stages, int KS, uint32_t idesc, uint32_t *status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (tc_smem(smem_raw) & 1023u)) & 1023u);
    const int stage_bytes = TC_A_BYTES + N * 128;
    const int NS = N > 64 ? 64 : N;  // tokens per epilogue pass
    float *stg = reinterpret_cast<float *>(smem + (size_t)n_stages * stage_bytes);  // [NS][TCK_LD]
    TcShared *sh = reinterpret_cast<TcShared *>(reinterpret_cast<unsigned char *>(stg) + (size_t)NS * TCK_LD * 4);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (a.pdl_trigger == 0) grid_dep_launch();
    const int nkb = a.in / TC_BK;
    const bool swiglu = a.epilogue == EPI_SWIGLU;
    const int ks = (int)tc_cluster_rank();
    const int rb = (int)blockIdx.x / KS;
    const int kb0 = (int)((long)ks * nkb / KS), kb1 = (int)((long)(ks + 1) * nkb / KS);
    const int n_units = kb1 - kb0;
    const int tm_cols = N < 32 ? 32 : N;

    if (tid == 0) {
        for (int i = 0; i < n_stages; ++i) {
            tc_mbar_init(tc_smem(&sh->full[i]), 1);
            tc_mbar_init(tc_smem(&sh->empty[i]), 1);
        }
        tc_mbar_init(tc_smem(&sh->tmem_full[0]), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&sh->tmem_base)), "r"(tm_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sh->tmem_base;

    bool ok = true;  // epilogue warps: the accumulator is complete
    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer (weights of the first ring before the dependency wait, as in gemm_tc_kernel)
        auto issue = [&](int j, bool weights, bool acts) {
            const int slot = j % n_stages;
            const uint32_t bar = tc_smem(&sh->full[slot]);
            const uint32_t dst = tc_smem(smem + (size_t)slot * stage_bytes);
            const int kx = (kb0 + j) * TC_BK;
            if (weights) {
                tc_mbar_expect_tx(bar, (uint32_t)stage_bytes);
                tc_tma_2d(dst, &map_w, kx, swiglu ? rb * 64 : rb * TC_BM, bar);
                tc_tma_2d(dst + TC_A_BYTES / 2, &map_w, kx, swiglu ? a.di + rb * 64 : rb * TC_BM + 64, bar);
            }
            if (acts) tc_tma_2d(dst + TC_A_BYTES, &map_x, kx, 0, bar);
        };
        const int first = n_units < n_stages ? n_units : n_stages;
        for (int j = 0; j < first; ++j) issue(j, true, false);
        grid_dep_wait();
        for (int j = 0; j < first; ++j) issue(j, false, true);
        for (int j = first; j < n_units && !sh->abort_flag; ++j) {
            const int slot = j % n_stages;
            const uint32_t parity = (uint32_t)(j / n_stages) & 1u;
            if (!tc_mbar_wait(tc_smem(&sh->empty[slot]), parity ^ 1u, &sh->abort_flag)) {
                atomicOr(status, 4u);
                sh->abort_flag = 1;
                break;
            }
            issue(j, true, true);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        for (int j = 0; j < n_units; ++j) {
            const int slot = j % n_stages;
            const uint32_t parity = (uint32_t)(j / n_stages) & 1u;
            if (!tc_mbar_wait(tc_smem(&sh->full[slot]), parity, &sh->abort_flag)) {
                atomicOr(status, 4u);
                sh->abort_flag = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = tc_smem(smem + (size_t)slot * stage_bytes), sb = sa + TC_A_BYTES;
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k)
                tc_mma_f16(tmem, tc_desc(sa + k * 32), tc_desc(sb + k * 32), idesc, (j > 0 || k > 0) ? 1u : 0u);
            tc_commit(tc_smem(&sh->empty[slot]));
        }
        tc_commit(tc_smem(&sh->tmem_full[0]));
    } else if (warp >= 2) {
        ok = tc_mbar_wait(tc_smem(&sh->tmem_full[0]), 0u, &sh->abort_flag);
        if (!ok) {
            atomicOr(status, 4u);
            sh->abort_flag = 1;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }

    // every thread of every CTA of the cluster walks the same number of passes and reaches both barriers of each
    for (int t0 = 0; t0 < N; t0 += NS) {
        if (warp >= 2) {
            // ---------------- accumulator columns [t0, t0 + NS) -> token-major staging tile
            const int q = warp & 3;
            const int row = q * 32 + lane;
            for (int c0 = 0; c0 < NS; c0 += 16) {
                uint32_t r[16];
                if (ok) {
                    tc_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(t0 + c0), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) stg[(size_t)(c0 + i) * TCK_LD + row] = ok ? __uint_as_float(r[i]) : 0.f;
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        tc_cluster_sync();  // every CTA of the row block has staged its partial tile

        if (warp >= 2 && t0 < a.n_tok) {
            // ---------------- this CTA's share of the items: chunk c of 8 rows (8 pairs for SwiGLU) with c % KS == ks
            const int et = tid - 64;
            const int chunks = swiglu ? 8 : 16;
            const int mine = (chunks - ks + KS - 1) / KS;  // chunks ks, ks + KS, ...
            TcPre pre[8];
            int cnt = 0;
            for (int idx = et; idx < mine * NS; idx += 128, ++cnt) {
                const int c = ks + (idx % mine) * KS, n = t0 + idx / mine;
                const int first = swiglu ? rb * 64 + 8 * c : rb * TC_BM + 8 * c;
                if (n < a.n_tok && first + 8 <= (swiglu ? a.di : a.out)) tc_prefetch<T>(a, n, first, pre[cnt]);
            }
            cnt = 0;
            for (int idx = et; idx < mine * NS; idx += 128, ++cnt) {
                const int c = ks + (idx % mine) * KS, nl = idx / mine, n = t0 + nl;
                const int first = swiglu ? rb * 64 + 8 * c : rb * TC_BM + 8 * c;
                if (!(n < a.n_tok && first + 8 <= (swiglu ? a.di : a.out))) continue;
                float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, u[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                const uint32_t sv = tc_smem(stg + (size_t)nl * TCK_LD + 8 * c);
                for (int p = 0; p < KS; ++p) {
                    const float4 lo = tc_ld_dsmem4(sv, (uint32_t)p), hi = tc_ld_dsmem4(sv + 16, (uint32_t)p);
                    v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w;
                    v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
                    if (swiglu) {
                        const float4 l2 = tc_ld_dsmem4(sv + 64 * 4, (uint32_t)p), h2 = tc_ld_dsmem4(sv + 64 * 4 + 16, (uint32_t)p);
                        u[0] += l2.x; u[1] += l2.y; u[2] += l2.z; u[3] += l2.w;
                        u[4] += h2.x; u[5] += h2.y; u[6] += h2.z; u[7] += h2.w;
                    }
                }
                tc_finish<T>(a, n, first, v, u, pre[cnt]);
            }
        }
        tc_cluster_sync();  // nobody overwrites or leaves while a peer may still read its tile
    }
    p2p_signal(a.push);  // no-op without tensor parallelism
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tm_cols) : "memory");
    }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*TcEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TcEncodeFn tc_encode_fn() {
    static TcEncodeFn fn = nullptr;
    static bool tried = false;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TcEncodeFn>(p);
    }
    return fn;
}

// 2-D map of a row-major [rows, cols] matrix of 16-bit elements; box = 64 columns x box_rows rows, 128-byte swizzle
static int tc_make_map(CUtensorMap *m, const void *base, int dt, uint64_t rows, uint64_t cols, uint64_t row_stride,
                       uint32_t box_rows) {
    TcEncodeFn fn = tc_encode_fn();
    if (!fn) {
        set_error("gemm_tc: cuTensorMapEncodeTiled is not available");
        return LCU_ERR_CUDA;
    }
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstr[1] = {row_stride * 2};
    cuuint32_t box[2] = {TC_BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, dt == LCU_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                    const_cast<void *>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("gemm_tc: cuTensorMapEncodeTiled failed with %d (base %p, %llu x %llu, stride %llu)", (int)r, base,
                  (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)row_stride);
        return LCU_ERR_CUDA;
    }
    return LCU_OK;
}

// status word for callers that have no context (the stand-alone operator)
static __device__ uint32_t g_tc_fallback_status;

static thread_local float *g_tc_ws = nullptr;
static thread_local size_t g_tc_ws_bytes = 0;
static thread_local unsigned *g_tc_tickets = nullptr;
static thread_local int g_tc_n_tickets = 0;
static thread_local uint32_t *g_tc_status = nullptr;

void gemm_tc_set_scratch(void *ws, size_t ws_bytes, unsigned *tickets, int n_tickets, uint32_t *status) {
    g_tc_ws = reinterpret_cast<float *>(ws);
    g_tc_ws_bytes = ws_bytes;
    g_tc_tickets = tickets;
    g_tc_n_tickets = n_tickets;
    g_tc_status = status;
}

bool gemm_tc_supported(int in, int w_q8) { return !w_q8 && in >= TC_BK && in % TC_BK == 0 && tc_encode_fn() != nullptr; }

static size_t tc_smem_bytes(int N, int stages) {
    return 1024 + (size_t)stages * (TC_A_BYTES + N * 128) + (size_t)TC_BM * (N + 1) * 4 + sizeof(TcShared) + 64;
}

template <class T>
static int tc_launch_t(const GemvArgs &a, int dt, cudaStream_t s, bool pdl, bool dry) {
    auto kernel = gemm_tc_kernel<T>;
    const int N = a.n_tok <= 16 ? 16 : (a.n_tok <= 32 ? 32 : (a.n_tok <= 64 ? 64 : (a.n_tok <= 128 ? 128 : 256)));
    int stages = 8;
    while (stages > 2 && tc_smem_bytes(N, stages) > (size_t)227 * 1024) --stages;
    const size_t smem = tc_smem_bytes(N, stages);
    static std::mutex mu;
    static std::map<int, uint32_t *> done;  // device -> fallback status word (also marks the attribute as set)
    int dev = 0;
    cudaGetDevice(&dev);
    uint32_t *status = g_tc_status;
    {
        std::lock_guard<std::mutex> lk(mu);
        auto it = done.find(dev);
        if (it == done.end()) {
            LCU_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            LCU_CHECK_CUDA(cudaFuncSetAttribute(gemm_tck_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            void *p = nullptr;
            LCU_CHECK_CUDA(cudaGetSymbolAddress(&p, g_tc_fallback_status));
            it = done.emplace(dev, reinterpret_cast<uint32_t *>(p)).first;
        }
        if (!status) status = it->second;
    }
    if (dry) return LCU_OK;
    const int n_pairs = a.out / 2;
    const int sms = sm_count();
    const uint32_t fmt = dt == LCU_BF16 ? 1u : 0u;
    CUtensorMap mw, mx;
    int rc;
    // 16-byte epilogue accesses need aligned, 8-divisible outputs
    bool vec_ok = a.stride_y % 8 == 0 && ((uintptr_t)a.y % 16) == 0 && (a.epilogue == EPI_SWIGLU ? a.di % 8 == 0 : a.out % 8 == 0);
    if (a.epilogue == EPI_RESIDUAL) vec_ok = vec_ok && a.stride_res % 8 == 0 && ((uintptr_t)a.res % 16) == 0;
    if (a.epilogue == EPI_ROPE_KV)
        vec_ok = vec_ok && a.dh % 8 == 0 && a.qd % 8 == 0 && a.kvd % 8 == 0 && ((uintptr_t)a.kv_pool % 16) == 0 &&
                 ((uintptr_t)a.sin_t % 16) == 0 && ((uintptr_t)a.cos_t % 16) == 0;
    const int vec = vec_ok ? 1 : 0;
    // ---- weight rows on M (any output shape; row blocks of 128)
    rc = tc_make_map(&mw, a.w, dt, (uint64_t)a.out, (uint64_t)a.in, (uint64_t)a.in, 64);
    if (rc) return rc;
    // the activation map has exactly n_tok rows: the rest of the N-row box is out of bounds and zero-filled
    rc = tc_make_map(&mx, a.x, dt, (uint64_t)a.n_tok, (uint64_t)a.in, (uint64_t)a.stride_x, (uint32_t)N);
    if (rc) return rc;
    // ---- few row blocks: the CTAs of a row block form a cluster and merge through distributed shared memory
    {
        // 1: where it measured faster than the stream-K split (64-token blocks: 6.23 -> 6.00 ms per 8B batch-64 step;
        // very few row blocks: 11.2 -> 8.7 ms for one rank's share of the 70B shape; with 16..32 tokens and 32..48 row
        // blocks the balanced stream-K split wins: 4.75 against 4.95 ms), 2: wherever it applies, 0: never
        const int cluster_mode = tuning().tc_cluster;
        const int n_rb_c = (n_pairs + 63) / 64, nkb_c = a.in / TC_BK;
        int KS = sms / n_rb_c;
        if (KS > 8) KS = 8;
        if (KS < 1) KS = 1;
        while (KS > 1 && nkb_c / KS < 4) --KS;
        // blocks of more than 64 tokens exist in this form only (clusters of one CTA where the matrix has row blocks to spare)
        // 1: where it measured faster than the stream-K split: 64-token blocks, and matrices whose row blocks leave room
        // for clusters of four and more (8B batch 32, per launch: O 20.9 -> 18.3 us, down 35.4 -> 32.9 us; the 48-row-block
        // QKV matrix with clusters of three 26.8 -> 34.5 us, so it stays on stream-K)
        const bool cluster_on = N > 64 || cluster_mode == 2 || (cluster_mode == 1 && (N == 64 || n_rb_c * 4 <= sms));
        if (vec && cluster_on && (KS >= 2 || N > 64)) {
            const int stage_bytes = TC_A_BYTES + N * 128;
            const int NS = N > 64 ? 64 : N;
            const size_t fixed = 1024 + (size_t)NS * TCK_LD * 4 + sizeof(TcShared) + 64;
            int st = (int)(((size_t)227 * 1024 - fixed) / stage_bytes);
            if (st > TC_MAX_STAGES) st = TC_MAX_STAGES;
            const uint32_t idesc_c = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(n_rb_c * KS);
            cfg.blockDim = dim3(TC_THREADS);
            cfg.dynamicSmemBytes = fixed + (size_t)st * stage_bytes;
            cfg.stream = s;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)KS;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = pdl ? 2 : 1;
            LCU_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemm_tck_kernel<T>, a, mw, mx, N, st, KS, idesc_c, status));
            g_linear_last_ctas = n_rb_c * KS;
            return LCU_OK;
        }
    }
    if (N > 64) {
        // the 16-byte epilogue does not apply to this shape: 64-token passes of the general form
        for (int t0 = 0; t0 < a.n_tok; t0 += 64) {
            GemvArgs b = a;
            b.n_tok = a.n_tok - t0 < 64 ? a.n_tok - t0 : 64;
            b.x = reinterpret_cast<const unsigned char *>(a.x) + (size_t)t0 * a.stride_x * 2;
            b.y = reinterpret_cast<unsigned char *>(a.y) + (size_t)t0 * a.stride_y * 2;
            if (a.res) b.res = reinterpret_cast<const unsigned char *>(a.res) + (size_t)t0 * a.stride_res * 2;
            if (a.pos) { b.pos = a.pos + t0; b.tok_seq = a.tok_seq + t0; }
            int rc2 = tc_launch_t<T>(b, dt, s, pdl, dry);
            if (rc2) return rc2;
        }
        return LCU_OK;
    }
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
    // Work split (stream-K): the (row block, K block) units are dealt to the SMs in equal contiguous ranges, so
    // the launch is balanced whatever the row-block count; row blocks cut between CTAs are summed through scratch.
    // Without scratch, or when the vector epilogue does not apply, ranges are whole row blocks.
    const int n_rb = (n_pairs + 63) / 64, nkb = a.in / TC_BK, total = n_rb * nkb;
    int units = (total + sms - 1) / sms;
    if (units < 8) units = 8;  // at least 8 K blocks (128 KB of weights) per CTA
    // a row block is shared by at most 6 CTAs: the merge loads 6 segments at once, beyond that it walks them one
    // round trip at a time (a [1280 x 8192] projection cut 15 ways took 41 us for 21 MB)
    if (units < (nkb + 4) / 5) units = (nkb + 4) / 5;
    int max_seg = (nkb + units - 1) / units + 1;
    const bool cut = vec && g_tc_ws && g_tc_tickets && n_rb <= g_tc_n_tickets &&
                     (size_t)n_rb * max_seg * N * TC_BM * 4 <= g_tc_ws_bytes;
    if (!cut || units % nkb == 0) {
        units = nkb * ((n_rb + sms - 1) / sms);
        max_seg = 1;
    }
    dim3 grid((total + units - 1) / units);
    LCU_CHECK_CUDA(launch_kernel(kernel, grid, dim3(TC_THREADS), smem, s, pdl, a, mw, mx, n_pairs, N, stages, units, max_seg, vec,
                                 idesc, g_tc_ws, g_tc_tickets, status));
    g_linear_last_ctas = (int)grid.x;
    return LCU_OK;
}

int gemm_tc_launch(const GemvArgs &a, int dt, cudaStream_t s, bool pdl, bool dry) {
    LCU_REQUIRE(a.n_tok >= 1 && a.n_tok <= 256, "gemm_tc: n_tok = %d (1..256)", a.n_tok);
    LCU_REQUIRE(dry || gemm_tc_supported(a.in, a.w_q8), "gemm_tc: in = %d unsupported", a.in);
    LCU_REQUIRE(a.out > 0 && a.out % 2 == 0, "gemm_tc: out = %d must be even", a.out);
    LCU_REQUIRE(a.prologue == PRO_NONE && !a.x_rows, "gemm_tc: takes prepared activations only");
    LCU_REQUIRE(a.stride_x % 8 == 0, "gemm_tc: x row stride %d must be a multiple of 8 elements", a.stride_x);
    LCU_REQUIRE(dry || (((uintptr_t)a.x | (uintptr_t)a.w) % 16) == 0, "gemm_tc: operands must be 16-byte aligned");
    if (a.epilogue == EPI_SWIGLU) LCU_REQUIRE(a.out == 2 * a.di, "gemm_tc: swiglu needs out == 2*di");
    if (dt == LCU_F16) return tc_launch_t<__half>(a, dt, s, pdl, dry);
    if (dt == LCU_BF16) return tc_launch_t<__nv_bfloat16>(a, dt, s, pdl, dry);
    set_error("gemm_tc: activation dtype %d unsupported", dt);
    return LCU_ERR_INVALID;
}

int gemm_tc_warm(int dt) {
    GemvArgs a{};
    a.in = 256; a.out = 256; a.n_tok = 16; a.stride_x = 256; a.epilogue = EPI_STORE;
    return gemm_tc_launch(a, dt, nullptr, false, true);
}

}  // namespace lcu
