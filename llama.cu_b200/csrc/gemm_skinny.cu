// Batched `Linear` for 5..64 tokens per pass — batched decode rounds and prefill chunks
// (llama.cu/src/op/linear.rs:17-120; the reference calls cuBLAS GemmEx with m = out,
// n = bucketed token count, k = in).  Still HBM-bound (<= 64 flop per weight byte), so the
// design goal is the GEMV's: stream every weight byte exactly once with many 128-bit loads
// in flight; tensor cores (mma.sync m16n8k16, f32 accumulate) only keep the arithmetic
// off the critical path.
//
//   - a warp owns 8 row PAIRS (16 weight rows = the M of the MMA; the token block is N);
//     the MMA's rows g and g+8 are the two rows of pair g (adjacent rows, or gate row p and
//     up row p + di), so a thread ends up holding both values of a pair for its two tokens
//     and the RoPE / SwiGLU / residual epilogues need no data exchange;
//   - weights go global -> registers directly as MMA A-fragments: each lane loads 16
//     contiguous bytes (one 256-bit load) of row g and of row g+8, so the 4 lanes of a quad read a
//     whole 128-byte line; the K positions inside a 64-wide block are permuted (lane t supplies
//     k = 16t..16t+15), which is harmless because the activation B-fragments read from shared
//     memory use the same permutation;
//   - a CTA is 8 warps = 128 weight rows sharing one activation chunk (256 K values of every
//     token, double-buffered in shared memory with cp.async, rows beyond the round zero-filled),
//     so activations are re-read from L2 once per 128 rows only;
//   - matrices with few rows are split along K across CTAs (grid.y) to fill the SMs; partial
//     sums go through scratch memory and the last CTA of a row block to arrive (atomic
//     ticket) adds them in split order, then runs the fused epilogue of the GEMV
//     (gemv_epilogue) for each (pair, token).
#include <cstdlib>
#include <map>
#include <mutex>
#include <type_traits>

#include "gemv.cuh"

namespace lcu {

constexpr int SK_THREADS = 256;
constexpr int SK_KBC = 4;             // 64-wide K blocks per activation chunk
constexpr int SK_XK = SK_KBC * 64;    // K elements per chunk
constexpr int SK_BP = 64;             // row pairs per CTA (8 warps x 8 pairs = 128 weight rows)

__device__ __forceinline__ void sk_cp_async_16(void *smem_dst, const void *gsrc, bool valid) {
    unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gsrc), "r"(sz) : "memory");
}

// grid = (row blocks of 64 pairs, K splits).  With more than one K split the partial sums go through
// `ws` [split][pair][token][2] and the last CTA of a row block to arrive (ticket) adds them in split
// order and runs the epilogue, so the result does not depend on which CTA finishes last.
// Fused epilogue of a thread's 2 x NTL (pair, token) values.  The residual is updated in place, so the compiler cannot
// move the residual loads of one item above the stores of the previous one: they are all fetched first.
template <class T, int NTL>
__device__ __forceinline__ void sk_finish(const GemvArgs &a, int pair, int t4, float acc[NTL][4]) {
    if (a.epilogue == EPI_RESIDUAL && a.push.n == 0) {
        const size_t r = (size_t)pair * 2;
        uint32_t res[NTL][2];
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int n = nt * 8 + 2 * t4 + k;
                res[nt][k] = n < a.n_tok ? *reinterpret_cast<const uint32_t *>(reinterpret_cast<const T *>(a.res) + (size_t)n * a.stride_res + r) : 0u;
            }
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int n = nt * 8 + 2 * t4 + k;
                if (n >= a.n_tok) continue;
                const float2 rf = Act<T>::to_f2(res[nt][k]);
                *reinterpret_cast<uint32_t *>(reinterpret_cast<T *>(a.y) + (size_t)n * a.stride_y + r) =
                    Act<T>::pack(acc[nt][k] + rf.x, acc[nt][2 + k] + rf.y);
            }
        return;
    }
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) {
        const int n0 = nt * 8 + 2 * t4;
        if (n0 < a.n_tok) gemv_epilogue<T>(a, pair, n0, acc[nt][0], acc[nt][2]);
        if (n0 + 1 < a.n_tok) gemv_epilogue<T>(a, pair, n0 + 1, acc[nt][1], acc[nt][3]);
    }
}

// Q8 = true (f16 activations only): weights are the repacked Q8_0 planes, int8 [out, in] then f16 scales
// [out, in/32].  Inside a 64-wide K block lane t4 owns k = 8 t4 .. 8 t4 + 7 of EACH 32-wide quantisation block
// (two 8-byte loads per row), so every pair of MMAs stays inside one quantisation block: its products are summed
// exactly (integers times f16 activations, f32 accumulation) into a temporary accumulator which is then scaled
// by the block's scale of row g / row g + 8 — the same arithmetic as scale * q dequantised in f32.
template <class T, int NTL, bool Q8>
__global__ void __launch_bounds__(SK_THREADS, (NTL <= 4 ? 2 : 1)) gemm_skinny_kernel(const GemvArgs a, int n_pairs, float *ws,
                                                                    unsigned *tickets) {
    constexpr int N = 8 * NTL;
    constexpr int ROWB = SK_XK * 2 + 16;  // bytes per activation row in shared memory (+16: bank skew)
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (a.pdl_trigger == 0) grid_dep_launch();
    const int g = lane >> 2, t4 = lane & 3;
    const int ksplit = gridDim.y, ks = blockIdx.y;
    const int Kper = a.in / ksplit;
    const int k0 = ks * Kper;
    const int nch = (Kper + SK_XK - 1) / SK_XK;
    const bool swiglu = a.epilogue == EPI_SWIGLU;

    const int pair = blockIdx.x * SK_BP + warp * 8 + g;
    const bool pv = pair < n_pairs;
    const size_t ra = swiglu ? (size_t)pair : (size_t)pair * 2;
    const size_t rb = swiglu ? (size_t)pair + a.di : ra + 1;
    const unsigned char *wbase = reinterpret_cast<const unsigned char *>(a.w);
    // inside a 64-wide K block lane t4 owns K values [16*t4, 16*t4 + 16): one 256-bit load per row,
    // and the 4 lanes of a quad read one full 128-byte line
    const unsigned char *wa = Q8 ? wbase + (pv ? ra : 0) * (size_t)a.in + (size_t)k0 + 8 * t4
                                 : wbase + (pv ? ra : 0) * (size_t)a.in * 2 + ((size_t)k0 + 16 * t4) * 2;
    const unsigned char *wb = Q8 ? wbase + (pv ? rb : 0) * (size_t)a.in + (size_t)k0 + 8 * t4
                                 : wbase + (pv ? rb : 0) * (size_t)a.in * 2 + ((size_t)k0 + 16 * t4) * 2;
    // Q8: the 8 scales of a 256-wide chunk are 16 contiguous bytes per row
    const uint16_t *sbase = reinterpret_cast<const uint16_t *>(a.w_scales);
    const uint16_t *sa = Q8 ? sbase + (pv ? ra : 0) * (size_t)(a.in / 32) + k0 / 32 : nullptr;
    const uint16_t *sb = Q8 ? sbase + (pv ? rb : 0) * (size_t)(a.in / 32) + k0 / 32 : nullptr;
    const T *xg = reinterpret_cast<const T *>(a.x);

    float acc[NTL][4];
#pragma unroll
    for (int i = 0; i < NTL; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    auto load_x_chunk = [&](int c, int buf) {
        unsigned char *dst = smem + (size_t)buf * N * ROWB;
        constexpr int PIECES = N * (SK_XK / 8);  // 16-byte pieces per chunk
        for (int i = tid; i < PIECES; i += SK_THREADS) {
            int n = i / (SK_XK / 8), piece = i - n * (SK_XK / 8);
            int kk = c * SK_XK + piece * 8;
            bool valid = n < a.n_tok && kk < Kper;
            const T *src = valid ? xg + (size_t)n * a.stride_x + k0 + kk : xg;
            sk_cp_async_16(dst + (size_t)n * ROWB + (size_t)piece * 16, src, valid);
        }
    };
    // weights: a rolling window of SK_KBC 64-wide blocks per row in registers; block kb of the next
    // chunk is requested as soon as block kb of this chunk has been multiplied
    u32x8 wra[Q8 ? 1 : SK_KBC], wrb[Q8 ? 1 : SK_KBC];
    uint2 qa[Q8 ? SK_KBC : 1][2], qb[Q8 ? SK_KBC : 1][2];  // Q8: [64-block][quantisation block] 8 int8 each
    uint4 sca = make_uint4(0, 0, 0, 0), scb = sca, sca_n = sca, scb_n = sca;  // Q8: 8 f16 scales of this / the next chunk
    auto load_w = [&](int c, int kb) {
        int kk = c * SK_XK + kb * 64;
        bool v = pv && kk < Kper;
        if constexpr (Q8) {
            qa[kb][0] = v ? ld_stream_64(wa + kk) : make_uint2(0, 0);
            qa[kb][1] = v ? ld_stream_64(wa + kk + 32) : make_uint2(0, 0);
            qb[kb][0] = v ? ld_stream_64(wb + kk) : make_uint2(0, 0);
            qb[kb][1] = v ? ld_stream_64(wb + kk + 32) : make_uint2(0, 0);
            if (kb == 0) {
                sca_n = v ? __ldg(reinterpret_cast<const uint4 *>(sa + kk / 32)) : make_uint4(0, 0, 0, 0);
                scb_n = v ? __ldg(reinterpret_cast<const uint4 *>(sb + kk / 32)) : make_uint4(0, 0, 0, 0);
            }
        } else {
            u32x8 z;
            z.lo = z.hi = make_uint4(0, 0, 0, 0);
            wra[kb] = v ? ld_stream_256(wa + (size_t)kk * 2) : z;
            wrb[kb] = v ? ld_stream_256(wb + (size_t)kk * 2) : z;
        }
    };
#pragma unroll
    for (int kb = 0; kb < SK_KBC; ++kb) load_w(0, kb);
    grid_dep_wait();
    load_x_chunk(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    for (int c = 0; c < nch; ++c) {
        if (c + 1 < nch) load_x_chunk(c + 1, (c + 1) & 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const unsigned char *xs = smem + (size_t)(c & 1) * N * ROWB + (size_t)t4 * (Q8 ? 16 : 32);
        if constexpr (Q8) {
            sca = sca_n;
            scb = scb_n;
        }
#pragma unroll
        for (int kb = 0; kb < SK_KBC; ++kb) {
            if constexpr (Q8) {
                const uint32_t sw_a[4] = {sca.x, sca.y, sca.z, sca.w}, sw_b[4] = {scb.x, scb.y, scb.z, scb.w};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t af[4], bf[4];
                    q8x4_to_h2(qa[kb][h].x, af[0], af[1]);
                    q8x4_to_h2(qa[kb][h].y, af[2], af[3]);
                    q8x4_to_h2(qb[kb][h].x, bf[0], bf[1]);
                    q8x4_to_h2(qb[kb][h].y, bf[2], bf[3]);
                    // scale of quantisation block 2 kb + h of this chunk: half (2 kb + h) of the 8 loaded
                    const __half2 pa = *reinterpret_cast<const __half2 *>(&sw_a[kb]);
                    const __half2 pb = *reinterpret_cast<const __half2 *>(&sw_b[kb]);
                    const float fa = h ? __high2float(pa) : __low2float(pa), fb = h ? __high2float(pb) : __low2float(pb);
#pragma unroll
                    for (int nt = 0; nt < NTL; ++nt) {
                        const uint4 xv = *reinterpret_cast<const uint4 *>(xs + (size_t)(nt * 8 + g) * ROWB + kb * 128 + h * 64);
                        float tmp[4] = {0.f, 0.f, 0.f, 0.f};
                        mma16816<T>(tmp, af[0], bf[0], af[1], bf[1], xv.x, xv.y);
                        mma16816<T>(tmp, af[2], bf[2], af[3], bf[3], xv.z, xv.w);
                        acc[nt][0] = fmaf(fa, tmp[0], acc[nt][0]);
                        acc[nt][1] = fmaf(fa, tmp[1], acc[nt][1]);
                        acc[nt][2] = fmaf(fb, tmp[2], acc[nt][2]);
                        acc[nt][3] = fmaf(fb, tmp[3], acc[nt][3]);
                    }
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) {
                    const uint4 *xp = reinterpret_cast<const uint4 *>(xs + (size_t)(nt * 8 + g) * ROWB + kb * 128);
                    const uint4 x0 = xp[0], x1 = xp[1];
                    mma16816<T>(acc[nt], wra[kb].lo.x, wrb[kb].lo.x, wra[kb].lo.y, wrb[kb].lo.y, x0.x, x0.y);
                    mma16816<T>(acc[nt], wra[kb].lo.z, wrb[kb].lo.z, wra[kb].lo.w, wrb[kb].lo.w, x0.z, x0.w);
                    mma16816<T>(acc[nt], wra[kb].hi.x, wrb[kb].hi.x, wra[kb].hi.y, wrb[kb].hi.y, x1.x, x1.y);
                    mma16816<T>(acc[nt], wra[kb].hi.z, wrb[kb].hi.z, wra[kb].hi.w, wrb[kb].hi.w, x1.z, x1.w);
                }
            }
            if (c + 1 < nch) load_w(c + 1, kb);
        }
        __syncthreads();
    }

    if (ksplit == 1) {
        // a thread holds both rows of its pair for tokens 2t and 2t+1 of every token tile
        if (pv) sk_finish<T, NTL>(a, pair, t4, acc);
        p2p_signal(a.push);
        return;
    }
    // ---- split K: partials to scratch, the last CTA of the row block adds them in split order
    if (pv) {
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) {
            float4 v = make_float4(acc[nt][0], acc[nt][2], acc[nt][1], acc[nt][3]);  // (tok 2t: va, vb), (tok 2t+1: va, vb)
            *reinterpret_cast<float4 *>(ws + (((size_t)ks * n_pairs + pair) * N + nt * 8 + 2 * t4) * 2) = v;
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned ticket = atomicAdd(&tickets[blockIdx.x], 1u);
        s_last = ticket == (unsigned)ksplit - 1;
        if (s_last) tickets[blockIdx.x] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!s_last) {
        p2p_signal(a.push);
        return;
    }
    __threadfence();
    if (pv) {
        // the partial sums of two token tiles at a time are all requested before the first add (one L2 round trip
        // per two tiles instead of one per split and tile)
#pragma unroll
        for (int nt0 = 0; nt0 < NTL; nt0 += 2) {
            float4 part[2][8];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < ksplit)
                        part[i][j] = __ldcg(reinterpret_cast<const float4 *>(ws + (((size_t)j * n_pairs + pair) * N + (nt0 + i) * 8 + 2 * t4) * 2));
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < ksplit) { sum.x += part[i][j].x; sum.y += part[i][j].y; sum.z += part[i][j].z; sum.w += part[i][j].w; }
                acc[nt0 + i][0] = sum.x; acc[nt0 + i][2] = sum.y; acc[nt0 + i][1] = sum.z; acc[nt0 + i][3] = sum.w;
            }
        }
        sk_finish<T, NTL>(a, pair, t4, acc);
    }
    p2p_signal(a.push);
}

// ------------------------------------------------------------------ host side

bool gemm_skinny_supported(int in, int w_q8) { return in >= SK_XK && in % 32 == 0 && (!w_q8 || in % SK_XK == 0); }

// Scratch for split-K partial sums and the per-row-block tickets, handed over by the context.
static thread_local float *g_ws = nullptr;
static thread_local size_t g_ws_bytes = 0;
static thread_local unsigned *g_tickets = nullptr;
static thread_local int g_n_tickets = 0;

void gemm_skinny_set_scratch(void *ws, size_t ws_bytes, unsigned *tickets, int n_tickets) {
    g_ws = reinterpret_cast<float *>(ws);
    g_ws_bytes = ws_bytes;
    g_tickets = tickets;
    g_n_tickets = n_tickets;
}

// K splits across CTAs: the count that fills the SMs best (whole waves), smallest on ties.
static int sk_choose_ksplit(int in, int n_pairs, int n) {
    const int row_blocks = (n_pairs + SK_BP - 1) / SK_BP;
    const int sms = sm_count();
    int best = 1;
    double best_eff = -1.0;
    for (int ks = 1; ks <= 8; ks *= 2) {
        if (in % (ks * 32) || in / ks < SK_XK) break;
        if (ks > 1 && (!g_ws || (size_t)ks * n_pairs * n * 2 * 4 > g_ws_bytes || row_blocks > g_n_tickets)) break;
        int ctas = row_blocks * ks;
        int waves = (ctas + sms - 1) / sms;
        double eff = (double)ctas / ((double)waves * sms);
        if (ks > 1) eff -= 0.03 * (ks > 2 ? 2 : 1);  // partial sums cost traffic: prefer fewer splits when close
        if (eff > best_eff + 1e-9) { best_eff = eff; best = ks; }
    }
    return best;
}

template <class T, int NTL, bool Q8>
static int sk_inst(const GemvArgs &a, int n_pairs, cudaStream_t s, bool pdl, bool dry) {
    auto kernel = gemm_skinny_kernel<T, NTL, Q8>;
    constexpr int N = 8 * NTL;
    size_t smem = (size_t)2 * N * (SK_XK * 2 + 16);
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
    int ksplit = sk_choose_ksplit(a.in, n_pairs, N);
    if (Q8) while (ksplit > 1 && (a.in / ksplit) % SK_XK) ksplit /= 2;  // a K range must hold whole scale groups
    dim3 grid((n_pairs + SK_BP - 1) / SK_BP, ksplit);
    LCU_CHECK_CUDA(launch_kernel(kernel, grid, dim3(SK_THREADS), smem, s, pdl, a, n_pairs, g_ws, g_tickets));
    g_linear_last_ctas = (int)(grid.x * grid.y);
    return LCU_OK;
}

template <class T>
static int sk_t(const GemvArgs &a, cudaStream_t s, bool pdl, bool dry) {
    int n_pairs = a.out / 2;
    int ntl = a.n_tok <= 16 ? 2 : (a.n_tok <= 32 ? 4 : 8);
    if (a.w_q8) {
        if constexpr (std::is_same<T, __half>::value) {
            switch (ntl) {
            case 2: return sk_inst<T, 2, true>(a, n_pairs, s, pdl, dry);
            case 4: return sk_inst<T, 4, true>(a, n_pairs, s, pdl, dry);
            default: return sk_inst<T, 8, true>(a, n_pairs, s, pdl, dry);
            }
        } else {
            set_error("gemm_skinny: Q8_0 weights need f16 activations");
            return LCU_ERR_INVALID;
        }
    }
    switch (ntl) {
    case 2: return sk_inst<T, 2, false>(a, n_pairs, s, pdl, dry);
    case 4: return sk_inst<T, 4, false>(a, n_pairs, s, pdl, dry);
    default: return sk_inst<T, 8, false>(a, n_pairs, s, pdl, dry);
    }
}

int gemm_skinny_launch(const GemvArgs &a, int dt, cudaStream_t s, bool pdl, bool dry) {
    LCU_REQUIRE(a.n_tok >= 1 && a.n_tok <= 64, "gemm_skinny: n_tok = %d (1..64)", a.n_tok);
    LCU_REQUIRE(gemm_skinny_supported(a.in, a.w_q8), "gemm_skinny: in = %d unsupported", a.in);
    LCU_REQUIRE(a.out > 0 && a.out % 2 == 0, "gemm_skinny: out = %d must be even", a.out);
    LCU_REQUIRE(a.prologue == PRO_NONE && !a.x_rows, "gemm_skinny: takes prepared activations only");
    LCU_REQUIRE(a.stride_x % 8 == 0, "gemm_skinny: x row stride %d must be a multiple of 8 elements", a.stride_x);
    if (a.epilogue == EPI_SWIGLU) LCU_REQUIRE(a.out == 2 * a.di, "gemm_skinny: swiglu needs out == 2*di");
    if (dt == LCU_F16) return sk_t<__half>(a, s, pdl, dry);
    if (dt == LCU_BF16) return sk_t<__nv_bfloat16>(a, s, pdl, dry);
    set_error("gemm_skinny: activation dtype %d unsupported", dt);
    return LCU_ERR_INVALID;
}

int gemm_skinny_warm(int in, int out, int dt, int w_q8) {
    if (!gemm_skinny_supported(in, w_q8)) return LCU_OK;
    for (int n = 16; n <= 64; n *= 2) {
        GemvArgs a{};
        a.in = in; a.out = out; a.n_tok = n; a.stride_x = in; a.epilogue = EPI_STORE; a.w_q8 = w_q8;
        int rc = gemm_skinny_launch(a, dt, nullptr, false, true);
        if (rc) return rc;
    }
    return LCU_OK;
}

}  // namespace lcu
