// Weight-streaming GEMV for 1..4 tokens — the `Linear` operator of the decode step
// (llama.cu/src/op/linear.rs:17-120: y = x·Wᵀ (+ residual), f32 accumulation, one
// rounding) with the neighbouring operators fused in:
//   prologue  RMSNorm of the input rows (op/rms_norm.cuh) — each CTA normalises x itself;
//   epilogue  residual add (linear.rs:35-46), RoPE + KV-cache append on the fused QKV
//             projection (op/rope.cuh, the append half of attention_kv_cached,
//             exec/step.rs:140-184), or SwiGLU on the fused gate|up projection
//             (op/swiglu.cuh).
// Every fused value is first rounded to the activation dtype where the reference
// materialises a tensor, so the fusion does not move a rounding point.
//
// The step is HBM-bound: each weight byte is read once per step, so the kernel is built
// around keeping 128-bit streaming loads in flight on every SM.
//   - grid: one or two CTAs per SM, each owning a contiguous, balanced range of row PAIRS
//     (pairs because RoPE rotates adjacent rows and SwiGLU joins row i with row i+di);
//   - inside a CTA the K dimension is split across KS warps (x RS row sub-groups); a warp
//     keeps 2*RP rows x KI 16-byte vectors in registers, loaded one group ahead of their
//     use — the loads of group g+1 are in flight while group g is reduced and stored;
//   - the first group's loads are issued BEFORE griddepcontrol.wait, so under programmatic
//     dependent launch the weights of this GEMV already stream while the previous kernel
//     of the step drains; only then are the activations staged to shared memory;
//   - Q8_0 weights (int8 quants + one f16 scale per 32) are dequantised in registers;
//   - nothing an epilogue needs is fetched behind the weight stream: the per-token constants of the
//     RoPE / KV-append epilogue sit in shared memory before the dependency wait, the residual pair of
//     a row pair is requested at the start of its group;
//   - the prologue is a template parameter, so the plain kernels carry no RMSNorm code; the one-token
//     RMSNorm form works from registers with the norm weights fetched before the wait.
#include <type_traits>

#include "gemv.cuh"

#include <cstdlib>
#include <map>
#include <mutex>

namespace lcu {

// int8 -> f32 without I2F: bytes xor 0x80 become 0..255, placed in the mantissa of 2^23.
__device__ __forceinline__ void q8x4_to_f32(uint32_t q, float f[4]) {
    uint32_t u = q ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.f;
}

template <class T>
__device__ __forceinline__ void vec8_to_f32(const uint4 &v, float f[8]) {
    float2 a = Act<T>::to_f2(v.x), b = Act<T>::to_f2(v.y), c = Act<T>::to_f2(v.z), d = Act<T>::to_f2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// PRO: 0 = activations staged as they are, 1 = RMSNorm (any token count, f32 or 16-bit norm weights), 2 = RMSNorm of one
// token from registers
template <class T, bool Q8, int NT, int KI, int RP, int PRO>
__global__ void __launch_bounds__(512, (NT == 1 && !Q8) ? 2 : 1) gemv_kernel(const GemvArgs a, int KS, int RS, int n_pairs) {
    constexpr int R = 2 * RP;
    constexpr int VE = Q8 ? 16 : 8;  // weights per 16-byte vector
    extern __shared__ __align__(16) unsigned char smem[];
    T *xs = reinterpret_cast<T *>(smem);                                        // [NT][in]
    float *part = reinterpret_cast<float *>(smem + (size_t)NT * a.in * sizeof(T));  // [2][nwarps][R*NT]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int ks = warp % KS, rs = warp / KS;
    const int nvec = a.in / VE;
    const size_t row_bytes = Q8 ? (size_t)a.in : (size_t)a.in * 2;
    const bool swiglu = a.epilogue == EPI_SWIGLU;

    const int p_begin = (int)((long long)n_pairs * blockIdx.x / gridDim.x);
    const int p_end = (int)((long long)n_pairs * (blockIdx.x + 1) / gridDim.x);
    const int group_pairs = RS * RP;
    const int n_groups = (p_end - p_begin + group_pairs - 1) / group_pairs;

    uint4 wreg[R][KI];
    uint16_t sreg[Q8 ? R : 1][Q8 ? KI : 1];
    const unsigned char *wbase = reinterpret_cast<const unsigned char *>(a.w);
    const uint16_t *sbase = reinterpret_cast<const uint16_t *>(a.w_scales);

    auto load_group = [&](int g) {
#pragma unroll
        for (int rp = 0; rp < RP; ++rp) {
            int p = p_begin + g * group_pairs + rs * RP + rp;
            bool pv = p < p_end && rs < RS;
            size_t ra = swiglu ? (size_t)p : (size_t)p * 2;
            size_t rb = swiglu ? (size_t)p + a.di : ra + 1;
#pragma unroll
            for (int ki = 0; ki < KI; ++ki) {
                int kv = (ks + KS * ki) * 32 + lane;
                bool v = pv && kv < nvec;
                wreg[2 * rp][ki] = v ? ld_stream_128(wbase + ra * row_bytes + (size_t)kv * 16) : make_uint4(0, 0, 0, 0);
                wreg[2 * rp + 1][ki] = v ? ld_stream_128(wbase + rb * row_bytes + (size_t)kv * 16) : make_uint4(0, 0, 0, 0);
                if constexpr (Q8) {
                    sreg[2 * rp][ki] = v ? __ldg(sbase + ra * (size_t)(a.in / 32) + (kv >> 1)) : (uint16_t)0;
                    sreg[2 * rp + 1][ki] = v ? __ldg(sbase + rb * (size_t)(a.in / 32) + (kv >> 1)) : (uint16_t)0;
                }
            }
        }
    };

    // Order of the first requests matters: L1 hands data back in request order, so activations asked for AFTER the
    // first weight group would only arrive with it (about 3 us under full load) and the RMSNorm arithmetic would then
    // run with the memory pipe idle.  The activations are therefore requested first, as asynchronous copies straight
    // into shared memory (no registers held), the first weight group right behind them, and the norm is computed
    // while those weights are in flight.  early_prefetch == 3 keeps the older order (weights, then activations).
    const bool x_first = a.early_prefetch == 1;
    if (a.early_prefetch == 3 && n_groups > 0) load_group(0);
    // RoPE / KV-append epilogue: position, cache page and the sin / cos rows of every token come from the round's
    // descriptor and constant tables, not from the predecessor -- staged in shared memory here, before the dependency
    // wait, so that the epilogues of the row groups (and the kernel's tail) hold no chain of global loads
    __shared__ RopeStage rope_stage;
    const bool rope_staged = a.epilogue == EPI_ROPE_KV && a.dh <= 128;
    if (rope_staged) {
        const int half_dh = a.dh >> 1;
        for (int i = threadIdx.x; i < a.n_tok * half_dh; i += blockDim.x) {
            const int t = i / half_dh, e = i - t * half_dh;
            const uint32_t p = a.pos[t];
            rope_stage.sn[t][e] = a.sin_t[(size_t)p * half_dh + e];
            rope_stage.cs[t][e] = a.cos_t[(size_t)p * half_dh + e];
            if (e == 0) {
                rope_stage.pos[t] = p;
                rope_stage.page[t] = a.page_table[(size_t)a.tok_seq[t] * a.pt_stride + (p >> a.geom.page_shift)];
            }
        }
    }
    // One token, RMSNorm, at most two vectors per thread: the norm weights are constants and are fetched BEFORE the
    // dependency wait, the activations go from global memory straight to registers, are squared, scaled and written to
    // shared memory once -- two barriers and one L2 round trip after the wait instead of four and two.  Same summation
    // order and the same products as the general path below.
    const int nv8 = a.in / 8;
    constexpr bool lean = PRO == 2;
    uint4 nwv[2];
    if constexpr (lean) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            nwv[j] = i < nv8 ? __ldg(reinterpret_cast<const uint4 *>(a.norm_w) + i) : make_uint4(0, 0, 0, 0);
        }
    }
    if (a.pdl_trigger == 0) grid_dep_launch();
    grid_dep_wait();
    if (a.early_prefetch == 0 && n_groups > 0) load_group(0);

    if constexpr (lean) {
        const size_t row = a.x_rows ? a.x_rows[0] : 0;
        const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.x) + row * a.stride_x);
        uint4 xv[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            xv[j] = i < nv8 ? src[i] : make_uint4(0, 0, 0, 0);
        }
        if (x_first && n_groups > 0) load_group(0);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float f[8];
            vec8_to_f32<T>(xv[j], f);
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
        }
        ss = warp_sum(ss);
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        float v = 0.f;
        for (int w = 0; w < nwarps; ++w) v += part[w];
        const float rms = rsqrtf(v / (float)a.in + a.eps);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < nv8) {
                float f[8], wf[8];
                vec8_to_f32<T>(xv[j], f);
                vec8_to_f32<T>(nwv[j], wf);
                uint4 o;
                o.x = Act<T>::pack(rms * f[0] * wf[0], rms * f[1] * wf[1]);
                o.y = Act<T>::pack(rms * f[2] * wf[2], rms * f[3] * wf[3]);
                o.z = Act<T>::pack(rms * f[4] * wf[4], rms * f[5] * wf[5]);
                o.w = Act<T>::pack(rms * f[6] * wf[6], rms * f[7] * wf[7]);
                reinterpret_cast<uint4 *>(xs)[i] = o;
            }
        }
        __syncthreads();
    } else {
        // ---- stage the activations (optionally RMS-normalised) in shared memory
        const T *xg = reinterpret_cast<const T *>(a.x);
        for (int t = 0; t < NT; ++t) {
            uint4 *dst = reinterpret_cast<uint4 *>(xs + (size_t)t * a.in);
            if (t < a.n_tok) {
                size_t row = a.x_rows ? a.x_rows[t] : (size_t)t;
                const uint4 *src = reinterpret_cast<const uint4 *>(xg + row * a.stride_x);
                if (x_first) {
                    for (int i = threadIdx.x; i < nv8; i += blockDim.x) {
                        unsigned d = (unsigned)__cvta_generic_to_shared(dst + i);
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + i) : "memory");
                    }
                } else {
                    for (int i = threadIdx.x; i < nv8; i += blockDim.x) dst[i] = src[i];
                }
            } else {
                for (int i = threadIdx.x; i < nv8; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
            }
        }
        if (x_first) {
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (n_groups > 0) load_group(0);
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if constexpr (PRO == 1) {
            float ss[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                ss[t] = 0.f;
                const uint4 *src = reinterpret_cast<const uint4 *>(xs + (size_t)t * a.in);
                for (int i = threadIdx.x; i < nv8; i += blockDim.x) {
                    float f[8];
                    vec8_to_f32<T>(src[i], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss[t] += f[j] * f[j];
                }
                ss[t] = warp_sum(ss[t]);
                if (lane == 0) part[t * 16 + warp] = ss[t];
            }
            __syncthreads();
            float rms[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                float v = 0.f;
                for (int w = 0; w < nwarps; ++w) v += part[t * 16 + w];
                rms[t] = rsqrtf(v / (float)a.in + a.eps);
            }
            __syncthreads();
            for (int i = threadIdx.x; i < nv8; i += blockDim.x) {
                float wf[8];
                if (a.norm_f32) {
                    const float4 *nw = reinterpret_cast<const float4 *>(a.norm_w);
                    float4 w0 = nw[2 * i], w1 = nw[2 * i + 1];
                    wf[0] = w0.x; wf[1] = w0.y; wf[2] = w0.z; wf[3] = w0.w;
                    wf[4] = w1.x; wf[5] = w1.y; wf[6] = w1.z; wf[7] = w1.w;
                } else {
                    vec8_to_f32<T>(reinterpret_cast<const uint4 *>(a.norm_w)[i], wf);
                }
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    uint4 *row = reinterpret_cast<uint4 *>(xs + (size_t)t * a.in);
                    float f[8];
                    vec8_to_f32<T>(row[i], f);
                    uint4 o;
                    o.x = Act<T>::pack(rms[t] * f[0] * wf[0], rms[t] * f[1] * wf[1]);
                    o.y = Act<T>::pack(rms[t] * f[2] * wf[2], rms[t] * f[3] * wf[3]);
                    o.z = Act<T>::pack(rms[t] * f[4] * wf[4], rms[t] * f[5] * wf[5]);
                    o.w = Act<T>::pack(rms[t] * f[6] * wf[6], rms[t] * f[7] * wf[7]);
                    row[i] = o;
                }
            }
            __syncthreads();
        }
    }

    // ---- main loop over row groups
    for (int g = 0; g < n_groups; ++g) {
        // the finishing lanes ask for their residual pair now: it arrives while the group is multiplied and reduced
        EpiPre pre;
        if (rope_staged) pre.rope = &rope_stage;
        if (a.epilogue == EPI_RESIDUAL && ks == 0 && rs < RS && lane < RP * NT) {
            const int rp = lane / NT, t = lane - rp * NT;
            const int p = p_begin + g * group_pairs + rs * RP + rp;
            if (p < p_end && t < a.n_tok) {
                pre.res = *reinterpret_cast<const uint32_t *>(reinterpret_cast<const T *>(a.res) + (size_t)t * a.stride_res + (size_t)p * 2);
                pre.has_res = true;
            }
        }
        float acc[R][NT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int t = 0; t < NT; ++t) acc[r][t] = 0.f;

#pragma unroll
        for (int ki = 0; ki < KI; ++ki) {
            int kv = (ks + KS * ki) * 32 + lane;
            if (kv < nvec) {
                if constexpr (!Q8) {
                    uint4 xv[NT];
#pragma unroll
                    for (int t = 0; t < NT; ++t) xv[t] = reinterpret_cast<const uint4 *>(xs + (size_t)t * a.in)[kv];
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int t = 0; t < NT; ++t) acc[r][t] = dot8_mixed<T>(wreg[r][ki], xv[t], acc[r][t]);
                } else if constexpr (std::is_same<T, __half>::value) {
                    // Q8_0 with f16 activations: int8 -> f16 pairs (prmt + one hsub2 per pair, exact), then the same
                    // mixed-precision FMA as the f16 path: integer x activation products are exact in f32, summed in
                    // element order, scaled by the block's scale -- the value of scale * q dequantised in f32
                    uint4 xv[NT][2];
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const uint4 *xp = reinterpret_cast<const uint4 *>(xs + (size_t)t * a.in) + 2 * kv;
                        xv[t][0] = xp[0];
                        xv[t][1] = xp[1];
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        uint4 w0, w1;
                        q8x4_to_h2(wreg[r][ki].x, w0.x, w0.y);
                        q8x4_to_h2(wreg[r][ki].y, w0.z, w0.w);
                        q8x4_to_h2(wreg[r][ki].z, w1.x, w1.y);
                        q8x4_to_h2(wreg[r][ki].w, w1.z, w1.w);
                        float sc = __half2float(__ushort_as_half(sreg[r][ki]));
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            float d = dot8_mixed<T>(w0, xv[t][0], 0.f);
                            d = dot8_mixed<T>(w1, xv[t][1], d);
                            acc[r][t] = fmaf(sc, d, acc[r][t]);
                        }
                    }
                } else {
                    float xf[NT][16];
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const uint4 *xv = reinterpret_cast<const uint4 *>(xs + (size_t)t * a.in) + 2 * kv;
                        vec8_to_f32<T>(xv[0], xf[t]);
                        vec8_to_f32<T>(xv[1], xf[t] + 8);
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        float wf[16];
                        q8x4_to_f32(wreg[r][ki].x, wf);
                        q8x4_to_f32(wreg[r][ki].y, wf + 4);
                        q8x4_to_f32(wreg[r][ki].z, wf + 8);
                        q8x4_to_f32(wreg[r][ki].w, wf + 12);
                        float sc = __half2float(__ushort_as_half(sreg[r][ki]));
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            float d = 0.f;
#pragma unroll
                            for (int j = 0; j < 16; ++j) d = fmaf(wf[j], xf[t][j], d);
                            acc[r][t] = fmaf(sc, d, acc[r][t]);
                        }
                    }
                }
            }
        }
        // next group's weights go in flight before this group is reduced
        if (g + 1 < n_groups) load_group(g + 1);

        float *pbuf = part + (size_t)(g & 1) * nwarps * (R * NT);
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                float v = warp_sum(acc[r][t]);
                if (lane == 0) pbuf[warp * (R * NT) + r * NT + t] = v;
            }
        __syncthreads();
        if (ks == 0 && rs < RS && lane < RP * NT) {
            int rp = lane / NT, t = lane - rp * NT;
            int p = p_begin + g * group_pairs + rs * RP + rp;
            if (p < p_end && t < a.n_tok) {
                float va = 0.f, vb = 0.f;
                for (int k = 0; k < KS; ++k) {
                    const float *src = pbuf + (size_t)(rs * KS + k) * (R * NT);
                    va += src[(2 * rp) * NT + t];
                    vb += src[(2 * rp + 1) * NT + t];
                }
                gemv_epilogue<T>(a, p, t, va, vb, pre);
            }
        }
    }
    if (a.pdl_trigger == 1) grid_dep_launch();
    p2p_signal(a.push);
}

// ------------------------------------------------------------------ host side

thread_local int g_linear_last_ctas = 0;

struct GemvPlan {
    int KS, RS, KI, RP, nwarps;
};

// Splits the 16-byte vector columns of a row (n32 warp-wide columns) over KS warps x KI
// vectors with the least padding, preferring few vectors per warp, then fills the CTA
// with RS row sub-groups up to 16 warps.
static GemvPlan plan_for(int in, bool q8, int nt) {
    int nvec = in / (q8 ? 16 : 8);
    int n32 = (nvec + 31) / 32;
    GemvPlan best = {1, 16, 1, 1, 16};
    long best_cost = -1;
    const int kis[4] = {1, 2, 4, 8};
    for (int kii = 0; kii < 4; ++kii) {
        int ki = kis[kii];
        int ks = (n32 + ki - 1) / ki;
        if (ks > 16) continue;
        int rs = 16 / ks;
        int waste = ks * ki - n32;          // padded vector columns per row
        int idle = 16 - ks * rs;            // warps the CTA cannot use
        long cost = (long)waste * 1000 / (ks * ki) * 4 + idle * 30 + ki * 5;
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = {ks, rs, ki, 1, ks * rs};
        }
    }
    int rp = 4 / best.KI;
    if (rp < 1) rp = 1;
    int cap = 8 / nt;  // keep 2*RP*NT accumulators <= 16
    if (cap < 1) cap = 1;
    if (rp > cap) rp = cap;
    if (q8 && rp > tuning().q8_rows) rp = tuning().q8_rows;
    best.RP = rp;
    return best;
}

template <class T, bool Q8, int NT, int KI, int RP, int PRO>
static int launch_inst(const GemvArgs &a, const GemvPlan &pl, int n_pairs, cudaStream_t s, bool pdl, bool dry) {
    auto kernel = gemv_kernel<T, Q8, NT, KI, RP, PRO>;
    // activations + double-buffered per-warp partial sums (also the RMSNorm scratch)
    size_t smem = (size_t)NT * a.in * sizeof(T) + (size_t)2 * 16 * (2 * RP * NT) * sizeof(float);
    int block = pl.nwarps * 32;

    struct Info { int ctas_per_sm; };
    static std::mutex mu;
    static std::map<std::pair<int, std::pair<int, size_t>>, Info> cache;  // (device, (block, smem))
    int dev = 0;
    cudaGetDevice(&dev);
    Info info;
    {
        std::lock_guard<std::mutex> lk(mu);
        auto key = std::make_pair(dev, std::make_pair(block, smem));
        auto it = cache.find(key);
        if (it == cache.end()) {
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemv smem)");
            }
            int occ = 0;
            cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, block, smem);
            if (e != cudaSuccess) return cuda_fail(e, "occupancy(gemv)");
            if (occ < 1) {
                set_error("gemv: configuration does not fit on an SM (in = %d, smem = %zu)", a.in, smem);
                return LCU_ERR_INVALID;
            }
            int cap = tuning().gemv_ctas_per_sm;
            info.ctas_per_sm = occ > cap ? cap : occ;
            cache[key] = info;
        } else {
            info = it->second;
        }
    }
    int group_pairs = pl.RS * RP;
    int max_ctas = sm_count() * info.ctas_per_sm;
    int want = (n_pairs + group_pairs - 1) / group_pairs;
    int grid = want < max_ctas ? want : max_ctas;
    if (grid < 1) grid = 1;
    if (dry) return LCU_OK;  // attributes and occupancy are now cached for this configuration
    LCU_CHECK_CUDA(launch_kernel(kernel, dim3(grid), dim3(block), smem, s, pdl, a, pl.KS, pl.RS, n_pairs));
    g_linear_last_ctas = grid;
    return LCU_OK;
}

template <class T, bool Q8, int NT>
static int launch_nt(const GemvArgs &a, const GemvPlan &pl, int n_pairs, cudaStream_t s, bool pdl, bool dry) {
    // prologue variant: the one-token register form needs 16-bit norm weights and at most two vectors per thread
    const int pro = a.prologue != PRO_RMSNORM ? 0 : ((NT == 1 && !a.norm_f32 && a.lean_norm && a.in / 8 <= 2 * pl.nwarps * 32) ? 2 : 1);
#define LCU_GEMV_CASE(KI_, RP_)                                                                                   \
    if (pl.KI == KI_ && pl.RP == RP_) {                                                                           \
        if (pro == 0) return launch_inst<T, Q8, NT, KI_, RP_, 0>(a, pl, n_pairs, s, pdl, dry);                    \
        if (pro == 1) return launch_inst<T, Q8, NT, KI_, RP_, 1>(a, pl, n_pairs, s, pdl, dry);                    \
        if constexpr (NT == 1) return launch_inst<T, Q8, NT, KI_, RP_, 2>(a, pl, n_pairs, s, pdl, dry);           \
    }
    if constexpr (Q8) {
        LCU_GEMV_CASE(1, 4) LCU_GEMV_CASE(1, 2) LCU_GEMV_CASE(2, 2) LCU_GEMV_CASE(4, 1) LCU_GEMV_CASE(8, 1)
    } else if constexpr (NT == 1) {
        LCU_GEMV_CASE(1, 4) LCU_GEMV_CASE(2, 2) LCU_GEMV_CASE(4, 1) LCU_GEMV_CASE(8, 1)
    } else if constexpr (NT == 2) {
        LCU_GEMV_CASE(1, 4) LCU_GEMV_CASE(2, 2) LCU_GEMV_CASE(4, 1) LCU_GEMV_CASE(8, 1)
    } else {
        LCU_GEMV_CASE(1, 2) LCU_GEMV_CASE(2, 2) LCU_GEMV_CASE(4, 1) LCU_GEMV_CASE(8, 1)
    }
#undef LCU_GEMV_CASE
    set_error("gemv: no kernel for KI = %d, RP = %d, NT = %d", pl.KI, pl.RP, NT);
    return LCU_ERR_INVALID;
}

template <class T, bool Q8>
static int launch_t(const GemvArgs &a, cudaStream_t s, bool pdl, bool dry) {
    int nt = a.n_tok <= 1 ? 1 : (a.n_tok == 2 ? 2 : 4);
    GemvPlan pl = plan_for(a.in, Q8, nt);
    int n_pairs = a.out / 2;
    switch (nt) {
    case 1: return launch_nt<T, Q8, 1>(a, pl, n_pairs, s, pdl, dry);
    case 2: return launch_nt<T, Q8, 2>(a, pl, n_pairs, s, pdl, dry);
    default: return launch_nt<T, Q8, 4>(a, pl, n_pairs, s, pdl, dry);
    }
}

int gemv_max_tokens(int in) {
    for (int nt = 4; nt > 1; nt >>= 1)
        if ((size_t)nt * in * 2 + 8192 <= (size_t)227 * 1024) return nt;
    return 1;
}

int gemv_launch(const GemvArgs &a, int dt, cudaStream_t s, bool pdl, bool dry) {
    LCU_REQUIRE(a.n_tok >= 1 && a.n_tok <= 4, "gemv: n_tok = %d (1..4)", a.n_tok);
    LCU_REQUIRE(a.out > 0 && a.out % 2 == 0, "gemv: out = %d must be even", a.out);
    LCU_REQUIRE(a.in > 0 && a.in % (a.w_q8 ? 32 : 8) == 0, "gemv: in = %d must be a multiple of %d", a.in,
                a.w_q8 ? 32 : 8);
    LCU_REQUIRE(a.stride_x % 8 == 0, "gemv: x row stride %d must be a multiple of 8 elements", a.stride_x);
    LCU_REQUIRE(a.n_tok <= gemv_max_tokens(a.in), "gemv: in = %d too large for %d tokens at once", a.in, a.n_tok);
    if (a.epilogue == EPI_SWIGLU) LCU_REQUIRE(a.out == 2 * a.di, "gemv: swiglu needs out == 2*di");
    if (a.epilogue == EPI_ROPE_KV)
        LCU_REQUIRE(a.out == a.qd + 2 * a.kvd && a.dh % 2 == 0, "gemv: rope/kv epilogue shape mismatch");
    GemvArgs b = a;
    b.lean_norm = tuning().gemv_lean_norm;
    if (dt == LCU_F16) return b.w_q8 ? launch_t<__half, true>(b, s, pdl, dry) : launch_t<__half, false>(b, s, pdl, dry);
    if (dt == LCU_BF16) {
        LCU_REQUIRE(!b.w_q8, "gemv: Q8_0 weights are supported with f16 activations only");
        return launch_t<__nv_bfloat16, false>(b, s, pdl, dry);
    }
    set_error("gemv: activation dtype %d unsupported", dt);
    return LCU_ERR_INVALID;
}

}  // namespace lcu

namespace lcu {
// Sets the shared-memory attribute and caches the occupancy of every kernel variant a
// context with these shapes can launch, so that nothing of the kind happens inside a
// stream capture.
int gemv_warm(int in, int out, bool q8, int dt) {
    for (int nt = 1; nt <= gemv_max_tokens(in); nt *= 2) {
        GemvArgs a{};
        a.in = in; a.out = out; a.n_tok = nt; a.w_q8 = q8; a.stride_x = in; a.epilogue = EPI_STORE;
        // every prologue variant: none, RMSNorm with 16-bit and with f32 norm weights
        for (int v = 0; v < 3; ++v) {
            a.prologue = v == 0 ? PRO_NONE : PRO_RMSNORM;
            a.norm_f32 = v == 2;
            int rc = gemv_launch(a, dt, nullptr, false, true);
            if (rc) return rc;
        }
    }
    return LCU_OK;
}
}  // namespace lcu
