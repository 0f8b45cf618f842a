// Stand-alone operators of the decode path: embedding gather, device-side token
// feedback, RMSNorm, RoPE, SwiGLU, add.  Each is the sm_100a counterpart of one NVRTC
// kernel of llama.cu/src/op/*.cuh with the same arithmetic and rounding points; the
// fused step uses them only where a fusion into a GEMV/GEMM is not available.
#include "common.cuh"

namespace lcu {

// ------------------------------------------------------------------ embedding
// op/embedding.cuh:1-9 moves rows as opaque byte units; here one block per row, 128-bit
// units when the row allows it.
template <class U>
__global__ void embedding_kernel(U *__restrict__ out, const U *__restrict__ table,
                                 const uint32_t *__restrict__ index, int units) {
    // a programmatic dependent (the first projection of the step) may start now: it streams its first weights while
    // this copy runs and waits for it before touching the activations
    grid_dep_launch();
    grid_dep_wait();
    size_t row = index[blockIdx.x];
    const U *src = table + row * units;
    U *dst = out + (size_t)blockIdx.x * units;
    for (int i = threadIdx.x; i < units; i += blockDim.x) dst[i] = src[i];
}

int op_embedding(void *out, const void *table, const uint32_t *index, int n, size_t row_bytes, cudaStream_t s,
                 bool pdl) {
    if (n <= 0) return LCU_OK;
    if (row_bytes % 16 == 0) {
        int units = (int)(row_bytes / 16);
        int block = units < 256 ? ((units + 31) / 32) * 32 : 256;
        LCU_CHECK_CUDA(launch_kernel(embedding_kernel<uint4>, dim3(n), dim3(block), 0, s, pdl, (uint4 *)out,
                                     (const uint4 *)table, index, units));
    } else {
        LCU_REQUIRE(row_bytes % 2 == 0, "embedding: row of %zu bytes is not a multiple of 2", row_bytes);
        int units = (int)(row_bytes / 2);
        LCU_CHECK_CUDA(launch_kernel(embedding_kernel<uint16_t>, dim3(n), dim3(256), 0, s, pdl, (uint16_t *)out,
                                     (const uint16_t *)table, index, units));
    }
    return LCU_OK;
}

// op/fast_embedding.cuh:7-15: tokens[map[i].v] = kv_pairs[map[i].k].k
__global__ void fast_embedding_kernel(uint32_t *__restrict__ tokens, const lcu_kv_pair *__restrict__ pairs,
                                      const uint2 *__restrict__ map, int n) {
    grid_dep_launch();
    grid_dep_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        uint2 m = map[i];
        tokens[m.y] = pairs[m.x].idx;
    }
}

int op_fast_embedding(uint32_t *tokens, const lcu_kv_pair *pairs, const uint32_t *map, int n, cudaStream_t s,
                      bool pdl) {
    if (n <= 0) return LCU_OK;
    LCU_CHECK_CUDA(launch_kernel(fast_embedding_kernel, dim3((n + 255) / 256), dim3(256), 0, s, pdl, tokens, pairs,
                                 (const uint2 *)map, n));
    return LCU_OK;
}

// ------------------------------------------------------------------ rms_norm
// op/rms_norm.cuh:6-81: f32 sum of squares over the row, rms = rsqrtf(acc/d + eps),
// y = Ta(rms * x * w).  One block per row; 128-bit loads when d and the strides allow.
template <class T, class Tw>
__global__ void rms_norm_kernel(T *__restrict__ y, int sy, const T *__restrict__ x, int sx,
                                const Tw *__restrict__ w, float eps, int d) {
    grid_dep_launch();  // a GEMM launched with the programmatic attribute may start streaming its weights now
    const T *xr = x + (size_t)blockIdx.x * sx;
    T *yr = y + (size_t)blockIdx.x * sy;
    // 128-bit path when the row and both strides allow it; the row stays in registers between passes
    const bool vec = (d % 8 == 0) && (sx % 8 == 0) && (sy % 8 == 0) && d <= 8 * 4 * (int)blockDim.x &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w)) % 16 == 0);
    // 16-bit norm weights are constants: they are requested before the dependency wait (and, in any case, together with
    // the row instead of after the reduction: one round trip to L2 less on the critical path)
    uint4 wk[4];
    if constexpr (sizeof(Tw) == 2) {
        if (vec) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int i = threadIdx.x + j * blockDim.x;
                wk[j] = i < d / 8 ? __ldg(reinterpret_cast<const uint4 *>(w) + i) : make_uint4(0, 0, 0, 0);
            }
        }
    }
    grid_dep_wait();
    uint4 keep[4];
    float acc = 0.f;
    if (vec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int i = threadIdx.x + j * blockDim.x;
            if (i < d / 8) {
                keep[j] = reinterpret_cast<const uint4 *>(xr)[i];
                const uint32_t u[4] = {keep[j].x, keep[j].y, keep[j].z, keep[j].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float2 f = Act<T>::to_f2(u[k]);
                    acc += f.x * f.x;
                    acc += f.y * f.y;
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float v = Act<T>::to_f(xr[i]);
            acc += v * v;
        }
    }
    __shared__ float part[32];
    __shared__ float rms_s;
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) rms_s = rsqrtf(v / (float)d + eps);
    }
    __syncthreads();
    float rms = rms_s;
    if (vec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int i = threadIdx.x + j * blockDim.x;
            if (i < d / 8) {
                float wf[8];
                if constexpr (sizeof(Tw) == 4) {
                    float4 w0 = reinterpret_cast<const float4 *>(w)[2 * i], w1 = reinterpret_cast<const float4 *>(w)[2 * i + 1];
                    wf[0] = w0.x; wf[1] = w0.y; wf[2] = w0.z; wf[3] = w0.w; wf[4] = w1.x; wf[5] = w1.y; wf[6] = w1.z; wf[7] = w1.w;
                } else {
                    const uint4 wv = wk[j];
                    float2 a = Act<T>::to_f2(wv.x), b = Act<T>::to_f2(wv.y), c = Act<T>::to_f2(wv.z), e = Act<T>::to_f2(wv.w);
                    wf[0] = a.x; wf[1] = a.y; wf[2] = b.x; wf[3] = b.y; wf[4] = c.x; wf[5] = c.y; wf[6] = e.x; wf[7] = e.y;
                }
                float2 f0 = Act<T>::to_f2(keep[j].x), f1 = Act<T>::to_f2(keep[j].y), f2 = Act<T>::to_f2(keep[j].z),
                       f3 = Act<T>::to_f2(keep[j].w);
                uint4 o;
                o.x = Act<T>::pack(rms * f0.x * wf[0], rms * f0.y * wf[1]);
                o.y = Act<T>::pack(rms * f1.x * wf[2], rms * f1.y * wf[3]);
                o.z = Act<T>::pack(rms * f2.x * wf[4], rms * f2.y * wf[5]);
                o.w = Act<T>::pack(rms * f3.x * wf[6], rms * f3.y * wf[7]);
                reinterpret_cast<uint4 *>(yr)[i] = o;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = Act<T>::to_f(xr[i]);
        float ww;
        if constexpr (sizeof(Tw) == 4) ww = w[i];
        else ww = Act<T>::to_f(w[i]);
        yr[i] = Act<T>::from_f(rms * v * ww);
    }
}

template <class T>
static int rms_norm_t(void *y, int sy, const void *x, int sx, const void *w, int w_dt, float eps, int n, int d,
                      cudaStream_t s, bool pdl) {
    int block = d >= 1024 ? 256 : (d >= 256 ? 128 : 32);
    if (w_dt == LCU_F32)
        LCU_CHECK_CUDA(launch_kernel(rms_norm_kernel<T, float>, dim3(n), dim3(block), 0, s, pdl, (T *)y, sy,
                                     (const T *)x, sx, (const float *)w, eps, d));
    else
        LCU_CHECK_CUDA(launch_kernel(rms_norm_kernel<T, T>, dim3(n), dim3(block), 0, s, pdl, (T *)y, sy,
                                     (const T *)x, sx, (const T *)w, eps, d));
    return LCU_OK;
}

int op_rms_norm(void *y, int sy, const void *x, int sx, const void *w, int w_dt, float eps, int n, int d, int dt,
                cudaStream_t s, bool pdl) {
    if (n <= 0) return LCU_OK;
    LCU_REQUIRE(dt == LCU_F16 || dt == LCU_BF16, "rms_norm: activation dtype %d unsupported", dt);
    LCU_REQUIRE(w_dt == dt || w_dt == LCU_F32, "rms_norm: weight dtype %d must be the activation dtype or f32", w_dt);
    LCU_REQUIRE(d > 0, "rms_norm: d = %d", d);
    return dt == LCU_F16 ? rms_norm_t<__half>(y, sy, x, sx, w, w_dt, eps, n, d, s, pdl)
                         : rms_norm_t<__nv_bfloat16>(y, sy, x, sx, w, w_dt, eps, n, d, s, pdl);
}

// ------------------------------------------------------------------ rope
// op/rope.cuh:1-35: (a,b) = x[2i], x[2i+1]; y[2i] = a*cos - b*sin; y[2i+1] = a*sin + b*cos
// with f32 tables indexed [pos, i].  One thread per pair, 32-bit loads/stores.
template <class T>
__global__ void rope_kernel(T *__restrict__ y, int sty, int shy, const T *__restrict__ x, int stx, int shx,
                            const uint32_t *__restrict__ pos, const float *__restrict__ sin_t,
                            const float *__restrict__ cos_t, int nh, int half_dh) {
    grid_dep_wait();
    int t = blockIdx.y;
    int idx = blockIdx.x * blockDim.x + threadIdx.x;  // over nh * half_dh
    if (idx >= nh * half_dh) return;
    int h = idx / half_dh, i = idx - h * half_dh;
    uint32_t p = pos[t];
    float sn = sin_t[(size_t)p * half_dh + i], cs = cos_t[(size_t)p * half_dh + i];
    const T *xp = x + (size_t)t * stx + (size_t)h * shx + 2 * i;
    T *yp = y + (size_t)t * sty + (size_t)h * shy + 2 * i;
    float a = Act<T>::to_f(xp[0]), b = Act<T>::to_f(xp[1]);
    yp[0] = Act<T>::from_f(a * cs - b * sn);
    yp[1] = Act<T>::from_f(a * sn + b * cs);
}

int op_rope(void *y, int sty, int shy, const void *x, int stx, int shx, const uint32_t *pos, const float *sin_t,
            const float *cos_t, int n, int nh, int dh, int dt, cudaStream_t s, bool pdl) {
    if (n <= 0) return LCU_OK;
    LCU_REQUIRE(dt == LCU_F16 || dt == LCU_BF16, "rope: activation dtype %d unsupported", dt);
    LCU_REQUIRE(dh > 0 && dh % 2 == 0 && nh > 0, "rope: nh = %d, dh = %d", nh, dh);
    int total = nh * (dh / 2);
    dim3 grid((total + 255) / 256, n), block(256);
    if (dt == LCU_F16)
        LCU_CHECK_CUDA(launch_kernel(rope_kernel<__half>, grid, block, 0, s, pdl, (__half *)y, sty, shy,
                                     (const __half *)x, stx, shx, pos, sin_t, cos_t, nh, dh / 2));
    else
        LCU_CHECK_CUDA(launch_kernel(rope_kernel<__nv_bfloat16>, grid, block, 0, s, pdl, (__nv_bfloat16 *)y, sty,
                                     shy, (const __nv_bfloat16 *)x, stx, shx, pos, sin_t, cos_t, nh, dh / 2));
    return LCU_OK;
}

// ------------------------------------------------------------------ swiglu
// op/swiglu.cuh:1-20: out = gate * sigmoid(gate) * up, sigmoid = fdividef(1, 1 + expf(-x))
__device__ __forceinline__ float swiglu_f(float gate, float up) {
    return gate * __fdividef(1.f, 1.f + expf(-gate)) * up;
}

template <class T>
__global__ void swiglu_kernel(T *__restrict__ out, int so, const T *__restrict__ gate, int sg,
                              const T *__restrict__ up, int su, int di) {
    grid_dep_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= di) return;
    int t = blockIdx.y;
    float g = Act<T>::to_f(gate[(size_t)t * sg + i]), u = Act<T>::to_f(up[(size_t)t * su + i]);
    out[(size_t)t * so + i] = Act<T>::from_f(swiglu_f(g, u));
}

int op_swiglu(void *out, int so, const void *gate, int sg, const void *up, int su, int n, int di, int dt,
              cudaStream_t s, bool pdl) {
    if (n <= 0) return LCU_OK;
    LCU_REQUIRE(dt == LCU_F16 || dt == LCU_BF16, "swiglu: activation dtype %d unsupported", dt);
    dim3 grid((di + 255) / 256, n), block(256);
    if (dt == LCU_F16)
        LCU_CHECK_CUDA(launch_kernel(swiglu_kernel<__half>, grid, block, 0, s, pdl, (__half *)out, so,
                                     (const __half *)gate, sg, (const __half *)up, su, di));
    else
        LCU_CHECK_CUDA(launch_kernel(swiglu_kernel<__nv_bfloat16>, grid, block, 0, s, pdl, (__nv_bfloat16 *)out, so,
                                     (const __nv_bfloat16 *)gate, sg, (const __nv_bfloat16 *)up, su, di));
    return LCU_OK;
}

// ------------------------------------------------------------------ add
// op/add.cuh:1-18: y = k == 0 ? b : k*x + b  (bias path of qwen2-style models)
template <class T>
__global__ void add_kernel(T *__restrict__ y, int sny, int sdy, const T *__restrict__ x, int snx, int sdx,
                           const T *__restrict__ b, int snb, int sdb, float k, int d) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d) return;
    int t = blockIdx.y;
    float bv = Act<T>::to_f(b[(size_t)t * snb + (size_t)i * sdb]);
    float r = k == 0.f ? bv : k * Act<T>::to_f(x[(size_t)t * snx + (size_t)i * sdx]) + bv;
    y[(size_t)t * sny + (size_t)i * sdy] = Act<T>::from_f(r);
}

int op_add(void *y, int sny, int sdy, const void *x, int snx, int sdx, const void *b, int snb, int sdb, float k,
           int n, int d, int dt, cudaStream_t s) {
    if (n <= 0) return LCU_OK;
    LCU_REQUIRE(dt == LCU_F16 || dt == LCU_BF16, "add: activation dtype %d unsupported", dt);
    dim3 grid((d + 255) / 256, n), block(256);
    if (dt == LCU_F16)
        add_kernel<__half><<<grid, block, 0, s>>>((__half *)y, sny, sdy, (const __half *)x, snx, sdx,
                                                  (const __half *)b, snb, sdb, k, d);
    else
        add_kernel<__nv_bfloat16><<<grid, block, 0, s>>>((__nv_bfloat16 *)y, sny, sdy, (const __nv_bfloat16 *)x, snx,
                                                         sdx, (const __nv_bfloat16 *)b, snb, sdb, k, d);
    LCU_CHECK_CUDA(cudaGetLastError());
    return LCU_OK;
}

}  // namespace lcu
