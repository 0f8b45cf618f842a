// Shared device/host helpers for the sm_100a decode kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/lcu.h"

namespace lcu {

// ------------------------------------------------------------------ errors
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define LCU_CHECK_CUDA(expr)                                   \
    do {                                                       \
        cudaError_t e__ = (expr);                              \
        if (e__ != cudaSuccess) return ::lcu::cuda_fail(e__, #expr); \
    } while (0)

#define LCU_REQUIRE(cond, ...)             \
    do {                                   \
        if (!(cond)) {                     \
            ::lcu::set_error(__VA_ARGS__); \
            return LCU_ERR_INVALID;        \
        }                                  \
    } while (0)

inline cudaStream_t as_stream(lcu_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Process-wide tuning values (lcu_set_tuning); the defaults are what the committed measurements use.
struct Tuning {
    int pdl_edges = -1;            // bit per layer edge launched as a programmatic dependent; -1: 28 (GEMV rounds) / 30 (batched)
    int gemv_lean_norm = 1;        // GEMV: one-token RMSNorm prologue from registers
    int rms_pdl = 1;               // batched rounds on the tcgen05 kernels: the stand-alone RMSNorm is a programmatic dependent
    int gemv_ctas_per_sm = 2;      // GEMV CTAs per SM (read at a shape's first launch)
    int q8_rows = 4;               // Q8_0 GEMV: row pairs per thread
    int tc = 1;                    // 0: keep the tcgen05 kernel out (mma.sync kernel for every batched round)
    int tc_block = 256;            // most tokens one tcgen05 launch takes (64, 128, 256): prefill rounds are cut into such blocks
    int tc_cluster = 1;            // cluster split-K form of the tcgen05 kernel: 0 never, 1 where it measured faster, 2 wherever it applies
    int p2p_scatter_ranks = 8;     // ranks from which the peer all-reduce takes the reduce-scatter + all-gather form
    long p2p_scatter_min = 131072; // ... for rounds of at least this many bytes
};
Tuning &tuning();
int sm_count();  // SMs of the current device (cached per device)

// ------------------------------------------------------------------ scalar types
template <class T> struct Act;  // activation dtype traits
template <> struct Act<__half> {
    using T2 = __half2;
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ float2 to_f2(uint32_t u) {
        return __half22float2(*reinterpret_cast<__half2 *>(&u));
    }
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
};
template <> struct Act<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float2 to_f2(uint32_t u) {
        // bf16 -> f32 is a 16-bit shift
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    }
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
};

// round-trip through the activation dtype: the reference materialises every operator
// output in that type, so fused kernels round at the same places
template <class T> __device__ __forceinline__ float round_act(float v) { return Act<T>::to_f(Act<T>::from_f(v)); }

// acc += a.lo * b.lo; acc += a.hi * b.hi for two packed 16-bit floats per operand, with the
// sm_100 mixed-precision FMA (f16/bf16 inputs, f32 accumulate, one rounding): the same value
// as converting both inputs to f32 and calling fmaf, without the two conversions.
template <class T> __device__ __forceinline__ float fma2_mixed(uint32_t a, uint32_t b, float acc);
template <> __device__ __forceinline__ float fma2_mixed<__half>(uint32_t a, uint32_t b, float acc) {
    asm("{\n .reg .b16 al, ah, bl, bh;\n mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n"
        " fma.rn.f32.f16 %0, al, bl, %0;\n fma.rn.f32.f16 %0, ah, bh, %0;\n}"
        : "+f"(acc) : "r"(a), "r"(b));
    return acc;
}
template <> __device__ __forceinline__ float fma2_mixed<__nv_bfloat16>(uint32_t a, uint32_t b, float acc) {
    asm("{\n .reg .b16 al, ah, bl, bh;\n mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n"
        " fma.rn.f32.bf16 %0, al, bl, %0;\n fma.rn.f32.bf16 %0, ah, bh, %0;\n}"
        : "+f"(acc) : "r"(a), "r"(b));
    return acc;
}
// dot product of 8 + 8 packed values accumulated in element order 0..7
template <class T> __device__ __forceinline__ float dot8_mixed(const uint4 &w, const uint4 &x, float acc) {
    acc = fma2_mixed<T>(w.x, x.x, acc);
    acc = fma2_mixed<T>(w.y, x.y, acc);
    acc = fma2_mixed<T>(w.z, x.z, acc);
    acc = fma2_mixed<T>(w.w, x.w, acc);
    return acc;
}

// int8 x 4 -> two f16x2 without I2F: bytes xor 0x80 land in the mantissa of 1024.0 (0x64xx = 1024 + byte),
// minus 1152 gives the signed value exactly.
__device__ __forceinline__ void q8x4_to_h2(uint32_t q, uint32_t &h01, uint32_t &h23) {
    const uint32_t u = q ^ 0x80808080u;
    const __half2 bias = __halves2half2(__ushort_as_half((unsigned short)0x6480), __ushort_as_half((unsigned short)0x6480));
    uint32_t ua = __byte_perm(u, 0x64646464u, 0x4140), ub = __byte_perm(u, 0x64646464u, 0x4342);
    __half2 a = __hsub2(*reinterpret_cast<__half2 *>(&ua), bias);
    __half2 b = __hsub2(*reinterpret_cast<__half2 *>(&ub), bias);
    h01 = *reinterpret_cast<uint32_t *>(&a);
    h23 = *reinterpret_cast<uint32_t *>(&b);
}

// ------------------------------------------------------------------ memory access
// 128-bit streaming load for data read exactly once per step (weights): no L1 allocation,
// read-only path.
__device__ __forceinline__ uint4 ld_stream_128(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// 256-bit streaming load (sm_100): 32 bytes per lane, so the 4 lanes of a quad cover one
// 128-byte line; evict-first in L2 because weights are used once per step.
struct u32x8 {
    uint4 lo, hi;
};
__device__ __forceinline__ u32x8 ld_stream_256(const void *p) {
    u32x8 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x), "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_64(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialisation
// attribute may start while its predecessor drains; everything it does before
// grid_dep_wait() must touch only memory no earlier kernel of the step writes (weights).
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ------------------------------------------------------------------ launch helper
// Launches with (optionally) the programmatic stream serialisation attribute.
template <class... KArgs, class... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl,
                          Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// KV page pool geometry: page p, layer l, kv in {0,1}, head h, slot t -> element offset.
// A page holds `page_tokens` tokens of every layer: [layer][k|v][kv head][token][dh].
struct KvGeom {
    int n_layers, nkvh, dh, page_tokens, page_shift;
    size_t page_elems;  // n_layers * 2 * nkvh * page_tokens * dh
    __host__ __device__ __forceinline__ size_t block_off(int page, int layer, int kv, int head) const {
        return (size_t)page * page_elems + ((size_t)(layer * 2 + kv) * nkvh + head) * ((size_t)page_tokens * dh);
    }
};

#ifdef __CUDACC__
// D += A(16x16, row) x B(16x8, col) on the legacy tensor-core path, f32 accumulation
template <class T> __device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                            uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__half>(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                                    uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#endif

}  // namespace lcu
