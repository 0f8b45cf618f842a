// Second witness for the parity tests — TEST INFRASTRUCTURE, not product code.
//
// Wraps the reference's own device code, compiled from the reference sources where they
// lie (the directory is given with -I at build time, nothing is copied), behind plain
// C entry points so that the GPU tests can run the reference's kernels and the CUDA
// library's kernels on the same inputs.  The `extern "C" __global__` wrappers and the
// launch geometry restate what the reference's Rust wrappers generate at run time for
// NVRTC: llama.cu/src/op/rms_norm.rs:62-104, rope.rs:59-137, swiglu.rs:66-95,
// embedding.rs:30-69, fast_embedding.rs:28-63, add.rs:57-92.
// The sampler (random_sample/sample.cu) is compiled as its own object and linked in.
#include <cub/block/block_load.cuh>
#include <cub/block/block_reduce.cuh>
#include <cub/block/block_store.cuh>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace ref_rms {
#include <rms_norm.cuh>
}
namespace ref_rope {
#include <rope.cuh>
}
namespace ref_swiglu {
#include <swiglu.cuh>
}
namespace ref_embd {
#include <embedding.cuh>
}
namespace ref_fast {
#include <fast_embedding.cuh>
}

// ---- rms_norm: one instantiation per hidden size the configs use (rms_norm.rs:62-90)
template <unsigned D, class Tw>
__global__ void k_rms_pad(half *y, int sy, const half *x, int sx, const Tw *w, float eps) {
    ref_rms::padding<D>(y, sy, x, sx, w, eps);
}
template <unsigned ITEMS, class Tw>
__global__ void k_rms_fold(half *y, int sy, const half *x, int sx, const Tw *w, float eps, unsigned d) {
    ref_rms::folding<1024, ITEMS>(y, sy, x, sx, w, eps, d);
}

template <class Tw>
static int launch_rms(half *y, int sy, const half *x, int sx, const Tw *w, float eps, int n, int d,
                      cudaStream_t s) {
    if (d <= 1024) {
        switch (d) {
        case 64: k_rms_pad<64, Tw><<<n, d, 0, s>>>(y, sy, x, sx, w, eps); break;
        case 128: k_rms_pad<128, Tw><<<n, d, 0, s>>>(y, sy, x, sx, w, eps); break;
        case 256: k_rms_pad<256, Tw><<<n, d, 0, s>>>(y, sy, x, sx, w, eps); break;
        case 512: k_rms_pad<512, Tw><<<n, d, 0, s>>>(y, sy, x, sx, w, eps); break;
        case 1024: k_rms_pad<1024, Tw><<<n, d, 0, s>>>(y, sy, x, sx, w, eps); break;
        default: return -1;
        }
    } else {
        if (d % 32) return -1;
        int items = (d / 32 + 31) / 32;  // to_divid.div_ceil(num_warps_block), rms_norm.rs:82-84
        switch (items) {
        case 2: k_rms_fold<2, Tw><<<n, 1024, 0, s>>>(y, sy, x, sx, w, eps, d); break;
        case 4: k_rms_fold<4, Tw><<<n, 1024, 0, s>>>(y, sy, x, sx, w, eps, d); break;
        case 8: k_rms_fold<8, Tw><<<n, 1024, 0, s>>>(y, sy, x, sx, w, eps, d); break;
        default: return -1;
        }
    }
    return (int)cudaGetLastError();
}

extern "C" int ref_rms_norm_f16(void *y, int sy, const void *x, int sx, const void *w, int w_is_f32,
                                float eps, int n, int d, cudaStream_t s) {
    return w_is_f32 ? launch_rms((half *)y, sy, (const half *)x, sx, (const float *)w, eps, n, d, s)
                    : launch_rms((half *)y, sy, (const half *)x, sx, (const half *)w, eps, n, d, s);
}

// ---- rope (rope.rs:86-107,121-137): grid (y=n, x=nh/nh_l), block (y=nh_l, x=dh/2)
__global__ void k_rope(half *y, int sty, int shy, const half *x, int stx, int shx,
                       const unsigned *pos, const float *sin_t, const float *cos_t) {
    ref_rope::padding<unsigned, half>(y, sty, shy, x, stx, shx, pos, sin_t, cos_t);
}
extern "C" int ref_rope_f16(void *y, int sty, int shy, const void *x, int stx, int shx, const unsigned *pos,
                            const float *sin_t, const float *cos_t, int n, int nh, int dh, cudaStream_t s) {
    int half_dh = dh / 2, max_l = 1024 / half_dh;
    if (max_l > nh) max_l = nh;
    int nh_l = 1;
    for (int c = max_l; c >= 1; --c)
        if (nh % c == 0) { nh_l = c; break; }
    dim3 grid(nh / nh_l, n), block(half_dh, nh_l);
    k_rope<<<grid, block, 0, s>>>((half *)y, sty, shy, (const half *)x, stx, shx, pos, sin_t, cos_t);
    return (int)cudaGetLastError();
}

// ---- swiglu (swiglu.rs:66-74): grid (y=n, x=di/blk), blk = gcd(1024, di)
__global__ void k_swiglu(half *out, int so, const half *gate, int sg, const half *up, int su) {
    ref_swiglu::kernel(out, so, gate, sg, up, su);
}
static int gcd_i(int a, int b) { while (b) { int r = a % b; a = b; b = r; } return a; }
extern "C" int ref_swiglu_f16(void *out, int so, const void *gate, int sg, const void *up, int su,
                              int n, int di, cudaStream_t s) {
    int blk = gcd_i(1024, di);
    dim3 grid(di / blk, n);
    k_swiglu<<<grid, blk, 0, s>>>((half *)out, so, (const half *)gate, sg, (const half *)up, su);
    return (int)cudaGetLastError();
}

// ---- embedding (embedding.rs:30-51): rows moved as 32-, 16-, 8-... byte units
template <class U>
__global__ void k_embd(U *out, const U *table, const unsigned *index) { ref_embd::kernel(out, table, index); }
extern "C" int ref_embedding(void *out, const void *table, const unsigned *index, int n, int row_bytes,
                             cudaStream_t s) {
    if (row_bytes % 32 == 0)
        k_embd<<<n, row_bytes / 32, 0, s>>>((double4 *)out, (const double4 *)table, index);
    else if (row_bytes % 16 == 0)
        k_embd<<<n, row_bytes / 16, 0, s>>>((float4 *)out, (const float4 *)table, index);
    else if (row_bytes % 2 == 0)
        k_embd<<<n, row_bytes / 2, 0, s>>>((short *)out, (const short *)table, index);
    else
        return -1;
    return (int)cudaGetLastError();
}

// ---- fast_embedding (fast_embedding.rs:28-44): one block of map.len() threads
__global__ void k_fast(unsigned *tokens, const ref_fast::KV<half> *pairs, const ref_fast::KV<unsigned> *map) {
    ref_fast::kernel(tokens, pairs, map);
}
extern "C" int ref_fast_embedding(unsigned *tokens, const void *kv_pairs, const void *map, int n_map,
                                  cudaStream_t s) {
    if (n_map <= 0) return 0;
    k_fast<<<1, n_map, 0, s>>>(tokens, (const ref_fast::KV<half> *)kv_pairs, (const ref_fast::KV<unsigned> *)map);
    return (int)cudaGetLastError();
}
