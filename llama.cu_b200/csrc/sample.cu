// Arg-max and random sampling over rows of logits — the sm_100a counterpart of
// librandom_sample.so (llama.cu/src/op/random_sample/sample.cuh).
//
// Arg-max (sample.cuh:13-25, cub::DeviceReduce::ArgMax): largest value, lowest index
// among equals.  The reference calls it once per output row from a host loop
// (exec/output_head.rs:104-113); here two launches cover every row: per-chunk partial
// (value, index) pairs by warp shuffles, then one block per row folds the partials.
//
// Sampling (sample.cuh:156-209): the reference radix-sorts all logits descending, turns
// them into weights w0 = 1, wi = exp((xi - x0)/T), prefix-sums them and returns the
// first entry whose prefix reaches random * min(top_p * total, prefix[top_k - 1]).
// Logits are 16-bit, so a full sort is unnecessary: one block per row builds a 65536-bin
// histogram of the order-preserving key, scans the bins from the largest key down
// (weights and prefixes in f64 — the reference keeps them in f16), finds the bin where
// the threshold falls and the rank inside it, and picks the element of that rank by
// ascending index, which is exactly the order a stable descending sort produces.
#include "sample.cuh"

#include <mutex>

namespace lcu {

template <class T> __device__ __forceinline__ float bits_to_f(uint16_t b);
template <> __device__ __forceinline__ float bits_to_f<__half>(uint16_t b) { return __half2float(__ushort_as_half(b)); }
template <> __device__ __forceinline__ float bits_to_f<__nv_bfloat16>(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

struct ArgPair {
    float v;
    uint32_t i;
    uint16_t bits;
};
__device__ __forceinline__ bool arg_better(float v, uint32_t i, float bv, uint32_t bi) {
    return v > bv || (v == bv && i < bi);
}

template <class T>
__global__ void __launch_bounds__(256) argmax_partial_kernel(const uint16_t *__restrict__ logits, size_t n, int nblk,
                                                             float *__restrict__ pv, uint32_t *__restrict__ pi) {
    grid_dep_launch();
    grid_dep_wait();
    const int row = blockIdx.y, blk = blockIdx.x;
    const uint16_t *x = logits + (size_t)row * n;
    size_t begin = (size_t)blk * ARGMAX_CHUNK, end = begin + ARGMAX_CHUNK;
    if (end > n) end = n;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    if (((reinterpret_cast<uintptr_t>(x) | (n * 2)) & 15) == 0) {
        // rows that start on 16 bytes: eight values per load (the order of the visits does not matter, ties go to the
        // lower index through arg_better)
        for (size_t i = begin + 8 * (size_t)threadIdx.x; i < end; i += 8 * (size_t)blockDim.x) {
            const uint4 q = *reinterpret_cast<const uint4 *>(x + i);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float v = bits_to_f<T>((uint16_t)(w[k >> 1] >> ((k & 1) * 16)));
                if (arg_better(v, (uint32_t)(i + k), bv, bi) || bi == 0xffffffffu) { bv = v; bi = (uint32_t)(i + k); }
            }
        }
    } else {
        for (size_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
            float v = bits_to_f<T>(x[i]);
            if (arg_better(v, (uint32_t)i, bv, bi) || bi == 0xffffffffu) { bv = v; bi = (uint32_t)i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0xffffffffu && (bi == 0xffffffffu || arg_better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (si[w] != 0xffffffffu && (bi == 0xffffffffu || arg_better(sv[w], si[w], bv, bi))) { bv = sv[w]; bi = si[w]; }
        pv[(size_t)row * nblk + blk] = bv;
        pi[(size_t)row * nblk + blk] = bi;
    }
}

template <class T>
__global__ void __launch_bounds__(256) argmax_final_kernel(const uint16_t *__restrict__ logits, size_t n, int nblk,
                                                           const float *__restrict__ pv, const uint32_t *__restrict__ pi,
                                                           const lcu_sample_args *__restrict__ args,
                                                           lcu_kv_pair *__restrict__ out, lcu_kv_pair *__restrict__ out_copy) {
    grid_dep_launch();
    grid_dep_wait();
    const int row = blockIdx.x;
    if (args) {  // rows that sample are written by the sampling kernel
        lcu_sample_args a = args[row];
        if (!(a.temperature == 0.f || a.top_k == 1)) return;
    }
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (int b = threadIdx.x; b < nblk; b += blockDim.x) {
        float v = pv[(size_t)row * nblk + b];
        uint32_t i = pi[(size_t)row * nblk + b];
        if (i != 0xffffffffu && (bi == 0xffffffffu || arg_better(v, i, bv, bi))) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0xffffffffu && (bi == 0xffffffffu || arg_better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (si[w] != 0xffffffffu && (bi == 0xffffffffu || arg_better(sv[w], si[w], bv, bi))) { bv = sv[w]; bi = si[w]; }
        lcu_kv_pair r;
        r.idx = bi;
        r.val = logits[(size_t)row * n + bi];
        r.pad = 0;
        out[row] = r;
        if (out_copy) out_copy[row] = r;
    }
}

// order-preserving 16-bit key of an f16 / bf16 bit pattern (larger value -> larger key)
__device__ __forceinline__ uint32_t key_of(uint16_t b) { return (b & 0x8000u) ? (uint32_t)(~b & 0xffffu) : (uint32_t)(b | 0x8000u); }
__device__ __forceinline__ uint16_t bits_of(uint32_t k) { return (k & 0x8000u) ? (uint16_t)(k ^ 0x8000u) : (uint16_t)(~k & 0xffffu); }

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_BINS = 65536;
constexpr int BINS_PER_THREAD = SAMPLE_BINS / SAMPLE_THREADS;

template <class T>
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_row_kernel(const uint16_t *__restrict__ logits, size_t n,
                                                                    const lcu_sample_args *__restrict__ args,
                                                                    const float *__restrict__ randoms,
                                                                    uint32_t *__restrict__ hist_all,
                                                                    lcu_kv_pair *__restrict__ out,
                                                                    lcu_kv_pair *__restrict__ out_copy) {
    grid_dep_launch();
    grid_dep_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const lcu_sample_args sa = args[row];
    if (sa.temperature == 0.f || sa.top_k == 1) return;  // arg-max rows are handled elsewhere
    const uint16_t *x = logits + (size_t)row * n;
    uint32_t *hist = hist_all + (size_t)row * SAMPLE_BINS;

    __shared__ double s_w[SAMPLE_THREADS];
    __shared__ unsigned long long s_c[SAMPLE_THREADS];
    __shared__ int s_max;
    __shared__ double s_total, s_cumk;
    __shared__ int s_bin, s_rank, s_found;
    __shared__ uint32_t s_cnt[32];

    for (int b = tid; b < SAMPLE_BINS; b += SAMPLE_THREADS) hist[b] = 0;
    if (tid == 0) { s_max = -1; s_bin = -1; s_rank = 1; s_found = 0; s_cumk = -1.0; }
    __syncthreads();
    for (size_t i = tid; i < n; i += SAMPLE_THREADS) atomicAdd(&hist[key_of(x[i])], 1u);
    __syncthreads();

    // thread `tid` owns bins hi, hi-1, ..., hi-63 (descending keys); thread 0 holds the largest keys
    const int hi = SAMPLE_BINS - 1 - tid * BINS_PER_THREAD;
    int mymax = -1;
    for (int j = 0; j < BINS_PER_THREAD; ++j)
        if (hist[hi - j]) { mymax = hi - j; break; }
    if (mymax >= 0) atomicMax(&s_max, mymax);
    __syncthreads();
    const int maxbin = s_max;
    const float xmax = bits_to_f<T>(bits_of((uint32_t)maxbin));
    auto weight = [&](int b) -> double {
        if (b == maxbin) return 1.0;
        return (double)expf((bits_to_f<T>(bits_of((uint32_t)b)) - xmax) / sa.temperature);
    };

    double wsum = 0.0;
    unsigned long long csum = 0;
    for (int j = 0; j < BINS_PER_THREAD; ++j) {
        uint32_t c = hist[hi - j];
        if (c) { wsum += (double)c * weight(hi - j); csum += c; }
    }
    s_w[tid] = wsum;
    s_c[tid] = csum;
    __syncthreads();
    // exclusive prefix over threads (thread order == descending key order)
    if (tid == 0) {
        double aw = 0.0;
        unsigned long long ac = 0;
        for (int i = 0; i < SAMPLE_THREADS; ++i) {
            double w = s_w[i];
            unsigned long long c = s_c[i];
            s_w[i] = aw;
            s_c[i] = ac;
            aw += w;
            ac += c;
        }
        s_total = aw;
    }
    __syncthreads();
    const double total = s_total, w_before = s_w[tid];
    const unsigned long long c_before = s_c[tid];
    unsigned long long topk = sa.top_k > n ? n : sa.top_k;

    // prefix[top_k - 1]
    if (csum && c_before < topk && topk <= c_before + csum) {
        double aw = w_before;
        unsigned long long ac = c_before;
        for (int j = 0; j < BINS_PER_THREAD; ++j) {
            uint32_t c = hist[hi - j];
            if (!c) continue;
            double w = weight(hi - j);
            if (ac + c >= topk) { s_cumk = aw + (double)(topk - ac) * w; break; }
            aw += (double)c * w;
            ac += c;
        }
    }
    __syncthreads();
    double lim = (double)sa.top_p * total;
    if (s_cumk >= 0.0 && s_cumk < lim) lim = s_cumk;
    const double thr = (double)randoms[row] * lim;

    // first entry (descending order) whose inclusive prefix reaches thr: the owner is the
    // thread whose bins contain the crossing (or the first non-empty thread when thr <= 0)
    if (csum && w_before + wsum >= thr && (w_before < thr || c_before == 0)) {
        double aw = w_before;
        int last_bin = -1;
        uint32_t last_c = 1;
        bool found = false;
        for (int j = 0; j < BINS_PER_THREAD && !found; ++j) {
            uint32_t c = hist[hi - j];
            if (!c) continue;
            double w = weight(hi - j);
            double incl = aw + (double)c * w;
            last_bin = hi - j;
            last_c = c;
            if (incl >= thr) {
                long long r = 1;
                if (thr > aw) {
                    r = (long long)ceil((thr - aw) / w);
                    if (r < 1) r = 1;
                    if (r > (long long)c) r = c;
                }
                s_bin = hi - j;
                s_rank = (int)r;
                found = true;
            }
            aw = incl;
        }
        if (!found) {  // the stepwise prefix fell short of the thread total by rounding
            s_bin = last_bin;
            s_rank = (int)last_c;
        }
    }
    __syncthreads();
    int bin = s_bin, rank = s_rank;
    if (bin < 0) {  // threshold beyond the total by rounding: take the very last entry
        __shared__ int s_min;
        if (tid == 0) s_min = SAMPLE_BINS;
        __syncthreads();
        int mymin = SAMPLE_BINS;
        for (int j = BINS_PER_THREAD - 1; j >= 0; --j)
            if (hist[hi - j]) { mymin = hi - j; break; }
        if (mymin < SAMPLE_BINS) atomicMin(&s_min, mymin);
        __syncthreads();
        bin = s_min;
        rank = (int)hist[bin];
    }

    // the rank-th (1-based) lowest index whose key is `bin`
    const int lane = tid & 31, warp = tid >> 5;
    uint32_t seen = 0;
    for (size_t base = 0; base < n; base += SAMPLE_THREADS) {
        size_t i = base + tid;
        bool hit = i < n && key_of(x[i]) == (uint32_t)bin;
        unsigned bal = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) s_cnt[warp] = __popc(bal);
        __syncthreads();
        uint32_t before = seen, chunk = 0;
        for (int w = 0; w < 32; ++w) {
            if (w < warp) before += s_cnt[w];
            chunk += s_cnt[w];
        }
        uint32_t my = before + __popc(bal & ((1u << lane) - 1)) + 1;
        if (hit && my == (uint32_t)rank) {
            lcu_kv_pair r;
            r.idx = (uint32_t)i;
            r.val = x[i];
            r.pad = 0;
            out[row] = r;
            if (out_copy) out_copy[row] = r;
            s_found = 1;
        }
        seen += chunk;
        __syncthreads();
        if (s_found || seen >= (uint32_t)rank) break;
    }
}

// ------------------------------------------------------------------ host side

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
static int n_blocks(size_t n) { return (int)((n + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK); }

size_t argmax_workspace_bytes(int rows, size_t n) { return 2 * align256((size_t)rows * n_blocks(n) * 4); }
size_t sample_workspace_bytes(int rows, size_t n) {
    return argmax_workspace_bytes(rows, n) + align256((size_t)rows * SAMPLE_BINS * 4);
}

int sample_rows(lcu_kv_pair *out, lcu_kv_pair *out_copy, const void *logits, int rows, size_t n,
                const lcu_sample_args *args_dev, const float *randoms_dev, int dt, void *workspace,
                size_t workspace_len, cudaStream_t s, bool pdl, bool any_sampling) {
    if (rows <= 0) return LCU_OK;
    LCU_REQUIRE(dt == LCU_F16 || dt == LCU_BF16, "sample: logits dtype %d unsupported", dt);
    LCU_REQUIRE(n > 0 && n < 0xffffffffull, "sample: n = %zu", n);
    if (!args_dev) any_sampling = false;
    size_t need = any_sampling ? sample_workspace_bytes(rows, n) : argmax_workspace_bytes(rows, n);
    LCU_REQUIRE(workspace && workspace_len >= need, "sample: workspace of %zu bytes, %zu needed", workspace_len, need);
    LCU_REQUIRE(!any_sampling || randoms_dev, "sample: sampling rows need random numbers");
    int nblk = n_blocks(n);
    unsigned char *p = reinterpret_cast<unsigned char *>(workspace);
    float *pv = reinterpret_cast<float *>(p);
    uint32_t *pi = reinterpret_cast<uint32_t *>(p + align256((size_t)rows * nblk * 4));
    uint32_t *hist = reinterpret_cast<uint32_t *>(p + argmax_workspace_bytes(rows, n));
    const uint16_t *lg = reinterpret_cast<const uint16_t *>(logits);
    if (dt == LCU_F16) {
        LCU_CHECK_CUDA(launch_kernel(argmax_partial_kernel<__half>, dim3(nblk, rows), dim3(256), 0, s, pdl, lg, n, nblk, pv, pi));
        LCU_CHECK_CUDA(launch_kernel(argmax_final_kernel<__half>, dim3(rows), dim3(256), 0, s, pdl, lg, n, nblk,
                                     (const float *)pv, (const uint32_t *)pi, args_dev, out, out_copy));
        if (any_sampling)
            LCU_CHECK_CUDA(launch_kernel(sample_row_kernel<__half>, dim3(rows), dim3(SAMPLE_THREADS), 0, s, false, lg, n,
                                         args_dev, randoms_dev, hist, out, out_copy));
    } else {
        LCU_CHECK_CUDA(launch_kernel(argmax_partial_kernel<__nv_bfloat16>, dim3(nblk, rows), dim3(256), 0, s, pdl, lg, n, nblk, pv, pi));
        LCU_CHECK_CUDA(launch_kernel(argmax_final_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, pdl, lg, n, nblk,
                                     (const float *)pv, (const uint32_t *)pi, args_dev, out, out_copy));
        if (any_sampling)
            LCU_CHECK_CUDA(launch_kernel(sample_row_kernel<__nv_bfloat16>, dim3(rows), dim3(SAMPLE_THREADS), 0, s, false, lg,
                                         n, args_dev, randoms_dev, hist, out, out_copy));
    }
    return LCU_OK;
}

}  // namespace lcu

// ------------------------------------------------------------------ arg-max without any allocation
//
// Some hosts cannot hand this library a workspace and cannot let it allocate one: a serving
// loop that must never call cudaMalloc on its hot path (the call synchronises the whole
// device and would stall every other stream), a host whose device memory is owned
// entirely by an external pool it may not touch from here, or code that is already
// recording a stream capture, where allocation is not permitted.  For them the partial
// (value, index) pairs of the two-stage arg-max live in a fixed array inside the library
// image.  Every GPU that loads the library carries this array until the process exits.
namespace lcu {
constexpr size_t NOALLOC_SLOTS = 8192;  // rows x ceil(n / ARGMAX_CHUNK) partial pairs at most
static __device__ __align__(256) unsigned char g_noalloc_scratch[2 * NOALLOC_SLOTS * 4 + 512];
}  // namespace lcu

extern "C" int lcu_argmax_rows_noalloc(lcu_kv_pair *out, const void *logits, int rows, size_t n, int dt,
                                       lcu_stream_t stream) {
    using namespace lcu;
    LCU_REQUIRE(out && logits, "argmax_rows_noalloc: null argument");
    LCU_REQUIRE(rows >= 1 && n >= 1, "argmax_rows_noalloc: rows = %d, n = %zu", rows, n);
    size_t slots = (size_t)rows * ((n + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK);
    if (slots > NOALLOC_SLOTS || argmax_workspace_bytes(rows, n) > sizeof(g_noalloc_scratch)) {
        set_error("argmax_rows_noalloc: %d rows of %zu logits need %zu partial slots, the built-in scratch holds %zu "
                  "(use lcu_op_sample_rows with a caller workspace for larger problems)",
                  rows, n, slots, NOALLOC_SLOTS);
        return LCU_ERR_INVALID;
    }
    // The array's name is only a host-side handle; its device address is looked up once per
    // device, with that device current, and kept.
    static std::mutex mu;
    static void *addr[64] = {nullptr};
    int dev = 0;
    LCU_CHECK_CUDA(cudaGetDevice(&dev));
    LCU_REQUIRE(dev >= 0 && dev < 64, "argmax_rows_noalloc: device index %d out of range", dev);
    void *ws = nullptr;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!addr[dev]) {
            void *p = nullptr;
            LCU_CHECK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
            addr[dev] = p;
        }
        ws = addr[dev];
    }
    return sample_rows(out, nullptr, logits, rows, n, nullptr, nullptr, dt, ws, sizeof(g_noalloc_scratch), as_stream(stream),
                       false, false);
}
