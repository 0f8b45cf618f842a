// Local half of the peer-memory all-reduce (protocol in p2p.cuh): wait for every rank's partial, sum
// the slots in rank order, write the residual stream, re-arm the counter.
#include "common.cuh"
#include "p2p.cuh"

namespace lcu {

namespace {

constexpr long long P2P_WAIT_CYCLES = 4000000000ll;  // about two seconds of SM clock

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct ReduceSrc {
    const unsigned char *slot[P2P_MAX_RANKS];
};

// header words of a region: [0..1] arrival counters, [2..3] departure tickets (per parity)
template <class T>
__global__ void __launch_bounds__(256) p2p_reduce_kernel(unsigned *header, int parity, ReduceSrc src, int n_ranks, T *y,
                                                         size_t n_vec, unsigned expected, uint32_t *status) {
    unsigned *arrive = header + parity, *leave = header + 2 + parity;
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        // once a wait has run out the group is broken: later waits give up at once instead of adding seconds each
        const long long limit = (*reinterpret_cast<volatile uint32_t *>(status) & 48u) ? 20000ll : P2P_WAIT_CYCLES;
        while (ld_acquire_sys(arrive) < expected) {
            if (clock64() - t0 > limit) {  // a peer never pushed: report and carry on
                atomicOr(status, 16u);
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 v[P2P_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < P2P_MAX_RANKS; ++r)
            if (r < n_ranks) v[r] = __ldcg(reinterpret_cast<const uint4 *>(src.slot[r]) + i);
#pragma unroll
        for (int r = 0; r < P2P_MAX_RANKS; ++r) {
            if (r < n_ranks) {
                const float2 a = Act<T>::to_f2(v[r].x), b = Act<T>::to_f2(v[r].y), c = Act<T>::to_f2(v[r].z),
                             d = Act<T>::to_f2(v[r].w);
                acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
                acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
            }
        }
        uint4 o;
        o.x = Act<T>::pack(acc[0], acc[1]); o.y = Act<T>::pack(acc[2], acc[3]);
        o.z = Act<T>::pack(acc[4], acc[5]); o.w = Act<T>::pack(acc[6], acc[7]);
        reinterpret_cast<uint4 *>(y)[i] = o;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(leave, 1u);
        if (t == gridDim.x - 1) {  // everyone of this launch has seen the counter: re-arm it
            *reinterpret_cast<volatile unsigned *>(leave) = 0u;
            *reinterpret_cast<volatile unsigned *>(arrive) = 0u;
            __threadfence();
        }
    }
}

struct BcastDst {
    unsigned char *base[P2P_MAX_RANKS];
};

__global__ void __launch_bounds__(256) p2p_broadcast_kernel(BcastDst peers, int n_ranks, int rank, int root, uint32_t *data,
                                                            int n_words, uint32_t *status) {
    if (rank == root) {
        for (int r = 0; r < n_ranks; ++r) {
            if (r == root) continue;
            uint32_t *dst = reinterpret_cast<uint32_t *>(peers.base[r] + 256);
            for (int i = threadIdx.x; i < n_words; i += blockDim.x) dst[i] = data[i];
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < (unsigned)n_ranks && (int)threadIdx.x != root)
            atomicAdd_system(reinterpret_cast<unsigned *>(peers.base[threadIdx.x]) + 4, 1u);
        return;
    }
    unsigned *flag = reinterpret_cast<unsigned *>(peers.base[rank]) + 4;
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        const long long limit = (*reinterpret_cast<volatile uint32_t *>(status) & 48u) ? 20000ll : P2P_WAIT_CYCLES;
        while (ld_acquire_sys(flag) == 0u) {
            if (clock64() - t0 > limit) {
                atomicOr(status, 32u);
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    const uint32_t *src = reinterpret_cast<const uint32_t *>(peers.base[rank] + 256);
    for (int i = threadIdx.x; i < n_words; i += blockDim.x) data[i] = __ldcg(src + i);
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned *>(flag) = 0u;
}

}  // namespace

size_t p2p_header_bytes(size_t bcast_bytes) { return (256 + bcast_bytes + 255) / 256 * 256; }
size_t p2p_region_bytes(int n_ranks, size_t slot_bytes, size_t bcast_bytes) {
    return p2p_header_bytes(bcast_bytes) + (size_t)2 * n_ranks * slot_bytes;
}

static inline unsigned char *slot_ptr(void *base, const P2pState &st, int parity, int src) {
    return reinterpret_cast<unsigned char *>(base) + st.hdr_bytes + ((size_t)parity * st.n + src) * st.slot_bytes;
}

void p2p_make_push(const P2pState &st, size_t byte_off, P2pPush *push) {
    push->n = st.n;
    for (int r = 0; r < P2P_MAX_RANKS; ++r) {
        push->slot[r] = r < st.n ? slot_ptr(st.base[r], st, st.parity, st.rank) + byte_off : nullptr;
        push->arrive[r] = r < st.n ? reinterpret_cast<unsigned *>(st.base[r]) + st.parity : nullptr;
    }
}

int p2p_reduce_launch(P2pState &st, void *y, size_t elems, int dt, unsigned expected, uint32_t *status, cudaStream_t s) {
    LCU_REQUIRE(st.ready, "p2p all-reduce: peers are not attached");
    LCU_REQUIRE(elems % 8 == 0 && elems * 2 <= st.slot_bytes, "p2p all-reduce: %zu elements do not fit the slot", elems);
    ReduceSrc src;
    for (int r = 0; r < P2P_MAX_RANKS; ++r)
        src.slot[r] = r < st.n ? slot_ptr(st.own, st, st.parity, r) : nullptr;
    const size_t n_vec = elems / 8;
    int grid = (int)((n_vec + 255) / 256);
    if (grid > 64) grid = 64;
    unsigned *header = reinterpret_cast<unsigned *>(st.own);
    if (dt == LCU_BF16)
        LCU_CHECK_CUDA(launch_kernel(p2p_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, false, header, st.parity, src, st.n,
                                     reinterpret_cast<__nv_bfloat16 *>(y), n_vec, expected, status));
    else
        LCU_CHECK_CUDA(launch_kernel(p2p_reduce_kernel<__half>, dim3(grid), dim3(256), 0, s, false, header, st.parity, src, st.n,
                                     reinterpret_cast<__half *>(y), n_vec, expected, status));
    st.parity ^= 1;
    return LCU_OK;
}

int p2p_broadcast_launch(P2pState &st, void *data, size_t bytes, int root, uint32_t *status, cudaStream_t s) {
    LCU_REQUIRE(st.ready, "p2p broadcast: peers are not attached");
    LCU_REQUIRE(bytes % 4 == 0 && 256 + bytes <= st.hdr_bytes, "p2p broadcast: %zu bytes do not fit the buffer", bytes);
    BcastDst peers;
    for (int r = 0; r < P2P_MAX_RANKS; ++r) peers.base[r] = r < st.n ? reinterpret_cast<unsigned char *>(st.base[r]) : nullptr;
    LCU_CHECK_CUDA(launch_kernel(p2p_broadcast_kernel, dim3(1), dim3(256), 0, s, false, peers, st.n, st.rank, root,
                                 reinterpret_cast<uint32_t *>(data), (int)(bytes / 4), status));
    return LCU_OK;
}

}  // namespace lcu
