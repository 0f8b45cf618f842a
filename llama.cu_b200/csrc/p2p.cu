// Local half of the peer-memory all-reduce (protocol in p2p.cuh): wait for every rank's partial, sum
// the slots in rank order, write the residual stream, re-arm the counter.
#include <cstring>

#include "common.cuh"
#include "p2p.cuh"

namespace lcu {

namespace {

// Longest a kernel here spins on a peer before it gives up: about two seconds of SM clock unless the host set
// another limit (p2p_set_wait_limit_us; kept in constant memory so that captured graphs see a later change too).
__constant__ long long c_wait_cycles = 4000000000ll;
__device__ __forceinline__ long long p2p_wait_cycles() { return c_wait_cycles; }

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
    grid_dep_launch();
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        // once a wait has run out the group is broken: later waits give up at once instead of adding seconds each
        const long long limit = (*reinterpret_cast<volatile uint32_t *>(status) & 48u) ? 20000ll : p2p_wait_cycles();
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

struct GatherDst {
    unsigned char *gather[P2P_MAX_RANKS];  // every rank's gather buffer of this parity
    unsigned *garrive[P2P_MAX_RANKS];      // every rank's second counter of this parity
};

// Scatter form: this rank owns columns [rank * cols, (rank + 1) * cols) of every token row.
template <class T>
__global__ void __launch_bounds__(256) p2p_reduce_scatter_kernel(unsigned *header, int parity, ReduceSrc src, GatherDst dst,
                                                                 int n_ranks, int rank, T *y, int n_tok, int d, int cols,
                                                                 unsigned expected, uint32_t *status) {
    unsigned *arrive = header + parity, *leave = header + 2 + parity, *garrive = header + 5 + parity;
    grid_dep_launch();
    const long long limit = (*reinterpret_cast<volatile uint32_t *>(status) & 48u) ? 20000ll : p2p_wait_cycles();
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        while (ld_acquire_sys(arrive) < expected) {
            if (clock64() - t0 > limit) {
                atomicOr(status, 16u);
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    // phase A: sum my column slice of every token, store it into every rank's gather buffer
    const int vec_per_row = cols / 8;
    const size_t n_vec = (size_t)n_tok * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / vec_per_row), v = (int)(i - (size_t)t * vec_per_row);
        const size_t off = ((size_t)t * d + (size_t)rank * cols) / 8 + v;  // in 16-byte vectors
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 vv[P2P_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < P2P_MAX_RANKS; ++r)
            if (r < n_ranks) vv[r] = __ldcg(reinterpret_cast<const uint4 *>(src.slot[r]) + off);
#pragma unroll
        for (int r = 0; r < P2P_MAX_RANKS; ++r) {
            if (r < n_ranks) {
                const float2 a = Act<T>::to_f2(vv[r].x), b = Act<T>::to_f2(vv[r].y), c = Act<T>::to_f2(vv[r].z),
                             e = Act<T>::to_f2(vv[r].w);
                acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
                acc[4] += c.x; acc[5] += c.y; acc[6] += e.x; acc[7] += e.y;
            }
        }
        uint4 o;
        o.x = Act<T>::pack(acc[0], acc[1]); o.y = Act<T>::pack(acc[2], acc[3]);
        o.z = Act<T>::pack(acc[4], acc[5]); o.w = Act<T>::pack(acc[6], acc[7]);
#pragma unroll
        for (int r = 0; r < P2P_MAX_RANKS; ++r)
            if (r < n_ranks) reinterpret_cast<uint4 *>(dst.gather[r])[off] = o;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < (unsigned)n_ranks) atomicAdd_system(dst.garrive[threadIdx.x], 1u);
    // phase B: every owner's every CTA has delivered -> copy the gathered rows to the residual stream
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        const unsigned want = (unsigned)n_ranks * gridDim.x;
        while (ld_acquire_sys(garrive) < want) {
            if (clock64() - t0 > limit) {
                atomicOr(status, 16u);
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    const uint4 *g = reinterpret_cast<const uint4 *>(dst.gather[rank]);
    const size_t all_vec = (size_t)n_tok * d / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < all_vec; i += (size_t)gridDim.x * blockDim.x)
        reinterpret_cast<uint4 *>(y)[i] = __ldcg(g + i);
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(leave, 1u);
        if (t == gridDim.x - 1) {
            *reinterpret_cast<volatile unsigned *>(leave) = 0u;
            *reinterpret_cast<volatile unsigned *>(arrive) = 0u;
            *reinterpret_cast<volatile unsigned *>(garrive) = 0u;
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
        const long long limit = (*reinterpret_cast<volatile uint32_t *>(status) & 48u) ? 20000ll : p2p_wait_cycles();
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

// ---- LM head sharded by vocabulary rows: candidates of the other ranks travel to the lead rank
__global__ void __launch_bounds__(64) p2p_head_push_kernel(lcu_kv_pair *dst, unsigned *counter, const lcu_kv_pair *local, int rows,
                                                           uint32_t idx_offset) {
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
        lcu_kv_pair p = local[i];
        p.idx += idx_offset;
        dst[i] = p;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd_system(counter, 1u);
}

template <class T>
__global__ void __launch_bounds__(64) p2p_head_pick_kernel(const lcu_kv_pair *cands, unsigned *counter, int n_ranks, int max_seqs,
                                                           const lcu_kv_pair *local, int rows, lcu_kv_pair *out,
                                                           lcu_kv_pair *out_copy, uint32_t *status) {
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        const long long limit = (*reinterpret_cast<volatile uint32_t *>(status) & 48u) ? 20000ll : p2p_wait_cycles();
        while (ld_acquire_sys(counter) < (unsigned)(n_ranks - 1)) {
            if (clock64() - t0 > limit) {  // a rank never delivered its candidates: report, keep the local winner
                atomicOr(status, 16u);
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
        lcu_kv_pair best = local[i];
        float bv = Act<T>::to_f(*reinterpret_cast<const T *>(&best.val));
        for (int r = 1; r < n_ranks; ++r) {
            const unsigned long long raw = __ldcg(reinterpret_cast<const unsigned long long *>(cands + (size_t)r * max_seqs + i));
            lcu_kv_pair c;
            memcpy(&c, &raw, 8);
            const float cv = Act<T>::to_f(*reinterpret_cast<const T *>(&c.val));
            if (cv > bv || (cv == bv && c.idx < best.idx)) { best = c; bv = cv; }
        }
        out[i] = best;
        if (out_copy) out_copy[i] = best;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        *reinterpret_cast<volatile unsigned *>(counter) = 0u;
        __threadfence();
    }
}

}  // namespace

int p2p_set_wait_limit_us(long long us) {
    LCU_REQUIRE(us >= 1 && us <= 60ll * 1000 * 1000, "wait limit of %lld us (1 us .. 60 s)", us);
    const long long cycles = us * 2000;  // SM clock of this part tops out just under 2 GHz
    LCU_CHECK_CUDA(cudaMemcpyToSymbol(c_wait_cycles, &cycles, sizeof(cycles)));
    return LCU_OK;
}

size_t p2p_header_bytes(size_t bcast_bytes, size_t cand_bytes) { return (256 + bcast_bytes + cand_bytes + 255) / 256 * 256; }
size_t p2p_region_bytes(int n_ranks, size_t slot_bytes, size_t bcast_bytes, size_t cand_bytes) {
    return p2p_header_bytes(bcast_bytes, cand_bytes) + (size_t)2 * n_ranks * slot_bytes + (size_t)2 * slot_bytes;
}

static inline unsigned char *slot_ptr(void *base, const P2pState &st, int parity, int src) {
    return reinterpret_cast<unsigned char *>(base) + st.hdr_bytes + ((size_t)parity * st.n + src) * st.slot_bytes;
}

static inline unsigned char *gather_ptr(void *base, const P2pState &st, int parity) {
    return reinterpret_cast<unsigned char *>(base) + st.hdr_bytes + ((size_t)2 * st.n + parity) * st.slot_bytes;
}

void p2p_make_push(const P2pState &st, size_t byte_off, P2pPush *push, int scatter_cols) {
    push->n = st.n;
    push->scatter_cols = scatter_cols;
    for (int r = 0; r < P2P_MAX_RANKS; ++r) {
        push->slot[r] = r < st.n ? slot_ptr(st.base[r], st, st.parity, st.rank) + byte_off : nullptr;
        push->arrive[r] = r < st.n ? reinterpret_cast<unsigned *>(st.base[r]) + st.parity : nullptr;
    }
}

int p2p_reduce_launch(P2pState &st, void *y, int n_tok, int d, int dt, unsigned expected, int scatter_cols, uint32_t *status,
                      cudaStream_t s, bool pdl) {
    const size_t elems = (size_t)n_tok * d;
    LCU_REQUIRE(st.ready, "p2p all-reduce: peers are not attached");
    LCU_REQUIRE(elems % 8 == 0 && elems * 2 <= st.slot_bytes, "p2p all-reduce: %zu elements do not fit the slot", elems);
    ReduceSrc src;
    for (int r = 0; r < P2P_MAX_RANKS; ++r)
        src.slot[r] = r < st.n ? slot_ptr(st.own, st, st.parity, r) : nullptr;
    unsigned *header = reinterpret_cast<unsigned *>(st.own);
    if (scatter_cols) {
        LCU_REQUIRE(scatter_cols * st.n == d && scatter_cols % 8 == 0, "p2p all-reduce: %d columns per rank do not tile d = %d", scatter_cols, d);
        GatherDst dst;
        for (int r = 0; r < P2P_MAX_RANKS; ++r) {
            dst.gather[r] = r < st.n ? gather_ptr(st.base[r], st, st.parity) : nullptr;
            dst.garrive[r] = r < st.n ? reinterpret_cast<unsigned *>(st.base[r]) + 5 + st.parity : nullptr;
        }
        const size_t n_vec = (size_t)n_tok * scatter_cols / 8;
        int grid = (int)((n_vec + 255) / 256);
        if (grid > 32) grid = 32;
        if (grid < 1) grid = 1;
        if (dt == LCU_BF16)
            LCU_CHECK_CUDA(launch_kernel(p2p_reduce_scatter_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, pdl, header, st.parity,
                                         src, dst, st.n, st.rank, reinterpret_cast<__nv_bfloat16 *>(y), n_tok, d, scatter_cols,
                                         expected, status));
        else
            LCU_CHECK_CUDA(launch_kernel(p2p_reduce_scatter_kernel<__half>, dim3(grid), dim3(256), 0, s, pdl, header, st.parity, src,
                                         dst, st.n, st.rank, reinterpret_cast<__half *>(y), n_tok, d, scatter_cols, expected,
                                         status));
        st.parity ^= 1;
        return LCU_OK;
    }
    const size_t n_vec = elems / 8;
    int grid = (int)((n_vec + 255) / 256);
    if (grid > 64) grid = 64;
    if (dt == LCU_BF16)
        LCU_CHECK_CUDA(launch_kernel(p2p_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, pdl, header, st.parity, src, st.n,
                                     reinterpret_cast<__nv_bfloat16 *>(y), n_vec, expected, status));
    else
        LCU_CHECK_CUDA(launch_kernel(p2p_reduce_kernel<__half>, dim3(grid), dim3(256), 0, s, pdl, header, st.parity, src, st.n,
                                     reinterpret_cast<__half *>(y), n_vec, expected, status));
    st.parity ^= 1;
    return LCU_OK;
}

int p2p_head_push_launch(P2pState &st, const void *local_pairs, int rows, uint32_t idx_offset, cudaStream_t s) {
    LCU_REQUIRE(st.ready && st.rank != 0 && rows <= st.max_seqs, "p2p head push: bad state (rank %d, %d rows)", st.rank, rows);
    unsigned char *lead = reinterpret_cast<unsigned char *>(st.base[0]);
    lcu_kv_pair *dst = reinterpret_cast<lcu_kv_pair *>(lead + st.cand_off) + (size_t)st.rank * st.max_seqs;
    LCU_CHECK_CUDA(launch_kernel(p2p_head_push_kernel, dim3(1), dim3(64), 0, s, false, dst, reinterpret_cast<unsigned *>(lead) + 7,
                                 reinterpret_cast<const lcu_kv_pair *>(local_pairs), rows, idx_offset));
    return LCU_OK;
}

int p2p_head_pick_launch(P2pState &st, const void *local_pairs, int rows, int dt, void *out, void *out_copy, uint32_t *status,
                         cudaStream_t s) {
    LCU_REQUIRE(st.ready && st.rank == 0 && rows <= st.max_seqs, "p2p head pick: bad state (rank %d, %d rows)", st.rank, rows);
    unsigned char *own = reinterpret_cast<unsigned char *>(st.own);
    const lcu_kv_pair *cands = reinterpret_cast<const lcu_kv_pair *>(own + st.cand_off);
    unsigned *counter = reinterpret_cast<unsigned *>(own) + 7;
    if (dt == LCU_BF16)
        LCU_CHECK_CUDA(launch_kernel(p2p_head_pick_kernel<__nv_bfloat16>, dim3(1), dim3(64), 0, s, false, cands, counter, st.n,
                                     st.max_seqs, reinterpret_cast<const lcu_kv_pair *>(local_pairs), rows,
                                     reinterpret_cast<lcu_kv_pair *>(out), reinterpret_cast<lcu_kv_pair *>(out_copy), status));
    else
        LCU_CHECK_CUDA(launch_kernel(p2p_head_pick_kernel<__half>, dim3(1), dim3(64), 0, s, false, cands, counter, st.n, st.max_seqs,
                                     reinterpret_cast<const lcu_kv_pair *>(local_pairs), rows, reinterpret_cast<lcu_kv_pair *>(out),
                                     reinterpret_cast<lcu_kv_pair *>(out_copy), status));
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
