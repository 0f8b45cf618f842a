// All-reduce of the tensor-parallel decode step over NVLink peer memory, fused with the producing
// linear layer.  Replaces the `AllReduce` node the reference places after the output and the down
// projection (llama.cu/src/op/all_reduce.rs:1-41, one ncclAllReduce per node).
//
// Protocol (one process per GPU, memory shared through CUDA IPC):
//   * every rank owns a region  [2 parities][n_ranks sources][max_tokens x d]  plus two arrival
//     counters and two departure tickets;
//   * the epilogue of the producing kernel stores its partial row block into slot (parity, me) of
//     EVERY rank's region (plain peer stores), fences, and each of its CTAs adds 1 to every rank's
//     arrival counter of that parity;
//   * a small local kernel on each rank waits (bounded) until its counter reaches
//     n_ranks x producer CTAs, sums the n_ranks slots in rank order in f32, rounds once and writes
//     the residual stream; the last of its CTAs to leave zeroes the counter.
// Large rounds (scatter form): pushing every partial to every rank costs (n_ranks - 1) x the message
// per rank on NVLink.  Instead rank k OWNS columns [k d/n, (k+1) d/n): producers store a partial only
// into the owner's region, the owner's kernel sums its column slice and stores the result into the
// "gather" buffer of every rank, raises their second counter, waits for its own second counter
// (every owner, every CTA) and copies the gathered rows to the residual stream: 2 (n-1)/n of the
// message per rank instead of (n-1), for one more hop.
// Two parities alternate from one all-reduce to the next.  A rank can only push into parity p again
// after it has passed its own reduction of parity p^1, which needs every rank's push of p^1, which
// every rank issues after finishing its reduction of p: so a slot and its counter are never written
// while they are still being read or reset.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace lcu {

constexpr int P2P_MAX_RANKS = 8;

// What a producing kernel needs: where to store and whom to tell.  n == 0: plain local output.
struct P2pPush {
    void *slot[P2P_MAX_RANKS];          // slot (parity, me) in rank r's region, offset like `y`
    unsigned *arrive[P2P_MAX_RANKS];    // rank r's arrival counter of this parity
    int n;
    int scatter_cols;                   // 0: store to every rank; else columns per owner, store to rank col / scatter_cols
};

#ifdef __CUDACC__
// Called by every thread of a producing CTA once all its output stores are issued.
__device__ __forceinline__ void p2p_signal(const P2pPush &p) {
    if (p.n == 0) return;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < (unsigned)p.n) atomicAdd_system(p.arrive[threadIdx.x], 1u);
}
#endif

struct P2pState {
    int rank = 0, n = 0;
    void *own = nullptr;                     // this rank's region (cudaMalloc)
    void *base[P2P_MAX_RANKS] = {nullptr};   // every rank's region as mapped here
    size_t slot_bytes = 0;                   // max_tokens * d * 2
    size_t hdr_bytes = 0;                    // counters (first 256 bytes) + broadcast buffer + head candidates
    size_t cand_off = 0;                     // byte offset of the head candidates [n_ranks][max_seqs] (8 bytes each)
    int max_seqs = 0;
    int parity = 0;                          // of the next all-reduce
    bool ready = false;
};

// Region layout: words 0..1 arrival counters, 2..3 departure tickets (per parity), 4 broadcast flag, 5..6 second
// (gather) counters, 7 head-candidate counter; from byte 256 the broadcast buffer (bcast_bytes), then the head
// candidates (cand_bytes); from hdr_bytes the slots [2][n_ranks][slot_bytes], then the gather buffers [2][slot_bytes].
size_t p2p_header_bytes(size_t bcast_bytes, size_t cand_bytes);
size_t p2p_region_bytes(int n_ranks, size_t slot_bytes, size_t bcast_bytes, size_t cand_bytes);
// Fills `push` for the next all-reduce (current parity) with a byte offset into the slot; scatter_cols as in P2pPush.
void p2p_make_push(const P2pState &st, size_t byte_off, P2pPush *push, int scatter_cols = 0);
// Enqueues the local reduction of n_tok rows of d elements (2-byte activation type): waits for `expected` arrivals,
// y = sum over ranks of the slots (scatter_cols != 0: the scatter form above); then flips the parity.
// status: device word that gets bit 16 on a timed-out wait.
// pdl: launched as a programmatic dependent of the producing projection — the kernel only spins on counters that the
// producers (this rank's included) raise after their last access, so it never waits for the producer grid itself, and
// it releases its own dependents at once.
int p2p_reduce_launch(P2pState &st, void *y, int n_tok, int d, int dt, unsigned expected, int scatter_cols, uint32_t *status,
                      cudaStream_t s, bool pdl = false);

// LM head sharded by vocabulary rows: every rank arg-maxes its slice; the others store their candidate pairs (index made
// global) into the lead rank's region and raise its counter (push), the lead rank waits (bounded) for n_ranks - 1
// arrivals and keeps, per row, the largest value / lowest index (pick), writing `out` and `out_copy`.
int p2p_head_push_launch(P2pState &st, const void *local_pairs, int rows, uint32_t idx_offset, cudaStream_t s);
int p2p_head_pick_launch(P2pState &st, const void *local_pairs, int rows, int dt, void *out, void *out_copy, uint32_t *status,
                         cudaStream_t s);

// Limit of every bounded peer wait of the calling thread's current device, in microseconds (default about 2 s).
int p2p_set_wait_limit_us(long long us);

// Token broadcast from rank `root` (the reference's `share_inputs`, exec/engine.rs:264-274): the root stores
// `bytes` (a multiple of 4, at most the broadcast buffer) into every other rank's buffer and raises their flag;
// the others wait (bounded) for the flag, copy the buffer to `data` and lower the flag.  Ranks are kept in step
// by the all-reduces between two broadcasts, so one buffer is enough.
int p2p_broadcast_launch(P2pState &st, void *data, size_t bytes, int root, uint32_t *status, cudaStream_t s);

}  // namespace lcu
