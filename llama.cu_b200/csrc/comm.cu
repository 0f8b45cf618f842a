// Collectives for the tensor-parallel step: NCCL found at run time with dlopen, so the
// library itself has no link-time dependency on it (the host process usually has NCCL
// loaded already).  Counterpart of the reference's use of crate `nccl`:
// `CommunicatorGroup::new` (llama.cu/src/exec/engine.rs:86), `all_reduce`
// (op/all_reduce.rs:36-40) and `broadcast` (exec/group.rs:114-115) — with one process per
// GPU instead of one thread per GPU, hence the unique-id handshake.
#include <dlfcn.h>

#include <cstring>

#include <mutex>

#include "ops.cuh"

namespace lcu {

namespace {
struct NcclId {  // ncclUniqueId, passed by value: 128 bytes
    char b[128];
};
struct Nccl {
    void *lib = nullptr;
    int (*GetUniqueId)(void *) = nullptr;
    int (*CommInitRank)(void **, int, NcclId, int) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*Broadcast)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};
Nccl g_nccl;
std::mutex g_mu;

int load_nccl() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_nccl.lib) return LCU_OK;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    void *lib = nullptr;
    for (const char *n : names) {
        lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (lib) break;
    }
    if (!lib) {
        set_error("NCCL library not found (libnccl.so.2): %s", dlerror());
        return LCU_ERR_COMM;
    }
    Nccl n;
    n.lib = lib;
    n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
    n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
    n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
    n.AllReduce = reinterpret_cast<decltype(n.AllReduce)>(dlsym(lib, "ncclAllReduce"));
    n.Broadcast = reinterpret_cast<decltype(n.Broadcast)>(dlsym(lib, "ncclBroadcast"));
    n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
    if (!n.GetUniqueId || !n.CommInitRank || !n.CommDestroy || !n.AllReduce || !n.Broadcast) {
        set_error("NCCL library lacks an expected symbol");
        return LCU_ERR_COMM;
    }
    g_nccl = n;
    return LCU_OK;
}

int nccl_fail(int rc, const char *what) {
    set_error("NCCL error %d (%s) in %s", rc, g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?", what);
    return LCU_ERR_COMM;
}
}  // namespace

int comm_all_reduce(void *comm, void *y, const void *x, size_t count, int dt, cudaStream_t s) {
    if (!comm) {
        set_error("all_reduce: no communicator");
        return LCU_ERR_COMM;
    }
    int rc = load_nccl();
    if (rc) return rc;
    // ncclDataType_t: ncclFloat16 = 6, ncclFloat32 = 7, ncclBfloat16 = 9; ncclSum = 0
    int nt = dt == LCU_F16 ? 6 : (dt == LCU_BF16 ? 9 : (dt == LCU_F32 ? 7 : -1));
    if (nt < 0) {
        set_error("all_reduce: dtype %d unsupported", dt);
        return LCU_ERR_INVALID;
    }
    int e = g_nccl.AllReduce(x, y, count, nt, 0, comm, s);
    if (e) return nccl_fail(e, "ncclAllReduce");
    return LCU_OK;
}

// == `comm.broadcast(tok_buf, None, 0, stream)` (llama.cu/src/exec/group.rs:114-115)
int comm_broadcast(void *comm, void *buf, size_t bytes, int root, cudaStream_t s) {
    if (!comm) {
        set_error("broadcast: no communicator");
        return LCU_ERR_COMM;
    }
    int rc = load_nccl();
    if (rc) return rc;
    int e = g_nccl.Broadcast(buf, buf, bytes, 0 /* ncclInt8 */, root, comm, s);
    if (e) return nccl_fail(e, "ncclBroadcast");
    return LCU_OK;
}

}  // namespace lcu

using namespace lcu;

extern "C" {

int lcu_comm_unique_id(void *id128) {
    LCU_REQUIRE(id128, "comm_unique_id: null argument");
    int rc = load_nccl();
    if (rc) return rc;
    int e = g_nccl.GetUniqueId(id128);
    if (e) return nccl_fail(e, "ncclGetUniqueId");
    return LCU_OK;
}

int lcu_comm_init_rank(const void *id128, int rank, int size, void **comm_out) {
    LCU_REQUIRE(id128 && comm_out && size >= 1 && rank >= 0 && rank < size, "comm_init_rank: bad arguments");
    int rc = load_nccl();
    if (rc) return rc;
    NcclId id;
    memcpy(id.b, id128, 128);
    void *comm = nullptr;
    int e = g_nccl.CommInitRank(&comm, size, id, rank);
    if (e) return nccl_fail(e, "ncclCommInitRank");
    *comm_out = comm;
    return LCU_OK;
}

int lcu_comm_destroy(void *comm) {
    if (!comm) return LCU_OK;
    int rc = load_nccl();
    if (rc) return rc;
    int e = g_nccl.CommDestroy(comm);
    if (e) return nccl_fail(e, "ncclCommDestroy");
    return LCU_OK;
}

}  // extern "C"
