// Stand-alone operators (ops.cu) and the collective wrapper (comm.cu).  Interface only.
#pragma once
#include "common.cuh"

namespace lcu {

int op_embedding(void *out, const void *table, const uint32_t *index, int n, size_t row_bytes, cudaStream_t s,
                 bool pdl);
int op_fast_embedding(uint32_t *tokens, const lcu_kv_pair *pairs, const uint32_t *map, int n, cudaStream_t s, bool pdl);
int op_rms_norm(void *y, int sy, const void *x, int sx, const void *w, int w_dt, float eps, int n, int d, int dt,
                cudaStream_t s, bool pdl);
int op_rope(void *y, int sty, int shy, const void *x, int stx, int shx, const uint32_t *pos, const float *sin_t,
            const float *cos_t, int n, int nh, int dh, int dt, cudaStream_t s, bool pdl);
int op_swiglu(void *out, int so, const void *gate, int sg, const void *up, int su, int n, int di, int dt,
              cudaStream_t s, bool pdl);
int op_add(void *y, int sny, int sdy, const void *x, int snx, int sdx, const void *b, int snb, int sdb, float k,
           int n, int d, int dt, cudaStream_t s);

// NCCL through dlopen (comm.cu)
int comm_all_reduce(void *comm, void *y, const void *x, size_t count, int dt, cudaStream_t s);
int comm_broadcast(void *comm, void *buf, size_t bytes, int root, cudaStream_t s);

}  // namespace lcu
