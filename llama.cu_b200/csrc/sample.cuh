// Arg-max and temperature / top-k / top-p sampling over rows of logits.  Interface only.
#pragma once
#include "common.cuh"

namespace lcu {

constexpr int ARGMAX_CHUNK = 4096;  // logits per partial-reduction block

size_t argmax_workspace_bytes(int rows, size_t n);
size_t sample_workspace_bytes(int rows, size_t n);  // covers argmax too
// args_dev == nullptr: every row is arg-max.  out_copy may be nullptr.
int sample_rows(lcu_kv_pair *out, lcu_kv_pair *out_copy, const void *logits, int rows, size_t n,
                const lcu_sample_args *args_dev, const float *randoms_dev, int dt, void *workspace,
                size_t workspace_len, cudaStream_t s, bool pdl, bool any_sampling);

}  // namespace lcu
