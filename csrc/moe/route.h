// Host interface of the MoE routing kernels (see route.cu).
#pragma once
#include <cuda_runtime.h>

namespace vade {

// logits fp32 [T][ld] with E router columns followed by the shared-expert gate column.
// Outputs: ids/wts [T][k], sg [T], tasks int4 [max_tasks], meta {tasks, rows, tasks wanted},
// row_token [rows], slot_row [T][k + ns].  counts [n_local] must be zero on entry and is zero on exit.
void moe_route(const float* logits, int ld, int T, int E, int k, bool renorm, int e0, int n_local, int ns, int bn,
               int* ids, float* wts, float* sg, int* counts, int* pos, int* offsets, int* tasks, int* meta, int max_tasks,
               int* row_token, int* slot_row, cudaStream_t s);

}  // namespace vade
