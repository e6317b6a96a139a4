// Host interface of the output-head reductions (see head.cu).
#pragma once
#include <cuda_runtime.h>

namespace vade {

// Greedy token per row: the largest logit, ties to the lowest id.  With chunk scratch
// (rows * ceil(n / argmax_chunk()) floats and ints) wide rows are reduced in two stages.
void argmax_rows(const float* logits, long long ld, int rows, int n, int id0, float* best_val, long long* best_id,
                 float* chunk_val, int* chunk_idx, cudaStream_t s);
int argmax_chunk();

}  // namespace vade
