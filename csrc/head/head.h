// Host interface of the output-head reductions (see head.cu).
#pragma once
#include <cuda_runtime.h>

namespace vade {

void argmax_rows(const float* logits, long long ld, int rows, int n, int id0, float* best_val, long long* best_id, cudaStream_t s);

}  // namespace vade
