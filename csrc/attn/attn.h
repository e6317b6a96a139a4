// Host interface of the gated paged attention kernels (see attn.cu).
#pragma once
#include <cuda_runtime.h>

namespace vade {

const char* attn_prep(const void* qkv, int ld, int rows, int nq, int nkv, int hd, const float* q_norm, const float* k_norm,
                      const int* positions, const int* row_slot, const int* block_table, int max_pages, void* q_out,
                      void* k_pages, void* v_pages, int rot, double theta, float eps, cudaStream_t s);

// split = true: decode class (fixed 256-key splits, `partial` is fp32 scratch of
// rows * nq * n_split * 258 floats); split = false: prefill class, single pass.
const char* attn_rows(const void* q, const void* qkv, int ld, const void* k_pages, const void* v_pages, const int* positions,
                      const int* row_slot, const int* block_table, int max_pages, int rows, int nq, int nkv, int hd,
                      bool split, float* partial, int n_split, void* out, cudaStream_t s);

int attn_split_keys();

}  // namespace vade
