// Host interface of the residual-stream row kernels (see rows.cu).
#pragma once
#include <cuda_runtime.h>

namespace vade {

void embed(const void* table_bf16, const long long* tokens, float* x, int rows, int H, cudaStream_t s);
void rmsnorm(const void* x, bool x_is_bf16, const float* w, void* h_bf16, int rows, int H, float eps, int ldh, int h_off, cudaStream_t s);
void fold_add_norm(const float* parts, long long part_stride, int n_parts, float* x, const float* w, void* h_bf16,
                   int rows, int H, float eps, cudaStream_t s);
void combine_add_norm(const void* y_bf16, const int* slot_row, const int* ids, const float* wts, const float* sg, int k, int ns,
                      float* x, const float* w, void* h_bf16, int rows, int H, float eps, cudaStream_t s);
// SwiGLU over fp32 K-range partials [n_parts][rows][2 * I] of interleaved gate/up columns (n_parts <= 8).
void swiglu_fold(const float* parts, long long part_stride, int n_parts, const int* n_rows, void* mid_bf16, int max_rows, int I, cudaStream_t s);
void gather_rows(const void* x_bf16, const int* row_token, const int* n_rows, void* xs_bf16, int max_rows, int H, cudaStream_t s);

}  // namespace vade
