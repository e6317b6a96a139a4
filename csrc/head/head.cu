// Output-head reductions over fp32 logits rows: greedy argmax (ties to the lowest id) and the
// merge of per-rank (value, id) candidates of a vocabulary-parallel head.
#include <cuda_runtime.h>
#include <cstdint>
#include <cfloat>
#include "head.h"

namespace vade {

__global__ void argmax_rows_kernel(const float* __restrict__ logits, long long ld, int n, int id0,
                                   float* __restrict__ best_val, long long* __restrict__ best_id) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const long long row = blockIdx.x;
    const float* p = logits + row * ld;
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = p[i];
        if (v > bv) { bv = v; bi = i; }            // ascending i per thread: ties keep the lower id
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (blockDim.x >> 5); ++w)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        best_val[row] = bv;
        best_id[row] = static_cast<long long>(bi) + id0;
    }
}

// Two-stage form for wide vocabularies: stage 1 reduces chunks of 4096 logits (one CTA each, 16 loads
// per thread issued together), stage 2 joins the chunk winners of a row in ascending chunk order.
constexpr int kChunk = 4096;

__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float* __restrict__ logits, long long ld, int n, float* __restrict__ cval, int* __restrict__ cidx, int n_chunks) {
    __shared__ float sv[8];
    __shared__ int si[8];
    const long long row = blockIdx.y;
    const int base = blockIdx.x * kChunk;
    const float* p = logits + row * ld + base;
    float v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) { const int i = u * 256 + threadIdx.x; v[u] = base + i < n ? p[i] : -FLT_MAX; }
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
#pragma unroll
    for (int u = 0; u < 16; ++u) if (v[u] > bv) { bv = v[u]; bi = base + u * 256 + threadIdx.x; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        cval[row * n_chunks + blockIdx.x] = bv;
        cidx[row * n_chunks + blockIdx.x] = bi;
    }
}

__global__ void __launch_bounds__(32)
argmax_join_kernel(const float* __restrict__ cval, const int* __restrict__ cidx, int n_chunks, int id0,
                   float* __restrict__ best_val, long long* __restrict__ best_id) {
    const long long row = blockIdx.x;
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < n_chunks; c += 32) {
        const float v = cval[row * n_chunks + c];
        const int i = cidx[row * n_chunks + c];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) { best_val[row] = bv; best_id[row] = static_cast<long long>(bi) + id0; }
}

void argmax_rows(const float* logits, long long ld, int rows, int n, int id0, float* best_val, long long* best_id,
                 float* chunk_val, int* chunk_idx, cudaStream_t s) {
    if (chunk_val == nullptr || n <= kChunk) {
        argmax_rows_kernel<<<rows, 1024, 0, s>>>(logits, ld, n, id0, best_val, best_id);
        return;
    }
    const int n_chunks = (n + kChunk - 1) / kChunk;
    argmax_chunks_kernel<<<dim3(n_chunks, rows), 256, 0, s>>>(logits, ld, n, chunk_val, chunk_idx, n_chunks);
    argmax_join_kernel<<<rows, 32, 0, s>>>(chunk_val, chunk_idx, n_chunks, id0, best_val, best_id);
}

int argmax_chunk() { return kChunk; }

}  // namespace vade
