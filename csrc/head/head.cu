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

void argmax_rows(const float* logits, long long ld, int rows, int n, int id0, float* best_val, long long* best_id, cudaStream_t s) {
    argmax_rows_kernel<<<rows, 1024, 0, s>>>(logits, ld, n, id0, best_val, best_id);
}

}  // namespace vade
