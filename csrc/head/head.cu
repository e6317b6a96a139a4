// Output-head reductions over fp32 logits rows: greedy argmax (ties to the lowest id) and the
// merge of per-rank (value, id) candidates of a vocabulary-parallel head.
#include <cuda_runtime.h>
#include <cstdint>
#include <cfloat>
#include "../common/ptx.cuh"
#include "../common/launch.h"
#include "head.h"

namespace vade {

__global__ void argmax_rows_kernel(const float* __restrict__ logits, long long ld, int n, int id0,
                                   float* __restrict__ best_val, long long* __restrict__ best_id) {
    chain_release();
    chain_wait();
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

// Two-stage form for wide or vocabulary-parallel heads: stage 1 reduces chunks of 4096 logits (one CTA
// each, 16 loads per thread issued together) to (value, global id) pairs; with a peer exchange the pairs
// go to every rank's copy of the candidate table [rank][row][chunk].  Stage 2 joins a row's candidates
// in ascending (rank, chunk) order: larger value wins, ties to the lower id, so every rank picks the
// same token.
constexpr int kChunk = 4096;

__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float* __restrict__ logits, long long ld, int n, int id0, uint2* __restrict__ cand, int n_chunks,
                     int rows, const PeerExchange px) {
    chain_release();
    chain_wait();
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
        const uint2 c = make_uint2(__float_as_uint(bv), static_cast<uint32_t>(bi + id0));
        if (px.n == 0) {
            cand[row * n_chunks + blockIdx.x] = c;
        } else {
            const long long at = static_cast<long long>(exchange_parity(px)) * px.half_stride
                               + (static_cast<long long>(px.self) * rows + row) * n_chunks + blockIdx.x;
            for (int d = 0; d < px.n; ++d) reinterpret_cast<uint2*>(px.out[d])[at] = c;
            __threadfence_system();
            exchange_arrive(px, gridDim.x * gridDim.y);
        }
    }
}

__global__ void __launch_bounds__(32)
argmax_join_kernel(const uint2* __restrict__ cand_in, int n_cand_per_rank, int ranks, const uint32_t* flags, int self,
                   long long half_stride, uint32_t* status, float* __restrict__ best_val, long long* __restrict__ best_id) {
    chain_release();
    chain_wait();
    const long long row = blockIdx.x;
    const int rows = gridDim.x;
    const uint2* cand = cand_in;
    if (flags != nullptr) cand += static_cast<long long>(exchange_wait(flags, ranks, self, status)) * half_stride;
    float bv = -FLT_MAX;
    long long bi = 0x7fffffffffffll;
    for (int c = threadIdx.x; c < ranks * n_cand_per_rank; c += 32) {
        const int r = c / n_cand_per_rank, ch = c % n_cand_per_rank;
        const uint2 u = cand[(static_cast<long long>(r) * rows + row) * n_cand_per_rank + ch];
        const float v = __uint_as_float(u.x);
        const long long i = u.y;
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) { best_val[row] = bv; best_id[row] = bi; }
}

void argmax_rows(const float* logits, long long ld, int rows, int n, int id0, float* best_val, long long* best_id,
                 void* cand, const HeadExchange* hx, uint32_t* status, cudaStream_t s) {
    if (cand == nullptr && hx == nullptr) {
        launch_chained(argmax_rows_kernel, dim3(rows), dim3(1024), 0, s, logits, ld, n, id0, best_val, best_id);
        return;
    }
    const int n_chunks = (n + kChunk - 1) / kChunk;
    PeerExchange px{};
    if (hx != nullptr) {
        for (int i = 0; i < hx->ranks; ++i) { px.out[i] = hx->out[i]; px.flags[i] = hx->flags[i]; }
        px.local = hx->local; px.half_stride = hx->half_stride; px.n = hx->ranks; px.self = hx->self; px.local_only_from = 0x7fffffff;
    }
    launch_chained(argmax_chunks_kernel, dim3(dim3(n_chunks, rows)), dim3(256), 0, s, logits, ld, n, id0, static_cast<uint2*>(cand), n_chunks, rows, px);
    if (hx != nullptr)
        launch_chained(argmax_join_kernel, dim3(rows), dim3(32), 0, s, static_cast<const uint2*>(hx->out[hx->self]), n_chunks, hx->ranks, hx->flags[hx->self],
                                              hx->self, hx->half_stride, status, best_val, best_id);
    else
        launch_chained(argmax_join_kernel, dim3(rows), dim3(32), 0, s, static_cast<const uint2*>(cand), n_chunks, 1, nullptr, 0, 0, status, best_val, best_id);
}

int argmax_chunk() { return kChunk; }

}  // namespace vade
