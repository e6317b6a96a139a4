// Row kernels around the fp32 residual stream: embedding gather, RMSNorm (1 + w), the fold of
// canonical-range partial sums fused with the residual add and the next norm, and the ordered
// MoE combine fused with the residual add and the next norm.
//
// One CTA per token row; every reduction is a fixed tree (per-thread ascending strides, then a
// 32-lane butterfly, then warps in index order), so a row's bits never depend on the rows beside it.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "../common/ptx.cuh"
#include "rows.h"

namespace vade {

constexpr int kRowThreads = 256;

// Sum over the block in a fixed order; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    const int nw = blockDim.x >> 5;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}

__global__ void embed_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ tokens,
                             float* __restrict__ x, int H) {
    const long long row = blockIdx.x;
    const __nv_bfloat16* src = table + tokens[row] * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) x[row * H + i] = __bfloat162float(src[i]);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// h = bf16( x * rsqrt(mean(x^2) + eps) * (1 + w) ); input fp32 or bf16
template <typename TIn>
__global__ void rmsnorm_kernel(const TIn* __restrict__ x, const float* __restrict__ w, __nv_bfloat16* __restrict__ h,
                               int H, float eps, int ldh, int h_off) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = to_f32(x[row * H + i]); ss += v * v; }
    const float inv = rsqrtf(block_sum(ss, red) / H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        h[row * ldh + h_off + i] = __float2bfloat16_rn(to_f32(x[row * H + i]) * inv * (1.f + w[i]));
}

// x += ((p0+p1)+(p2+p3))+((p4+p5)+(p6+p7));  h = norm(x) if w != nullptr
__global__ void fold_add_norm_kernel(const float* __restrict__ parts, long long part_stride, int n_parts,
                                     float* __restrict__ x, const float* __restrict__ w, __nv_bfloat16* __restrict__ h,
                                     int H, float eps) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float* p = parts + row * H + i;
        float s;
        if (n_parts == 8) {
            s = ((p[0] + p[part_stride]) + (p[2 * part_stride] + p[3 * part_stride]))
              + ((p[4 * part_stride] + p[5 * part_stride]) + (p[6 * part_stride] + p[7 * part_stride]));
        } else if (n_parts == 4) {
            s = (p[0] + p[part_stride]) + (p[2 * part_stride] + p[3 * part_stride]);
        } else if (n_parts == 2) {
            s = p[0] + p[part_stride];
        } else {
            s = p[0];
        }
        const float v = x[row * H + i] + s;
        x[row * H + i] = v;
        ss += v * v;
    }
    if (w == nullptr) return;
    const float inv = rsqrtf(block_sum(ss, red) / H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        h[row * H + i] = __float2bfloat16_rn(x[row * H + i] * inv * (1.f + w[i]));
}

// x[t] += sum over the token's slots in ascending expert id of weight * y[row_of(t, slot)], then the
// shared virtual experts (ids above every routed id) in order; h = norm(x) if w != nullptr.
// y is bf16 [rows][H]; slot_row[t][slot] gives the row of y (or -1 if the slot is not present).
__global__ void combine_add_norm_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ slot_row,
                                        const int* __restrict__ ids, const float* __restrict__ wts, const float* __restrict__ sg,
                                        int k, int ns, float* __restrict__ x, const float* __restrict__ w,
                                        __nv_bfloat16* __restrict__ h, int H, float eps) {
    __shared__ float red[32];
    __shared__ int order[64];
    __shared__ float ow[64];
    __shared__ int orow[64];
    const long long t = blockIdx.x;
    const int slots = k + ns;
    if (threadIdx.x == 0) {
        // insertion sort of the k routed slots by expert id (ids are distinct per token)
        for (int j = 0; j < k; ++j) order[j] = j;
        for (int a = 1; a < k; ++a) {
            const int cur = order[a];
            const int key = ids[t * k + cur];
            int b = a - 1;
            while (b >= 0 && ids[t * k + order[b]] > key) { order[b + 1] = order[b]; --b; }
            order[b + 1] = cur;
        }
        for (int j = 0; j < k; ++j) { ow[j] = wts[t * k + order[j]]; orow[j] = slot_row[t * slots + order[j]]; }
        for (int j = 0; j < ns; ++j) { ow[k + j] = sg[t]; orow[k + j] = slot_row[t * slots + k + j]; }
    }
    __syncthreads();
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < slots; ++j) {
            const int r = orow[j];
            if (r >= 0) acc += ow[j] * __bfloat162float(y[static_cast<long long>(r) * H + i]);
        }
        const float v = x[t * H + i] + acc;
        x[t * H + i] = v;
        ss += v * v;
    }
    if (w == nullptr) return;
    const float inv = rsqrtf(block_sum(ss, red) / H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        h[t * H + i] = __float2bfloat16_rn(x[t * H + i] * inv * (1.f + w[i]));
}

// rows of xs = rows of x picked by row_token (the MoE dispatch gather into expert-sorted order)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_token,
                                   const int* __restrict__ n_rows, __nv_bfloat16* __restrict__ xs, int H) {
    const int r = blockIdx.x;
    if (r >= *n_rows) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(row_token[r]) * H);
    uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<long long>(r) * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

void embed(const void* table, const long long* tokens, float* x, int rows, int H, cudaStream_t s) {
    embed_kernel<<<rows, kRowThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(table), tokens, x, H);
}
void rmsnorm(const void* x, bool x_is_bf16, const float* w, void* h, int rows, int H, float eps, int ldh, int h_off, cudaStream_t s) {
    if (x_is_bf16)
        rmsnorm_kernel<__nv_bfloat16><<<rows, kRowThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), w, static_cast<__nv_bfloat16*>(h), H, eps, ldh, h_off);
    else
        rmsnorm_kernel<float><<<rows, kRowThreads, 0, s>>>(static_cast<const float*>(x), w, static_cast<__nv_bfloat16*>(h), H, eps, ldh, h_off);
}
void fold_add_norm(const float* parts, long long part_stride, int n_parts, float* x, const float* w, void* h,
                   int rows, int H, float eps, cudaStream_t s) {
    fold_add_norm_kernel<<<rows, kRowThreads, 0, s>>>(parts, part_stride, n_parts, x, w, static_cast<__nv_bfloat16*>(h), H, eps);
}
void combine_add_norm(const void* y, const int* slot_row, const int* ids, const float* wts, const float* sg, int k, int ns,
                      float* x, const float* w, void* h, int rows, int H, float eps, cudaStream_t s) {
    combine_add_norm_kernel<<<rows, kRowThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(y), slot_row, ids, wts, sg, k, ns, x, w,
                                                        static_cast<__nv_bfloat16*>(h), H, eps);
}
void gather_rows(const void* x, const int* row_token, const int* n_rows, void* xs, int max_rows, int H, cudaStream_t s) {
    gather_rows_kernel<<<max_rows, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(x), row_token, n_rows, static_cast<__nv_bfloat16*>(xs), H);
}

}  // namespace vade
