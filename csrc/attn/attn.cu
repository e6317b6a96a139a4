// Gated attention over the paged KV cache (head dimension 256, GQA).
//
//   attn_prep    per (row, head): q/k RMSNorm (1 + w), partial rotary embedding on the first `rot`
//                dims (rotate-half), q written as bf16 rows, k/v appended to the row's cache page
//   attn_rows    one CTA per (row, kv head[, key split]); one warp per query head of the group;
//                lanes own 8 of the 256 dims; online softmax over the row's visible keys.
//                Decode class: keys are cut into fixed 256-key splits (independent of the batch),
//                partials {m, l, acc} go to scratch and attn_merge joins them in split order.
//                Prefill class: one pass over all keys, output written directly.
//   output       attention * sigmoid(gate), bf16, gate read from the q projection rows
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cfloat>
#include "../common/ptx.cuh"
#include "attn.h"

namespace vade {

constexpr int kHD = 256;
constexpr int kPage = 64;
constexpr int kSplit = 256;

__global__ void attn_prep_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int nq, int nkv,
                                 const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                 const int* __restrict__ positions, const int* __restrict__ row_slot,
                                 const int* __restrict__ block_table, int max_pages,
                                 __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pages,
                                 __nv_bfloat16* __restrict__ v_pages, int rot, double log_theta, float eps) {
    __shared__ float xs[kHD];
    __shared__ float red[8];
    const int row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    const int pos = positions[row];
    const __nv_bfloat16* base = qkv + static_cast<long long>(row) * ld;
    const bool is_q = head < nq;
    const int kvh = is_q ? 0 : (head - nq);
    const __nv_bfloat16* src = is_q ? base + head * 2 * kHD : base + nq * 2 * kHD + kvh * kHD;
    const float x = __bfloat162float(src[d]);
    float ss = x * x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((d & 31) == 0) red[d >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float w = is_q ? q_norm[d] : k_norm[d];
    const float xn = x * rsqrtf(tot / kHD + eps) * (1.f + w);
    xs[d] = xn;
    __syncthreads();
    float y = xn;
    const int half = rot >> 1;
    if (d < rot) {
        const int i = d < half ? d : d - half;
        const double ang = static_cast<double>(pos) * exp(-log_theta * (2.0 * i) / rot);
        double sn, cs;
        sincos(ang, &sn, &cs);
        const float c = static_cast<float>(cs), s = static_cast<float>(sn);
        y = d < half ? xs[d] * c - xs[d + half] * s : xs[d] * c + xs[d - half] * s;
    }
    if (is_q) {
        q_out[(static_cast<long long>(row) * nq + head) * kHD + d] = __float2bfloat16_rn(y);
    } else {
        const int page = block_table[static_cast<long long>(row_slot[row]) * max_pages + pos / kPage];
        const long long at = ((static_cast<long long>(page) * kPage + pos % kPage) * nkv + kvh) * kHD + d;
        k_pages[at] = __float2bfloat16_rn(y);
        v_pages[at] = base[nq * 2 * kHD + nkv * kHD + kvh * kHD + d];
    }
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

template <bool SPLIT>
__global__ void attn_rows_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ qkv, int ld,
                                 const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                                 const int* __restrict__ positions, const int* __restrict__ row_slot,
                                 const int* __restrict__ block_table, int max_pages, int nq, int nkv, float scale,
                                 float* __restrict__ partial, int n_split, __nv_bfloat16* __restrict__ out) {
    const int row = blockIdx.x, kvh = blockIdx.y, split = SPLIT ? blockIdx.z : 0;
    const int group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = kvh * group + warp;
    const int len = positions[row] + 1;
    const int k0 = SPLIT ? split * kSplit : 0;
    const int k1 = SPLIT ? min(len, k0 + kSplit) : len;
    if (k0 >= len) return;
    float qv[8];
    unpack8(*reinterpret_cast<const uint4*>(q + (static_cast<long long>(row) * nq + head) * kHD + lane * 8), qv);
#pragma unroll
    for (int i = 0; i < 8; ++i) qv[i] *= scale;
    const int* table = block_table + static_cast<long long>(row_slot[row]) * max_pages;
    float m = -FLT_MAX, l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int key = k0; key < k1; ++key) {
        const long long at = ((static_cast<long long>(table[key / kPage]) * kPage + key % kPage) * nkv + kvh) * kHD + lane * 8;
        float kf[8], vf[8];
        unpack8(*reinterpret_cast<const uint4*>(k_pages + at), kf);
        unpack8(*reinterpret_cast<const uint4*>(v_pages + at), vf);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += qv[i] * kf[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float mn = fmaxf(m, s);
        const float corr = __expf(m - mn);
        const float p = __expf(s - mn);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = acc[i] * corr + p * vf[i];
        m = mn;
    }
    if (SPLIT) {
        float* dst = partial + ((static_cast<long long>(row) * nq + head) * n_split + split) * (kHD + 2);
        if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[2 + lane * 8 + i] = acc[i];
    } else {
        const __nv_bfloat16* gate = qkv + static_cast<long long>(row) * ld + head * 2 * kHD + kHD + lane * 8;
        __nv_bfloat16* dst = out + (static_cast<long long>(row) * nq + head) * kHD + lane * 8;
        const float inv = 1.f / l;
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = __float2bfloat16_rn(acc[i] * inv * sigmoidf_(__bfloat162float(gate[i])));
    }
}

__global__ void attn_merge_kernel(const float* __restrict__ partial, int n_split, const int* __restrict__ positions,
                                  const __nv_bfloat16* __restrict__ qkv, int ld, int nq, __nv_bfloat16* __restrict__ out) {
    const int row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    const int used = (positions[row] + kSplit) / kSplit;          // ceil((pos + 1) / split)
    const float* src = partial + (static_cast<long long>(row) * nq + head) * n_split * (kHD + 2);
    float M = -FLT_MAX;
    for (int s = 0; s < used; ++s) M = fmaxf(M, src[s * (kHD + 2)]);
    float L = 0.f, o = 0.f;
    for (int s = 0; s < used; ++s) {
        const float e = __expf(src[s * (kHD + 2)] - M);
        L += src[s * (kHD + 2) + 1] * e;
        o += src[s * (kHD + 2) + 2 + d] * e;
    }
    const float gate = __bfloat162float(qkv[static_cast<long long>(row) * ld + head * 2 * kHD + kHD + d]);
    out[(static_cast<long long>(row) * nq + head) * kHD + d] = __float2bfloat16_rn(o / L * sigmoidf_(gate));
}

const char* attn_prep(const void* qkv, int ld, int rows, int nq, int nkv, int hd, const float* q_norm, const float* k_norm,
                      const int* positions, const int* row_slot, const int* block_table, int max_pages, void* q_out,
                      void* k_pages, void* v_pages, int rot, double theta, float eps, cudaStream_t s) {
    if (hd != kHD) return "attention kernels handle head dimension 256";
    attn_prep_kernel<<<dim3(rows, nq + nkv), kHD, 0, s>>>(static_cast<const __nv_bfloat16*>(qkv), ld, nq, nkv, q_norm, k_norm, positions,
                                                         row_slot, block_table, max_pages, static_cast<__nv_bfloat16*>(q_out),
                                                         static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages),
                                                         rot, log(theta), eps);
    return cudaGetLastError() == cudaSuccess ? nullptr : "attn_prep launch failed";
}

const char* attn_rows(const void* q, const void* qkv, int ld, const void* k_pages, const void* v_pages, const int* positions,
                      const int* row_slot, const int* block_table, int max_pages, int rows, int nq, int nkv, int hd,
                      bool split, float* partial, int n_split, void* out, cudaStream_t s) {
    if (hd != kHD) return "attention kernels handle head dimension 256";
    const int group = nq / nkv;
    if (group < 1 || group > 32 || nq % nkv != 0) return "bad GQA group";
    const float scale = 1.0f / sqrtf(static_cast<float>(hd));
    const __nv_bfloat16 *qp = static_cast<const __nv_bfloat16*>(q), *qk = static_cast<const __nv_bfloat16*>(qkv);
    const __nv_bfloat16 *kp = static_cast<const __nv_bfloat16*>(k_pages), *vp = static_cast<const __nv_bfloat16*>(v_pages);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    if (split) {
        attn_rows_kernel<true><<<dim3(rows, nkv, n_split), group * 32, 0, s>>>(qp, qk, ld, kp, vp, positions, row_slot, block_table,
                                                                              max_pages, nq, nkv, scale, partial, n_split, o);
        attn_merge_kernel<<<dim3(rows, nq), kHD, 0, s>>>(partial, n_split, positions, qk, ld, nq, o);
    } else {
        attn_rows_kernel<false><<<dim3(rows, nkv, 1), group * 32, 0, s>>>(qp, qk, ld, kp, vp, positions, row_slot, block_table,
                                                                         max_pages, nq, nkv, scale, partial, 1, o);
    }
    return cudaGetLastError() == cudaSuccess ? nullptr : "attention launch failed";
}

int attn_split_keys() { return kSplit; }

}  // namespace vade
