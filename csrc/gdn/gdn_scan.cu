// Gated DeltaNet token mixer, one launch per layer: depthwise causal conv (kernel 4) + SiLU,
// l2-normalised q/k, gates, the delta-rule recurrence with the 128 x 128 fp32 state of each value
// head held in registers (one state column per thread), and the gated RMSNorm of the output.
//
//   per row:  S *= e^g;  delta = (v - S^T k) * beta;  S += k (x) delta;  o = S^T q
//             out = RMSNorm(o) * w * sigmoid(z)
//
// grid = (local key heads, sequences); block = (value heads per key head) x 128 threads.  A block
// walks the rows of its sequence in order (one row for a decode step, several for a verify pass,
// a whole tile for a prompt), so a sequence's bits do not depend on what else is in the batch.
// Sums over the 128 state rows are one ascending chain; sums across a head's 128 threads are a
// fixed butterfly + warp order.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "../common/ptx.cuh"
#include "gdn_scan.h"

namespace vade {

constexpr int kD = 128;      // key and value head dimension handled by this kernel

__device__ __forceinline__ float group_sum(float v, float* red, int g, int wg, int lane) {
    // sum over the 128 threads (4 warps) of value-head group g; all threads of the block call this
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[g * 4 + wg] = v;
    __syncthreads();
    return ((red[g * 4 + 0] + red[g * 4 + 1]) + (red[g * 4 + 2] + red[g * 4 + 3]));
}

// One projection value: a bf16 element, or the bf16 rounding of the ascending sum of fp32 K-range partials.
template <bool PARTS>
__device__ __forceinline__ float proj_at(const void* proj, long long row, int ld, int col, int n_parts, long long part_stride) {
    if (!PARTS) return __bfloat162float(static_cast<const __nv_bfloat16*>(proj)[row * ld + col]);
    const float* p = static_cast<const float*>(proj) + row * ld + col;
    if (n_parts == 4) {                         // the loads are independent; only the adds are ordered
        const float a0 = p[0], a1 = p[part_stride], a2 = p[2 * part_stride], a3 = p[3 * part_stride];
        return bf16_round(((a0 + a1) + a2) + a3);
    }
    float a = p[0];
    for (int i = 1; i < n_parts; ++i) a += p[i * part_stride];
    return bf16_round(a);
}

template <int REP, bool PARTS>
__global__ void __launch_bounds__(REP * 128, 1)
gdn_scan_kernel(const void* __restrict__ proj, int ld, int n_parts, long long part_stride, const float* __restrict__ conv_w,
                float* __restrict__ hist, float* __restrict__ state, const float* __restrict__ a_log,
                const float* __restrict__ dt_bias, const float* __restrict__ norm_w,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                __nv_bfloat16* __restrict__ out, int kh, int vh, float eps, int gate_silu) {
    extern __shared__ float sm[];
    constexpr int rep = REP;
    float* q_s = sm;                         // [rep][128]
    float* k_s = q_s + rep * kD;             // [rep][128]
    float* red = k_s + rep * kD;             // [rep][4] x 2
    const int khead = blockIdx.x;
    const int b = blockIdx.y;
    const int g = threadIdx.x >> 7;
    const int j = threadIdx.x & 127;
    const int wg = (threadIdx.x >> 5) & 3;
    const int lane = threadIdx.x & 31;
    const int vhead = khead * rep + g;
    const int slot = seq_slot[b];
    const int r0 = seq_start[b], r1 = seq_start[b + 1];
    const int C = 2 * kh * kD + vh * kD;
    const int cq = khead * kD + j, ck = kh * kD + khead * kD + j, cv = 2 * kh * kD + vhead * kD + j;
    const int oz = C + vhead * kD + j, ob = C + vh * kD + vhead, oa = C + vh * kD + vh + vhead;

    float wq[4], wk[4], wv[4], hq[3], hk[3], hv[3];
#pragma unroll
    for (int i = 0; i < 4; ++i) { wq[i] = conv_w[cq * 4 + i]; wk[i] = conv_w[ck * 4 + i]; wv[i] = conv_w[cv * 4 + i]; }
    float* hbase = hist + static_cast<long long>(slot) * 3 * C;
#pragma unroll
    for (int i = 0; i < 3; ++i) { hq[i] = hbase[i * C + cq]; hk[i] = hbase[i * C + ck]; hv[i] = hbase[i * C + cv]; }

    float S[kD];
    float* sp = state + ((static_cast<long long>(slot) * vh + vhead) * kD) * kD + j;
#pragma unroll
    for (int i = 0; i < kD; ++i) S[i] = sp[i * kD];

    const float neg_a = -__expf(a_log[vhead]);
    const float dtb = dt_bias[vhead];
    const float nw = norm_w[j];
    const float qscale = rsqrtf(static_cast<float>(kD));

    for (int r = r0; r < r1; ++r) {
        const float xq = proj_at<PARTS>(proj, r, ld, cq, n_parts, part_stride);
        const float xk = proj_at<PARTS>(proj, r, ld, ck, n_parts, part_stride);
        const float xv = proj_at<PARTS>(proj, r, ld, cv, n_parts, part_stride);
        const float xb = proj_at<PARTS>(proj, r, ld, ob, n_parts, part_stride);
        const float xa = proj_at<PARTS>(proj, r, ld, oa, n_parts, part_stride);
        const float z = proj_at<PARTS>(proj, r, ld, oz, n_parts, part_stride);
        float aq = 0.f, ak = 0.f, av = 0.f;
        aq += hq[0] * wq[0]; aq += hq[1] * wq[1]; aq += hq[2] * wq[2]; aq += xq * wq[3];
        ak += hk[0] * wk[0]; ak += hk[1] * wk[1]; ak += hk[2] * wk[2]; ak += xk * wk[3];
        av += hv[0] * wv[0]; av += hv[1] * wv[1]; av += hv[2] * wv[2]; av += xv * wv[3];
        hq[0] = hq[1]; hq[1] = hq[2]; hq[2] = xq;
        hk[0] = hk[1]; hk[1] = hk[2]; hk[2] = xk;
        hv[0] = hv[1]; hv[1] = hv[2]; hv[2] = xv;
        const float q = siluf_(aq), k = siluf_(ak), v = siluf_(av);
        const float ssq = group_sum(q * q, red, g, wg, lane);
        const float ssk = group_sum(k * k, red + rep * 4, g, wg, lane);
        q_s[g * kD + j] = q * rsqrtf(ssq + 1e-6f) * qscale;
        k_s[g * kD + j] = k * rsqrtf(ssk + 1e-6f);
        const float beta = sigmoidf_(xb);
        const float ax = xa + dtb;
        const float sp_ = ax > 20.f ? ax : log1pf(__expf(ax));
        const float decay = __expf(neg_a * sp_);
        __syncthreads();
        const float* qv = q_s + g * kD;
        const float* kv = k_s + g * kD;
        float mem = 0.f;
#pragma unroll
        for (int i = 0; i < kD; ++i) { S[i] *= decay; mem += S[i] * kv[i]; }
        const float delta = (v - mem) * beta;
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < kD; ++i) { S[i] += kv[i] * delta; o += S[i] * qv[i]; }
        const float sso = group_sum(o * o, red, g, wg, lane);
        const float gz = gate_silu ? siluf_(z) : sigmoidf_(z);
        out[static_cast<long long>(r) * (vh * kD) + vhead * kD + j] = __float2bfloat16_rn(o * rsqrtf(sso / kD + eps) * nw * gz);
    }
#pragma unroll
    for (int i = 0; i < kD; ++i) sp[i * kD] = S[i];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        hbase[i * C + cv] = hv[i];
        if (g == 0) { hbase[i * C + cq] = hq[i]; hbase[i * C + ck] = hk[i]; }
    }
}

const char* gdn_scan(const void* proj, bool parts, int n_parts, long long part_stride, int ld, const float* conv_w, float* hist,
                     float* state, const float* a_log, const float* dt_bias, const float* norm_w, const int* seq_slot,
                     const int* seq_start, int n_seq, void* out, int kh, int vh, int kd, int vd, float eps, bool gate_silu,
                     cudaStream_t s) {
    if (kd != kD || vd != kD) return "gdn_scan handles head dimension 128";
    if (vh % kh != 0 || vh / kh > 3) return "value heads per key head must be 1, 2 or 3";
    const int rep = vh / kh;
    const size_t smem = (2 * rep * kD + 2 * rep * 4) * sizeof(float);
    const dim3 grid(kh, n_seq);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    const int gs = gate_silu ? 1 : 0;
#define VADE_GDN(REP, PARTS) gdn_scan_kernel<REP, PARTS><<<grid, REP * 128, smem, s>>>(proj, ld, n_parts, part_stride, conv_w, hist, \
        state, a_log, dt_bias, norm_w, seq_slot, seq_start, o, kh, vh, eps, gs)
    if (parts) {
        if (rep == 1) VADE_GDN(1, true); else if (rep == 2) VADE_GDN(2, true); else VADE_GDN(3, true);
    } else {
        if (rep == 1) VADE_GDN(1, false); else if (rep == 2) VADE_GDN(2, false); else VADE_GDN(3, false);
    }
#undef VADE_GDN
    return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_scan launch failed";
}

}  // namespace vade
