// Gated attention over the paged KV cache (head dimension 256, GQA).
//
//   attn_prep    per (row, head): q/k RMSNorm (1 + w), partial rotary embedding on the first `rot`
//                dims (rotate-half), q written as bf16 rows, k/v appended to the row's cache page
//   attn_rows    one CTA per (row, kv head[, key split]); one warp per query head of the group;
//                lanes own 8 of the 256 dims; online softmax over the row's visible keys.
//                Decode class: keys are cut into fixed 128-key splits (independent of the batch),
//                partials {m, l, acc} go to scratch and attn_merge joins them in split order.
//                Prefill class: one pass over all keys, output written directly.
//   output       attention * sigmoid(gate), bf16, gate read from the q projection rows
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cfloat>
#include "../common/ptx.cuh"
#include "../common/launch.h"
#include "attn.h"
#include "attn_static.h"
#include <mutex>

namespace vade {

constexpr int kHD = 256;
constexpr int kPage = 64;
constexpr int kSplit = 128;

// One projection value: a bf16 element, or the bf16 rounding of the ascending sum of fp32 K-range partials.
template <bool PARTS>
__device__ __forceinline__ float qkv_at(const void* qkv, long long row, int ld, int col, int n_parts, long long part_stride) {
    if (!PARTS) return __bfloat162float(static_cast<const __nv_bfloat16*>(qkv)[row * ld + col]);
    const float* p = static_cast<const float*>(qkv) + row * ld + col;
    if (n_parts == 4) {
        const float a0 = p[0], a1 = p[part_stride], a2 = p[2 * part_stride], a3 = p[3 * part_stride];
        return bf16_round(((a0 + a1) + a2) + a3);
    }
    float a = p[0];
    for (int i = 1; i < n_parts; ++i) a += p[i * part_stride];
    return bf16_round(a);
}

template <bool PARTS>
__global__ void attn_prep_kernel(const void* __restrict__ qkv, int ld, int n_parts, long long part_stride, int nq, int nkv,
                                 const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                 const int* __restrict__ positions, const int* __restrict__ row_slot,
                                 const int* __restrict__ block_table, int max_pages,
                                 __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ gate_out,
                                 __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages, int rot,
                                 double log_theta, float eps) {
    chain_release();
    chain_wait();
    __shared__ float xs[kHD];
    __shared__ float red[8];
    const int row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    const int pos = positions[row];
    const bool is_q = head < nq;
    const int kvh = is_q ? 0 : (head - nq);
    const int col = is_q ? head * 2 * kHD + d : nq * 2 * kHD + kvh * kHD + d;
    const float x = qkv_at<PARTS>(qkv, row, ld, col, n_parts, part_stride);
    // the other value this thread forwards: the head's output gate (query heads) or the value row (kv heads)
    const float other = qkv_at<PARTS>(qkv, row, ld, is_q ? col + kHD : col + nkv * kHD, n_parts, part_stride);
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
        gate_out[(static_cast<long long>(row) * nq + head) * kHD + d] = __float2bfloat16_rn(other);
    } else {
        const int page = block_table[static_cast<long long>(row_slot[row]) * max_pages + pos / kPage];
        const long long at = ((static_cast<long long>(page) * kPage + pos % kPage) * nkv + kvh) * kHD + d;
        k_pages[at] = __float2bfloat16_rn(y);
        v_pages[at] = __float2bfloat16_rn(other);
    }
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// One warp = one query head.  Keys are visited 32 at a time: lane j scores key j against the whole
// query (query in shared memory, key row read as 16-byte pieces), the 32 scores are merged into the
// running softmax with one butterfly, then lane d accumulates dims 8d..8d+7 of the output over
// the 32 value rows (row reads are coalesced, probabilities come by shuffle).  The visiting order
// (ascending key groups of 32, ascending key inside a group) is fixed, so a row's result depends
// only on its own keys.
template <bool SPLIT>
__global__ void __launch_bounds__(512)
attn_rows_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ gate_buf,
                 const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                 const int* __restrict__ positions, const int* __restrict__ row_slot,
                 const int* __restrict__ block_table, int max_pages, int nq, int nkv, float scale,
                 float* __restrict__ partial, int n_split, __nv_bfloat16* __restrict__ out) {
    chain_release();
    chain_wait();
    extern __shared__ float q_s[];                 // [group][256]
    const int row = blockIdx.x, kvh = blockIdx.y, split = SPLIT ? blockIdx.z : 0;
    const int group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = kvh * group + warp;
    const int len = positions[row] + 1;
    const int k0 = SPLIT ? split * kSplit : 0;
    const int k1 = SPLIT ? min(len, k0 + kSplit) : len;
    if (k0 >= len) return;
    {
        float qv[8];
        unpack8(*reinterpret_cast<const uint4*>(q + (static_cast<long long>(row) * nq + head) * kHD + lane * 8), qv);
#pragma unroll
        for (int i = 0; i < 8; ++i) q_s[warp * kHD + lane * 8 + i] = qv[i] * scale;
    }
    __syncwarp();
    const float4* qs4 = reinterpret_cast<const float4*>(q_s + warp * kHD);
    const int* table = block_table + static_cast<long long>(row_slot[row]) * max_pages;
    const long long head_off = static_cast<long long>(kvh) * kHD;
    const long long row_stride = static_cast<long long>(nkv) * kHD;
    float m = -FLT_MAX, l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int kb = k0; kb < k1; kb += 32) {
        // all 32 keys of a group sit in one 64-key page (groups start on multiples of 32)
        const long long page_base = (static_cast<long long>(table[kb / kPage]) * kPage + (kb % kPage)) * row_stride + head_off;
        const int key = kb + lane;
        const bool live = key < k1;
        float s = -FLT_MAX;
        if (live) {
            const uint4* kr = reinterpret_cast<const uint4*>(k_pages + page_base + lane * row_stride);
            float s0 = 0.f, s1 = 0.f;              // even / odd 8-column pieces, joined once at the end
#pragma unroll
            for (int c0 = 0; c0 < kHD / 8; c0 += 8) {
                uint4 kk[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) kk[u] = kr[c0 + u];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    float kf[8];
                    unpack8(kk[u], kf);
                    const float4 qa = qs4[2 * (c0 + u)], qb = qs4[2 * (c0 + u) + 1];
                    float& t = (u & 1) ? s1 : s0;
                    t += qa.x * kf[0]; t += qa.y * kf[1]; t += qa.z * kf[2]; t += qa.w * kf[3];
                    t += qb.x * kf[4]; t += qb.y * kf[5]; t += qb.z * kf[6]; t += qb.w * kf[7];
                }
            }
            s = s0 + s1;
        }
        float gm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
        const float mn = fmaxf(m, gm);
        const float corr = __expf(m - mn);
        const float p = live ? __expf(s - mn) : 0.f;
        float ps = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = l * corr + ps;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= corr;
        m = mn;
        const int nk = min(32, k1 - kb);
        const __nv_bfloat16* vr = v_pages + page_base + lane * 8;
#pragma unroll
        for (int j0 = 0; j0 < 32; j0 += 8) {
            uint4 vv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                vv[u] = (j0 + u < nk) ? *reinterpret_cast<const uint4*>(vr + (j0 + u) * row_stride) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float pj = __shfl_sync(0xffffffffu, p, j0 + u);
                float vf[8];
                unpack8(vv[u], vf);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += pj * vf[i];
            }
        }
    }
    if (SPLIT) {
        float* dst = partial + ((static_cast<long long>(row) * nq + head) * n_split + split) * (kHD + 2);
        if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[2 + lane * 8 + i] = acc[i];
    } else {
        const __nv_bfloat16* gate = gate_buf + (static_cast<long long>(row) * nq + head) * kHD + lane * 8;
        __nv_bfloat16* dst = out + (static_cast<long long>(row) * nq + head) * kHD + lane * 8;
        const float inv = 1.f / l;
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = __float2bfloat16_rn(acc[i] * inv * sigmoidf_(__bfloat162float(gate[i])));
    }
}

// Decode-class split: one CTA per (row, kv head, 128-key split).  The split's K and V rows are staged in
// shared memory with 16-byte asynchronous copies that are all in flight at once (one memory round
// trip per split), then each warp (= one query head of the group) visits the keys in the same fixed
// order as attn_rows_kernel: ascending groups of 32, lane j scoring key j, one butterfly per group.
constexpr int kKStride = kHD + 8;          // padded K row (elements): conflict-free 16-byte reads down a column of rows

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}

__global__ void __launch_bounds__(512)
attn_split_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                  const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ positions,
                  const int* __restrict__ row_slot, const int* __restrict__ block_table, int max_pages, int nq, int nkv,
                  float scale, float* __restrict__ partial, int n_split) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) uint8_t smem_attn[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_attn);                  // [128][264]
    __nv_bfloat16* Vs = Ks + kSplit * kKStride;                                       // [128][256]
    float* q_s = reinterpret_cast<float*>(Vs + kSplit * kHD);                         // [group][256]
    const int row = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = kvh * group + warp;
    const int len = positions[row] + 1;
    const int k0 = split * kSplit;
    if (k0 >= len) return;
    const int nk = min(kSplit, len - k0);
    const int* table = block_table + static_cast<long long>(row_slot[row]) * max_pages;
    const int page0 = table[k0 / kPage];
    const int page1 = (nk > kPage) ? table[k0 / kPage + 1] : page0;
    const long long row_stride = static_cast<long long>(nkv) * kHD;
    for (int idx = threadIdx.x; idx < nk * (kHD / 8); idx += blockDim.x) {
        const int key = idx >> 5, c = idx & 31;
        const long long at = (static_cast<long long>(key < kPage ? page0 : page1) * kPage + (key & (kPage - 1))) * row_stride
                           + static_cast<long long>(kvh) * kHD + c * 8;
        cp_async16(Ks + key * kKStride + c * 8, k_pages + at);
        cp_async16(Vs + key * kHD + c * 8, v_pages + at);
    }
    {
        float qv[8];
        unpack8(*reinterpret_cast<const uint4*>(q + (static_cast<long long>(row) * nq + head) * kHD + lane * 8), qv);
#pragma unroll
        for (int i = 0; i < 8; ++i) q_s[warp * kHD + lane * 8 + i] = qv[i] * scale;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const float4* qs4 = reinterpret_cast<const float4*>(q_s + warp * kHD);
    float m = -FLT_MAX, l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int kb = 0; kb < nk; kb += 32) {
        const bool live = kb + lane < nk;
        float s = -FLT_MAX;
        if (live) {
            const uint4* kr = reinterpret_cast<const uint4*>(Ks + (kb + lane) * kKStride);
            float s0 = 0.f, s1 = 0.f;              // even / odd 8-column pieces, joined once at the end
#pragma unroll 8
            for (int c = 0; c < kHD / 8; ++c) {
                float kf[8];
                unpack8(kr[c], kf);
                const float4 qa = qs4[2 * c], qb = qs4[2 * c + 1];
                float& t = (c & 1) ? s1 : s0;
                t += qa.x * kf[0]; t += qa.y * kf[1]; t += qa.z * kf[2]; t += qa.w * kf[3];
                t += qb.x * kf[4]; t += qb.y * kf[5]; t += qb.z * kf[6]; t += qb.w * kf[7];
            }
            s = s0 + s1;
        }
        float gm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
        const float mn = fmaxf(m, gm);
        const float corr = __expf(m - mn);
        const float p = live ? __expf(s - mn) : 0.f;
        float ps = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = l * corr + ps;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= corr;
        m = mn;
        const int cnt = min(32, nk - kb);
        const __nv_bfloat16* vr = Vs + kb * kHD + lane * 8;
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (j < cnt) {
                float vf[8];
                unpack8(*reinterpret_cast<const uint4*>(vr + j * kHD), vf);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += pj * vf[i];
            }
        }
    }
    float* dst = partial + ((static_cast<long long>(row) * nq + head) * n_split + split) * (kHD + 2);
    if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[2 + lane * 8 + i] = acc[i];
}

// Joins the split partials of one (row, head) in a fixed order: 1024 threads = 4 split classes
// (s mod 4) x 256 dims; the four class sums are added as (c0 + c1) + (c2 + c3).
__global__ void __launch_bounds__(1024)
attn_merge_kernel(const float* __restrict__ partial, int n_split, const int* __restrict__ positions,
                  const __nv_bfloat16* __restrict__ gate_buf, int nq, __nv_bfloat16* __restrict__ out) {
    chain_release();
    chain_wait();
    extern __shared__ float sm_merge[];            // e[n_split], then 32 reduction words, then 4 x 256 class sums
    const int row = blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, cls = tid >> 8, d = tid & 255, lane = tid & 31, warp = tid >> 5;
    const int used = (positions[row] + kSplit) / kSplit;          // ceil((pos + 1) / split)
    const float* src = partial + (static_cast<long long>(row) * nq + head) * n_split * (kHD + 2);
    float* e_s = sm_merge;
    float* red = sm_merge + n_split;
    float* cls_sum = red + 32;
    // pass 1: block max of m_s
    float mx = -FLT_MAX;
    for (int s = tid; s < used; s += 1024) { const float v = src[s * (kHD + 2)]; e_s[s] = v; mx = fmaxf(mx, v); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    float M = red[0];
#pragma unroll
    for (int i = 1; i < 32; ++i) M = fmaxf(M, red[i]);
    __syncthreads();
    // pass 2: weights e_s = exp(m_s - M) and L = sum_s l_s * e_s (thread-strided, then fixed tree)
    float lp = 0.f;
    for (int s = tid; s < used; s += 1024) { const float e = __expf(e_s[s] - M); e_s[s] = e; lp += src[s * (kHD + 2) + 1] * e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lp += __shfl_xor_sync(0xffffffffu, lp, o);
    if (lane == 0) red[warp] = lp;
    __syncthreads();
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) L += red[i];
    // pass 3: weighted sum of the accumulators, splits of class cls in ascending order
    float o = 0.f;
    int s = cls;
    for (; s + 28 < used; s += 32) {
        float a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) a[u] = src[(s + 4 * u) * (kHD + 2) + 2 + d];
#pragma unroll
        for (int u = 0; u < 8; ++u) o += a[u] * e_s[s + 4 * u];
    }
    for (; s < used; s += 4) o += src[s * (kHD + 2) + 2 + d] * e_s[s];
    cls_sum[cls * kHD + d] = o;
    __syncthreads();
    if (cls == 0) {
        const float tot = (cls_sum[d] + cls_sum[kHD + d]) + (cls_sum[2 * kHD + d] + cls_sum[3 * kHD + d]);
        const float gate = __bfloat162float(gate_buf[(static_cast<long long>(row) * nq + head) * kHD + d]);
        out[(static_cast<long long>(row) * nq + head) * kHD + d] = __float2bfloat16_rn(tot / L * sigmoidf_(gate));
    }
}

const char* attn_prep(const void* qkv, bool parts, int n_parts, long long part_stride, int ld, int rows, int nq, int nkv, int hd,
                      const float* q_norm, const float* k_norm, const int* positions, const int* row_slot, const int* block_table,
                      int max_pages, void* q_out, void* gate_out, void* k_pages, void* v_pages, int rot, double theta, float eps,
                      cudaStream_t s) {
    if (hd != kHD) return "attention kernels handle head dimension 256";
    const dim3 grid(rows, nq + nkv);
    __nv_bfloat16 *qo = static_cast<__nv_bfloat16*>(q_out), *go = static_cast<__nv_bfloat16*>(gate_out);
    __nv_bfloat16 *kp = static_cast<__nv_bfloat16*>(k_pages), *vp = static_cast<__nv_bfloat16*>(v_pages);
    if (parts)
        launch_chained(attn_prep_kernel<true>, dim3(grid), dim3(kHD), 0, s, qkv, ld, n_parts, part_stride, nq, nkv, q_norm, k_norm, positions, row_slot,
                                                    block_table, max_pages, qo, go, kp, vp, rot, log(theta), eps);
    else
        launch_chained(attn_prep_kernel<false>, dim3(grid), dim3(kHD), 0, s, qkv, ld, n_parts, part_stride, nq, nkv, q_norm, k_norm, positions, row_slot,
                                                     block_table, max_pages, qo, go, kp, vp, rot, log(theta), eps);
    return cudaGetLastError() == cudaSuccess ? nullptr : "attn_prep launch failed";
}

const char* attn_rows(const void* q, const void* gate, const void* k_pages, const void* v_pages, const int* positions,
                      const int* row_slot, const int* block_table, int max_pages, int rows, int nq, int nkv, int hd,
                      bool split, float* partial, int n_split, void* out, cudaStream_t s) {
    if (hd != kHD) return "attention kernels handle head dimension 256";
    const int group = nq / nkv;
    if (group < 1 || group > 16 || nq % nkv != 0) return "GQA group must be 1..16";
    const float scale = 1.0f / sqrtf(static_cast<float>(hd));
    const __nv_bfloat16 *qp = static_cast<const __nv_bfloat16*>(q), *gp = static_cast<const __nv_bfloat16*>(gate);
    const __nv_bfloat16 *kp = static_cast<const __nv_bfloat16*>(k_pages), *vp = static_cast<const __nv_bfloat16*>(v_pages);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    const size_t sm = group * kHD * sizeof(float);
    if (split) {
        const size_t sm_split = static_cast<size_t>(kSplit) * (kKStride + kHD) * 2 + sm;
        const size_t sm_merge = (static_cast<size_t>(n_split) + 32 + 4 * kHD) * sizeof(float);
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(attn_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
                cudaFuncSetAttribute(attn_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess)
                return "cannot raise shared memory limit";
            configured = true;
        }
        if (sm_merge > 64 * 1024) return "context too long for the split merge";
        launch_chained(attn_split_kernel, dim3(dim3(rows, nkv, n_split)), dim3(group * 32), sm_split, s, qp, kp, vp, positions, row_slot, block_table,
                                                                                max_pages, nq, nkv, scale, partial, n_split);
        launch_chained(attn_merge_kernel, dim3(dim3(rows, nq)), dim3(1024), sm_merge, s, partial, n_split, positions, gp, nq, o);
    } else {
        launch_chained(attn_rows_kernel<false>, dim3(dim3(rows, nkv, 1)), dim3(group * 32), sm, s, qp, gp, kp, vp, positions, row_slot, block_table,
                                                                          max_pages, nq, nkv, scale, partial, 1, o);
    }
    return cudaGetLastError() == cudaSuccess ? nullptr : "attention launch failed";
}

int attn_split_keys() { return kSplit; }

}  // namespace vade

// ---------------------------------------------------------------------------------------------
// Entry point that allocates nothing (see attn_static.h): the split partials go to an array that
// is part of the library image.  In host code the array's name is only a stand-in; the device
// address comes from cudaGetSymbolAddress, looked up once per device.
static __device__ __align__(256) float vade_attn_static_scratch[VADE_ATTN_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the static array on the current device (nullptr on failure).
float* static_scratch_on_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, vade_attn_static_scratch) != cudaSuccess) return nullptr;
        g_scratch_addr[dev] = static_cast<float*>(p);
    }
    return g_scratch_addr[dev];
}
}  // namespace

extern "C" __attribute__((visibility("default")))
int vade_attn_decode_static(const void* q, const void* gate, const void* k_pages, const void* v_pages, const int* positions,
                            const int* row_slot, const int* block_table, int max_pages, int rows, int nq, int nkv, int hd,
                            int max_len, void* out, cudaStream_t stream) {
    if (!q || !gate || !k_pages || !v_pages || !positions || !row_slot || !block_table || !out) return VADE_ATTN_STATIC_BAD_ARGUMENT;
    if (rows <= 0 || nq <= 0 || nkv <= 0 || max_len <= 0 || max_pages <= 0) return VADE_ATTN_STATIC_BAD_ARGUMENT;
    const int n_split = (max_len + vade::attn_split_keys() - 1) / vade::attn_split_keys();
    const unsigned long long need = 1ull * rows * nq * n_split * (hd + 2);
    if (need > VADE_ATTN_STATIC_SCRATCH_FLOATS) return VADE_ATTN_STATIC_TOO_LARGE;
    float* scratch = static_scratch_on_current_device();
    if (scratch == nullptr) return VADE_ATTN_STATIC_CUDA_ERROR;
    const char* err = vade::attn_rows(q, gate, k_pages, v_pages, positions, row_slot, block_table, max_pages, rows, nq, nkv, hd,
                                      true, scratch, n_split, out, stream);
    if (err == nullptr) return VADE_ATTN_STATIC_OK;
    return (hd != 256 || nq % nkv != 0 || nq / nkv > 16) ? VADE_ATTN_STATIC_BAD_ARGUMENT : VADE_ATTN_STATIC_CUDA_ERROR;
}

extern "C" __attribute__((visibility("default")))
unsigned long long vade_attn_static_scratch_bytes(void) {
    return 4ull * VADE_ATTN_STATIC_SCRATCH_FLOATS;
}
