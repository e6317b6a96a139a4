// MoE routing on the device: softmax -> top-k (ties to the lower expert id) -> renormalise, then the
// expert-sorted row layout the grouped GEMM consumes.
//
//   route_count   one warp per token: fp32 softmax numerators, k selection rounds, weights; each
//                 selected pair of a LOCAL expert takes a position inside its expert with an
//                 integer atomic (positions only decide which row of the gathered matrix a pair
//                 occupies, never any arithmetic)
//   scan_tasks    one CTA: prefix sums over local + shared experts, task table for the grouped
//                 GEMM ({expert, first row, rows}), totals; re-zeroes the counters for the next call
//   scatter_rows  one thread per (token, slot): row_token[] (gather list) and slot_row[][] (where
//                 the combine finds each slot's output; -1 when another rank owns the expert)
#include <cuda_runtime.h>
#include <cstdint>
#include <cfloat>
#include "../common/ptx.cuh"
#include "route.h"

namespace vade {

constexpr int kMaxPerLane = 32;      // up to 1024 experts

__global__ void route_count_kernel(const float* __restrict__ logits, int ld, int T, int E, int k, int renorm,
                                   int e0, int n_local, int* __restrict__ ids, float* __restrict__ wts,
                                   float* __restrict__ sg, int* __restrict__ counts, int* __restrict__ pos) {
    const int warps_per_block = blockDim.x >> 5;
    const int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    const float* row = logits + static_cast<long long>(t) * ld;
    const int per = (E + 31) / 32;
    float v[kMaxPerLane];
    float mx = -FLT_MAX;
#pragma unroll 4
    for (int i = 0; i < per; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? row[e] : -FLT_MAX;
        mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int i = 0; i < per; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? __expf(v[i] - mx) : -1.f;      // numerators; -1 marks "not a candidate"
        if (e < E) sum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float sel_w = 0.f;
    int sel_e = -1;
    float picked = 0.f;
    for (int r = 0; r < k; ++r) {
        float bv = -1.f;
        int be = 0x7fffffff;
        for (int i = 0; i < per; ++i) {
            const int e = i * 32 + lane;
            if (v[i] > bv) { bv = v[i]; be = e; }       // ascending e inside the lane: ties keep the lower id
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        if ((be & 31) == lane) v[be >> 5] = -1.f;
        if (lane == r) { sel_w = bv; sel_e = be; }
        picked += bv;
    }
    if (lane < k) {
        const float w = renorm ? sel_w / picked : sel_w / sum;
        ids[t * k + lane] = sel_e;
        wts[t * k + lane] = w;
        const int le = sel_e - e0;
        pos[t * k + lane] = (le >= 0 && le < n_local) ? atomicAdd(&counts[le], 1) : -1;
    }
    if (lane == 0) sg[t] = sigmoidf_(row[E]);
}

__global__ void scan_tasks_kernel(int* __restrict__ counts, int n_local, int ns, int T, int bn,
                                  int* __restrict__ offsets, int4* __restrict__ tasks, int* __restrict__ meta, int max_tasks) {
    // meta[0] = number of tasks, meta[1] = number of rows
    if (threadIdx.x != 0) return;
    int row = 0, nt = 0;
    const int ne = n_local + ns;
    for (int e = 0; e < ne; ++e) {
        const int c = e < n_local ? counts[e] : T;
        offsets[e] = row;
        for (int r = 0; r < c; r += bn) {
            if (nt < max_tasks) tasks[nt] = make_int4(e, row + r, min(bn, c - r), 0);
            ++nt;
        }
        row += c;
        if (e < n_local) counts[e] = 0;
    }
    meta[0] = min(nt, max_tasks);
    meta[1] = row;
    meta[2] = nt;          // > max_tasks would mean the host bound was wrong; the host checks in debug runs
}

__global__ void scatter_rows_kernel(const int* __restrict__ ids, const int* __restrict__ pos, const int* __restrict__ offsets,
                                    int T, int k, int ns, int e0, int n_local, int* __restrict__ row_token, int* __restrict__ slot_row) {
    const int slots = k + ns;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * slots) return;
    const int t = idx / slots, j = idx % slots;
    int row = -1;
    if (j < k) {
        const int p = pos[t * k + j];
        if (p >= 0) row = offsets[ids[t * k + j] - e0] + p;
    } else {
        row = offsets[n_local + (j - k)] + t;
    }
    slot_row[idx] = row;
    if (row >= 0) row_token[row] = t;
}

void moe_route(const float* logits, int ld, int T, int E, int k, bool renorm, int e0, int n_local, int ns, int bn,
               int* ids, float* wts, float* sg, int* counts, int* pos, int* offsets, int* tasks, int* meta, int max_tasks,
               int* row_token, int* slot_row, cudaStream_t s) {
    const int wpb = 4;
    route_count_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, s>>>(logits, ld, T, E, k, renorm ? 1 : 0, e0, n_local, ids, wts, sg, counts, pos);
    scan_tasks_kernel<<<1, 32, 0, s>>>(counts, n_local, ns, T, bn, offsets, reinterpret_cast<int4*>(tasks), meta, max_tasks);
    const int total = T * (k + ns);
    scatter_rows_kernel<<<(total + 255) / 256, 256, 0, s>>>(ids, pos, offsets, T, k, ns, e0, n_local, row_token, slot_row);
}

}  // namespace vade
