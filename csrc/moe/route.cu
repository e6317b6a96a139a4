// MoE routing on the device: softmax -> top-k (ties to the lower expert id) -> renormalise, then the
// row layout the grouped GEMM consumes.  Router logits may arrive as several K-range partials
// (fp32 [parts][T][ld]); they are added in ascending part order before the softmax.
//
// The row layout is GLOBAL: it covers every expert of the model and is a pure function of the routing,
// so every rank of an expert-parallel group computes the same layout, runs tasks only for the experts
// it holds, and finds every other rank's outputs at the same row numbers after the exchange.
//
// Large passes (prompt tiles):
//   route_topk       one warp per token: ids, weights, shared gate
//   route_positions  one CTA per expert: the position of each (token, slot) pair inside its expert is
//                    the number of earlier pairs (token-major order) of that expert: a stable count,
//                    no atomics, identical on every rank
//   scan_tasks       one CTA: prefix sums over all experts + shared virtual experts, task table
//                    {local expert, first row, rows, first output row} for the experts this rank holds
//   scatter_rows     one thread per (token, slot): row_token[] (gather list) and slot_row[][]
// Small passes (decode / verify, T <= 16):
//   route_small      one CTA does all of it without a gather: every ACTIVE expert (ascending id) gets
//                    a 16-row block and, on the rank that holds it, one task over all T token rows (the
//                    token tile is 16 wide anyway); outputs of tokens that did not pick it are never read.
#include <cuda_runtime.h>
#include <cstdint>
#include <cfloat>
#include "../common/ptx.cuh"
#include "../common/launch.h"
#include "route.h"

namespace vade {

// top-k of one token by one warp.  PER = ceil(E / 32) logits per lane, kept in registers.
template <int PER>
__device__ __forceinline__ void warp_topk(const float* __restrict__ logits, long long part_stride, int n_parts, int E, int k,
                                          int renorm, int lane, float& sel_w, int& sel_e, float& gate_logit) {
    float v[PER];
    float mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        float a = -FLT_MAX;
        if (e < E) {
            a = logits[e];
            for (int p = 1; p < n_parts; ++p) a += logits[p * part_stride + e];
        }
        v[i] = a;
        mx = fmaxf(mx, a);
    }
    gate_logit = logits[E];
    for (int p = 1; p < n_parts; ++p) gate_logit += logits[p * part_stride + E];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? __expf(v[i] - mx) : -1.f;      // numerators; -1 marks "not a candidate"
        if (e < E) sum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float picked = 0.f;
    sel_w = 0.f;
    sel_e = -1;
    for (int r = 0; r < k; ++r) {
        float bv = -1.f;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * 32 + lane;
            if (v[i] > bv) { bv = v[i]; be = e; }       // ascending e inside the lane: ties keep the lower id
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (i * 32 + lane == be) v[i] = -1.f;
        if (lane == r) { sel_w = bv; sel_e = be; }
        picked += bv;
    }
    sel_w = renorm ? sel_w / picked : sel_w / sum;
}

template <int PER>
__global__ void route_topk_kernel(const float* __restrict__ logits, long long part_stride, int n_parts, int ld, int T, int E,
                                  int k, int renorm, int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ sg) {
    chain_release();
    chain_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    float w, gl;
    int e;
    warp_topk<PER>(logits + static_cast<long long>(t) * ld, part_stride, n_parts, E, k, renorm, lane, w, e, gl);
    if (lane < k) {
        ids[t * k + lane] = e;
        wts[t * k + lane] = w;
    }
    if (lane == 0) sg[t] = sigmoidf_(gl);
}

// pos[p] = number of pairs p' < p with ids[p'] == ids[p]; counts[e] = pairs of expert e.
__global__ void __launch_bounds__(256)
route_positions_kernel(const int* __restrict__ ids, int P, int* __restrict__ pos, int* __restrict__ counts) {
    chain_release();
    chain_wait();
    __shared__ int wsum[8];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int running = 0;
    for (int base = 0; base < P; base += 256) {
        const int p = base + threadIdx.x;
        const bool match = p < P && ids[p] == e;
        const unsigned bal = __ballot_sync(0xffffffffu, match);
        if (lane == 0) wsum[warp] = __popc(bal);
        __syncthreads();
        int woff = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) { const int c = wsum[w]; if (w < warp) woff += c; total += c; }
        if (match) pos[p] = running + woff + __popc(bal & ((1u << lane) - 1u));
        running += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = running;
}

// Inclusive scan of two integers across the block (1024 threads), fixed order.
__device__ __forceinline__ void block_scan2(int& a, int& b, int* sa, int* sb) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int ta = __shfl_up_sync(0xffffffffu, a, o), tb = __shfl_up_sync(0xffffffffu, b, o);
        if (lane >= o) { a += ta; b += tb; }
    }
    if (lane == 31) { sa[warp] = a; sb[warp] = b; }
    __syncthreads();
    if (warp == 0) {
        int wa = sa[lane], wb = sb[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int ta = __shfl_up_sync(0xffffffffu, wa, o), tb = __shfl_up_sync(0xffffffffu, wb, o);
            if (lane >= o) { wa += ta; wb += tb; }
        }
        sa[lane] = wa; sb[lane] = wb;
    }
    __syncthreads();
    if (warp > 0) { a += sa[warp - 1]; b += sb[warp - 1]; }
    __syncthreads();
}

// meta: [0] tasks of this rank, [1] rows of the global layout, [2] tasks wanted (> max_tasks: the host
// bound was wrong), [4] first and [5] end row of this rank's routed experts, [6] first shared row.
__global__ void __launch_bounds__(1024, 1)
scan_tasks_kernel(const int* __restrict__ counts, int E, int e0, int n_local, int ns, int T, int bn,
                  int* __restrict__ offsets, int4* __restrict__ tasks, int* __restrict__ meta, int max_tasks) {
    chain_release();
    chain_wait();
    __shared__ int sa[32], sb[32];
    const int ne = E + ns;
    int carry_rows = 0, carry_tasks = 0;
    for (int base = 0; base < ne; base += 1024) {
        const int e = base + threadIdx.x;
        const bool local = e < ne && ((e >= e0 && e < e0 + n_local) || e >= E);
        const int c = e < ne ? (e < E ? counts[e] : T) : 0;
        const int nt = local ? (c + bn - 1) / bn : 0;
        int ic = c, it = nt;
        block_scan2(ic, it, sa, sb);
        const int row_off = carry_rows + ic - c, task_off = carry_tasks + it - nt;
        if (e < ne) {
            offsets[e] = row_off;
            const int le = e < E ? e - e0 : n_local + (e - E);
            for (int r = 0; r < nt; ++r)
                if (task_off + r < max_tasks)
                    tasks[task_off + r] = make_int4(le, row_off + r * bn, min(bn, c - r * bn), row_off + r * bn);
            if (e == e0) meta[4] = row_off;
            if (e == e0 + n_local - 1) meta[5] = row_off + c;
            if (e == E) meta[6] = row_off;
        }
        carry_rows += sa[31];
        carry_tasks += sb[31];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        meta[0] = min(carry_tasks, max_tasks);
        meta[1] = carry_rows;
        meta[2] = carry_tasks;
        if (ns == 0) meta[6] = carry_rows;
        if (n_local == 0) { meta[4] = 0; meta[5] = 0; }
    }
}

__global__ void scatter_rows_kernel(const int* __restrict__ ids, const int* __restrict__ pos, const int* __restrict__ offsets,
                                    int T, int k, int ns, int E, int* __restrict__ row_token, int* __restrict__ slot_row) {
    chain_release();
    chain_wait();
    const int slots = k + ns;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * slots) return;
    const int t = idx / slots, j = idx % slots;
    const int row = j < k ? offsets[ids[t * k + j]] + pos[t * k + j] : offsets[E + (j - k)] + t;
    slot_row[idx] = row;
    row_token[row] = t;
}

// T <= 16 rows, n_local <= 1024 experts, one CTA of 1024 threads.
template <int PER>
__global__ void __launch_bounds__(1024, 1)
route_small_kernel(const float* __restrict__ logits, long long part_stride, int n_parts, int ld, int T, int E, int k, int renorm,
                   int e0, int n_local, int ns, int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ sg,
                   int4* __restrict__ tasks_up, int4* __restrict__ tasks_down, int* __restrict__ meta, int* __restrict__ slot_row) {
    chain_release();
    chain_wait();
    extern __shared__ float lg[];              // [T][E + 1] logits with their K-range partials added
    __shared__ int present[1024];
    __shared__ int index_of[1024];
    __shared__ int sa[32], sb[32];
    __shared__ int sel[16 * 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    present[threadIdx.x] = 0;
    // all partial loads of an element are issued together, then added in ascending part order
    for (int i = threadIdx.x; i < T * (E + 1); i += blockDim.x) {
        const int t = i / (E + 1), e = i % (E + 1);
        const float* src = logits + static_cast<long long>(t) * ld + e;
        float a;
        if (n_parts == 8) {
            float p[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) p[u] = src[u * part_stride];
            a = p[0];
#pragma unroll
            for (int u = 1; u < 8; ++u) a += p[u];
        } else {
            a = src[0];
            for (int u = 1; u < n_parts; ++u) a += src[u * part_stride];
        }
        lg[i] = a;
    }
    __syncthreads();
    if (warp < T) {
        float w, gl;
        int e;
        warp_topk<PER>(lg + warp * (E + 1), 0, 1, E, k, renorm, lane, w, e, gl);
        if (lane < k) {
            ids[warp * k + lane] = e;
            wts[warp * k + lane] = w;
            sel[warp * 32 + lane] = e;
            present[e] = 1;
        }
        if (lane == 0) sg[warp] = sigmoidf_(gl);
    }
    __syncthreads();
    // global block index of every active expert (ascending id); this rank's tasks are the active experts it holds
    const int mine = threadIdx.x < E ? present[threadIdx.x] : 0;
    const int local = (mine && static_cast<int>(threadIdx.x) >= e0 && static_cast<int>(threadIdx.x) < e0 + n_local) ? 1 : 0;
    int inc = mine, inc_local = local;
    block_scan2(inc, inc_local, sa, sb);
    const int n_active = sa[31], n_active_local = sb[31];
    const int idx = inc - mine;
    index_of[threadIdx.x] = idx;
    if (local) {
        const int li = inc_local - 1;
        tasks_up[li] = make_int4(threadIdx.x - e0, 0, T, idx * 16);
        tasks_down[li] = make_int4(threadIdx.x - e0, idx * 16, T, idx * 16);
    }
    if (threadIdx.x < ns) {
        const int li = n_active_local + threadIdx.x, blk = n_active + threadIdx.x;
        tasks_up[li] = make_int4(n_local + threadIdx.x, 0, T, blk * 16);
        tasks_down[li] = make_int4(n_local + threadIdx.x, blk * 16, T, blk * 16);
    }
    if (threadIdx.x == 0) {
        meta[0] = n_active_local + ns;
        meta[1] = (n_active + ns) * 16;
        meta[2] = n_active_local + ns;
    }
    __syncthreads();
    const int slots = k + ns;
    for (int i = threadIdx.x; i < T * slots; i += blockDim.x) {
        const int t = i / slots, j = i % slots;
        slot_row[i] = (j < k ? index_of[sel[t * 32 + j]] : n_active + (j - k)) * 16 + t;
    }
}

template <int PER>
static void route_large(const float* logits, long long part_stride, int n_parts, int ld, int T, int E, int k, bool renorm,
                        int* ids, float* wts, float* sg, cudaStream_t s) {
    const int wpb = 4;
    launch_chained(route_topk_kernel<PER>, dim3((T + wpb - 1) / wpb), dim3(wpb * 32), 0, s, logits, part_stride, n_parts, ld, T, E, k, renorm ? 1 : 0, ids, wts, sg);
}

const char* moe_route(const float* logits, long long part_stride, int n_parts, int ld, int T, int E, int k, bool renorm, int e0,
                      int n_local, int ns, int bn, int* ids, float* wts, float* sg, int* counts, int* pos, int* offsets, int* tasks,
                      int* meta, int max_tasks, int* row_token, int* slot_row, cudaStream_t s) {
    if (E > 1024 || k > 32) return "router supports up to 1024 experts and top-32";
    if (E <= 128) route_large<4>(logits, part_stride, n_parts, ld, T, E, k, renorm, ids, wts, sg, s);
    else if (E <= 512) route_large<16>(logits, part_stride, n_parts, ld, T, E, k, renorm, ids, wts, sg, s);
    else route_large<32>(logits, part_stride, n_parts, ld, T, E, k, renorm, ids, wts, sg, s);
    launch_chained(route_positions_kernel, dim3(E), dim3(256), 0, s, ids, T * k, pos, counts);
    launch_chained(scan_tasks_kernel, dim3(1), dim3(1024), 0, s, counts, E, e0, n_local, ns, T, bn, offsets, reinterpret_cast<int4*>(tasks), meta, max_tasks);
    const int total = T * (k + ns);
    launch_chained(scatter_rows_kernel, dim3((total + 255) / 256), dim3(256), 0, s, ids, pos, offsets, T, k, ns, E, row_token, slot_row);
    return cudaGetLastError() == cudaSuccess ? nullptr : "route launch failed";
}

const char* moe_route_small(const float* logits, long long part_stride, int n_parts, int ld, int T, int E, int k, bool renorm, int e0,
                            int n_local, int ns, int* ids, float* wts, float* sg, int* tasks_up, int* tasks_down, int* meta,
                            int* slot_row, cudaStream_t s) {
    if (T > 16 || n_local > 1024 || E > 1024 || k > 32 || ns > 32) return "route_small handles up to 16 rows and 1024 experts";
    int4* tu = reinterpret_cast<int4*>(tasks_up);
    int4* td = reinterpret_cast<int4*>(tasks_down);
    const int rn = renorm ? 1 : 0;
    const size_t sm = static_cast<size_t>(T) * (E + 1) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(route_small_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * 1025 * 4);
        cudaFuncSetAttribute(route_small_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * 1025 * 4);
        cudaFuncSetAttribute(route_small_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * 1025 * 4);
        configured = true;
    }
    if (E <= 128) launch_chained(route_small_kernel<4>, dim3(1), dim3(1024), sm, s, logits, part_stride, n_parts, ld, T, E, k, rn, e0, n_local, ns, ids, wts, sg, tu, td, meta, slot_row);
    else if (E <= 512) launch_chained(route_small_kernel<16>, dim3(1), dim3(1024), sm, s, logits, part_stride, n_parts, ld, T, E, k, rn, e0, n_local, ns, ids, wts, sg, tu, td, meta, slot_row);
    else launch_chained(route_small_kernel<32>, dim3(1), dim3(1024), sm, s, logits, part_stride, n_parts, ld, T, E, k, rn, e0, n_local, ns, ids, wts, sg, tu, td, meta, slot_row);
    return cudaGetLastError() == cudaSuccess ? nullptr : "route_small launch failed";
}

}  // namespace vade
