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

// Routing of a small pass (T <= 16 rows, E <= 1024 experts) by ONE CTA of any width (a multiple of 32
// threads with E <= 4 * blockDim.x).  lg: shared memory for [T][E + 1] floats.
template <int PER>
__device__ void route_small_body(const float* __restrict__ logits, long long part_stride, int n_parts, int ld, int T, int E, int k,
                                 int renorm, int e0, int n_local, int ns, int* __restrict__ ids, float* __restrict__ wts,
                                 float* __restrict__ sg, int4* __restrict__ tasks_up, int4* __restrict__ tasks_down,
                                 int* __restrict__ meta, int* __restrict__ slot_row, int* __restrict__ row_token, float* lg) {
    // row_token == nullptr: every task multiplies all T rows and keeps row t of its 16-row block for token t.
    // row_token != nullptr (compact): a task multiplies only the tokens routed to its expert; block row p holds the
    // p-th such token in ascending token order and row_token[block * 16 + p] names it.
    __shared__ unsigned int tokmask[1024];
    __shared__ unsigned char present[1024];
    __shared__ short index_of[1024];
    __shared__ int sa[32], sb[32];
    __shared__ int sel[16 * 32];
    const int nthr = blockDim.x, nwarps = nthr >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 1024; i += nthr) { present[i] = 0; tokmask[i] = 0u; }
    // all partial loads of an element are issued together, then added in ascending part order
    for (int i = threadIdx.x; i < T * (E + 1); i += nthr) {
        const int t = i / (E + 1), e = i % (E + 1);
        const float* src = logits + static_cast<long long>(t) * ld + e;
        float a;
        if (n_parts == 8) {
            float p[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) p[u] = __ldcg(src + u * part_stride);
            a = p[0];
#pragma unroll
            for (int u = 1; u < 8; ++u) a += p[u];
        } else {
            a = __ldcg(src);
            for (int u = 1; u < n_parts; ++u) a += __ldcg(src + u * part_stride);
        }
        lg[i] = a;
    }
    __syncthreads();
    for (int row = warp; row < T; row += nwarps) {
        float w, gl;
        int e;
        warp_topk<PER>(lg + row * (E + 1), 0, 1, E, k, renorm, lane, w, e, gl);
        if (lane < k) {
            ids[row * k + lane] = e;
            wts[row * k + lane] = w;
            sel[row * 32 + lane] = e;
            present[e] = 1;
            atomicOr(&tokmask[e], 1u << row);               // a set of token rows: the order of arrival does not matter
        }
        if (lane == 0) sg[row] = sigmoidf_(gl);
    }
    __syncthreads();
    // global block index of every active expert (ascending id); this rank's tasks are the active experts it holds.
    // Thread i owns the experts [i * ept, (i + 1) * ept).
    const int ept = (E + nthr - 1) / nthr;
    const int first = threadIdx.x * ept;
    int cnt = 0, cnt_local = 0;
    for (int j = 0; j < ept; ++j) {
        const int e = first + j;
        if (e < E && present[e]) {
            ++cnt;
            if (e >= e0 && e < e0 + n_local) ++cnt_local;
        }
    }
    int inc = cnt, inc_local = cnt_local;
    block_scan2(inc, inc_local, sa, sb);
    const int n_active = sa[nwarps - 1], n_active_local = sb[nwarps - 1];
    // task order: the shared experts first (they hold every row of the pass, the longest tasks, so they start with
    // the first wave of CTAs instead of forming the tail), then this rank's active routed experts by ascending id
    int idx = inc - cnt, li = ns + inc_local - cnt_local;
    for (int j = 0; j < ept; ++j) {
        const int e = first + j;
        if (e < E && present[e]) {
            index_of[e] = static_cast<short>(idx);
            if (e >= e0 && e < e0 + n_local) {
                if (row_token == nullptr) {
                    tasks_up[li] = make_int4(e - e0, 0, T, idx * 16);
                    tasks_down[li] = make_int4(e - e0, idx * 16, T, idx * 16);
                } else {
                    unsigned int m = tokmask[e];
                    const int n = __popc(m);
                    tasks_up[li] = make_int4(e - e0, idx * 16, n, idx * 16);
                    tasks_down[li] = make_int4(e - e0, idx * 16, n, idx * 16);
                    for (int p = 0; m != 0u; ++p, m &= m - 1u) row_token[idx * 16 + p] = __ffs(m) - 1;
                }
                ++li;
            }
            ++idx;
        }
    }
    for (int i = threadIdx.x; i < ns; i += nthr) {
        const int lt = i, blk = n_active + i;
        tasks_up[lt] = make_int4(n_local + i, row_token == nullptr ? 0 : blk * 16, T, blk * 16);
        tasks_down[lt] = make_int4(n_local + i, blk * 16, T, blk * 16);
        if (row_token != nullptr)
            for (int t = 0; t < T; ++t) row_token[blk * 16 + t] = t;
    }
    if (threadIdx.x < 8) {
        int v = 0;
        if (threadIdx.x == 0 || threadIdx.x == 2) v = n_active_local + ns;
        if (threadIdx.x == 1) v = (n_active + ns) * 16;
        meta[threadIdx.x] = v;
    }
    __syncthreads();
    const int slots = k + ns;
    for (int i = threadIdx.x; i < T * slots; i += nthr) {
        const int t = i / slots, j = i % slots;
        int row = (j < k ? index_of[sel[t * 32 + j]] : n_active + (j - k)) * 16 + t;
        if (row_token != nullptr && j < k) {
            const int e = sel[t * 32 + j];
            row = index_of[e] * 16 + __popc(tokmask[e] & ((1u << t) - 1u));
        }
        slot_row[i] = row;
    }
}

template <int PER>
__global__ void __launch_bounds__(1024, 1)
route_small_kernel(const float* __restrict__ logits, long long part_stride, int n_parts, int ld, int T, int E, int k, int renorm,
                   int e0, int n_local, int ns, int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ sg,
                   int4* __restrict__ tasks_up, int4* __restrict__ tasks_down, int* __restrict__ meta, int* __restrict__ slot_row,
                   int* __restrict__ row_token) {
    chain_release();
    chain_wait();
    extern __shared__ float lg[];              // [T][E + 1] logits with their K-range partials added
    route_small_body<PER>(logits, part_stride, n_parts, ld, T, E, k, renorm, e0, n_local, ns, ids, wts, sg, tasks_up, tasks_down,
                          meta, slot_row, row_token, lg);
}

// ------------------------------------------------------------------ decode-class router
// Router logits of a few token rows as K-range partials by warp-level mma over the plain bf16 router
// rows (a stream over 2 MB: no tile reuse, so no shared-memory staging of the weights), and, for small
// passes, the routing itself by the last CTA to finish (a ticket in global memory).
//   warp = 16 router rows x one of 8 K ranges; thread (g, t) loads 16 bytes (8 columns) of rows g and
//   g + 8 per 32-column chunk, all chunks up front; the 16 K slots of an mma are a fixed permutation of
//   16 columns, applied to the token operand as well (see gemm/rows_mma.cu).
// grid = (row tiles / 8, 8 ranges, groups of NT * 8 token rows), 256 threads.
constexpr int kRouterThreads = 256;
constexpr int kRouterChunks = 8;               // 32-column chunks kept in flight per thread

struct RouterFuse {                            // routing by the last CTA (T <= 16); ticket == nullptr: logits only
    unsigned int* ticket;
    int E, k, renorm, e0, n_local, ns;
    int* ids; float* wts; float* sg; int4* tasks_up; int4* tasks_down; int* meta; int* slot_row; int* row_token;
};

template <int NT, int PER>
__global__ void __launch_bounds__(kRouterThreads)
router_rows_kernel(const __nv_bfloat16* __restrict__ w, int n_rows, int K, const __nv_bfloat16* __restrict__ x, int ldx, int T,
                   float* __restrict__ logits, long long part_stride, int ld, const RouterFuse f) {
    chain_release();
    extern __shared__ __align__(16) uint8_t dyn[];          // token columns of this range, later the routing's logits
    __shared__ int is_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x * (kRouterThreads / 32) + warp;
    const int range = blockIdx.y;
    const int rc = K / 8;                                    // columns per range
    const int col0 = range * rc;
    const int tok0 = blockIdx.z * (NT * 8);
    const int ntok = min(NT * 8, T - tok0);
    const int xstride = rc * 2 + 64;                         // bytes; odd multiple of 64 -> conflict-free 16-byte reads
    const int r0 = tile * 16 + g, r1 = r0 + 8;
    const bool ok0 = r0 < n_rows, ok1 = r1 < n_rows;
    const uint4* p0 = reinterpret_cast<const uint4*>(w + static_cast<long long>(ok0 ? r0 : 0) * K + col0) + t;
    const uint4* p1 = reinterpret_cast<const uint4*>(w + static_cast<long long>(ok1 ? r1 : 0) * K + col0) + t;
    const int chunks = rc / 32;

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    bool staged = false;
    for (int c0 = 0; c0 < chunks; c0 += kRouterChunks) {
        uint4 u0[kRouterChunks], u1[kRouterChunks];
#pragma unroll
        for (int i = 0; i < kRouterChunks; ++i) {
            u0[i] = u1[i] = make_uint4(0u, 0u, 0u, 0u);
            if (c0 + i < chunks) {
                if (ok0) u0[i] = __ldg(p0 + (c0 + i) * 4);
                if (ok1) u1[i] = __ldg(p1 + (c0 + i) * 4);
            }
        }
        if (!staged) {                                       // the router rows are immutable: only the token rows wait
            chain_wait();
            const int pieces = rc / 8;
            for (int p = threadIdx.x; p < NT * 8 * pieces; p += kRouterThreads) {
                const int j = p / pieces, q = p - j * pieces;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (j < ntok) v = *reinterpret_cast<const uint4*>(x + static_cast<long long>(tok0 + j) * ldx + col0 + q * 8);
                *reinterpret_cast<uint4*>(dyn + j * xstride + q * 16) = v;
            }
            __syncthreads();
            staged = true;
        }
#pragma unroll
        for (int i = 0; i < kRouterChunks; ++i) {
            if (c0 + i < chunks) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint4 bx = *reinterpret_cast<const uint4*>(dyn + (n * 8 + g) * xstride + (c0 + i) * 64 + t * 16);
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[n][0]), "+f"(acc[n][1]), "+f"(acc[n][2]), "+f"(acc[n][3])
                                 : "r"(u0[i].x), "r"(u1[i].x), "r"(u0[i].y), "r"(u1[i].y), "r"(bx.x), "r"(bx.y));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[n][0]), "+f"(acc[n][1]), "+f"(acc[n][2]), "+f"(acc[n][3])
                                 : "r"(u0[i].z), "r"(u1[i].z), "r"(u0[i].w), "r"(u1[i].w), "r"(bx.z), "r"(bx.w));
                }
            }
        }
    }
    float* out = logits + range * part_stride;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int j = n * 8 + 2 * t + e;
            if (j < ntok) {
                if (ok0) out[static_cast<long long>(tok0 + j) * ld + r0] = acc[n][e];
                if (ok1) out[static_cast<long long>(tok0 + j) * ld + r1] = acc[n][2 + e];
            }
        }
    }
    if (f.ticket == nullptr) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(f.ticket, 1u) == gridDim.x * gridDim.y - 1 ? 1 : 0;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x == 0) *f.ticket = 0u;
    route_small_body<PER>(logits, part_stride, 8, ld, T, f.E, f.k, f.renorm, f.e0, f.n_local, f.ns, f.ids, f.wts, f.sg, f.tasks_up,
                          f.tasks_down, f.meta, f.slot_row, f.row_token, reinterpret_cast<float*>(dyn));
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
                            int* slot_row, int* row_token, cudaStream_t s) {
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
    if (E <= 128) launch_chained(route_small_kernel<4>, dim3(1), dim3(1024), sm, s, logits, part_stride, n_parts, ld, T, E, k, rn, e0, n_local, ns, ids, wts, sg, tu, td, meta, slot_row, row_token);
    else if (E <= 512) launch_chained(route_small_kernel<16>, dim3(1), dim3(1024), sm, s, logits, part_stride, n_parts, ld, T, E, k, rn, e0, n_local, ns, ids, wts, sg, tu, td, meta, slot_row, row_token);
    else launch_chained(route_small_kernel<32>, dim3(1), dim3(1024), sm, s, logits, part_stride, n_parts, ld, T, E, k, rn, e0, n_local, ns, ids, wts, sg, tu, td, meta, slot_row, row_token);
    return cudaGetLastError() == cudaSuccess ? nullptr : "route_small launch failed";
}

template <int NT>
static const char* launch_router(const void* w, int n_rows, int K, const void* x, int ldx, int T, float* logits, long long part_stride,
                                 int ld, const RouterFuse& f, int E, cudaStream_t s) {
    const int tiles = (n_rows + 15) / 16;
    const dim3 grid((tiles + kRouterThreads / 32 - 1) / (kRouterThreads / 32), 8, (T + NT * 8 - 1) / (NT * 8));
    const int stage = NT * 8 * (K / 8 * 2 + 64);
    const int route = f.ticket != nullptr ? T * (E + 1) * static_cast<int>(sizeof(float)) : 0;
    const int sm = stage > route ? stage : route;
    auto k4 = router_rows_kernel<NT, 4>;
    auto k16 = router_rows_kernel<NT, 16>;
    auto k32 = router_rows_kernel<NT, 32>;
    auto kern = E <= 128 ? k4 : E <= 512 ? k16 : k32;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(k4, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        cudaFuncSetAttribute(k16, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        cudaFuncSetAttribute(k32, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        configured = true;
    }
    if (sm > 96 * 1024) return "router pass does not fit in shared memory";
    launch_chained(kern, grid, dim3(kRouterThreads), sm, s, static_cast<const __nv_bfloat16*>(w), n_rows, K,
                   static_cast<const __nv_bfloat16*>(x), ldx, T, logits, part_stride, ld, f);
    return cudaGetLastError() == cudaSuccess ? nullptr : "router launch failed";
}

const char* router_rows(const void* w, int n_rows, int K, const void* x, int ldx, int T, float* logits, long long part_stride, int ld,
                        unsigned int* ticket, int E, int k, bool renorm, int e0, int n_local, int ns, int* ids, float* wts, float* sg,
                        int* tasks_up, int* tasks_down, int* meta, int* slot_row, int* row_token, cudaStream_t s) {
    if (K % 512 != 0) return "router columns must be a multiple of 512";
    if ((reinterpret_cast<uintptr_t>(w) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0 || ldx % 8 != 0)
        return "router operands must be 16-byte aligned";
    RouterFuse f{};
    if (ticket != nullptr) {
        if (T > 16 || E > 1024 || k > 32 || ns > 32 || n_rows != E + 1) return "fused routing handles up to 16 rows and 1024 experts";
        f.ticket = ticket; f.E = E; f.k = k; f.renorm = renorm ? 1 : 0; f.e0 = e0; f.n_local = n_local; f.ns = ns;
        f.ids = ids; f.wts = wts; f.sg = sg; f.tasks_up = reinterpret_cast<int4*>(tasks_up); f.tasks_down = reinterpret_cast<int4*>(tasks_down);
        f.meta = meta; f.slot_row = slot_row; f.row_token = row_token;
    }
    if (T <= 8) return launch_router<1>(w, n_rows, K, x, ldx, T, logits, part_stride, ld, f, E, s);
    if (T <= 16) return launch_router<2>(w, n_rows, K, x, ldx, T, logits, part_stride, ld, f, E, s);
    if (T <= 32) return launch_router<4>(w, n_rows, K, x, ldx, T, logits, part_stride, ld, f, E, s);
    return launch_router<8>(w, n_rows, K, x, ldx, T, logits, part_stride, ld, f, E, s);
}

}  // namespace vade
