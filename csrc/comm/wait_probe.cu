// The consumer side of a cross-GPU exchange on its own, for tests and for `doctor`: one warp waits
// (bounded) for the flag words of an exchange exactly as the fold / combine / argmax-join kernels do.
// With a flag that nothing sets, the wait runs out after `limit_ns`, the status word is raised to
// 100 + the silent rank, the kernel returns and the context stays usable: the failure path of every
// fused exchange, exercised without a failing peer.
#include <cuda_runtime.h>
#include <cstdint>
#include "../common/ptx.cuh"
#include "../common/launch.h"
#include "wait_probe.h"

namespace vade {

__global__ void __launch_bounds__(32)
wait_probe_kernel(const uint32_t* __restrict__ flags, int n, int self, uint32_t* __restrict__ status, unsigned long long limit_ns,
                  uint32_t* __restrict__ half_out) {
    chain_release();
    chain_wait();
    const uint32_t half = exchange_wait(flags, n, self, status, limit_ns);
    if (threadIdx.x == 0) *half_out = half;
}

const char* wait_probe(const uint32_t* flags, int n, int self, uint32_t* status, unsigned long long limit_ns, uint32_t* half_out,
                       cudaStream_t s) {
    if (n < 1 || n > kMaxPeers || self < 0 || self >= n) return "wait_probe: bad rank count";
    if (limit_ns > 2000000000ull) return "wait_probe: the limit is capped at two seconds";
    launch_chained(wait_probe_kernel, dim3(1), dim3(32), 0, s, flags, n, self, status, limit_ns, half_out);
    return cudaGetLastError() == cudaSuccess ? nullptr : "wait_probe launch failed";
}

}  // namespace vade
