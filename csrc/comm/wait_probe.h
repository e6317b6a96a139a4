// Host interface of the bounded-wait probe (see wait_probe.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace vade {

// flags: the n flag words of one exchange on this rank; status: one word, raised on a timeout.
const char* wait_probe(const uint32_t* flags, int n, int self, uint32_t* status, unsigned long long limit_ns, uint32_t* half_out,
                       cudaStream_t s);

}  // namespace vade
