// Host interface of the output-head reductions (see head.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace vade {

// Vocabulary-parallel head: every rank's candidate table [2 halves][ranks][rows][chunks] of (value, id)
// pairs, the flag arrays of this exchange kind and this rank's sequence words (see PeerExchange).
struct HeadExchange {
    void* out[8] = {};
    uint32_t* flags[8] = {};
    uint32_t* local = nullptr;
    long long half_stride = 0;          // pairs between the two halves
    int ranks = 0;
    int self = 0;
};

// Greedy token per row: the largest logit, ties to the lowest id.  `cand` (rows * ceil(n / argmax_chunk())
// 8-byte pairs) enables the two-stage form on one GPU; `hx` the vocabulary-parallel form, where id0 is the
// first vocabulary id of this rank and every rank ends with the same winners.
void argmax_rows(const float* logits, long long ld, int rows, int n, int id0, float* best_val, long long* best_id,
                 void* cand, const HeadExchange* hx, uint32_t* status, cudaStream_t s);
int argmax_chunk();

// Compact top-k (k <= 64) of each row in canonical order (descending value, ascending id among equals).
// cand: rows * ceil(n / argmax_chunk()) * 64 eight-byte words of scratch.  Returns an error text or nullptr.
const char* topk_rows(const float* logits, long long ld, int rows, int n, int k, void* cand, float* vals, long long* ids, cudaStream_t s);

}  // namespace vade
