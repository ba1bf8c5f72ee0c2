// In-switch (NVLS multimem) all-reduce of a bf16 buffer in symmetric memory; see allreduce.cu.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace sharq {

constexpr int kAllReduceMaxRanks = 16;
constexpr int kAllReduceMaxCtas = 256;
constexpr int kAllReduceDefaultCtas = 64;

// bytes of flag words every rank must provide (zero-initialised once) next to its buffer
size_t allreduce_flag_bytes();

cudaError_t run_allreduce_multimem(void *multicast_data, void *const *rank_flag_ptrs, int rank, int world, size_t bytes,
                                   int max_ctas, int *error_flag, cudaStream_t stream);

}  // namespace sharq
