// In-switch (NVLS multimem) all-reduce of a bf16 buffer in symmetric memory; see allreduce.cu.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace sharq {

constexpr int kAllReduceMaxRanks = 16;
constexpr int kAllReduceMaxCtas = 256;
constexpr int kAllReduceDefaultCtas = 64;
constexpr int kAllReducePeerMaxRanks = 4;  // the peer-copy variant keeps one 16-byte vector per rank in registers

// Clock cycles a cross-rank flag wait may take before the kernel gives up with an error code
// (0 restores the default of about two seconds).  Host-side setting for later launches.
void set_allreduce_wait_limit(long long cycles);

// bytes of flag words every rank must provide (zero-initialised once) next to its buffer
size_t allreduce_flag_bytes();

// multicast_data != nullptr: in-switch variant; else the peer-copy variant on rank_data_ptrs
// (world <= kAllReducePeerMaxRanks).
cudaError_t run_allreduce(void *multicast_data, void *const *rank_data_ptrs, void *const *rank_flag_ptrs, int rank,
                          int world, size_t bytes, int max_ctas, int *error_flag, cudaStream_t stream);

}  // namespace sharq
