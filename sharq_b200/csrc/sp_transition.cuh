// Host launcher of the tensor-parallel layer transition kernel (sp_transition.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace sharq {

constexpr int kSpMaxRanks = 16;

struct SpTransitionArgs {
  const void *partial_blocks = nullptr;     // this GPU's collection buffer [world][m / world, k] bf16 (null: none)
  const void *residual_in = nullptr;        // this GPU's rows of the residual stream [m / world, k] bf16 (null: none)
  void *residual_out = nullptr;             // this GPU's rows of the new residual stream
  const void *gamma = nullptr;              // RMSNorm weight [k] bf16
  float eps = 0.0f;
  void *workspace = nullptr;                // sp_transition_workspace_bytes(m / world) bytes on this GPU
  float *scale_out = nullptr;               // one float on this GPU
  // this GPU's copy of the prepared activation of all m rows, inside a symmetric allocation ...
  void *a_comp = nullptr, *e = nullptr, *sfa_sparse = nullptr, *q_res = nullptr, *sf_res = nullptr;
  long long multicast_delta = 0;            // ... whose multicast address is the local address plus this
  void *const *rank_state_ptrs = nullptr;   // [world] every GPU's state words as mapped on this GPU
  int rank = 0, world = 1;
  int m = 0, k = 0;
  int *error_flag = nullptr;
};

// bytes of state every GPU provides in symmetric memory, zero-initialised once
size_t sp_transition_state_bytes();
// bytes of per-call scratch (per-row inv_rms of this GPU's rows)
size_t sp_transition_workspace_bytes(int rows);

// Clock cycles a wait of the kernel may take (0 restores the default of about ten seconds).
void set_sp_transition_wait_limit(long long cycles);

cudaError_t run_sp_transition(const SpTransitionArgs &args, cudaStream_t stream);

}  // namespace sharq
