// Host launcher of the block-scaled FP4 GEMMs (gemm.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace sharq {

constexpr int kGemmMaxPeers = 16;

struct GemmArgs {
  // Sparse main path operand (all three null => dense-only GEMM).
  const void *a_comp = nullptr;      // [m, k/4] compressed e2m1 pairs
  const void *e = nullptr;           // metadata, [k/256][ceil128(m)][16 B]
  const void *sfa_sparse = nullptr;  // UE4M3 per 32 along K, blocked layout
  // Dense operand (null => sparse-only GEMM).
  const void *a_dense = nullptr;    // [m, k/2] e2m1
  const void *sfa_dense = nullptr;  // UE4M3 per 16 along K, blocked layout
  // Weight: one payload, two views of its scales.
  const void *b = nullptr;           // [n, k/2] e2m1
  const void *sfb_sparse = nullptr;  // per 32 (used by the sparse pass)
  const void *sfb_dense = nullptr;   // per 16 (used by the dense pass)
  // Epilogue: d = bf16(alpha * acc + beta * c_in), then (+ bias) in bf16.
  const void *c_in = nullptr;  // [m, n] bf16, optional
  const void *bias = nullptr;  // [n] bf16, optional
  void *d = nullptr;           // [m, n] bf16
  const float *alpha_ptr = nullptr;  // device scalar; when non-null the factor is alpha * (*alpha_ptr)
  float alpha = 1.0f;
  float beta = 0.0f;
  int m = 0, n = 0, k = 0;
  int tile_n = 0;             // 0 = choose, else 128 or 256
  int *error_flag = nullptr;  // device int, set non-zero when a bounded wait ran out
  // Optional scratch of at least m * n * 4 bytes: lets a GEMM with M <= 128 split K over the SMs
  // (fp32 partial sums are accumulated there, a second kernel applies the epilogue).
  void *workspace = nullptr;
  size_t workspace_bytes = 0;
  // Scatter mode (scatter_world > 1, `d` unused): the m / scatter_world rows owned by GPU o are stored into
  // d_peer[o] (GPU o's collection buffer as mapped on this GPU, [scatter_world][m / scatter_world][n] bf16) at
  // block scatter_rank.  Needs m % (128 * scatter_world) == 0 and n % 8 == 0.
  void *d_peer[kGemmMaxPeers] = {};
  int scatter_world = 0, scatter_rank = 0;
};

cudaError_t run_gemm(const GemmArgs &args, cudaStream_t stream);

// Fused SharQ GEMM over the groups (experts) of a mixture-of-experts layer in one launch.  The
// activation rows are sorted by group, every group's segment padded to a multiple of 256 rows
// (m is the padded total); unit_group[u] (device, m / 256 entries) is the group of rows
// [256u, 256u + 256) or -1 for a unit without rows; row r of D is
// alpha * alpha_vec[group] * (A_sparse[r] + A_res[r]) . W[group]^T.
constexpr int kGemmMaxGroups = 16;
struct GroupedGemmArgs {
  const void *a_comp = nullptr, *e = nullptr, *sfa_sparse = nullptr, *a_dense = nullptr, *sfa_dense = nullptr;
  int groups = 0;
  const void *b[kGemmMaxGroups] = {}, *sfb_sparse[kGemmMaxGroups] = {}, *sfb_dense[kGemmMaxGroups] = {};
  const int *unit_group = nullptr;
  const float *alpha_vec = nullptr;
  float alpha = 1.0f;
  void *d = nullptr;
  int m = 0, n = 0, k = 0;
  int *error_flag = nullptr;
};
cudaError_t run_gemm_grouped(const GroupedGemmArgs &args, cudaStream_t stream);

}  // namespace sharq
