// Host launchers of the activation prepare kernels (prepare.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace sharq {

// Bytes of scratch the scaled / RMSNorm-fused prepare needs for M rows:
// [0,4) tensor absmax bits, [4,8) grid barrier counter, [256, 256 + 4*M) per-row inv_rms.
size_t prepare_workspace_bytes(int m);

// Prepare of an already scaled bf16 activation [m,k].  With q_sparse_dense != nullptr
// the debug variant runs (dense sparse payload instead of a_comp/e).
cudaError_t run_prepare(const void *x, int m, int k, void *a_comp, void *e, void *q_sparse_dense,
                        void *sfa_sparse, void *q_res, void *sf_res, cudaStream_t stream);

// Row statistics + prepare with the tensor scale (and RMSNorm when gamma != nullptr)
// applied inline.  inv_rms_external (optional) receives the per-row inv_rms instead of
// the workspace slot.  With absmax_ready (gamma == nullptr only) the workspace already
// holds the bits of max|x| and the statistics pass is skipped.  With residual (RMSNorm path
// only) the input is bf16(x + residual), which the statistics kernel also writes to sum_out.
cudaError_t run_scaled_prepare(const void *x, const void *gamma, float eps, int m, int k, void *workspace,
                               float *inv_rms_external, void *a_comp, void *e, void *sfa_sparse, void *q_res,
                               void *sf_res, float *scale_out, cudaStream_t stream, bool absmax_ready = false,
                               const void *residual = nullptr, void *sum_out = nullptr);

// Tensor-scale prepare of a grouped activation (mixture-of-experts layers): rows sorted by group in
// 256-row units (m a multiple of 256), unit_group[u] < 0 = unit without rows (its outputs are
// zero metadata / scales and untouched payload), amax_bits[g] = bits of max|x| over group g
// (already computed), scale_vec_out[g] = clamp(amax_g / 2688, 1e-9).  With src_row the output row r is
// prepared from input row src_row[r] of x (a gather; < 0: a padding row, all-zero scales).  Every group is divided by
// its own scale, exactly as a separate call per group would do.
cudaError_t run_grouped_prepare(const void *x, int m, int k, const unsigned int *amax_bits, const int *unit_group, int groups,
                                void *a_comp, void *e, void *sfa_sparse, void *q_res, void *sf_res, float *scale_vec_out,
                                cudaStream_t stream, const int *src_row = nullptr);

// Grid barriers of the one-launch prepare that ran out on the current device since the library
// was loaded (0 in a healthy process; -1 when the counter cannot be read).
int prepare_timeouts();

}  // namespace sharq
