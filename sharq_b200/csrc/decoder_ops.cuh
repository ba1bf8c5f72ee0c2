// Host launchers of the decoder-layer element-wise kernels (decoder_ops.cu).
#pragma once
#include <cuda_runtime.h>

namespace sharq {

// Rotary embedding in place on `heads` consecutive heads at the start of every row of a bf16
// matrix (row_stride elements between rows); position = row % seq_len; cos/sin: [seq_len, head_dim].
cudaError_t run_rope_inplace(void *x, long long rows, long long row_stride, int seq_len, int heads, int head_dim,
                             const void *cos_t, const void *sin_t, cudaStream_t stream);

// h[rows, ffn] = silu(gate) * up from gate_up[rows, 2*ffn] (gate first); amax_bits (optional) is
// zeroed and then raised to the bits of max|h|.
// With unit_group (device, one int per 256 rows, < 0 = unit without rows) the rows are a grouped
// activation: amax_bits has `groups` words, one per group, and rows of empty units are skipped.
cudaError_t run_swiglu_absmax(const void *gate_up, long long rows, int ffn, long long row_stride, void *h,
                              unsigned int *amax_bits, cudaStream_t stream, const int *unit_group = nullptr, int groups = 1);

// max|x| per group of a grouped bf16 activation [rows, width] into amax_bits[groups] (zeroed first).
// With src_row, grouped row r is input row src_row[r] of x (< 0: a padding row without data).
cudaError_t run_abs_stats_grouped(const void *x, long long rows, int width, unsigned int *amax_bits, const int *unit_group,
                                  int groups, cudaStream_t stream, const int *src_row = nullptr);

// out[t, :] = sum over the top_k slots of token t, in ascending expert order, of y[dest[t, j], :] * w[t, j]
// with bf16 roundings after every product and every addition (selected: expert index per slot).
cudaError_t run_moe_combine(void *out, const void *y, const int *dest, const long long *selected, const void *w,
                            long long tokens, int top_k, int width, cudaStream_t stream);

// out[rows, k] = bf16(s * rsqrt(mean(s^2) + eps) * gamma), s = bf16(x + residual) stored to sum_out
// (residual == nullptr: s = x, sum_out unused); K a multiple of 8, at most 8192.
cudaError_t run_add_rmsnorm(const void *x, const void *residual, void *sum_out, const void *gamma, float eps, long long rows,
                            int k, void *out, cudaStream_t stream);

// out[rows[i], :] += y[i, :] * w[i] in bf16 (distinct rows inside [0, out_rows), others skipped; width a multiple of 8).
cudaError_t run_scatter_add_scaled(void *out, const void *y, const long long *rows, const void *w, long long n_rows,
                                   int width, long long out_rows, cudaStream_t stream);

}  // namespace sharq
