// extern "C" boundary of the library (declared in include/sharq_b200.h): argument
// checks with the reference's error conditions, then the launchers.
#include "../../include/sharq_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "allreduce.cuh"
#include "common.cuh"
#include "decoder_ops.cuh"
#include "gemm.cuh"
#include "prepare.cuh"
#include "quant.cuh"
#include "sp_transition.cuh"

namespace {

thread_local char g_error[512] = "";
int g_tile_n = 0;

int fail(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return 1;
}

int check_cuda(cudaError_t err, const char *what) {
  if (err == cudaSuccess) return 0;
  return fail("%s: %s", what, cudaGetErrorString(err));
}

inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }

#define SHARQ_REQUIRE(cond, ...) \
  do {                           \
    if (!(cond)) return fail(__VA_ARGS__); \
  } while (0)

}  // namespace

extern "C" {

int sharq_version(void) { return 100; }

const char *sharq_last_error(void) { return g_error; }

int sharq_get_sparse_nvfp4_buffer_sizes(int m, int n, int k, int64_t out[4]) {
  SHARQ_REQUIRE(m > 0 && n > 0 && k > 0 && out, "M, N, K must be positive");
  out[0] = (int64_t)sharq::a_comp_bytes(m, k);
  out[1] = (int64_t)sharq::e_bytes(m, k);
  out[2] = (int64_t)sharq::sf_alloc_bytes(m, k);
  out[3] = (int64_t)sharq::sf_alloc_bytes(n, k);
  return 0;
}

int sharq_get_fused_sparse_residual_buffer_sizes(int m, int n, int k, int64_t out[5]) {
  SHARQ_REQUIRE(m > 0 && k > 0 && out, "M, K must be positive");
  (void)n;
  out[0] = (int64_t)sharq::a_comp_bytes(m, k);
  out[1] = (int64_t)sharq::e_bytes(m, k);
  out[2] = (int64_t)sharq::sf_alloc_bytes(m, k);
  out[3] = (int64_t)m * (int64_t)(k / 2);
  out[4] = (int64_t)sharq::sf_alloc_bytes(m, k);
  return 0;
}

int sharq_fused_sparse_residual_quantize_x(const void *x, int m, int n, int k, void *a_comp, void *e, void *sfa_sparse,
                                           void *q_res, void *sf_res, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && k > 0, "X must be shaped [M, K]");
  SHARQ_REQUIRE(k % 128 == 0, "fused_sparse_residual_quantize_x currently requires K to be a multiple of 128, got %d", k);
  SHARQ_REQUIRE(x && a_comp && e && sfa_sparse && q_res && sf_res, "null buffer");
  return check_cuda(sharq::run_prepare(x, m, k, a_comp, e, nullptr, sfa_sparse, q_res, sf_res, as_stream(stream)),
                    "fused_sparse_residual_quantize_x");
}

int sharq_fused_sparse_residual_quantize_x_debug(const void *x, int m, int n, int k, void *q_sparse, void *sfa_sparse,
                                                 void *q_res, void *sf_res, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && k > 0, "X must be shaped [M, K]");
  SHARQ_REQUIRE(k % 128 == 0,
                "fused_sparse_residual_quantize_x_debug currently requires K to be a multiple of 128, got %d", k);
  SHARQ_REQUIRE(x && q_sparse && sfa_sparse && q_res && sf_res, "null buffer");
  return check_cuda(sharq::run_prepare(x, m, k, nullptr, nullptr, q_sparse, sfa_sparse, q_res, sf_res, as_stream(stream)),
                    "fused_sparse_residual_quantize_x_debug");
}

size_t sharq_prepare_workspace_bytes(int m) { return sharq::prepare_workspace_bytes(m); }

int sharq_prepare_timeouts(void) { return sharq::prepare_timeouts(); }

int sharq_fused_rmsnorm_sparse_residual_quantize_x(const void *x, const void *gamma, float eps, int m, int n, int k,
                                                   void *workspace, size_t workspace_bytes, void *a_comp, void *e,
                                                   void *sfa_sparse, void *q_res, void *sf_res, float *scale_out,
                                                   void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && k > 0, "X must be shaped [M, K]");
  SHARQ_REQUIRE(k % 128 == 0,
                "fused_rmsnorm_sparse_residual_quantize_x currently requires K to be a multiple of 128, got %d", k);
  SHARQ_REQUIRE(k / 32 <= 1024, "fused_rmsnorm_sparse_residual_quantize_x requires K/32 <= 1024, got %d", k / 32);
  SHARQ_REQUIRE(x && gamma && a_comp && e && sfa_sparse && q_res && sf_res, "null buffer");
  SHARQ_REQUIRE(workspace && workspace_bytes >= sharq::prepare_workspace_bytes(m), "workspace too small: need %zu bytes",
                sharq::prepare_workspace_bytes(m));
  return check_cuda(sharq::run_scaled_prepare(x, gamma, eps, m, k, workspace, nullptr, a_comp, e, sfa_sparse, q_res,
                                              sf_res, scale_out, as_stream(stream)),
                    "fused_rmsnorm_sparse_residual_quantize_x");
}

int sharq_fused_add_rmsnorm_sparse_residual_quantize_x(const void *x, const void *residual, void *sum_out,
                                                       const void *gamma, float eps, int m, int n, int k, void *workspace,
                                                       size_t workspace_bytes, void *a_comp, void *e, void *sfa_sparse,
                                                       void *q_res, void *sf_res, float *scale_out, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && k > 0, "X must be shaped [M, K]");
  SHARQ_REQUIRE(k % 128 == 0,
                "fused_add_rmsnorm_sparse_residual_quantize_x requires K to be a multiple of 128, got %d", k);
  SHARQ_REQUIRE(k / 32 <= 1024, "fused_add_rmsnorm_sparse_residual_quantize_x requires K/32 <= 1024, got %d", k / 32);
  SHARQ_REQUIRE(x && residual && sum_out && gamma && a_comp && e && sfa_sparse && q_res && sf_res, "null buffer");
  SHARQ_REQUIRE(workspace && workspace_bytes >= sharq::prepare_workspace_bytes(m), "workspace too small: need %zu bytes",
                sharq::prepare_workspace_bytes(m));
  return check_cuda(sharq::run_scaled_prepare(x, gamma, eps, m, k, workspace, nullptr, a_comp, e, sfa_sparse, q_res,
                                              sf_res, scale_out, as_stream(stream), false, residual, sum_out),
                    "fused_add_rmsnorm_sparse_residual_quantize_x");
}

int sharq_scaled_sparse_residual_quantize_x(const void *x, int m, int n, int k, void *workspace, size_t workspace_bytes,
                                            void *a_comp, void *e, void *sfa_sparse, void *q_res, void *sf_res,
                                            float *scale_out, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && k > 0, "X must be shaped [M, K]");
  SHARQ_REQUIRE(k % 128 == 0, "scaled_sparse_residual_quantize_x requires K to be a multiple of 128, got %d", k);
  SHARQ_REQUIRE(x && a_comp && e && sfa_sparse && q_res && sf_res, "null buffer");
  SHARQ_REQUIRE(workspace && workspace_bytes >= 256, "workspace too small: need 256 bytes");
  return check_cuda(sharq::run_scaled_prepare(x, nullptr, 0.0f, m, k, workspace, nullptr, a_comp, e, sfa_sparse, q_res,
                                              sf_res, scale_out, as_stream(stream)),
                    "scaled_sparse_residual_quantize_x");
}

int sharq_rope_inplace(void *x_bf16, int rows, int row_stride, int seq_len, int heads, int head_dim, const void *cos_bf16,
                       const void *sin_bf16, void *stream) {
  SHARQ_REQUIRE(x_bf16 && cos_bf16 && sin_bf16, "null buffer");
  SHARQ_REQUIRE(rows > 0 && seq_len > 0 && heads > 0, "rows, seq_len, heads must be positive");
  SHARQ_REQUIRE(head_dim > 0 && head_dim % 16 == 0, "head_dim must be a positive multiple of 16, got %d", head_dim);
  SHARQ_REQUIRE(row_stride >= heads * head_dim && row_stride % 8 == 0,
                "row_stride must cover heads * head_dim and be a multiple of 8");
  SHARQ_REQUIRE((reinterpret_cast<uintptr_t>(x_bf16) & 15) == 0, "x must be 16-byte aligned");
  SHARQ_REQUIRE(((reinterpret_cast<uintptr_t>(cos_bf16) | reinterpret_cast<uintptr_t>(sin_bf16)) & 15) == 0,
                "cos and sin must be 16-byte aligned");
  return check_cuda(sharq::run_rope_inplace(x_bf16, rows, row_stride, seq_len, heads, head_dim, cos_bf16, sin_bf16,
                                            as_stream(stream)),
                    "rope_inplace");
}

int sharq_scatter_add_scaled(void *out_bf16, int out_rows, const void *y_bf16, const int64_t *rows, const void *w_bf16,
                             int n_rows, int width, void *stream) {
  SHARQ_REQUIRE(out_bf16 && y_bf16 && rows && w_bf16, "null buffer");
  SHARQ_REQUIRE(n_rows >= 0 && out_rows >= 0 && width > 0 && width % 8 == 0,
                "n_rows and out_rows must be >= 0 and width a positive multiple of 8");
  SHARQ_REQUIRE(((reinterpret_cast<uintptr_t>(out_bf16) | reinterpret_cast<uintptr_t>(y_bf16)) & 15) == 0,
                "out and y must be 16-byte aligned");
  return check_cuda(sharq::run_scatter_add_scaled(out_bf16, y_bf16, reinterpret_cast<const long long *>(rows), w_bf16,
                                                  n_rows, width, out_rows, as_stream(stream)),
                    "scatter_add_scaled");
}

int sharq_add_rmsnorm(const void *x_bf16, const void *residual_bf16, void *sum_out_bf16, const void *gamma_bf16, float eps,
                      int rows, int k, void *out_bf16, void *stream) {
  SHARQ_REQUIRE(x_bf16 && gamma_bf16 && out_bf16, "null buffer");
  SHARQ_REQUIRE((residual_bf16 == nullptr) == (sum_out_bf16 == nullptr), "residual and sum_out go together");
  SHARQ_REQUIRE(rows >= 0 && k > 0 && k % 8 == 0 && k <= 8192, "rows must be >= 0 and K a multiple of 8, at most 8192, got %d", k);
  SHARQ_REQUIRE(((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(residual_bf16) |
                  reinterpret_cast<uintptr_t>(sum_out_bf16) | reinterpret_cast<uintptr_t>(gamma_bf16) |
                  reinterpret_cast<uintptr_t>(out_bf16)) & 15) == 0, "buffers must be 16-byte aligned");
  return check_cuda(sharq::run_add_rmsnorm(x_bf16, residual_bf16, sum_out_bf16, gamma_bf16, eps, rows, k, out_bf16,
                                           as_stream(stream)),
                    "add_rmsnorm");
}

int sharq_swiglu(const void *gate_up_bf16, int rows, int ffn, void *h_bf16, void *stream) {
  SHARQ_REQUIRE(gate_up_bf16 && h_bf16, "null buffer");
  SHARQ_REQUIRE(rows > 0 && ffn > 0 && ffn % 8 == 0, "rows must be positive and ffn a positive multiple of 8");
  return check_cuda(sharq::run_swiglu_absmax(gate_up_bf16, rows, ffn, 2LL * ffn, h_bf16, nullptr, as_stream(stream)),
                    "swiglu");
}

int sharq_swiglu_sparse_residual_quantize_x(const void *gate_up_bf16, int m, int n, int k, void *h_bf16, void *workspace,
                                            size_t workspace_bytes, void *a_comp, void *e, void *sfa_sparse, void *q_res,
                                            void *sf_res, float *scale_out, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && k > 0, "gate_up must be shaped [M, 2K]");
  SHARQ_REQUIRE(k % 128 == 0, "swiglu_sparse_residual_quantize_x requires K to be a multiple of 128, got %d", k);
  SHARQ_REQUIRE(gate_up_bf16 && h_bf16 && a_comp && e && sfa_sparse && q_res && sf_res, "null buffer");
  SHARQ_REQUIRE(workspace && workspace_bytes >= 256, "workspace too small: need 256 bytes");
  if (check_cuda(sharq::run_swiglu_absmax(gate_up_bf16, m, k, 2LL * k, h_bf16, static_cast<unsigned int *>(workspace),
                                          as_stream(stream)),
                 "swiglu_absmax"))
    return 1;
  return check_cuda(sharq::run_scaled_prepare(h_bf16, nullptr, 0.0f, m, k, workspace, nullptr, a_comp, e, sfa_sparse,
                                              q_res, sf_res, scale_out, as_stream(stream), /*absmax_ready=*/true),
                    "swiglu_sparse_residual_quantize_x");
}

int sharq_quantize_w32_shared(const void *w, int n, int k, void *qw, void *sfw_sparse, void *sfw_dense, void *stream) {
  SHARQ_REQUIRE(n > 0 && k > 0, "W must be shaped [N, K]");
  SHARQ_REQUIRE(k % 32 == 0, "quantize_w32_shared requires K to be a multiple of 32, got %d", k);
  SHARQ_REQUIRE(k / 32 <= 1024, "run_quantize_w32_bf16_nvfp4_shared requires hidden_dim / 32 <= 1024");
  SHARQ_REQUIRE(w && qw && sfw_sparse && sfw_dense, "null buffer");
  return check_cuda(sharq::run_quantize_w32_shared(w, n, k, qw, sfw_sparse, sfw_dense, as_stream(stream)),
                    "quantize_w32_shared");
}

int sharq_duplicate_sfa32_to_sfa16(const void *sfa_sparse, int m, int n, int k, void *sfa_dense, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && k > 0, "M, K must be positive");
  SHARQ_REQUIRE(k % 32 == 0, "run_duplicate_sfa32_to_sfa16 requires hidden_dim to be a multiple of 32");
  SHARQ_REQUIRE(k / 32 <= 1024, "run_duplicate_sfa32_to_sfa16 requires hidden_dim / 32 <= 1024");
  SHARQ_REQUIRE(sfa_sparse && sfa_dense, "null buffer");
  return check_cuda(sharq::run_duplicate_sf32_to_sf16(sfa_sparse, m, k, sfa_dense, as_stream(stream)),
                    "duplicate_sfa32_to_sfa16");
}

int sharq_quantize_nvfp4(const void *x, int rows, int k, void *q, void *sf, void *stream) {
  SHARQ_REQUIRE(rows > 0 && k > 0, "input must be shaped [rows, K]");
  SHARQ_REQUIRE(k % 16 == 0, "Unsupported hidden size %d: K must be a multiple of 16", k);
  SHARQ_REQUIRE(x && q && sf, "null buffer");
  return check_cuda(sharq::run_quantize_dense_nvfp4(x, rows, k, q, sf, as_stream(stream)), "quantize_nvfp4");
}

int sharq_compress_sparse_a(const void *a_q_dense, int m, int n, int k, void *a_comp, void *e, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && k > 0, "A_q_dense must be shaped [M, K/2]");
  SHARQ_REQUIRE(k % 32 == 0, "compress_sparse_a requires K to be a multiple of 32, got %d", k);
  SHARQ_REQUIRE(a_q_dense && a_comp && e, "null buffer");
  return check_cuda(sharq::run_compress_sparse_a(a_q_dense, m, k, a_comp, e, as_stream(stream)), "compress_sparse_a");
}

size_t sharq_allreduce_flag_bytes(void) { return sharq::allreduce_flag_bytes(); }

int sharq_allreduce_bf16_multimem(void *multicast_data, void *const *rank_flag_ptrs, int rank, int world,
                                  size_t n_bytes, int max_ctas, int *error_flag, void *stream) {
  SHARQ_REQUIRE(multicast_data && rank_flag_ptrs && error_flag, "multicast_data, rank_flag_ptrs, error_flag must be set");
  SHARQ_REQUIRE(world >= 1 && world <= sharq::kAllReduceMaxRanks, "world must be in [1, %d]", sharq::kAllReduceMaxRanks);
  SHARQ_REQUIRE(rank >= 0 && rank < world, "rank must be in [0, world)");
  SHARQ_REQUIRE(n_bytes > 0 && n_bytes % ((size_t)16 * world) == 0, "n_bytes must be a positive multiple of 16 * world");
  SHARQ_REQUIRE((reinterpret_cast<uintptr_t>(multicast_data) & 15) == 0, "multicast_data must be 16-byte aligned");
  for (int i = 0; i < world; ++i) SHARQ_REQUIRE(rank_flag_ptrs[i] != nullptr, "rank_flag_ptrs[%d] is NULL", i);
  return check_cuda(sharq::run_allreduce(multicast_data, nullptr, rank_flag_ptrs, rank, world, n_bytes, max_ctas, error_flag,
                                         as_stream(stream)),
                    "allreduce_multimem launch");
}

int sharq_allreduce_bf16_peer(void *const *rank_data_ptrs, void *const *rank_flag_ptrs, int rank, int world, size_t n_bytes,
                              int max_ctas, int *error_flag, void *stream) {
  SHARQ_REQUIRE(rank_data_ptrs && rank_flag_ptrs && error_flag, "rank_data_ptrs, rank_flag_ptrs, error_flag must be set");
  SHARQ_REQUIRE(world >= 1 && world <= sharq::kAllReducePeerMaxRanks, "world must be in [1, %d]",
                sharq::kAllReducePeerMaxRanks);
  SHARQ_REQUIRE(rank >= 0 && rank < world, "rank must be in [0, world)");
  SHARQ_REQUIRE(n_bytes > 0 && n_bytes % ((size_t)16 * world) == 0, "n_bytes must be a positive multiple of 16 * world");
  for (int i = 0; i < world; ++i) {
    SHARQ_REQUIRE(rank_data_ptrs[i] != nullptr && (reinterpret_cast<uintptr_t>(rank_data_ptrs[i]) & 15) == 0,
                  "rank_data_ptrs[%d] must be a 16-byte aligned pointer", i);
    SHARQ_REQUIRE(rank_flag_ptrs[i] != nullptr, "rank_flag_ptrs[%d] is NULL", i);
  }
  return check_cuda(sharq::run_allreduce(nullptr, rank_data_ptrs, rank_flag_ptrs, rank, world, n_bytes, max_ctas, error_flag,
                                         as_stream(stream)),
                    "allreduce_peer launch");
}

int sharq_grouped_sparse_residual_quantize_x(const void *x_bf16, const int *src_row, int m, int n, int k,
                                            const int *unit_group, int groups, void *amax_workspace, void *a_comp, void *e,
                                            void *sfa_sparse, void *q_res, void *sf_res, float *scale_vec_out, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && m % 256 == 0 && k > 0 && k % 128 == 0, "M must be a positive multiple of 256 and K of 128");
  SHARQ_REQUIRE(groups >= 1 && groups <= sharq::kGemmMaxGroups, "groups must be in [1, %d]", sharq::kGemmMaxGroups);
  SHARQ_REQUIRE(x_bf16 && unit_group && amax_workspace && a_comp && e && sfa_sparse && q_res && sf_res && scale_vec_out,
                "null buffer");
  auto *amax = static_cast<unsigned int *>(amax_workspace);
  if (check_cuda(sharq::run_abs_stats_grouped(x_bf16, m, k, amax, unit_group, groups, as_stream(stream), src_row),
                 "grouped absmax"))
    return 1;
  return check_cuda(sharq::run_grouped_prepare(x_bf16, m, k, amax, unit_group, groups, a_comp, e, sfa_sparse, q_res, sf_res,
                                               scale_vec_out, as_stream(stream), src_row),
                    "grouped_sparse_residual_quantize_x");
}

int sharq_grouped_swiglu_sparse_residual_quantize_x(const void *gate_up_bf16, int m, int n, int k, void *h_bf16,
                                                   const int *unit_group, int groups, void *amax_workspace, void *a_comp,
                                                   void *e, void *sfa_sparse, void *q_res, void *sf_res,
                                                   float *scale_vec_out, void *stream) {
  (void)n;
  SHARQ_REQUIRE(m > 0 && m % 256 == 0 && k > 0 && k % 128 == 0, "M must be a positive multiple of 256 and K of 128");
  SHARQ_REQUIRE(groups >= 1 && groups <= sharq::kGemmMaxGroups, "groups must be in [1, %d]", sharq::kGemmMaxGroups);
  SHARQ_REQUIRE(gate_up_bf16 && h_bf16 && unit_group && amax_workspace && a_comp && e && sfa_sparse && q_res && sf_res &&
                    scale_vec_out,
                "null buffer");
  auto *amax = static_cast<unsigned int *>(amax_workspace);
  if (check_cuda(sharq::run_swiglu_absmax(gate_up_bf16, m, k, 2LL * k, h_bf16, amax, as_stream(stream), unit_group, groups),
                 "grouped swiglu"))
    return 1;
  return check_cuda(sharq::run_grouped_prepare(h_bf16, m, k, amax, unit_group, groups, a_comp, e, sfa_sparse, q_res, sf_res,
                                               scale_vec_out, as_stream(stream)),
                    "grouped_swiglu_sparse_residual_quantize_x");
}

int sharq_linear_gemm_grouped(const void *a_comp, const void *e, const void *sfa_sparse, const void *q_res, const void *sf_res,
                              int groups, const void *const *qw, const void *const *sfw_sparse, const void *const *sfw_dense,
                              const int *unit_group, const float *alpha_vec, float alpha, int m, int n, int k, void *d,
                              int *error_flag, void *stream) {
  SHARQ_REQUIRE(m > 0 && m % 256 == 0 && n > 0 && k > 0 && k % 128 == 0,
                "M must be a positive multiple of 256, K a multiple of 128");
  SHARQ_REQUIRE(groups >= 1 && groups <= sharq::kGemmMaxGroups, "groups must be in [1, %d]", sharq::kGemmMaxGroups);
  SHARQ_REQUIRE(a_comp && e && sfa_sparse && q_res && sf_res && qw && sfw_sparse && sfw_dense && unit_group && alpha_vec && d &&
                    error_flag,
                "null buffer");
  sharq::GroupedGemmArgs g;
  g.a_comp = a_comp;
  g.e = e;
  g.sfa_sparse = sfa_sparse;
  g.a_dense = q_res;
  g.sfa_dense = sf_res;
  g.groups = groups;
  for (int i = 0; i < groups; ++i) {
    SHARQ_REQUIRE(qw[i] && sfw_sparse[i] && sfw_dense[i], "weight buffers of group %d missing", i);
    g.b[i] = qw[i];
    g.sfb_sparse[i] = sfw_sparse[i];
    g.sfb_dense[i] = sfw_dense[i];
  }
  g.unit_group = unit_group;
  g.alpha_vec = alpha_vec;
  g.alpha = alpha;
  g.d = d;
  g.m = m;
  g.n = n;
  g.k = k;
  g.error_flag = error_flag;
  return check_cuda(sharq::run_gemm_grouped(g, as_stream(stream)), "linear_gemm_grouped");
}

int sharq_moe_combine(void *out_bf16, const void *y_bf16, const int *dest, const int64_t *selected, const void *w_bf16,
                      int tokens, int top_k, int width, void *stream) {
  SHARQ_REQUIRE(out_bf16 && y_bf16 && dest && selected && w_bf16, "null buffer");
  SHARQ_REQUIRE(tokens >= 0 && top_k >= 1 && top_k <= 8 && width > 0 && width % 8 == 0,
                "tokens >= 0, top_k in [1, 8], width a positive multiple of 8");
  SHARQ_REQUIRE(((reinterpret_cast<uintptr_t>(out_bf16) | reinterpret_cast<uintptr_t>(y_bf16)) & 15) == 0,
                "out and y must be 16-byte aligned");
  return check_cuda(sharq::run_moe_combine(out_bf16, y_bf16, dest, reinterpret_cast<const long long *>(selected), w_bf16, tokens,
                                           top_k, width, as_stream(stream)),
                    "moe_combine");
}

int sharq_linear_gemm_scatter(const void *a_comp, const void *e, const void *sfa_sparse, const void *q_res, const void *sf_res,
                              const void *qw, const void *sfw_sparse, const void *sfw_dense, int m, int n, int k, float alpha,
                              const float *alpha_dev, void *const *d_rank_ptrs, int rank, int world, int *error_flag,
                              void *stream) {
  SHARQ_REQUIRE(world >= 2 && world <= sharq::kGemmMaxPeers, "world must be in [2, %d]", sharq::kGemmMaxPeers);
  SHARQ_REQUIRE(rank >= 0 && rank < world, "rank must be in [0, world)");
  SHARQ_REQUIRE(m > 0 && n > 0 && k > 0 && m % (128 * world) == 0 && n % 8 == 0 && k % 128 == 0,
                "needs M %% (128 * world) == 0, N %% 8 == 0, K %% 128 == 0");
  SHARQ_REQUIRE(a_comp && e && sfa_sparse && q_res && sf_res && qw && sfw_sparse && sfw_dense && d_rank_ptrs && error_flag,
                "null buffer");
  sharq::GemmArgs g;
  g.a_comp = a_comp;
  g.e = e;
  g.sfa_sparse = sfa_sparse;
  g.a_dense = q_res;
  g.sfa_dense = sf_res;
  g.b = qw;
  g.sfb_sparse = sfw_sparse;
  g.sfb_dense = sfw_dense;
  g.alpha = alpha;
  g.alpha_ptr = alpha_dev;
  g.m = m;
  g.n = n;
  g.k = k;
  g.tile_n = g_tile_n;
  g.error_flag = error_flag;
  g.scatter_world = world;
  g.scatter_rank = rank;
  for (int r = 0; r < world; ++r) {
    SHARQ_REQUIRE(d_rank_ptrs[r] != nullptr && (reinterpret_cast<uintptr_t>(d_rank_ptrs[r]) & 15) == 0,
                  "d_rank_ptrs[%d] must be a 16-byte aligned pointer", r);
    g.d_peer[r] = d_rank_ptrs[r];
  }
  return check_cuda(sharq::run_gemm(g, as_stream(stream)), "linear_gemm_scatter");
}

size_t sharq_tp_transition_state_bytes(void) { return sharq::sp_transition_state_bytes(); }

size_t sharq_tp_transition_workspace_bytes(int rows) { return rows > 0 ? sharq::sp_transition_workspace_bytes(rows) : 0; }

int sharq_tp_reduce_rmsnorm_prepare_allgather(const void *partial_blocks, const void *residual_in, void *residual_out,
                                              const void *rmsnorm_weight, float eps, int m, int n, int k, void *workspace,
                                              size_t workspace_bytes, void *a_comp, void *e, void *sfa_sparse, void *q_res,
                                              void *sf_res, long long multicast_delta, float *scale_out,
                                              void *const *rank_state_ptrs, int rank, int world, int *error_flag,
                                              void *stream) {
  (void)n;
  SHARQ_REQUIRE(world >= 1 && world <= sharq::kSpMaxRanks, "world must be in [1, %d]", sharq::kSpMaxRanks);
  SHARQ_REQUIRE(rank >= 0 && rank < world, "rank must be in [0, world)");
  SHARQ_REQUIRE(m > 0 && k > 0 && m % (128 * world) == 0,
                "M must be a positive multiple of 128 * world (every GPU owns whole 128-row bands), got M = %d, world = %d", m,
                world);
  SHARQ_REQUIRE(k % 128 == 0 && k / 32 <= 1024, "K must be a multiple of 128 with K/32 <= 1024, got %d", k);
  SHARQ_REQUIRE(partial_blocks || residual_in, "partial products or a residual (or both) must be given");
  SHARQ_REQUIRE(residual_out && rmsnorm_weight && a_comp && e && sfa_sparse && q_res && sf_res && scale_out && rank_state_ptrs &&
                    error_flag,
                "null buffer");
  SHARQ_REQUIRE(workspace && workspace_bytes >= sharq::sp_transition_workspace_bytes(m / world),
                "workspace too small: need %zu bytes", sharq::sp_transition_workspace_bytes(m / world));
  const void *aligned[] = {partial_blocks, residual_in, residual_out, rmsnorm_weight, a_comp, e, sfa_sparse, q_res, sf_res};
  for (const void *ptr : aligned)
    SHARQ_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, "buffers must be 16-byte aligned");
  SHARQ_REQUIRE((multicast_delta & 15) == 0, "multicast_delta must be a multiple of 16");
  for (int i = 0; i < world; ++i)
    SHARQ_REQUIRE(rank_state_ptrs[i] != nullptr && (reinterpret_cast<uintptr_t>(rank_state_ptrs[i]) & 15) == 0,
                  "rank_state_ptrs[%d] must be a 16-byte aligned pointer", i);
  sharq::SpTransitionArgs a;
  a.partial_blocks = partial_blocks;
  a.residual_in = residual_in;
  a.residual_out = residual_out;
  a.gamma = rmsnorm_weight;
  a.eps = eps;
  a.workspace = workspace;
  a.scale_out = scale_out;
  a.a_comp = a_comp;
  a.e = e;
  a.sfa_sparse = sfa_sparse;
  a.q_res = q_res;
  a.sf_res = sf_res;
  a.multicast_delta = multicast_delta;
  a.rank_state_ptrs = rank_state_ptrs;
  a.rank = rank;
  a.world = world;
  a.m = m;
  a.k = k;
  a.error_flag = error_flag;
  return check_cuda(sharq::run_sp_transition(a, as_stream(stream)), "tp_reduce_rmsnorm_prepare_allgather launch");
}

int sharq_set_wait_limit_cycles(long long cycles) {
  SHARQ_REQUIRE(cycles >= 0, "cycles must be >= 0 (0 restores the defaults)");
  sharq::set_allreduce_wait_limit(cycles);
  sharq::set_sp_transition_wait_limit(cycles);
  return 0;
}

int sharq_set_gemm_tile_n(int tile_n) {
  SHARQ_REQUIRE(tile_n == 0 || tile_n == 128 || tile_n == 256 || tile_n == 512, "tile_n must be 0, 128, 256 or 512");
  g_tile_n = tile_n;
  return 0;
}

size_t sharq_gemm_workspace_bytes(int m, int n) {
  return (m > 0 && m <= 128 && n > 0) ? (size_t)m * (size_t)n * sizeof(float) : 0;
}

int sharq_matmul(const void *a, const void *b, const void *sfa, const void *sfb, int m, int n, int k, float alpha,
                 const float *alpha_dev, const void *c_in, float beta, void *d, int *error_flag, void *stream) {
  return sharq_matmul_ws(a, b, sfa, sfb, m, n, k, alpha, alpha_dev, c_in, beta, d, nullptr, 0, error_flag, stream);
}

int sharq_matmul_ws(const void *a, const void *b, const void *sfa, const void *sfb, int m, int n, int k, float alpha,
                    const float *alpha_dev, const void *c_in, float beta, void *d, void *workspace,
                    size_t workspace_bytes, int *error_flag, void *stream) {
  SHARQ_REQUIRE(m > 0 && n > 0 && k > 0, "M, N, K must be positive");
  SHARQ_REQUIRE(k % 64 == 0, "matmul requires K to be a multiple of 64, got %d", k);
  SHARQ_REQUIRE(a && b && sfa && sfb && d && error_flag, "null buffer");
  SHARQ_REQUIRE(beta == 0.0f || c_in != nullptr, "C_in must be given when beta != 0");
  sharq::GemmArgs g;
  g.a_dense = a;
  g.sfa_dense = sfa;
  g.b = b;
  g.sfb_dense = sfb;
  g.c_in = c_in;
  g.d = d;
  g.alpha = alpha;
  g.alpha_ptr = alpha_dev;
  g.beta = beta;
  g.m = m;
  g.n = n;
  g.k = k;
  g.tile_n = g_tile_n;
  g.error_flag = error_flag;
  g.workspace = workspace;
  g.workspace_bytes = workspace ? workspace_bytes : 0;
  SHARQ_REQUIRE(workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                "workspace must be 16-byte aligned");
  return check_cuda(sharq::run_gemm(g, as_stream(stream)), "matmul");
}

int sharq_sparse_matmul(const void *a_comp, const void *b, const void *e, const void *sfa, const void *sfb, int m, int n,
                        int k, float alpha, const float *alpha_dev, float beta, void *d, int *error_flag, void *stream) {
  return sharq_sparse_matmul_ws(a_comp, b, e, sfa, sfb, m, n, k, alpha, alpha_dev, beta, d, nullptr, 0, error_flag, stream);
}

int sharq_sparse_matmul_ws(const void *a_comp, const void *b, const void *e, const void *sfa, const void *sfb, int m, int n,
                           int k, float alpha, const float *alpha_dev, float beta, void *d, void *workspace,
                           size_t workspace_bytes, int *error_flag, void *stream) {
  SHARQ_REQUIRE(m > 0 && n > 0 && k > 0, "M, N, K must be positive");
  SHARQ_REQUIRE(beta == 0.0f, "sparse_matmul currently requires beta == 0");
  SHARQ_REQUIRE(k % 128 == 0, "sparse_matmul requires K to be a multiple of 128, got %d", k);
  SHARQ_REQUIRE(a_comp && b && e && sfa && sfb && d && error_flag, "null buffer");
  sharq::GemmArgs g;
  g.a_comp = a_comp;
  g.e = e;
  g.sfa_sparse = sfa;
  g.b = b;
  g.sfb_sparse = sfb;
  g.d = d;
  g.alpha = alpha;
  g.alpha_ptr = alpha_dev;
  g.m = m;
  g.n = n;
  g.k = k;
  g.tile_n = g_tile_n;
  g.error_flag = error_flag;
  g.workspace = workspace;
  g.workspace_bytes = workspace ? workspace_bytes : 0;
  SHARQ_REQUIRE(workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                "workspace must be 16-byte aligned");
  return check_cuda(sharq::run_gemm(g, as_stream(stream)), "sparse_matmul");
}

int sharq_linear_gemm(const void *a_comp, const void *e, const void *sfa_sparse, const void *q_res, const void *sf_res,
                      const void *qw, const void *sfw_sparse, const void *sfw_dense, int m, int n, int k, float alpha,
                      const float *alpha_dev, const void *bias, void *d, int *error_flag, void *stream) {
  return sharq_linear_gemm_ws(a_comp, e, sfa_sparse, q_res, sf_res, qw, sfw_sparse, sfw_dense, m, n, k, alpha, alpha_dev, bias,
                              d, nullptr, 0, error_flag, stream);
}

int sharq_linear_gemm_ws(const void *a_comp, const void *e, const void *sfa_sparse, const void *q_res, const void *sf_res,
                         const void *qw, const void *sfw_sparse, const void *sfw_dense, int m, int n, int k, float alpha,
                         const float *alpha_dev, const void *bias, void *d, void *workspace, size_t workspace_bytes,
                         int *error_flag, void *stream) {
  SHARQ_REQUIRE(m > 0 && n > 0 && k > 0, "M, N, K must be positive");
  SHARQ_REQUIRE(k % 128 == 0, "linear_gemm requires K to be a multiple of 128, got %d", k);
  SHARQ_REQUIRE(a_comp && e && sfa_sparse && q_res && sf_res && qw && sfw_sparse && sfw_dense && d && error_flag,
                "null buffer");
  sharq::GemmArgs g;
  g.a_comp = a_comp;
  g.e = e;
  g.sfa_sparse = sfa_sparse;
  g.a_dense = q_res;
  g.sfa_dense = sf_res;
  g.b = qw;
  g.sfb_sparse = sfw_sparse;
  g.sfb_dense = sfw_dense;
  g.bias = bias;
  g.d = d;
  g.alpha = alpha;
  g.alpha_ptr = alpha_dev;
  g.m = m;
  g.n = n;
  g.k = k;
  g.tile_n = g_tile_n;
  g.error_flag = error_flag;
  g.workspace = workspace;
  g.workspace_bytes = workspace ? workspace_bytes : 0;
  SHARQ_REQUIRE(workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                "workspace must be 16-byte aligned");
  return check_cuda(sharq::run_gemm(g, as_stream(stream)), "linear_gemm");
}

}  // extern "C"
