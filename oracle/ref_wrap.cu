// extern "C" shims around the REFERENCE's own host launchers, so that tests can run the
// reference's CUDA kernels (compiled in place from the reference checkout, never copied)
// next to this project's kernels.  TEST INFRASTRUCTURE ONLY; built by oracle/build_ref.py
// into oracle/_ref/libsharq_ref.so when the reference checkout and CUTLASS headers are
// available.  Declarations below restate the reference's prototypes
// (kernels/include/fused_sparse_prepare.h, shared_weight_nvfp4.h, reorder.cuh, nvfp4.h,
// sparse_nvfp4.h of the reference project).
#include "fused_sparse_prepare.h"
#include "nvfp4.h"
#include "reorder.cuh"
#include "shared_weight_nvfp4.h"
#include "sparse_nvfp4.h"

extern "C" {

int ref_fused_sparse_residual_x(void *x, int m, int n, int k, void *a_comp, void *e, void *q_sparse_dense, void *sf_sparse,
                                void *q_res, void *sf_res) {
  run_fused_sparse_residual_x_bf16_nvfp4((bf16_t *)x, m, n, k, (uint8_t *)a_comp, (uint8_t *)e, (uint8_t *)q_sparse_dense,
                                         (sf_t *)sf_sparse, (uint8_t *)q_res, (sf_t *)sf_res);
  return (int)cudaGetLastError();
}

int ref_rmsnorm_row_stats(void *x, void *gamma, float eps, int m, int k, float *inv_rms, float *row_absmax) {
  run_fused_rmsnorm_row_stats_bf16((bf16_t *)x, (bf16_t *)gamma, eps, m, k, inv_rms, row_absmax);
  return (int)cudaGetLastError();
}

int ref_rmsnorm_sparse_residual_x(void *x, void *gamma, float *inv_rms, const float *scale, int m, int n, int k,
                                  void *a_comp, void *e, void *sf_sparse, void *q_res, void *sf_res) {
  run_fused_rmsnorm_sparse_residual_x_bf16_nvfp4((bf16_t *)x, (bf16_t *)gamma, inv_rms, scale, m, n, k, (uint8_t *)a_comp,
                                                 (uint8_t *)e, nullptr, (sf_t *)sf_sparse, (uint8_t *)q_res,
                                                 (sf_t *)sf_res);
  return (int)cudaGetLastError();
}

int ref_quantize_w32_shared(void *w, int n, int k, void *q, void *sf_sparse, void *sf_dense) {
  run_quantize_w32_bf16_nvfp4_shared((bf16_t *)w, n, k, (uint8_t *)q, (sf_t *)sf_sparse, (sf_t *)sf_dense);
  return (int)cudaGetLastError();
}

// identity reorder, KE = 0, K = 4096 or 14336 (two of the sizes the reference instantiates)
int ref_quantize_x_dense(void *x, int m, int k, int16_t *identity_index, void *q, void *sf) {
  if (k == 4096)
    run_reorder_x_bf16_nvfp4<16, 4096>((bf16_t *)x, m, identity_index, (uint8_t *)q, (sf_t *)sf, k, 0);
  else if (k == 14336)
    run_reorder_x_bf16_nvfp4<16, 14336>((bf16_t *)x, m, identity_index, (uint8_t *)q, (sf_t *)sf, k, 0);
  else if (k == 2048)
    run_reorder_x_bf16_nvfp4<16, 2048>((bf16_t *)x, m, identity_index, (uint8_t *)q, (sf_t *)sf, k, 0);
  else
    return -1;
  return (int)cudaGetLastError();
}

#ifdef SHARQ_REF_WITH_GEMM
// D = bf16(alpha * A.B^T + beta * C): the reference's CUTLASS dense and sparse GEMMs
int ref_matmul_dense(const void *a, const void *b, int m, int n, int k, void *c, void *d, const void *sfa, const void *sfb,
                     float alpha, float beta) {
  matmul_host_nvfp4_bf16((const cutlass::float_e2m1_t *)a, (const cutlass::float_e2m1_t *)b, m, n, k,
                         (cutlass::bfloat16_t *)c, (cutlass::bfloat16_t *)d, (const cutlass::float_ue4m3_t *)sfa,
                         (const cutlass::float_ue4m3_t *)sfb, alpha, beta, nullptr);
  return (int)cudaGetLastError();
}

int ref_matmul_sparse(const void *a_comp, const void *b, const void *e, int m, int n, int k, void *d, const void *sfa,
                      const void *sfb, float alpha) {
  sparse_nvfp4::matmul_host_sparse_nvfp4_bf16((const cutlass::float_e2m1_t *)a_comp, (const cutlass::float_e2m1_t *)b,
                                              (const uint8_t *)e, m, n, k, (cutlass::bfloat16_t *)d, (cutlass::bfloat16_t *)d,
                                              (const cutlass::float_ue4m3_t *)sfa, (const cutlass::float_ue4m3_t *)sfb, alpha,
                                              0.0f, nullptr);
  return (int)cudaGetLastError();
}

#endif  // SHARQ_REF_WITH_GEMM

}  // extern "C"
