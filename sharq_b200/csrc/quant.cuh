// Host launchers of the weight preparation / dense NVFP4 quantisation kernels (quant.cu).
#pragma once
#include <cuda_runtime.h>

namespace sharq {

cudaError_t run_quantize_w32_shared(const void *w, int n, int k, void *qw, void *sf_sparse, void *sf_dense,
                                    cudaStream_t stream);
cudaError_t run_duplicate_sf32_to_sf16(const void *sf32, int rows, int k, void *sf16, cudaStream_t stream);
cudaError_t run_quantize_dense_nvfp4(const void *x, int rows, int k, void *q, void *sf, cudaStream_t stream);
cudaError_t run_compress_sparse_a(const void *a_dense, int m, int k, void *a_comp, void *e, cudaStream_t stream);

}  // namespace sharq
