// Weight preparation and dense NVFP4 quantisation kernels for sm_100a.
//
// Replaces, behind the same buffer formats, the reference's
//   kernels/src/shared_weight_nvfp4.cu:20-189   (32-group shared weight payload, scale duplication)
//   kernels/src/reorder.cu:69-203,381-555 and kernels/src/down.cu:72-233 with identity
//   reorder and KE == 0                         (dense NVFP4 quantisation, 16-group scales)
//   kernels/src/bindings.cpp:164-230            (structured-sparse compressor, debug path)
// These run offline (weights) or in the dense-NVFP4 baseline mode, so they are written
// for clarity: one thread per scale group, 16-byte loads and stores.
#include "common.cuh"
#include "quant.cuh"

namespace sharq {

namespace {

__device__ __forceinline__ void unpack8(const uint4 &v, float *f) {
  uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    f[2 * t] = bf16_bits_to_float(w[t] & 0xFFFFu);
    f[2 * t + 1] = bf16_bits_to_float(w[t] >> 16);
  }
}

// One thread per 32-element group of one weight row.
__global__ void __launch_bounds__(256) quantize_w32_shared_kernel(const __nv_bfloat16 *__restrict__ w, int n, int k,
                                                                   uint8_t *__restrict__ qw,
                                                                   uint8_t *__restrict__ sf_sparse,
                                                                   uint8_t *__restrict__ sf_dense) {
  const int groups = k >> 5;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * groups) return;
  const int row = (int)(idx / groups), g = (int)(idx % groups);
  const uint4 *src = reinterpret_cast<const uint4 *>(w + (size_t)row * k + (size_t)g * 32);
  float x[32];
#pragma unroll
  for (int j = 0; j < 4; ++j) unpack8(__ldg(src + j), x + 8 * j);
  float mx = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fabsf(x[i]));
  float s = fminf(fmaxf(__fdiv_rn(mx, kFp4Max), kScaleEps), kFp8Max);
  uint32_t code = float_to_ue4m3(s);
  float inv = __frcp_rn(ue4m3_to_float(code));
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    out[j] = pack_e2m1x8(__fmul_rn(x[8 * j + 0], inv), __fmul_rn(x[8 * j + 1], inv), __fmul_rn(x[8 * j + 2], inv),
                         __fmul_rn(x[8 * j + 3], inv), __fmul_rn(x[8 * j + 4], inv), __fmul_rn(x[8 * j + 5], inv),
                         __fmul_rn(x[8 * j + 6], inv), __fmul_rn(x[8 * j + 7], inv));
  *reinterpret_cast<uint4 *>(qw + (size_t)row * (k / 2) + (size_t)g * 16) = make_uint4(out[0], out[1], out[2], out[3]);
  sf_sparse[sf_offset(row, g, groups)] = (uint8_t)code;
  // the two 16-group slots of the dense layout are neighbours: one 16-bit store
  *reinterpret_cast<uint16_t *>(sf_dense + sf_offset(row, 2 * g, k / 16)) = (uint16_t)(code | (code << 8));
}

__global__ void __launch_bounds__(256) duplicate_sf32_to_sf16_kernel(const uint8_t *__restrict__ sf32, int rows, int k,
                                                                      uint8_t *__restrict__ sf16) {
  const int groups = k >> 5;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * groups) return;
  const int row = (int)(idx / groups), g = (int)(idx % groups);
  uint32_t code = sf32[sf_offset(row, g, groups)];
  *reinterpret_cast<uint16_t *>(sf16 + sf_offset(row, 2 * g, k / 16)) = (uint16_t)(code | (code << 8));
}

// One thread per 16-element group.
__global__ void __launch_bounds__(256) quantize_dense_nvfp4_kernel(const __nv_bfloat16 *__restrict__ x, int rows, int k,
                                                                    uint8_t *__restrict__ q, uint8_t *__restrict__ sf) {
  const int groups = k >> 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * groups) return;
  const int row = (int)(idx / groups), g = (int)(idx % groups);
  const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)row * k + (size_t)g * 16);
  float v[16];
  unpack8(__ldg(src), v);
  unpack8(__ldg(src + 1), v + 8);
  float mx = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) mx = fmaxf(mx, fabsf(v[i]));
  float s = clamp_val(__fdiv_rn(mx, kFp4Max), kScaleEps, kFp8Max);
  uint32_t code = float_to_ue4m3(s);
  // The reference writes this reciprocal as a double division rounded to float; for
  // every UE4M3 value that equals the correctly rounded float reciprocal.
  float inv = __frcp_rn(ue4m3_to_float(code));
  uint32_t lo = pack_e2m1x8(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv), __fmul_rn(v[2], inv), __fmul_rn(v[3], inv),
                            __fmul_rn(v[4], inv), __fmul_rn(v[5], inv), __fmul_rn(v[6], inv), __fmul_rn(v[7], inv));
  uint32_t hi = pack_e2m1x8(__fmul_rn(v[8], inv), __fmul_rn(v[9], inv), __fmul_rn(v[10], inv), __fmul_rn(v[11], inv),
                            __fmul_rn(v[12], inv), __fmul_rn(v[13], inv), __fmul_rn(v[14], inv), __fmul_rn(v[15], inv));
  *reinterpret_cast<uint2 *>(q + (size_t)row * (k / 2) + (size_t)g * 8) = make_uint2(lo, hi);
  sf[sf_offset(row, g, groups)] = (uint8_t)code;
}

// One thread per 32-element group (four 8-element chunks): a dense payload that
// already holds at most two non-zero bytes per 4-byte chunk -> compressed bytes +
// metadata.  A byte counts as zero when both nibbles are +-0.
__global__ void __launch_bounds__(256) compress_sparse_a_kernel(const uint8_t *__restrict__ a_dense, int m, int k,
                                                                 uint8_t *__restrict__ a_comp, uint8_t *__restrict__ e) {
  const int groups = k >> 5;
  const int aligned_m = (m + 127) / 128 * 128;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)m * groups) return;
  const int row = (int)(idx / groups), g = (int)(idx % groups);
  uint4 v = *reinterpret_cast<const uint4 *>(a_dense + (size_t)row * (k / 2) + (size_t)g * 16);
  uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t comp[2] = {0, 0};
  uint32_t meta = 0;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t idx0 = 0, idx1 = 0, v0 = 0, v1 = 0;
    int cnt = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      uint32_t b = (w[c] >> (8 * p)) & 0xFFu;
      bool nz = (b & 0x77u) != 0;
      if (nz && cnt == 0) {
        idx0 = p;
        v0 = b;
      } else if (nz && cnt == 1) {
        idx1 = p;
        v1 = b;
      }
      cnt += nz ? 1 : 0;
    }
    if (cnt == 1 && idx0 == 3) {
      v1 = v0;
      v0 = 0;
      idx0 = 0;
      idx1 = 3;
    } else if (cnt == 1) {
      v1 = 0;
      idx1 = 3;
    }
    uint32_t two = v0 | (v1 << 8);
    comp[c >> 1] |= (c & 1) ? (two << 16) : two;
    meta |= (idx0 | (idx1 << 2)) << (4 * c);
  }
  *reinterpret_cast<uint2 *>(a_comp + (size_t)row * (k / 4) + (size_t)g * 8) = make_uint2(comp[0], comp[1]);
  *reinterpret_cast<uint16_t *>(e + (size_t)(g / 8) * aligned_m * 16 + (size_t)row * 16 + (size_t)(g % 8) * 2) =
      (uint16_t)meta;
}

inline unsigned blocks_for(long long items) { return (unsigned)((items + 255) / 256); }

}  // namespace

cudaError_t run_quantize_w32_shared(const void *w, int n, int k, void *qw, void *sf_sparse, void *sf_dense,
                                    cudaStream_t stream) {
  cudaError_t err = cudaMemsetAsync(sf_sparse, 0, sf_alloc_bytes(n, k), stream);
  if (err != cudaSuccess) return err;
  err = cudaMemsetAsync(sf_dense, 0, sf_alloc_bytes(n, k), stream);
  if (err != cudaSuccess) return err;
  quantize_w32_shared_kernel<<<blocks_for((long long)n * (k / 32)), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16 *>(w), n, k, static_cast<uint8_t *>(qw), static_cast<uint8_t *>(sf_sparse),
      static_cast<uint8_t *>(sf_dense));
  return cudaGetLastError();
}

cudaError_t run_duplicate_sf32_to_sf16(const void *sf32, int rows, int k, void *sf16, cudaStream_t stream) {
  cudaError_t err = cudaMemsetAsync(sf16, 0, sf_alloc_bytes(rows, k), stream);
  if (err != cudaSuccess) return err;
  duplicate_sf32_to_sf16_kernel<<<blocks_for((long long)rows * (k / 32)), 256, 0, stream>>>(
      static_cast<const uint8_t *>(sf32), rows, k, static_cast<uint8_t *>(sf16));
  return cudaGetLastError();
}

cudaError_t run_quantize_dense_nvfp4(const void *x, int rows, int k, void *q, void *sf, cudaStream_t stream) {
  quantize_dense_nvfp4_kernel<<<blocks_for((long long)rows * (k / 16)), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16 *>(x), rows, k, static_cast<uint8_t *>(q), static_cast<uint8_t *>(sf));
  return cudaGetLastError();
}

cudaError_t run_compress_sparse_a(const void *a_dense, int m, int k, void *a_comp, void *e, cudaStream_t stream) {
  cudaError_t err = cudaMemsetAsync(a_comp, 0, a_comp_bytes(m, k), stream);
  if (err != cudaSuccess) return err;
  err = cudaMemsetAsync(e, 0, e_bytes(m, k), stream);
  if (err != cudaSuccess) return err;
  compress_sparse_a_kernel<<<blocks_for((long long)m * (k / 32)), 256, 0, stream>>>(
      static_cast<const uint8_t *>(a_dense), m, k, static_cast<uint8_t *>(a_comp), static_cast<uint8_t *>(e));
  return cudaGetLastError();
}

}  // namespace sharq
