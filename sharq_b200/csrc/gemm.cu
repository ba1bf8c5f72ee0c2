// Block-scaled FP4 GEMMs for sm_100a, hand-written on tcgen05 / TMEM / TMA:
//   dense NVFP4      D = bf16(alpha * (A . B^T) + beta * C)         (one UE4M3 scale per 16 along K)
//   sparse NVFP4     the same with a pair-wise 4:8 compressed A     (one scale per 32 logical K)
//   fused SharQ      sparse main + dense residual against the SAME weight tile, both
//                    accumulated into one TMEM tile, one epilogue (+ optional bias).
// They replace the reference's CUTLASS-generated kernels behind the same buffers:
//   kernels/src/nvfp4.cu:432-455, kernels/src/sparse_nvfp4.cu:436-460 and the two-launch
//   composition at model/qLinearLayer.py:130-154.
//
// Kernel shape (one output tile of 128 x BN per CTA, K consumed in stages of 256):
//   warp 0    TMA producer: per stage three tensor-map loads (weight tile, dense A tile,
//             compressed A tile; 128-byte / 64-byte swizzle) and plain bulk copies of the
//             metadata tile and the scale-factor tiles, all landing on one mbarrier.
//   warp 1    MMA issuer: copies metadata and scale factors shared -> tensor memory
//             (tcgen05.cp), then issues 2 sparse (K=128) and 4 dense (K=64) MMAs per stage
//             into the same accumulator; tcgen05.commit releases the stage.
//   warps 2-5 epilogue: tcgen05.ld the accumulator, alpha/beta/bias, bf16, store.
// All mbarrier waits are bounded; a timed-out wait sets *error_flag and every role
// drains to the common exit, where tensor memory is released.
#include "common.cuh"
#include "gemm.cuh"
#include "sm100_ptx.cuh"

#include <cstring>
#include <mutex>

namespace sharq {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 256;           // logical K per stage
constexpr int kGemmThreads = 192;  // 6 warps

template <int BN, bool SPARSE, bool DENSE>
struct StageLayout {
  static constexpr int kBands = BN / 128;
  static constexpr int kWBytes = BN * 128;
  static constexpr int kADenseBytes = DENSE ? kBM * 128 : 0;
  static constexpr int kACompBytes = SPARSE ? kBM * 64 : 0;
  static constexpr int kEBytes = SPARSE ? 2048 : 0;
  static constexpr int kSfaSpBytes = SPARSE ? 1024 : 0;
  static constexpr int kSfbSpBytes = SPARSE ? kBands * 1024 : 0;
  static constexpr int kSfaDBytes = DENSE ? 2048 : 0;
  static constexpr int kSfbDBytes = DENSE ? kBands * 2048 : 0;
  static constexpr int kOffW = 0;
  static constexpr int kOffADense = kOffW + kWBytes;
  static constexpr int kOffAComp = kOffADense + kADenseBytes;
  static constexpr int kOffE = kOffAComp + kACompBytes;
  static constexpr int kOffSfaSp = kOffE + kEBytes;
  static constexpr int kOffSfbSp = kOffSfaSp + kSfaSpBytes;
  static constexpr int kOffSfaD = kOffSfbSp + kSfbSpBytes;
  static constexpr int kOffSfbD = kOffSfaD + kSfaDBytes;
  static constexpr int kStageBytes = (kOffSfbD + kSfbDBytes + 1023) / 1024 * 1024;
  static constexpr int kStages = (BN == 256) ? (SPARSE && DENSE ? 3 : 4) : 4;
  // tensor memory columns
  static constexpr int kColAcc = 0;
  static constexpr int kColE = BN;
  static constexpr int kColSfaSp = kColE + 4;
  static constexpr int kColSfbSp = kColSfaSp + 8;
  static constexpr int kColSfaD = kColSfbSp + 2 * (BN / 32);
  static constexpr int kColSfbD = kColSfaD + 16;
  static constexpr int kColEnd = kColSfbD + 4 * (BN / 32);
  static constexpr int kTmemCols = kColEnd <= 256 ? 256 : 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct GemmParams {
  const uint8_t *e;
  const uint8_t *sfa_sparse;
  const uint8_t *sfa_dense;
  const uint8_t *sfb_sparse;
  const uint8_t *sfb_dense;
  const __nv_bfloat16 *c_in;
  const __nv_bfloat16 *bias;
  __nv_bfloat16 *d;
  const float *alpha_ptr;
  float alpha;
  float beta;
  int m, n, k;
  int *error_flag;
};

template <int BN, bool SPARSE, bool DENSE>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a_dense,
                const __grid_constant__ CUtensorMap tm_a_comp, const GemmParams p) {
  using L = StageLayout<BN, SPARSE, DENSE>;
  constexpr int S = L::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + S * L::kStageBytes);
  uint64_t *empty_bar = full_bar + S;
  uint64_t *acc_bar = empty_bar + S;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_bar + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x;
  const int m_tile = blockIdx.y;
  const int k_stages = (p.k + kBK - 1) / kBK;
  const int aligned_m = (p.m + 127) / 128 * 128;
  const int tiles_sp = p.k / 128;  // 512-byte scale tiles per 128-row band, 32-group layout
  const int tiles_d = p.k / 64;    // same, 16-group layout

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
    }
    ptx::mbar_init(acc_bar, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(tmem_slot, L::kTmemCols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      ptx::tma_prefetch_desc(&tm_w);
      if (DENSE) ptx::tma_prefetch_desc(&tm_a_dense);
      if (SPARSE) ptx::tma_prefetch_desc(&tm_a_comp);
      for (int it = 0; it < k_stages; ++it) {
        const int s = it % S;
        const uint32_t ph = (uint32_t)(it / S) & 1u;
        if (!ptx::mbar_wait(empty_bar + s, ph ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicExch(p.error_flag, 1);
          break;
        }
        uint8_t *st = smem + s * L::kStageBytes;
        const int n_sp = SPARSE ? min(2, tiles_sp - 2 * it) : 0;
        const int n_d = DENSE ? min(4, tiles_d - 4 * it) : 0;
        uint32_t tx = L::kWBytes + L::kADenseBytes + L::kACompBytes + L::kEBytes;
        tx += (uint32_t)(n_sp * 512 * (1 + L::kBands) + n_d * 512 * (1 + L::kBands));
        ptx::mbar_arrive_expect_tx(full_bar + s, tx);
        ptx::tma_load_2d(st + L::kOffW, &tm_w, it * 128, n_tile * BN, full_bar + s);
        if (DENSE) {
          ptx::tma_load_2d(st + L::kOffADense, &tm_a_dense, it * 128, m_tile * kBM, full_bar + s);
          ptx::bulk_load_1d(st + L::kOffSfaD, p.sfa_dense + ((size_t)m_tile * tiles_d + 4 * (size_t)it) * 512,
                            (uint32_t)n_d * 512, full_bar + s);
          for (int b = 0; b < L::kBands; ++b)
            ptx::bulk_load_1d(st + L::kOffSfbD + b * 2048,
                              p.sfb_dense + ((size_t)(n_tile * L::kBands + b) * tiles_d + 4 * (size_t)it) * 512,
                              (uint32_t)n_d * 512, full_bar + s);
        }
        if (SPARSE) {
          ptx::tma_load_2d(st + L::kOffAComp, &tm_a_comp, it * 64, m_tile * kBM, full_bar + s);
          ptx::bulk_load_1d(st + L::kOffE, p.e + ((size_t)it * aligned_m + (size_t)m_tile * 128) * 16, 2048,
                            full_bar + s);
          ptx::bulk_load_1d(st + L::kOffSfaSp, p.sfa_sparse + ((size_t)m_tile * tiles_sp + 2 * (size_t)it) * 512,
                            (uint32_t)n_sp * 512, full_bar + s);
          for (int b = 0; b < L::kBands; ++b)
            ptx::bulk_load_1d(st + L::kOffSfbSp + b * 1024,
                              p.sfb_sparse + ((size_t)(n_tile * L::kBands + b) * tiles_sp + 2 * (size_t)it) * 512,
                              (uint32_t)n_sp * 512, full_bar + s);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc_d = ptx::make_idesc_nvf4(kBM, BN, false);
      constexpr uint32_t idesc_s = ptx::make_idesc_nvf4(kBM, BN, true);
      uint32_t accumulate = 0;
      bool ok = true;
      for (int it = 0; it < k_stages && ok; ++it) {
        const int s = it % S;
        const uint32_t ph = (uint32_t)(it / S) & 1u;
        if (!ptx::mbar_wait(full_bar + s, ph, abort_flag)) {
          *abort_flag = 1;
          atomicExch(p.error_flag, 2);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t st = ptx::smem_u32(smem + s * L::kStageBytes);
        const int n_sp = SPARSE ? min(2, tiles_sp - 2 * it) : 0;
        const int n_d = DENSE ? min(4, tiles_d - 4 * it) : 0;
        if (SPARSE) {
          ptx::tmem_cp_128x128b<1>(tmem_base + L::kColE, ptx::make_smem_desc(st + L::kOffE, 128, 0, 0));
          for (int t = 0; t < n_sp; ++t) {
            ptx::tmem_cp_32x128b_warpx4<1>(tmem_base + L::kColSfaSp + 4 * t,
                                           ptx::make_smem_desc(st + L::kOffSfaSp + t * 512, 128, 0, 0));
            for (int b = 0; b < L::kBands; ++b)
              ptx::tmem_cp_32x128b_warpx4<1>(tmem_base + L::kColSfbSp + t * (BN / 32) + 4 * b,
                                             ptx::make_smem_desc(st + L::kOffSfbSp + b * 1024 + t * 512, 128, 0, 0));
          }
        }
        if (DENSE) {
          for (int t = 0; t < n_d; ++t) {
            ptx::tmem_cp_32x128b_warpx4<1>(tmem_base + L::kColSfaD + 4 * t,
                                           ptx::make_smem_desc(st + L::kOffSfaD + t * 512, 128, 0, 0));
            for (int b = 0; b < L::kBands; ++b)
              ptx::tmem_cp_32x128b_warpx4<1>(tmem_base + L::kColSfbD + t * (BN / 32) + 4 * b,
                                             ptx::make_smem_desc(st + L::kOffSfbD + b * 2048 + t * 512, 128, 0, 0));
          }
        }
        if (SPARSE) {
          // compressed A: 64-byte swizzled rows, 32 bytes (128 logical K) per MMA;
          // weight: 128-byte swizzled rows, 64 bytes (128 K) per MMA.
          for (int t = 0; t < n_sp; ++t) {
            uint64_t da = ptx::make_smem_desc(st + L::kOffAComp + t * 32, 512, 16, 4);
            uint64_t db = ptx::make_smem_desc(st + L::kOffW + t * 64, 1024, 16, 2);
            ptx::mma_nvf4_sparse<1>(tmem_base + L::kColAcc, da, db, idesc_s, tmem_base + L::kColSfaSp + 4 * t,
                                    tmem_base + L::kColSfbSp + t * (BN / 32), tmem_base + L::kColE + 2 * t, accumulate);
            accumulate = 1;
          }
        }
        if (DENSE) {
          for (int t = 0; t < n_d; ++t) {
            uint64_t da = ptx::make_smem_desc(st + L::kOffADense + t * 32, 1024, 16, 2);
            uint64_t db = ptx::make_smem_desc(st + L::kOffW + t * 32, 1024, 16, 2);
            ptx::mma_nvf4_dense<1>(tmem_base + L::kColAcc, da, db, idesc_d, tmem_base + L::kColSfaD + 4 * t,
                                   tmem_base + L::kColSfbD + t * (BN / 32), accumulate);
            accumulate = 1;
          }
        }
        ptx::tc_commit<1>(empty_bar + s);
      }
      if (ok) ptx::tc_commit<1>(acc_bar);
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // tensor-memory lane quadrant this warp may read
    const int row = m_tile * kBM + quad * 32 + lane;
    bool ok = ptx::mbar_wait(acc_bar, 0, abort_flag);
    if (!ok) {
      *abort_flag = 1;
      atomicExch(p.error_flag, 3);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      ptx::tc_fence_after();
      const float alpha = p.alpha_ptr ? p.alpha * (*p.alpha_ptr) : p.alpha;
      const float beta = p.beta;
      const bool has_c = (p.c_in != nullptr) && (beta != 0.0f);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t acc[32];
        ptx::tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(L::kColAcc + c0), acc);
        ptx::tmem_ld_wait();
        const int col0 = n_tile * BN + c0;
        if (row < p.m && col0 < p.n) {
          const size_t off = (size_t)row * p.n + col0;
          const bool full = (col0 + 32 <= p.n) && ((p.n & 7) == 0);
#pragma unroll
          for (int v = 0; v < 4; ++v) {  // 8 columns per 16-byte store
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = alpha * __uint_as_float(acc[8 * v + i]);
            if (has_c) {
              if (full) {
                uint4 cv = *reinterpret_cast<const uint4 *>(p.c_in + off + 8 * v);
                uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  f[2 * i] = __fmaf_rn(beta, bf16_bits_to_float(cw[i] & 0xFFFFu), f[2 * i]);
                  f[2 * i + 1] = __fmaf_rn(beta, bf16_bits_to_float(cw[i] >> 16), f[2 * i + 1]);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (col0 + 8 * v + i < p.n) f[i] = __fmaf_rn(beta, __bfloat162float(p.c_in[off + 8 * v + i]), f[i]);
              }
            }
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t lo = float_to_bf16_bits(f[2 * i]), hi = float_to_bf16_bits(f[2 * i + 1]);
              if (p.bias != nullptr) {
                // bias is added to the bf16 result, as a separate bf16 add would
                const int cc = col0 + 8 * v + 2 * i;
                float b0 = cc < p.n ? __bfloat162float(p.bias[cc]) : 0.0f;
                float b1 = cc + 1 < p.n ? __bfloat162float(p.bias[cc + 1]) : 0.0f;
                lo = float_to_bf16_bits(bf16_bits_to_float(lo) + b0);
                hi = float_to_bf16_bits(bf16_bits_to_float(hi) + b1);
              }
              o[i] = lo | (hi << 16);
            }
            if (full) {
              *reinterpret_cast<uint4 *>(p.d + off + 8 * v) = make_uint4(o[0], o[1], o[2], o[3]);
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (col0 + 8 * v + i < p.n)
                  p.d[off + 8 * v + i] = __ushort_as_bfloat16((unsigned short)((o[i >> 1] >> (16 * (i & 1))) & 0xFFFFu));
            }
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, L::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D byte tensor [rows, row_bytes] with a [box_rows, box_bytes] box.
bool make_tmap_bytes(CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                     uint32_t box_bytes, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, bool SPARSE, bool DENSE>
cudaError_t launch(const GemmArgs &a, cudaStream_t stream) {
  using L = StageLayout<BN, SPARSE, DENSE>;
  static bool attr_set[64] = {};
  auto kernel = gemm_kernel<BN, SPARSE, DENSE>;
  int dev = 0;
  cudaError_t de = cudaGetDevice(&dev);
  if (de != cudaSuccess) return de;
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  CUtensorMap tm_w, tm_ad, tm_ac;
  memset(&tm_ad, 0, sizeof(tm_ad));
  memset(&tm_ac, 0, sizeof(tm_ac));
  if (!make_tmap_bytes(&tm_w, a.b, (uint64_t)a.n, (uint64_t)a.k / 2, BN, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return cudaErrorInvalidValue;
  if (DENSE && !make_tmap_bytes(&tm_ad, a.a_dense, (uint64_t)a.m, (uint64_t)a.k / 2, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return cudaErrorInvalidValue;
  if (SPARSE && !make_tmap_bytes(&tm_ac, a.a_comp, (uint64_t)a.m, (uint64_t)a.k / 4, kBM, 64, CU_TENSOR_MAP_SWIZZLE_64B))
    return cudaErrorInvalidValue;
  GemmParams p{};
  p.e = static_cast<const uint8_t *>(a.e);
  p.sfa_sparse = static_cast<const uint8_t *>(a.sfa_sparse);
  p.sfa_dense = static_cast<const uint8_t *>(a.sfa_dense);
  p.sfb_sparse = static_cast<const uint8_t *>(a.sfb_sparse);
  p.sfb_dense = static_cast<const uint8_t *>(a.sfb_dense);
  p.c_in = static_cast<const __nv_bfloat16 *>(a.c_in);
  p.bias = static_cast<const __nv_bfloat16 *>(a.bias);
  p.d = static_cast<__nv_bfloat16 *>(a.d);
  p.alpha_ptr = a.alpha_ptr;
  p.alpha = a.alpha;
  p.beta = a.beta;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.error_flag = a.error_flag;
  dim3 grid((a.n + BN - 1) / BN, (a.m + kBM - 1) / kBM);
  kernel<<<grid, kGemmThreads, L::kSmemBytes, stream>>>(tm_w, tm_ad, tm_ac, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t run_gemm(const GemmArgs &a, cudaStream_t stream) {
  const bool sparse = a.a_comp != nullptr;
  const bool dense = a.a_dense != nullptr;
  if (!sparse && !dense) return cudaErrorInvalidValue;
  const int bn = a.tile_n == 128 ? 128 : (a.tile_n == 256 ? 256 : (a.n % 256 == 0 && a.m > 128 ? 256 : 128));
  if (bn == 256) {
    if (sparse && dense) return launch<256, true, true>(a, stream);
    if (sparse) return launch<256, true, false>(a, stream);
    return launch<256, false, true>(a, stream);
  }
  if (sparse && dense) return launch<128, true, true>(a, stream);
  if (sparse) return launch<128, true, false>(a, stream);
  return launch<128, false, true>(a, stream);
}

}  // namespace sharq
