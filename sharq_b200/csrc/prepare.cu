// Activation prepare kernels for sm_100a: row statistics, and the fused
// [RMSNorm ->] tensor-scale -> pair-wise 4:8 sparse main path + dense NVFP4 residual.
//
// Replaces, behind the same buffer formats, the reference's
//   kernels/src/fused_sparse_prepare.cu:89-251          (prepare of a pre-scaled input)
//   kernels/src/fused_rmsnorm_sparse_prepare.cu:85-325  (row stats + RMSNorm-fused prepare)
//   kernels/src/bindings.cpp:270-274,320-326,337        (zero fills and the tensor-scale glue)
// and the host-side amax / divide passes of model/quantize.py:179-183.
//
// Work split: one thread owns one 32-element group (one sparse scale, two residual
// scales).  A warp covers 4 rows x 8 groups = 4 rows x 256 columns, which makes its
// metadata (4 rows x 16 B) and its packed outputs contiguous per row; a CTA of 8 warps
// covers 32 rows x 256 columns.  Every byte of every output buffer is written by the
// kernel (payload by its owner thread, padding rows/columns and the spare tail of
// each buffer with zeros), so callers may hand in uninitialised memory.
#include "common.cuh"
#include "prepare.cuh"

namespace sharq {

namespace {

constexpr int kRowsPerWarp = 4;
constexpr int kGroupsPerWarp = 8;
constexpr int kWarpsPerCta = 8;
constexpr int kRowsPerCta = kRowsPerWarp * kWarpsPerCta;  // 32
constexpr int kColsPerCta = kGroupsPerWarp * 32;          // 256
constexpr int kPrepareThreads = 32 * kWarpsPerCta;

// Read-only 16-byte load that allocates in L1: a lane reads its 64-byte group with four
// of these and the second load of each 32-byte sector is served by L1.
__device__ __forceinline__ uint4 ld_nc_16(const void *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }

__device__ __forceinline__ uint4 ld_ca_16(const void *p) {
  return *reinterpret_cast<const uint4 *>(p);
}

// ---------------------------------------------------------------------------
// Row statistics.
//   mode kRms : inv_rms[r] = rsqrtf(sum(x^2)/K + eps) with the reference's summation
//               order (each 32-group left to right, then the group sums left to
//               right), and the tensor-wide max of |bf16(x * inv_rms * gamma)|.
//   mode kAbs : only the tensor-wide max of |x|.
// The tensor max is accumulated with an integer atomicMax on the float bits (all
// candidates are non-negative).  One warp per row.
// ---------------------------------------------------------------------------
template <bool kRms>
__global__ void __launch_bounds__(256) row_stats_kernel(const __nv_bfloat16 *__restrict__ x,
                                                         const __nv_bfloat16 *__restrict__ gamma, float eps,
                                                         int m, int k, float *__restrict__ inv_rms,
                                                         unsigned int *__restrict__ amax_bits) {
  extern __shared__ float partial[];  // [warps][k/32]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = k >> 5;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= m) return;
  const __nv_bfloat16 *xr = x + (size_t)row * k;
  float inv = 1.0f;
  float mx = 0.0f;

  if (kRms) {
    float *my = partial + (size_t)warp * groups;
    for (int g = lane; g < groups; g += 32) {
      const uint4 *p = reinterpret_cast<const uint4 *>(xr + (size_t)g * 32);
      float s = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v = ld_ca_16(p + j);
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float a = bf16_bits_to_float(w[t] & 0xFFFFu);
          float b = bf16_bits_to_float(w[t] >> 16);
          s = __fmaf_rn(a, a, s);  // a*a is exact in float, so this equals s + a*a
          s = __fmaf_rn(b, b, s);
        }
      }
      my[g] = s;
    }
    __syncwarp();
    float total = 0.0f;
    if (lane == 0) {
      for (int g = 0; g < groups; ++g) total = __fadd_rn(total, my[g]);
      inv = rsqrtf(__fadd_rn(__fdiv_rn(total, (float)k), eps));
      inv_rms[row] = inv;
    }
    inv = __shfl_sync(0xffffffffu, inv, 0);
  }

  for (int c = lane; c < (k >> 3); c += 32) {
    uint4 v = ld_ca_16(reinterpret_cast<const uint4 *>(xr) + c);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if (kRms) {
      uint4 gv = *(reinterpret_cast<const uint4 *>(gamma) + c);
      uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float a = __fmul_rn(__fmul_rn(bf16_bits_to_float(w[t] & 0xFFFFu), inv), bf16_bits_to_float(gw[t] & 0xFFFFu));
        float b = __fmul_rn(__fmul_rn(bf16_bits_to_float(w[t] >> 16), inv), bf16_bits_to_float(gw[t] >> 16));
        mx = fmaxf(mx, fabsf(bf16_bits_to_float(float_to_bf16_bits(a))));
        mx = fmaxf(mx, fabsf(bf16_bits_to_float(float_to_bf16_bits(b))));
      }
    } else {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        mx = fmaxf(mx, fabsf(bf16_bits_to_float(w[t] & 0xFFFFu)));
        mx = fmaxf(mx, fabsf(bf16_bits_to_float(w[t] >> 16)));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) atomicMax(amax_bits, __float_as_uint(mx));
}

// ---------------------------------------------------------------------------
// The 32-element group: selection, sparse quantisation, residual quantisation.
// ---------------------------------------------------------------------------
struct GroupOut {
  uint32_t q_res[4];     // 16 B dense residual payload
  uint32_t a_comp[2];    // 8 B compressed sparse payload
  uint32_t q_sparse[4];  // 16 B dense sparse payload (debug output only)
  uint32_t meta;         // 2 B metadata (4 nibbles)
  uint32_t sf_sparse;    // 1 B
  uint32_t sf_res;       // 2 B (first 16-group in the low byte)
};

__device__ __forceinline__ float scale_from_max(float mx, uint32_t &code) {
  float s = clamp_val(__fdiv_rn(mx, kFp4Max), kScaleEps, kFp8Max);
  code = float_to_ue4m3(s);
  return ue4m3_to_float(code);
}

template <bool kDebug>
__device__ __forceinline__ void quantize_group32(float (&x)[32], GroupOut &o) {
  // -- pair selection per 8-element chunk (strict '>' : the earlier pair wins ties)
  uint32_t keep_pairs = 0;  // bit (4*chunk + pair)
  uint32_t meta = 0;
  uint32_t sel[4];          // idx0 | idx1 << 2 per chunk
  float sparse_max = 0.0f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float best0 = -1.0f, best1 = -1.0f;
    int i0 = 0, i1 = 1;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      float score = fmaxf(fabsf(x[8 * c + 2 * p]), fabsf(x[8 * c + 2 * p + 1]));
      bool gt0 = score > best0;
      bool gt1 = score > best1;
      // order of updates mirrors: if (gt0) {best1=best0; i1=i0; best0=score; i0=p;} else if (gt1) {best1=score; i1=p;}
      best1 = gt0 ? best0 : (gt1 ? score : best1);
      i1 = gt0 ? i0 : (gt1 ? p : i1);
      best0 = gt0 ? score : best0;
      i0 = gt0 ? p : i0;
    }
    int lo = min(i0, i1), hi = max(i0, i1);
    sel[c] = (uint32_t)(lo | (hi << 2));
    meta |= sel[c] << (4 * c);
    keep_pairs |= ((1u << lo) | (1u << hi)) << (4 * c);
    // best0/best1 are the two kept pair scores, so their max is the kept absmax
    sparse_max = fmaxf(sparse_max, fmaxf(best0, best1));
  }
  o.meta = meta;

  // -- sparse main path scale (one UE4M3 per 32 logical elements)
  uint32_t s_code;
  float s_q = scale_from_max(sparse_max, s_code);
  float s_r = __frcp_rn(s_q);
  o.sf_sparse = s_code;
  float half_s = 0.5f * s_q;  // exact

  // -- quantise every pair, keep the selected ones, form the residual
  float r[32];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    // the 4 pair-bytes of this chunk: quantise all 8 values, then mask to the kept pairs
    uint32_t all4 = pack_e2m1x8(__fmul_rn(x[8 * c + 0], s_r), __fmul_rn(x[8 * c + 1], s_r),
                                __fmul_rn(x[8 * c + 2], s_r), __fmul_rn(x[8 * c + 3], s_r),
                                __fmul_rn(x[8 * c + 4], s_r), __fmul_rn(x[8 * c + 5], s_r),
                                __fmul_rn(x[8 * c + 6], s_r), __fmul_rn(x[8 * c + 7], s_r));
    uint32_t dense4 = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int i = 8 * c + 2 * p;
      bool keep = (keep_pairs >> (4 * c + p)) & 1u;
      uint32_t byte = (all4 >> (8 * p)) & 0xFFu;
      float d0 = (float)e2m1_twice_magnitude(byte);
      float d1 = (float)e2m1_twice_magnitude(byte >> 4);
      d0 = (byte & 0x08u) ? -d0 : d0;
      d1 = (byte & 0x80u) ? -d1 : d1;
      // x - q*s with q*s = d * (s/2) exact, single rounding
      float r0 = __fmaf_rn(-d0, half_s, x[i]);
      float r1 = __fmaf_rn(-d1, half_s, x[i + 1]);
      r[i] = keep ? r0 : x[i];
      r[i + 1] = keep ? r1 : x[i + 1];
      dense4 |= keep ? (0xFFu << (8 * p)) : 0u;
    }
    dense4 &= all4;
    if (kDebug) o.q_sparse[c] = dense4;
    uint32_t b0 = (dense4 >> (8 * (sel[c] & 3u))) & 0xFFu;
    uint32_t b1 = (dense4 >> (8 * (sel[c] >> 2))) & 0xFFu;
    uint32_t two = b0 | (b1 << 8);
    if (c & 1)
      o.a_comp[c >> 1] |= two << 16;
    else
      o.a_comp[c >> 1] = two;
  }

  // -- dense residual, one scale per 16
  uint32_t sf_res = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) mx = fmaxf(mx, fabsf(r[16 * h + i]));
    uint32_t code;
    float rq = scale_from_max(mx, code);
    float rr = __frcp_rn(rq);
    sf_res |= code << (8 * h);
#pragma unroll
    for (int wv = 0; wv < 2; ++wv) {
      const int i = 16 * h + 8 * wv;
      uint32_t word = pack_e2m1x8(__fmul_rn(r[i + 0], rr), __fmul_rn(r[i + 1], rr), __fmul_rn(r[i + 2], rr),
                                  __fmul_rn(r[i + 3], rr), __fmul_rn(r[i + 4], rr), __fmul_rn(r[i + 5], rr),
                                  __fmul_rn(r[i + 6], rr), __fmul_rn(r[i + 7], rr));
      o.q_res[2 * h + wv] = word;
    }
  }
  o.sf_res = sf_res;
}

// ---------------------------------------------------------------------------
// Prepare kernel.
//   kMode 0: input already scaled (drop-in for fused_sparse_residual_quantize_x)
//   kMode 1: RMSNorm + tensor scale inline (needs inv_rms and the tensor absmax)
//   kMode 2: tensor scale inline only (x / scale rounded to bf16), scale from absmax
// grid.x = K tiles of 256 columns, grid.y = row tiles of 32 rows up to ceil128(M),
// plus kTailCtas extra CTAs in grid.y that zero the spare tail of each buffer.
// ---------------------------------------------------------------------------
struct PrepareParams {
  const __nv_bfloat16 *x;
  const __nv_bfloat16 *gamma;
  const float *inv_rms;
  const unsigned int *amax_bits;
  float *scale_out;  // optional, written by one thread (modes 1, 2)
  uint8_t *a_comp;
  uint8_t *e;
  uint8_t *q_sparse_dense;  // debug only
  uint8_t *sfa_sparse;
  uint8_t *q_res;
  uint8_t *sf_res;
  int m, k;
  int row_tiles;  // ceil128(m) / 32
};

constexpr int kTailCtas = 4;

__device__ __forceinline__ void zero_range(uint8_t *base, size_t begin, size_t end, int worker, int workers) {
  if (base == nullptr || begin >= end) return;
  // byte-wise head until 16-byte alignment, then 16-byte stores
  size_t a = (begin + 15) & ~(size_t)15;
  if (a > end) a = end;
  for (size_t i = begin + worker; i < a; i += workers) base[i] = 0;
  size_t n16 = (end - a) / 16;
  uint4 z = make_uint4(0, 0, 0, 0);
  for (size_t i = worker; i < n16; i += workers) reinterpret_cast<uint4 *>(base + a)[i] = z;
  for (size_t i = a + n16 * 16 + worker; i < end; i += workers) base[i] = 0;
}

template <int kMode, bool kDebug>
__global__ void __launch_bounds__(kPrepareThreads) prepare_kernel(const PrepareParams p) {
  const int m = p.m, k = p.k;
  const int groups32 = k >> 5;
  const int aligned_m = (m + 127) / 128 * 128;

  if ((int)blockIdx.y >= p.row_tiles) {
    // tail CTAs: zero what no owner thread writes
    const int worker = ((int)blockIdx.y - p.row_tiles) * gridDim.x * blockDim.x + blockIdx.x * blockDim.x + threadIdx.x;
    const int workers = kTailCtas * gridDim.x * blockDim.x;
    const size_t bands = (size_t)aligned_m / 128;
    zero_range(p.sfa_sparse, bands * (size_t)(groups32 / 4) * 512, sf_alloc_bytes(m, k), worker, workers);
    zero_range(p.sf_res, bands * (size_t)(k / 16 / 4) * 512, sf_alloc_bytes(m, k), worker, workers);
    if (!kDebug) zero_range(p.a_comp, (size_t)m * (k / 4), a_comp_bytes(m, k), worker, workers);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y * kRowsPerCta + warp * kRowsPerWarp + (lane >> 3);
  const int group = blockIdx.x * kGroupsPerWarp + (lane & 7);
  const bool row_ok = row < m;
  const bool col_ok = group < groups32;
  const bool live = row_ok && col_ok;

  GroupOut o;
  o.a_comp[0] = o.a_comp[1] = 0;
  o.meta = 0;
  o.sf_sparse = 0;
  o.sf_res = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.q_res[i] = o.q_sparse[i] = 0;

  if (live) {
    float x[32];
    const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (size_t)row * k + (size_t)group * 32);
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = ld_nc_16(src + j);

    float inv = 1.0f, scale = 1.0f;
    if (kMode != 0) {
      float amax = __uint_as_float(*p.amax_bits);
      // ATen divides a CUDA tensor by a host scalar by multiplying with the float
      // reciprocal; clamp(min=1e-9) follows (kernels/src/bindings.cpp:337 of the reference).
      scale = fmaxf(__fmul_rn(amax, 1.0f / 2688.0f), 1.0e-9f);
      if (p.scale_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *p.scale_out = scale;
    }
    if (kMode == 1) inv = p.inv_rms[row];

#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
      uint32_t gw[4] = {0, 0, 0, 0};
      if (kMode == 1) {
        uint4 gv = *(reinterpret_cast<const uint4 *>(p.gamma + (size_t)group * 32) + j);
        gw[0] = gv.x; gw[1] = gv.y; gw[2] = gv.z; gw[3] = gv.w;
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float a = bf16_bits_to_float(w[t] & 0xFFFFu);
        float b = bf16_bits_to_float(w[t] >> 16);
        if (kMode == 1) {
          a = __fmul_rn(__fmul_rn(a, inv), bf16_bits_to_float(gw[t] & 0xFFFFu));
          b = __fmul_rn(__fmul_rn(b, inv), bf16_bits_to_float(gw[t] >> 16));
          a = bf16_bits_to_float(float_to_bf16_bits(a));
          b = bf16_bits_to_float(float_to_bf16_bits(b));
        }
        if (kMode != 0) {
          a = bf16_bits_to_float(float_to_bf16_bits(__fdiv_rn(a, scale)));
          b = bf16_bits_to_float(float_to_bf16_bits(__fdiv_rn(b, scale)));
        }
        x[8 * j + 2 * t] = a;
        x[8 * j + 2 * t + 1] = b;
      }
    }
    quantize_group32<kDebug>(x, o);
  }

  // ---- stores
  if (live) {
    uint4 q = make_uint4(o.q_res[0], o.q_res[1], o.q_res[2], o.q_res[3]);
    *reinterpret_cast<uint4 *>(p.q_res + (size_t)row * (k / 2) + (size_t)group * 16) = q;
    if (kDebug) {
      uint4 qs = make_uint4(o.q_sparse[0], o.q_sparse[1], o.q_sparse[2], o.q_sparse[3]);
      *reinterpret_cast<uint4 *>(p.q_sparse_dense + (size_t)row * (k / 2) + (size_t)group * 16) = qs;
    } else {
      *reinterpret_cast<uint2 *>(p.a_comp + (size_t)row * (k / 4) + (size_t)group * 8) = make_uint2(o.a_comp[0], o.a_comp[1]);
    }
  }
  // Metadata: rows up to ceil128(M), columns up to ceil256(K); dead lanes write zeros.
  // One warp writes 4 rows x 16 B = 64 contiguous bytes.
  if (!kDebug) {
    // combine the 16-bit metadata of two neighbouring groups into one 32-bit store
    uint32_t mine = o.meta & 0xFFFFu;
    uint32_t other = __shfl_down_sync(0xffffffffu, mine, 1);
    if ((lane & 1) == 0) {
      uint8_t *dst = p.e + (size_t)blockIdx.x * aligned_m * 16 + (size_t)row * 16 + (size_t)(lane & 7) * 2;
      *reinterpret_cast<uint32_t *>(dst) = mine | (other << 16);
    }
  }
  // Scale factors: 4 neighbouring groups share one 32-bit word of the sparse layout,
  // 2 neighbouring groups (4 residual scales) one word of the dense layout.
  {
    uint32_t s = o.sf_sparse;
    uint32_t s1 = __shfl_down_sync(0xffffffffu, s, 1);
    uint32_t s2 = __shfl_down_sync(0xffffffffu, s, 2);
    uint32_t s3 = __shfl_down_sync(0xffffffffu, s, 3);
    uint32_t r2 = o.sf_res;
    uint32_t r2n = __shfl_down_sync(0xffffffffu, r2, 1);
    if (col_ok) {
      if ((lane & 3) == 0)
        *reinterpret_cast<uint32_t *>(p.sfa_sparse + sf_offset(row, group, groups32)) = s | (s1 << 8) | (s2 << 16) | (s3 << 24);
      if ((lane & 1) == 0)
        *reinterpret_cast<uint32_t *>(p.sf_res + sf_offset(row, 2 * group, k / 16)) = r2 | (r2n << 16);
    }
  }
}

}  // namespace

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------

size_t prepare_workspace_bytes(int m) { return 256 + (size_t)m * sizeof(float); }

static cudaError_t launch_prepare(int mode, bool debug, const PrepareParams &p, cudaStream_t stream) {
  dim3 grid((p.k + kColsPerCta - 1) / kColsPerCta, p.row_tiles + kTailCtas);
  dim3 block(kPrepareThreads);
  if (debug) {
    prepare_kernel<0, true><<<grid, block, 0, stream>>>(p);
  } else if (mode == 0) {
    prepare_kernel<0, false><<<grid, block, 0, stream>>>(p);
  } else if (mode == 1) {
    prepare_kernel<1, false><<<grid, block, 0, stream>>>(p);
  } else {
    prepare_kernel<2, false><<<grid, block, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

cudaError_t run_prepare(const void *x, int m, int k, void *a_comp, void *e, void *q_sparse_dense,
                        void *sfa_sparse, void *q_res, void *sf_res, cudaStream_t stream) {
  PrepareParams p{};
  p.x = static_cast<const __nv_bfloat16 *>(x);
  p.a_comp = static_cast<uint8_t *>(a_comp);
  p.e = static_cast<uint8_t *>(e);
  p.q_sparse_dense = static_cast<uint8_t *>(q_sparse_dense);
  p.sfa_sparse = static_cast<uint8_t *>(sfa_sparse);
  p.q_res = static_cast<uint8_t *>(q_res);
  p.sf_res = static_cast<uint8_t *>(sf_res);
  p.m = m;
  p.k = k;
  p.row_tiles = (m + 127) / 128 * 128 / kRowsPerCta;
  return launch_prepare(0, q_sparse_dense != nullptr, p, stream);
}

cudaError_t run_scaled_prepare(const void *x, const void *gamma, float eps, int m, int k, void *workspace,
                               float *inv_rms_external, void *a_comp, void *e, void *sfa_sparse, void *q_res,
                               void *sf_res, float *scale_out, cudaStream_t stream) {
  // workspace: [0,4) tensor absmax bits; [256, 256+4m) inv_rms
  auto *amax_bits = static_cast<unsigned int *>(workspace);
  float *inv_rms = inv_rms_external ? inv_rms_external
                                    : reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + 256);
  cudaError_t err = cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int), stream);
  if (err != cudaSuccess) return err;
  const int warps = 8;
  dim3 grid((m + warps - 1) / warps), block(32 * warps);
  const bool rms = gamma != nullptr;
  if (rms) {
    size_t smem = (size_t)warps * (k / 32) * sizeof(float);
    if (smem > 48 * 1024) {
      err = cudaFuncSetAttribute(row_stats_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return err;
    }
    row_stats_kernel<true><<<grid, block, smem, stream>>>(static_cast<const __nv_bfloat16 *>(x),
                                                         static_cast<const __nv_bfloat16 *>(gamma), eps, m, k,
                                                         inv_rms, amax_bits);
  } else {
    row_stats_kernel<false><<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), nullptr, 0.0f, m, k,
                                                        nullptr, amax_bits);
  }
  err = cudaGetLastError();
  if (err != cudaSuccess) return err;

  PrepareParams p{};
  p.x = static_cast<const __nv_bfloat16 *>(x);
  p.gamma = static_cast<const __nv_bfloat16 *>(gamma);
  p.inv_rms = inv_rms;
  p.amax_bits = amax_bits;
  p.scale_out = scale_out;
  p.a_comp = static_cast<uint8_t *>(a_comp);
  p.e = static_cast<uint8_t *>(e);
  p.sfa_sparse = static_cast<uint8_t *>(sfa_sparse);
  p.q_res = static_cast<uint8_t *>(q_res);
  p.sf_res = static_cast<uint8_t *>(sf_res);
  p.m = m;
  p.k = k;
  p.row_tiles = (m + 127) / 128 * 128 / kRowsPerCta;
  return launch_prepare(rms ? 1 : 2, false, p, stream);
}

}  // namespace sharq
