// Activation prepare kernels for sm_100a: row statistics, and the fused
// [RMSNorm ->] tensor-scale -> pair-wise 4:8 sparse main path + dense NVFP4 residual.
//
// Replaces, behind the same buffer formats, the reference's
//   kernels/src/fused_sparse_prepare.cu:89-251          (prepare of a pre-scaled input)
//   kernels/src/fused_rmsnorm_sparse_prepare.cu:85-325  (row stats + RMSNorm-fused prepare)
//   kernels/src/bindings.cpp:270-274,320-326,337        (zero fills and the tensor-scale glue)
// and the host-side amax / divide passes of model/quantize.py:179-183.
//
// Work split of the prepare kernel: one thread owns one 32-element group (one sparse scale,
// two residual scales).  A warp covers 4 rows x 8 groups = 4 rows x 256 columns, which makes
// its metadata (4 rows x 16 B) and its packed outputs contiguous per row; a CTA of 8 warps
// covers 32 rows x 256 columns.  Every byte of every output buffer is written by the kernel
// (payload by its owner thread, padding rows/columns and the spare tail of each buffer with
// zeros), so callers may hand in uninitialised memory.
//
// The kernel is instruction-bound, so the arithmetic is arranged to need few instructions
// while producing exactly the reference's bits:
//   * pair selection on integer keys: the pair score max(|a|,|b|) of two bf16-exact values
//     has 16 zero low bits as a float, so `bits | (3 - pair)` is a key whose integer order is
//     "larger score first, earlier pair first" - the reference's strict-'>' scan order;
//   * scale value and reciprocal of the 126 possible UE4M3 codes come from a shared-memory
//     table filled with ue4m3 -> float and the IEEE reciprocal;
//   * e2m1 encode/decode use the hardware conversions; x - q*s is one FMA (q*s is exact);
//   * x / scale (tensor scale) is y * (1/scale) when that product is provably on the same side
//     of every bf16 rounding boundary as the IEEE quotient, and an IEEE division otherwise.
#include "common.cuh"
#include "prepare.cuh"
#include "prepare_device.cuh"

#include <cstdlib>

namespace sharq {

using namespace prep;

namespace {

constexpr int kRowsPerWarp = 4;
constexpr int kGroupsPerWarp = 8;
constexpr int kWarpsPerCta = 8;
constexpr int kRowsPerCta = kRowsPerWarp * kWarpsPerCta;  // 32
constexpr int kColsPerCta = kGroupsPerWarp * 32;          // 256
constexpr int kPrepareThreads = 32 * kWarpsPerCta;

// Raise the tensor absmax (non-negative float bits, integer order = float order).  The read
// first keeps the number of same-address atomics small once the maximum has settled.
__device__ __forceinline__ void raise_amax(unsigned int *amax_bits, float mx) {
  const unsigned int bits = __float_as_uint(mx);
  if (bits > *reinterpret_cast<volatile unsigned int *>(amax_bits)) atomicMax(amax_bits, bits);
}

// ---------------------------------------------------------------------------
// Row statistics for the RMSNorm path, one CTA per row, one thread per 32-element group:
//   inv_rms[r] = rsqrtf(sum(x^2)/K + eps) with the reference's summation order (each group
//   left to right - an FMA chain whose products are exact - then the group sums left to
//   right by one thread), and the tensor-wide max of |bf16(x * inv_rms * gamma)|.
// Many rows are resident per SM, so the serial sums of different rows overlap.
// ---------------------------------------------------------------------------
// With kAdd the row is first formed as bf16(x + residual) (the decoder's residual add, rounded
// like the ATen add), stored to sum_out, and the statistics are those of the sum.
template <bool kAdd>
__global__ void __launch_bounds__(1024, 2) rms_stats_kernel(const __nv_bfloat16 *__restrict__ x,
                                                          const __nv_bfloat16 *__restrict__ residual,
                                                          __nv_bfloat16 *__restrict__ sum_out,
                                                          const __nv_bfloat16 *__restrict__ gamma, float eps, int k,
                                                          float *__restrict__ inv_rms,
                                                          unsigned int *__restrict__ amax_bits) {
  extern __shared__ float partial[];  // [k/32] group sums, then [0] is reused for inv_rms
  __shared__ float warp_max[32];
  const int groups = k >> 5;
  const int g = threadIdx.x;
  const int row = blockIdx.x;
  const bool live = g < groups;
  uint32_t w[16];
  if (live) {
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)row * k + (size_t)g * 32);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 v = __ldg(src + j);
      w[4 * j + 0] = v.x;
      w[4 * j + 1] = v.y;
      w[4 * j + 2] = v.z;
      w[4 * j + 3] = v.w;
    }
    if (kAdd) {
      const uint4 *rsrc = reinterpret_cast<const uint4 *>(residual + (size_t)row * k + (size_t)g * 32);
      uint4 *dst = reinterpret_cast<uint4 *>(sum_out + (size_t)row * k + (size_t)g * 32);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 r = __ldg(rsrc + j);
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int t = 0; t < 4; ++t)
          w[4 * j + t] = pack_bf16x2(__fadd_rn(lo_f(w[4 * j + t]), lo_f(rw[t])), __fadd_rn(hi_f(w[4 * j + t]), hi_f(rw[t])));
        dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
      }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float a = lo_f(w[i]), b = hi_f(w[i]);
      s = __fmaf_rn(a, a, s);  // a*a is exact in float, so this equals s + a*a
      s = __fmaf_rn(b, b, s);
    }
    partial[g] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.0f;
    for (int i = 0; i < groups; i += 4) {  // groups is a multiple of 4 (K % 128 == 0)
      float4 v = *reinterpret_cast<const float4 *>(partial + i);
      total = __fadd_rn(total, v.x);
      total = __fadd_rn(total, v.y);
      total = __fadd_rn(total, v.z);
      total = __fadd_rn(total, v.w);
    }
    float inv = rsqrtf(__fadd_rn(__fdiv_rn(total, (float)k), eps));
    inv_rms[row] = inv;
    warp_max[31] = inv;  // slot 31 is free: at most 32 warps, reduction uses [0, nwarps)
  }
  __syncthreads();
  const float inv = warp_max[31];
  __syncthreads();
  float mx = 0.0f;
  if (live) {
    const uint4 *gsrc = reinterpret_cast<const uint4 *>(gamma + (size_t)g * 32);
    __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 gv = __ldg(gsrc + j);
      uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float a = __fmul_rn(__fmul_rn(lo_f(w[4 * j + t]), inv), lo_f(gw[t]));
        float b = __fmul_rn(__fmul_rn(hi_f(w[4 * j + t]), inv), hi_f(gw[t]));
        m2 = __hmax2(m2, __habs2(__floats2bfloat162_rn(a, b)));
      }
    }
    mx = fmaxf(__bfloat162float(m2.x), __bfloat162float(m2.y));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  if (lane == 0) warp_max[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    mx = lane < nwarps ? warp_max[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) raise_amax(amax_bits, mx);
  }
}

// Tensor-wide max |x| of a bf16 tensor (non-RMSNorm path): flat grid-stride reduction.
__global__ void __launch_bounds__(256) abs_stats_kernel(const __nv_bfloat16 *__restrict__ x, size_t n16,
                                                         unsigned int *__restrict__ amax_bits) {
  __shared__ float warp_max[8];
  __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);
  const uint4 *src = reinterpret_cast<const uint4 *>(x);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = (i + u * stride < n16) ? __ldg(src + i + u * stride) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      m2 = __hmax2(m2, __habs2(*reinterpret_cast<__nv_bfloat162 *>(&v[u].x)));
      m2 = __hmax2(m2, __habs2(*reinterpret_cast<__nv_bfloat162 *>(&v[u].y)));
      m2 = __hmax2(m2, __habs2(*reinterpret_cast<__nv_bfloat162 *>(&v[u].z)));
      m2 = __hmax2(m2, __habs2(*reinterpret_cast<__nv_bfloat162 *>(&v[u].w)));
    }
  }
  float mx = fmaxf(__bfloat162float(m2.x), __bfloat162float(m2.y));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) warp_max[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    mx = lane < 8 ? warp_max[lane] : 0.0f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) raise_amax(amax_bits, mx);
  }
}

// ---------------------------------------------------------------------------
// Prepare kernel.
//   kMode 0: input already scaled (drop-in for fused_sparse_residual_quantize_x)
//   kMode 1: RMSNorm + tensor scale inline (needs inv_rms and the tensor absmax)
//   kMode 2: tensor scale inline only (x / scale rounded to bf16), scale from absmax
// Persistent: a fixed number of CTAs per SM loops over 32-row x 256-column tiles (rows up to
// ceil128(M)); every CTA first helps zero the spare tail of each buffer.
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
  // grouped activation of a mixture-of-experts layer (mode 2, absmax ready): rows sorted by group in
  // 256-row units; unit_group[u] < 0 = unit without rows; amax_bits and scale_vec_out have `groups` entries
  const int *unit_group;
  float *scale_vec_out;
  int groups;
  const int *src_row;  // optional gather: output row r is prepared from input row src_row[r] (< 0: a padding row of zeros)
};

constexpr int kPrepareCtasPerSm = 3;
constexpr size_t kInlineAbsmaxElements = 256 * 1024;  // up to 512 KB of input is scanned by every CTA

// kCtas: resident CTAs per SM the register allocation aims at.  The tensor-scale mode runs
// fastest with two (no spills) except on a gathered activation (src_row), where the third CTA
// hides more of the gather's latency (measured: 2048 x 14336 43.3 -> 41.1 us with two,
// 34816 x 4096 grouped 253 -> 264 us).
template <int kMode, bool kDebug, int kCtas = kPrepareCtasPerSm>
__global__ void __launch_bounds__(kPrepareThreads, kCtas) prepare_kernel(const PrepareParams p) {
  const int m = p.m, k = p.k;
  const int groups32 = k >> 5;
  const int aligned_m = (m + 127) / 128 * 128;

  __shared__ ScaleTables tbl;
  extern __shared__ uint4 gamma_smem[];  // mode 1: the whole RMSNorm weight, k bf16
  if (threadIdx.x < 128) {
    const float v = ue4m3_to_float(threadIdx.x);
    tbl.value[threadIdx.x] = v;
    tbl.recip[threadIdx.x] = __frcp_rn(v);  // code 0 is never looked up (scales are clamped to >= 2^-9)
  }
  if (kMode == 1) {
    const uint4 *gsrc = reinterpret_cast<const uint4 *>(p.gamma);
    for (int i = threadIdx.x; i < k / 8; i += blockDim.x) gamma_smem[i] = __ldg(gsrc + i);
  }
  __syncthreads();

  // zero what no owner thread writes: the spare tail of the scale buffers and of A_comp
  {
    const int worker = blockIdx.x * blockDim.x + threadIdx.x;
    const int workers = gridDim.x * blockDim.x;
    const size_t bands = (size_t)aligned_m / 128;
    zero_range(p.sfa_sparse, bands * (size_t)(groups32 / 4) * 512, sf_alloc_bytes(m, k), worker, workers);
    zero_range(p.sf_res, bands * (size_t)(k / 16 / 4) * 512, sf_alloc_bytes(m, k), worker, workers);
    if (!kDebug) zero_range(p.a_comp, (size_t)m * (k / 4), a_comp_bytes(m, k), worker, workers);
  }

  float scale = 1.0f, recip = 1.0f;
  if (kMode != 0) {
    float amax;
    if (kMode == 2 && p.amax_bits == nullptr) {
      // Small input (a decode step): every CTA finds max|x| of the whole tensor itself, which
      // replaces the memset and the statistics launch; the tensor is read from L2.
      __shared__ float cta_max[kWarpsPerCta];
      const uint4 *all = reinterpret_cast<const uint4 *>(p.x);
      const size_t n16 = (size_t)m * k / 8;
      __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);
      for (size_t i = threadIdx.x; i < n16; i += blockDim.x) {
        const uint4 v = __ldg(all + i);
        m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&v.x)));
        m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&v.y)));
        m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&v.z)));
        m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&v.w)));
      }
      float mx = fmaxf(__bfloat162float(m2.x), __bfloat162float(m2.y));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if ((threadIdx.x & 31) == 0) cta_max[threadIdx.x >> 5] = mx;
      __syncthreads();
      mx = cta_max[0];
#pragma unroll
      for (int w = 1; w < kWarpsPerCta; ++w) mx = fmaxf(mx, cta_max[w]);
      amax = mx;
    } else {
      amax = __uint_as_float(*p.amax_bits);
    }
    // ATen divides a CUDA tensor by a host scalar by multiplying with the float
    // reciprocal; clamp(min=1e-9) follows (kernels/src/bindings.cpp:337 of the reference).
    scale = fmaxf(__fmul_rn(amax, 1.0f / 2688.0f), 1.0e-9f);
    if (p.scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *p.scale_out = scale;
    if (kMode == 2 && p.unit_group != nullptr && blockIdx.x == 0 && (int)threadIdx.x < p.groups)
      p.scale_vec_out[threadIdx.x] = fmaxf(__fmul_rn(__uint_as_float(p.amax_bits[threadIdx.x]), 1.0f / 2688.0f), 1.0e-9f);
    if (kMode == 2) scale = round_to_bf16(scale);  // the divisor of the non-RMSNorm path, see round_to_bf16
    recip = __frcp_rn(scale);
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (k + kColsPerCta - 1) / kColsPerCta;
  const int total_tiles = k_tiles * p.row_tiles;
  const int row_in_tile = warp * kRowsPerWarp + (lane >> 3);
  const int group_in_tile = lane & 7;

  // persistent loop over 32-row x 256-column tiles; the next tile's 64 bytes are loaded
  // before the current tile is processed, so the loads overlap the arithmetic
  uint4 next[4];
  float next_inv = 0.0f;
  bool next_row_ok = true;
  auto issue_loads = [&](int tile) {
    const int row = (tile / k_tiles) * kRowsPerCta + row_in_tile;
    const int group = (tile % k_tiles) * kGroupsPerWarp + group_in_tile;
    if (tile < total_tiles && row < m && group < groups32) {
      int in_row = row;
      if (kMode == 2 && p.src_row != nullptr) in_row = p.src_row[row];
      next_row_ok = in_row >= 0;
      if (in_row >= 0) {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (size_t)in_row * k + (size_t)group * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) next[j] = __ldg(src + j);
      }
      if (kMode == 1) next_inv = p.inv_rms[row];
    }
  };
  issue_loads(blockIdx.x);

  for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const int k_tile = tile % k_tiles;
    const int row = (tile / k_tiles) * kRowsPerCta + row_in_tile;
    const int group = k_tile * kGroupsPerWarp + group_in_tile;
    const bool col_ok = group < groups32;
    bool live = row < m && col_ok;
    float t_scale = scale, t_recip = recip;
    if (kMode == 2 && p.unit_group != nullptr) {  // per-group tensor scale; a 32-row tile lies inside one 256-row unit
      const int grp = p.unit_group[((tile / k_tiles) * kRowsPerCta) >> 8];
      live = live && grp >= 0;
      t_scale = round_to_bf16(fmaxf(__fmul_rn(__uint_as_float(p.amax_bits[grp < 0 ? 0 : grp]), 1.0f / 2688.0f), 1.0e-9f));
      t_recip = __frcp_rn(t_scale);
    }

    uint32_t xw[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      xw[4 * j + 0] = next[j].x;
      xw[4 * j + 1] = next[j].y;
      xw[4 * j + 2] = next[j].z;
      xw[4 * j + 3] = next[j].w;
    }
    const float inv = next_inv;
    live = live && next_row_ok;
    issue_loads(tile + gridDim.x);

    GroupOut o;
    o.a_comp[0] = o.a_comp[1] = 0;
    o.meta = 0;
    o.sf_sparse = 0;
    o.sf_res = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) o.q_res[i] = o.q_sparse[i] = 0;

    if (live) {
      if (kMode == 1) {
        const uint4 *gsrc = gamma_smem + (size_t)group * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 gv = gsrc[j];
          uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const uint32_t w = xw[4 * j + t];
            const float a = __fmul_rn(__fmul_rn(lo_f(w), inv), lo_f(gw[t]));
            const float b = __fmul_rn(__fmul_rn(hi_f(w), inv), hi_f(gw[t]));
            xw[4 * j + t] = pack_bf16x2(a, b);
          }
        }
      }
      scale_quantize_group<kMode, kDebug>(xw, t_scale, t_recip, tbl, o, [&](uint32_t (&w)[16]) {
        // mode 2, rare: the group is read again for the division form
        const int in_row = p.src_row != nullptr ? p.src_row[row] : row;
        const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (size_t)in_row * k + (size_t)group * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 v = __ldg(src + j);
          w[4 * j + 0] = v.x;
          w[4 * j + 1] = v.y;
          w[4 * j + 2] = v.z;
          w[4 * j + 3] = v.w;
        }
      });

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
        uint8_t *dst = p.e + (size_t)k_tile * aligned_m * 16 + (size_t)row * 16 + (size_t)group_in_tile * 2;
        *reinterpret_cast<uint32_t *>(dst) = mine | (other << 16);
      }
    }
    // Scale factors: 4 neighbouring groups share one 32-bit word of the sparse layout,
    // 2 neighbouring groups (4 residual scales) one word of the dense layout.
    {
      uint32_t sv = o.sf_sparse;
      uint32_t s1 = __shfl_down_sync(0xffffffffu, sv, 1);
      uint32_t s2 = __shfl_down_sync(0xffffffffu, sv, 2);
      uint32_t s3 = __shfl_down_sync(0xffffffffu, sv, 3);
      uint32_t r2 = o.sf_res;
      uint32_t r2n = __shfl_down_sync(0xffffffffu, r2, 1);
      if (col_ok) {
        if ((lane & 3) == 0)
          *reinterpret_cast<uint32_t *>(p.sfa_sparse + sf_offset(row, group, groups32)) = sv | (s1 << 8) | (s2 << 16) | (s3 << 24);
        if ((lane & 1) == 0)
          *reinterpret_cast<uint32_t *>(p.sf_res + sf_offset(row, 2 * group, k / 16)) = r2 | (r2n << 16);
      }
    }
  }
}


// ---------------------------------------------------------------------------
// One-launch scaled prepare (modes 1 and 2 with their statistics pass folded in).
//
// A cooperative grid of one CTA per SM; CTA b owns a contiguous block of rows.  Phase 1: the
// CTA streams its rows through shared memory in chunks, computes the row statistics of the
// RMSNorm path in the reference's summation order (group sums as FMA chains, then left to
// right over the groups by one thread per row), replaces the cached rows by the normalised
// bf16 values and folds max|y| into the tensor absmax word.  All CTAs then meet at a
// grid-wide barrier (a counter in the caller's workspace, bounded spin), read the absmax and
// quantise: the last chunk straight from shared memory, earlier chunks (when the CTA's rows
// do not fit) from a second read of the input.  At 2048 x 4096 every row stays on chip, so
// the input is read from HBM exactly once and the statistics cost no launch of their own.
// ---------------------------------------------------------------------------
constexpr int kFusedSmemBudget = 200 * 1024;       // dynamic shared memory the row cache may use
constexpr long long kGridBarrierLimitCycles = 2000000000LL;  // about one second

__device__ int g_prepare_timeouts = 0;  // grid barriers that ran out (the result of such a call is wrong)

struct FusedParams {
  const __nv_bfloat16 *x;
  const __nv_bfloat16 *residual;  // kAdd: the input is bf16(x + residual) ...
  __nv_bfloat16 *sum_out;         // ... which is also written here
  const __nv_bfloat16 *gamma;
  float eps;
  float *inv_rms;            // [m], mode 1
  unsigned int *amax_bits;   // zero on entry
  unsigned int *arrive;      // zero on entry: grid barrier counter
  float *scale_out;
  uint8_t *a_comp, *e, *sfa_sparse, *q_res, *sf_res;
  int m, k;
  int rows_per_cta;
  int chunk_rows;  // rows of one shared-memory chunk
};

// stores of one quantised group: payloads by the owner lane, metadata and scale factors
// combined over neighbouring lanes (groups g, g+1[, g+2, g+3] of the same row)
__device__ __forceinline__ void store_group(const FusedParams &p, const GroupOut &o, int row, int group, bool live,
                                            bool in_padded, int aligned_m, int lane) {
  const int k = p.k, groups32 = k >> 5;
  if (live) {
    *reinterpret_cast<uint4 *>(p.q_res + (size_t)row * (k / 2) + (size_t)group * 16) =
        make_uint4(o.q_res[0], o.q_res[1], o.q_res[2], o.q_res[3]);
    *reinterpret_cast<uint2 *>(p.a_comp + (size_t)row * (k / 4) + (size_t)group * 8) = make_uint2(o.a_comp[0], o.a_comp[1]);
  }
  const uint32_t mine = o.meta & 0xFFFFu;
  const uint32_t other = __shfl_down_sync(0xffffffffu, mine, 1);
  if ((lane & 1) == 0 && in_padded)
    *reinterpret_cast<uint32_t *>(p.e + (size_t)(group >> 3) * aligned_m * 16 + (size_t)row * 16 + (size_t)(group & 7) * 2) =
        mine | (other << 16);
  const uint32_t sv = o.sf_sparse;
  const uint32_t s1 = __shfl_down_sync(0xffffffffu, sv, 1);
  const uint32_t s2 = __shfl_down_sync(0xffffffffu, sv, 2);
  const uint32_t s3 = __shfl_down_sync(0xffffffffu, sv, 3);
  const uint32_t r2 = o.sf_res;
  const uint32_t r2n = __shfl_down_sync(0xffffffffu, r2, 1);
  if (live) {
    if ((lane & 3) == 0)
      *reinterpret_cast<uint32_t *>(p.sfa_sparse + sf_offset(row, group, groups32)) = sv | (s1 << 8) | (s2 << 16) | (s3 << 24);
    if ((lane & 1) == 0) *reinterpret_cast<uint32_t *>(p.sf_res + sf_offset(row, 2 * group, k / 16)) = r2 | (r2n << 16);
  }
}

template <int kMode, bool kAdd, int kFusedThreads>
__global__ void __launch_bounds__(kFusedThreads, 1) prepare_fused_kernel(const FusedParams p) {
  static_assert(kMode == 1 || kMode == 2, "modes with a statistics pass");
  constexpr int kFusedWarps = kFusedThreads / 32;
  const int m = p.m, k = p.k;
  const int groups32 = k >> 5;
  const int groups_padded = ((k + 255) / 256) * 8;  // groups of the metadata tiles (256 columns each)
  const int aligned_m = (m + 127) / 128 * 128;
  const int row_vecs = k >> 3;                     // uint4 per row
  const int partial_stride = groups32 + 4;         // padded: 16-byte reads of neighbouring rows hit different banks
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  __shared__ ScaleTables tbl;
  __shared__ float warp_red[32];
  extern __shared__ uint4 fused_smem[];
  uint4 *gamma_s = fused_smem;                                      // mode 1: k bf16, pieces permuted like the cache
  uint4 *cache = fused_smem + (kMode == 1 ? row_vecs : 0);          // chunk_rows x k bf16
  float *partial = reinterpret_cast<float *>(cache + (size_t)p.chunk_rows * row_vecs);  // mode 1: chunk_rows x partial_stride
  float *inv_s = partial + (kMode == 1 ? p.chunk_rows * partial_stride : 0);            // mode 1: rows_per_cta

  if (threadIdx.x < 128) {
    const float v = ue4m3_to_float(threadIdx.x);
    tbl.value[threadIdx.x] = v;
    tbl.recip[threadIdx.x] = __frcp_rn(v);  // code 0 is never looked up (scales are clamped to >= 2^-9)
  }
  if (kMode == 1) {
    const uint4 *gsrc = reinterpret_cast<const uint4 *>(p.gamma);
    for (int i = threadIdx.x; i < row_vecs; i += kFusedThreads) gamma_s[cache_slot(i >> 2, i & 3)] = __ldg(gsrc + i);
  }

  // ---- zero what no owner thread writes: padding rows of the metadata and scale-factor
  // bands, the spare band of the scale buffers, the tail of A_comp
  {
    const int worker = blockIdx.x * kFusedThreads + threadIdx.x;
    const int workers = gridDim.x * kFusedThreads;
    const size_t bands = (size_t)aligned_m / 128;
    zero_range(p.sfa_sparse, bands * (size_t)(groups32 / 4) * 512, sf_alloc_bytes(m, k), worker, workers);
    zero_range(p.sf_res, bands * (size_t)(k / 16 / 4) * 512, sf_alloc_bytes(m, k), worker, workers);
    zero_range(p.a_comp, (size_t)m * (k / 4), a_comp_bytes(m, k), worker, workers);
    const int pad_rows = aligned_m - m;
    const int k_tiles = groups_padded >> 3;
    const int w_sp = groups32 >> 2, w_res = k >> 6;  // 32-bit scale words per row
    const int per_row = k_tiles * 4 + w_sp + w_res;  // 32-bit words to clear per padding row
    for (long long i = worker; i < (long long)pad_rows * per_row; i += workers) {
      const int row = m + (int)(i / per_row);
      int j = (int)(i % per_row);
      if (j < k_tiles * 4) {
        *reinterpret_cast<uint32_t *>(p.e + ((size_t)(j >> 2) * aligned_m + row) * 16 + (size_t)(j & 3) * 4) = 0u;
      } else if ((j -= k_tiles * 4) < w_sp) {
        *reinterpret_cast<uint32_t *>(p.sfa_sparse + sf_offset(row, 4 * j, groups32)) = 0u;
      } else {
        j -= w_sp;
        *reinterpret_cast<uint32_t *>(p.sf_res + sf_offset(row, 4 * j, k / 16)) = 0u;
      }
    }
  }

  const int row_begin = min(m, (int)blockIdx.x * p.rows_per_cta);
  const int row_end = min(m, row_begin + p.rows_per_cta);
  const int rows = row_end - row_begin;
  const int chunks = rows > 0 ? (rows + p.chunk_rows - 1) / p.chunk_rows : 0;
  const int first_chunk_rows = rows - (chunks - 1) * p.chunk_rows;  // the short chunk goes first, the cached (last) one is full
  auto chunk_first_row = [&](int c) { return c == 0 ? 0 : first_chunk_rows + (c - 1) * p.chunk_rows; };
  auto chunk_size = [&](int c) { return c == 0 ? first_chunk_rows : p.chunk_rows; };
  const __nv_bfloat16 *src = kAdd ? p.sum_out : p.x;  // what a second read of the (summed) input reads
  // no barrier here: the tables and gamma are first read after the barriers of phase 1 / the grid barrier

  // ------------------------------------------------------------------ phase 1: statistics
  __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);
  for (int c = 0; c < chunks; ++c) {
    const int c_rows = chunk_size(c), c_row0 = row_begin + chunk_first_row(c);
    if (c > 0) __syncthreads();  // the previous chunk's cache and partial sums are no longer read
    // two tasks (32-element groups) per iteration, all loads issued before the first use
    const int n_tasks = c_rows * groups32;
    for (int t0 = threadIdx.x; t0 < n_tasks; t0 += 2 * kFusedThreads) {
      uint32_t w[2][16];
      int rl[2], g[2];
      bool on[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int t = t0 + u * kFusedThreads;
        on[u] = t < n_tasks;
        rl[u] = on[u] ? t / groups32 : 0;
        g[u] = on[u] ? t - rl[u] * groups32 : 0;
      }
      uint4 xv[2][4], rv[2][4];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (on[u]) {
          const size_t off = (size_t)(c_row0 + rl[u]) * k + (size_t)g[u] * 32;
          const uint4 *xs = reinterpret_cast<const uint4 *>(p.x + off);
#pragma unroll
          for (int j = 0; j < 4; ++j) xv[u][j] = __ldg(xs + j);
          if (kAdd) {
            const uint4 *rs = reinterpret_cast<const uint4 *>(p.residual + off);
#pragma unroll
            for (int j = 0; j < 4; ++j) rv[u][j] = __ldg(rs + j);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (!on[u]) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          w[u][4 * j + 0] = xv[u][j].x;
          w[u][4 * j + 1] = xv[u][j].y;
          w[u][4 * j + 2] = xv[u][j].z;
          w[u][4 * j + 3] = xv[u][j].w;
        }
        if (kAdd) {
          uint4 *dst = reinterpret_cast<uint4 *>(p.sum_out + (size_t)(c_row0 + rl[u]) * k + (size_t)g[u] * 32);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t rw[4] = {rv[u][j].x, rv[u][j].y, rv[u][j].z, rv[u][j].w};
#pragma unroll
            for (int q = 0; q < 4; ++q)
              w[u][4 * j + q] = pack_bf16x2(__fadd_rn(lo_f(w[u][4 * j + q]), lo_f(rw[q])),
                                            __fadd_rn(hi_f(w[u][4 * j + q]), hi_f(rw[q])));
            dst[j] = make_uint4(w[u][4 * j], w[u][4 * j + 1], w[u][4 * j + 2], w[u][4 * j + 3]);
          }
        }
        uint4 *row_cache = cache + (size_t)rl[u] * row_vecs;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          row_cache[cache_slot(g[u], j)] = make_uint4(w[u][4 * j], w[u][4 * j + 1], w[u][4 * j + 2], w[u][4 * j + 3]);
        if (kMode == 1) {
          float sq = 0.0f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a = lo_f(w[u][i]), b = hi_f(w[u][i]);
            sq = __fmaf_rn(a, a, sq);  // a*a is exact in float, so this equals sq + a*a
            sq = __fmaf_rn(b, b, sq);
          }
          partial[rl[u] * partial_stride + g[u]] = sq;
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[u][i])));
        }
      }
    }
    if (kMode == 1) {
      __syncthreads();
      if (threadIdx.x < c_rows) {
        const float4 *pr = reinterpret_cast<const float4 *>(partial + threadIdx.x * partial_stride);
        float total = 0.0f;
        for (int i = 0; i < groups32 / 4; ++i) {  // groups32 is a multiple of 4 (K % 128 == 0)
          const float4 v = pr[i];
          total = __fadd_rn(total, v.x);
          total = __fadd_rn(total, v.y);
          total = __fadd_rn(total, v.z);
          total = __fadd_rn(total, v.w);
        }
        const float inv = rsqrtf(__fadd_rn(__fdiv_rn(total, (float)k), p.eps));
        inv_s[chunk_first_row(c) + threadIdx.x] = inv;
        p.inv_rms[c_row0 + threadIdx.x] = inv;
      }
      __syncthreads();
      // normalise in place: the cache then holds y = bf16(x * inv_rms * gamma)
      for (int t = threadIdx.x; t < c_rows * groups32; t += kFusedThreads) {
        const int rl = t / groups32, g = t - rl * groups32;
        const float inv = inv_s[chunk_first_row(c) + rl];
        uint4 *row_cache = cache + (size_t)rl * row_vecs;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int slot = cache_slot(g, j);
          const uint4 xv = row_cache[slot];
          const uint4 gv = gamma_s[slot];
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
          uint32_t y[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            y[q] = pack_bf16x2(__fmul_rn(__fmul_rn(lo_f(xw[q]), inv), lo_f(gw[q])),
                               __fmul_rn(__fmul_rn(hi_f(xw[q]), inv), hi_f(gw[q])));
            m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&y[q])));
          }
          row_cache[slot] = make_uint4(y[0], y[1], y[2], y[3]);
        }
      }
    }
  }

  // ---- CTA absmax -> tensor absmax, grid barrier, tensor scale
  {
    float mx = fmaxf(__bfloat162float(m2.x), __bfloat162float(m2.y));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) warp_red[warp] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
      for (int w = 1; w < kFusedWarps; ++w) mx = fmaxf(mx, warp_red[w]);
      if (mx > 0.0f) atomicMax(p.amax_bits, __float_as_uint(mx));
      __threadfence();
      atomicAdd(p.arrive, 1u);
      const long long t0 = clock64();
      while (ld_acquire_gpu(p.arrive) < gridDim.x) {
        if (clock64() - t0 > kGridBarrierLimitCycles) {
          atomicAdd(&g_prepare_timeouts, 1);
          break;
        }
      }
    }
    __syncthreads();
  }
  const float amax = __uint_as_float(ld_acquire_gpu(p.amax_bits));
  // ATen divides a CUDA tensor by a host scalar by multiplying with the float
  // reciprocal; clamp(min=1e-9) follows (kernels/src/bindings.cpp:337 of the reference).
  const float scale = fmaxf(__fmul_rn(amax, 1.0f / 2688.0f), 1.0e-9f);
  if (p.scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *p.scale_out = scale;
  const float div = kMode == 2 ? round_to_bf16(scale) : scale;  // see round_to_bf16
  const float recip = __frcp_rn(div);

  // ------------------------------------------------------------------ phase 2: quantise
  const int tasks_per_row = (groups_padded + 31) >> 5;  // a warp takes 32 neighbouring groups of one row
  for (int c = chunks - 1; c >= 0; --c) {
    const bool cached = c == chunks - 1;
    const int c_rows = chunk_size(c), c_row0 = row_begin + chunk_first_row(c);
    for (int wt = warp; wt < c_rows * tasks_per_row; wt += kFusedWarps) {
      const int rl = wt / tasks_per_row;
      const int group = (wt - rl * tasks_per_row) * 32 + lane;
      const int row = c_row0 + rl;
      const bool live = group < groups32;
      uint32_t xw[16];
      GroupOut o;
      o.a_comp[0] = o.a_comp[1] = 0;
      o.meta = 0;
      o.sf_sparse = 0;
      o.sf_res = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) o.q_res[i] = o.q_sparse[i] = 0;
      // the group's 32 values from the row cache or, for a chunk that is not cached, from global memory
      auto load_group = [&](uint32_t (&w)[16]) {
        if (cached) {
          const uint4 *row_cache = cache + (size_t)rl * row_vecs;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v = row_cache[cache_slot(group, j)];
            w[4 * j + 0] = v.x;
            w[4 * j + 1] = v.y;
            w[4 * j + 2] = v.z;
            w[4 * j + 3] = v.w;
          }
        } else {
          // plain loads: with kAdd these bytes were written by this CTA in phase 1
          const uint4 *xs = reinterpret_cast<const uint4 *>(src + (size_t)row * k + (size_t)group * 32);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v = xs[j];
            w[4 * j + 0] = v.x;
            w[4 * j + 1] = v.y;
            w[4 * j + 2] = v.z;
            w[4 * j + 3] = v.w;
          }
        }
      };
      if (live) {
        load_group(xw);
        if (!cached) {
          if (kMode == 1) {
            const float inv = inv_s[chunk_first_row(c) + rl];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 gv = gamma_s[cache_slot(group, j)];
              const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint32_t w = xw[4 * j + q];
                xw[4 * j + q] = pack_bf16x2(__fmul_rn(__fmul_rn(lo_f(w), inv), lo_f(gw[q])),
                                            __fmul_rn(__fmul_rn(hi_f(w), inv), hi_f(gw[q])));
              }
            }
          }
        }
        scale_quantize_group<kMode, false>(xw, div, recip, tbl, o, load_group);
      }
      store_group(p, o, row, group, live, group < groups_padded, aligned_m, lane);
    }
  }
}

}  // namespace

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------

size_t prepare_workspace_bytes(int m) { return 256 + (size_t)m * sizeof(float); }

// SM count of the current device (queried once per device).
static cudaError_t current_sms(int *dev_out, int *sms_out) {
  static int sms[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (sms[dev] == 0 && (e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  *dev_out = dev;
  *sms_out = sms[dev];
  return cudaSuccess;
}

static int prepare_grid(const PrepareParams &p) {
  int dev = 0, sms = 0;
  const int tiles = ((p.k + kColsPerCta - 1) / kColsPerCta) * p.row_tiles;
  if (current_sms(&dev, &sms) != cudaSuccess) return tiles < 1024 ? tiles : 1024;
  const int full = sms * kPrepareCtasPerSm;
  return tiles < full ? tiles : full;
}

static cudaError_t launch_prepare(int mode, bool debug, const PrepareParams &p, cudaStream_t stream) {
  dim3 grid(prepare_grid(p));
  dim3 block(kPrepareThreads);
  if (debug) {
    prepare_kernel<0, true><<<grid, block, 0, stream>>>(p);
  } else if (mode == 0) {
    prepare_kernel<0, false><<<grid, block, 0, stream>>>(p);
  } else if (mode == 1) {
    const size_t gamma_bytes = (size_t)p.k * sizeof(__nv_bfloat16);
    static bool attr_set[64] = {};
    int dev = 0;
    if (gamma_bytes > 48 * 1024 && cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(prepare_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
      if (e != cudaSuccess) return e;
      attr_set[dev] = true;
    }
    prepare_kernel<1, false><<<grid, block, gamma_bytes, stream>>>(p);
  } else if (p.src_row != nullptr) {
    prepare_kernel<2, false><<<grid, block, 0, stream>>>(p);
  } else {
    prepare_kernel<2, false, 2><<<grid, block, 0, stream>>>(p);
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

// One cooperative launch for statistics + prepare (see prepare_fused_kernel).  Returns
// cudaErrorNotSupported when the shape does not fit or the device cannot launch it, in which
// case the caller falls back to the separate statistics and prepare kernels.
template <int kMode, bool kAdd, int kThreads>
static cudaError_t launch_fused_t(const FusedParams &p_in, cudaStream_t stream) {
  static bool attr_set[64] = {};
  static int coop[64] = {};  // 0 unknown, 1 yes, -1 no
  int dev = 0, sms = 0;
  cudaError_t e = current_sms(&dev, &sms);
  if (e != cudaSuccess) return e;
  if (coop[dev] == 0) {
    int v = 0;
    coop[dev] = (cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && v) ? 1 : -1;
  }
  if (coop[dev] < 0) return cudaErrorNotSupported;
  FusedParams p = p_in;
  const int groups32 = p.k / 32;
  p.rows_per_cta = (p.m + sms - 1) / sms;
  const size_t row_bytes = (size_t)p.k * 2 + (kMode == 1 ? (size_t)(groups32 + 4) * 4 : 0);
  const size_t fixed = (kMode == 1 ? (size_t)p.k * 2 + (size_t)p.rows_per_cta * 4 : 0);
  if (fixed + row_bytes > (size_t)kFusedSmemBudget) return cudaErrorNotSupported;
  const size_t capacity = ((size_t)kFusedSmemBudget - fixed) / row_bytes;
  p.chunk_rows = (int)(capacity < (size_t)p.rows_per_cta ? capacity : (size_t)p.rows_per_cta);
  const size_t smem = fixed + (size_t)p.chunk_rows * row_bytes + 16;
  auto kernel = prepare_fused_kernel<kMode, kAdd, kThreads>;
  if (!attr_set[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFusedSmemBudget + 16);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.gridDim = dim3(sms);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

// 512 threads per CTA: measured against 448, 768 and 896 (more threads spill or idle in the
// partly filled last round of 56 warp tasks per CTA at 2048 x 4096)
template <int kMode, bool kAdd>
static cudaError_t launch_fused(const FusedParams &p, cudaStream_t stream) {
  return launch_fused_t<kMode, kAdd, 512>(p, stream);
}

static bool fused_prepare_enabled() {
  static const bool on = [] {
    const char *v = getenv("SHARQ_PREPARE_FUSED");  // tuning hook: 0 selects the separate statistics + prepare kernels
    return !(v != nullptr && v[0] == '0');
  }();
  return on;
}

int prepare_timeouts() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_prepare_timeouts, sizeof(v)) != cudaSuccess) return -1;
  return v;
}

cudaError_t run_scaled_prepare(const void *x, const void *gamma, float eps, int m, int k, void *workspace,
                               float *inv_rms_external, void *a_comp, void *e, void *sfa_sparse, void *q_res,
                               void *sf_res, float *scale_out, cudaStream_t stream, bool absmax_ready,
                               const void *residual, void *sum_out) {
  if (residual != nullptr && (gamma == nullptr || sum_out == nullptr)) return cudaErrorInvalidValue;
  // workspace: [0,4) tensor absmax bits; [256, 256+4m) inv_rms
  auto *amax_bits = static_cast<unsigned int *>(workspace);
  float *inv_rms = inv_rms_external ? inv_rms_external
                                    : reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + 256);
  cudaError_t err = cudaSuccess;
  const bool rms = gamma != nullptr;
  // a small non-RMSNorm input (a decode step): the prepare kernel finds max|x| itself
  const bool inline_absmax = !rms && !absmax_ready && (size_t)m * k <= kInlineAbsmaxElements;
  // One cooperative launch pays while the per-SM row caches hold most of the tensor; beyond that
  // the separate statistics and prepare kernels (more resident warps per SM) are faster.  Measured
  // crossovers (us, one launch / separate): RMSNorm 4096 x 4096 35.0 / 37.0, 8192 x 4096
  // 65.7 / 63.8, 16384 x 4096 136 / 118; tensor scale 2048 x 7168 24.9 / 25.0, 4096 x 4096 28.7 / 27.0.
  const size_t elements = (size_t)m * (size_t)k;
  const bool one_launch_pays = elements < (rms ? ((size_t)1 << 25) : ((size_t)1 << 24));
  if (!absmax_ready && !inline_absmax && one_launch_pays && fused_prepare_enabled()) {
    FusedParams f{};
    f.x = static_cast<const __nv_bfloat16 *>(x);
    f.residual = static_cast<const __nv_bfloat16 *>(residual);
    f.sum_out = static_cast<__nv_bfloat16 *>(sum_out);
    f.gamma = static_cast<const __nv_bfloat16 *>(gamma);
    f.eps = eps;
    f.inv_rms = inv_rms;
    f.amax_bits = amax_bits;
    f.arrive = amax_bits + 1;
    f.scale_out = scale_out;
    f.a_comp = static_cast<uint8_t *>(a_comp);
    f.e = static_cast<uint8_t *>(e);
    f.sfa_sparse = static_cast<uint8_t *>(sfa_sparse);
    f.q_res = static_cast<uint8_t *>(q_res);
    f.sf_res = static_cast<uint8_t *>(sf_res);
    f.m = m;
    f.k = k;
    if ((err = cudaMemsetAsync(amax_bits, 0, 2 * sizeof(unsigned int), stream)) != cudaSuccess) return err;
    err = !rms ? launch_fused<2, false>(f, stream)
               : (residual != nullptr ? launch_fused<1, true>(f, stream) : launch_fused<1, false>(f, stream));
    if (err == cudaSuccess) return cudaSuccess;
    (void)cudaGetLastError();  // not launchable here: the separate kernels below do the same work
    if (err != cudaErrorNotSupported && err != cudaErrorCooperativeLaunchTooLarge) return err;
    err = cudaSuccess;
  }
  if (absmax_ready) {
    // the producer of x already left max|x| in the workspace: no statistics pass
    if (rms) return cudaErrorInvalidValue;
  } else if (inline_absmax) {
    amax_bits = nullptr;
  } else if ((err = cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int), stream)) != cudaSuccess) {
    return err;
  } else if (rms) {
    const int groups = k / 32;
    const int threads = (groups + 31) / 32 * 32;
    if (residual != nullptr) {
      rms_stats_kernel<true><<<m, threads, (size_t)groups * sizeof(float), stream>>>(
          static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(residual),
          static_cast<__nv_bfloat16 *>(sum_out), static_cast<const __nv_bfloat16 *>(gamma), eps, k, inv_rms, amax_bits);
      x = sum_out;  // the prepare reads the sum
    } else {
      rms_stats_kernel<false><<<m, threads, (size_t)groups * sizeof(float), stream>>>(
          static_cast<const __nv_bfloat16 *>(x), nullptr, nullptr, static_cast<const __nv_bfloat16 *>(gamma), eps, k,
          inv_rms, amax_bits);
    }
  } else {
    const size_t n16 = (size_t)m * k / 8;
    size_t blocks = (n16 + 255) / 256;
    int dev = 0, sms = 0;
    if (current_sms(&dev, &sms) != cudaSuccess) sms = 128;
    if (blocks > (size_t)sms * 8) blocks = (size_t)sms * 8;
    abs_stats_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), n16, amax_bits);
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

cudaError_t run_grouped_prepare(const void *x, int m, int k, const unsigned int *amax_bits, const int *unit_group, int groups,
                                void *a_comp, void *e, void *sfa_sparse, void *q_res, void *sf_res, float *scale_vec_out,
                                cudaStream_t stream, const int *src_row) {
  if (m <= 0 || m % 256 != 0 || groups < 1) return cudaErrorInvalidValue;
  PrepareParams p{};
  p.x = static_cast<const __nv_bfloat16 *>(x);
  p.amax_bits = amax_bits;
  p.a_comp = static_cast<uint8_t *>(a_comp);
  p.e = static_cast<uint8_t *>(e);
  p.sfa_sparse = static_cast<uint8_t *>(sfa_sparse);
  p.q_res = static_cast<uint8_t *>(q_res);
  p.sf_res = static_cast<uint8_t *>(sf_res);
  p.m = m;
  p.k = k;
  p.row_tiles = m / kRowsPerCta;
  p.unit_group = unit_group;
  p.scale_vec_out = scale_vec_out;
  p.groups = groups;
  p.src_row = src_row;
  return launch_prepare(2, false, p, stream);
}

}  // namespace sharq
