// Device code shared by the activation prepare kernels (prepare.cu) and the tensor-parallel
// transition kernel (sp_transition.cu): bf16 packing helpers, the 32-element group (pair
// selection, sparse main path, dense residual), the tensor-scale division, and small utilities.
#pragma once

#include "common.cuh"

namespace sharq {
namespace prep {

__device__ __forceinline__ float lo_f(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// two floats -> packed bf16x2 (a in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}

// ---------------------------------------------------------------------------
// The 32-element group: selection, sparse quantisation, residual quantisation.
// ---------------------------------------------------------------------------
struct ScaleTables {
  float value[128];  // ue4m3 code -> float
  float recip[128];  // IEEE 1.0f / value
};

struct GroupOut {
  uint32_t q_res[4];     // 16 B dense residual payload
  uint32_t a_comp[2];    // 8 B compressed sparse payload
  uint32_t q_sparse[4];  // 16 B dense sparse payload (debug output only)
  uint32_t meta;         // 2 B metadata (4 nibbles)
  uint32_t sf_sparse;    // 1 B
  uint32_t sf_res;       // 2 B (first 16-group in the low byte)
  uint32_t second_min;   // smallest (key - 4) of the second selected pair over the four chunks (see kTinyKey)
};

// four packed e2m1x2 bytes -> four half2 words (element 2i of byte i in the low half)
__device__ __forceinline__ void decode_e2m1x8(uint32_t word, uint32_t (&h)[4]) {
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t"
      "}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(word));
}

__device__ __forceinline__ uint32_t scale_code_from_max(float mx) {
  return float_to_ue4m3(clamp_val(__fdiv_rn(mx, kFp4Max), kScaleEps, kFp8Max));
}

template <bool kDebug>
__device__ __forceinline__ void quantize_group32(const uint32_t (&xw)[16], const ScaleTables &tbl, GroupOut &o) {
  float x[32];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    x[2 * i] = lo_f(xw[i]);
    x[2 * i + 1] = hi_f(xw[i]);
  }

  // -- pair selection per 8-element chunk on integer keys
  uint32_t lo_idx[4], hi_idx[4];
  uint32_t max_key = 0;
  uint32_t meta = 0;
  uint32_t second_min = 0xFFFFFFFFu;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t key[4];
#pragma unroll
    for (int p = 0; p < 4; ++p)
      key[p] = __float_as_uint(fmaxf(fabsf(x[8 * c + 2 * p]), fabsf(x[8 * c + 2 * p + 1]))) | (uint32_t)(3 - p);
    const uint32_t m01 = max(key[0], key[1]), n01 = min(key[0], key[1]);
    const uint32_t m23 = max(key[2], key[3]), n23 = min(key[2], key[3]);
    const uint32_t best = max(m01, m23);
    const uint32_t second = max(min(m01, m23), max(n01, n23));
    const uint32_t ib = 3u - (best & 3u), is = 3u - (second & 3u);
    lo_idx[c] = min(ib, is);
    hi_idx[c] = max(ib, is);
    meta |= (lo_idx[c] | (hi_idx[c] << 2)) << (4 * c);
    max_key = max(max_key, best);
    second_min = min(second_min, second - 4u);  // an all-zero pair (key < 4) wraps to a huge value
  }
  o.meta = meta;
  o.second_min = second_min;

  // -- sparse main path scale (one UE4M3 per 32 logical elements)
  const uint32_t s_code = scale_code_from_max(__uint_as_float(max_key & 0xFFFF0000u));
  const float s_q = tbl.value[s_code];
  const float s_r = tbl.recip[s_code];
  o.sf_sparse = s_code;

  // -- quantise every pair, mask to the selected ones, form the residual
  float r[32];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t all4 = pack_e2m1x8(__fmul_rn(x[8 * c + 0], s_r), __fmul_rn(x[8 * c + 1], s_r),
                                      __fmul_rn(x[8 * c + 2], s_r), __fmul_rn(x[8 * c + 3], s_r),
                                      __fmul_rn(x[8 * c + 4], s_r), __fmul_rn(x[8 * c + 5], s_r),
                                      __fmul_rn(x[8 * c + 6], s_r), __fmul_rn(x[8 * c + 7], s_r));
    const uint32_t mask4 = (0xFFu << (8 * lo_idx[c])) | (0xFFu << (8 * hi_idx[c]));
    const uint32_t dense4 = all4 & mask4;  // dropped pairs become +0,+0: their residual is x itself
    if (kDebug) o.q_sparse[c] = dense4;
    uint32_t h[4];
    decode_e2m1x8(dense4, h);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float2 q = __half22float2(*reinterpret_cast<__half2 *>(&h[p]));
      // q * s_q is exact (2-bit x 4-bit significands), so the FMA rounds once like x - (q*s)
      r[8 * c + 2 * p] = __fmaf_rn(-q.x, s_q, x[8 * c + 2 * p]);
      r[8 * c + 2 * p + 1] = __fmaf_rn(-q.y, s_q, x[8 * c + 2 * p + 1]);
    }
    // the two kept pair-bytes, ascending pair order
    const uint32_t two = __byte_perm(dense4, 0u, lo_idx[c] | (hi_idx[c] << 4) | 0x4400u);
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
    const uint32_t code = scale_code_from_max(mx);
    const float rr = tbl.recip[code];
    sf_res |= code << (8 * h);
#pragma unroll
    for (int wv = 0; wv < 2; ++wv) {
      const int i = 16 * h + 8 * wv;
      o.q_res[2 * h + wv] =
          pack_e2m1x8(__fmul_rn(r[i + 0], rr), __fmul_rn(r[i + 1], rr), __fmul_rn(r[i + 2], rr), __fmul_rn(r[i + 3], rr),
                      __fmul_rn(r[i + 4], rr), __fmul_rn(r[i + 5], rr), __fmul_rn(r[i + 6], rr), __fmul_rn(r[i + 7], rr));
    }
  }
  o.sf_res = sf_res;
}

// bf16(y / scale) of a whole 32-element group, y already bf16-exact floats.
// q = y * recip is within 2 ulp of the true quotient; when q is more than 4 ulp away from
// every bf16 rounding boundary (low 16 bits == 0x8000) the IEEE quotient rounds to the same
// bf16 value.  The boundary test is done on packed halves: the low
// 16 bits of both products of a word go into one register (one byte permute), 0x8004 is added
// to each half (a carry out of the low half can only raise the high half by one, which the
// wider threshold absorbs), and a packed unsigned minimum over the group is compared once.
// A group in which any product lies within the window is redone with IEEE divisions.
__device__ __forceinline__ void scale_group32(uint32_t (&w)[16], float scale, float recip) {
  uint32_t out[16];
  uint32_t nearest = 0xFFFFFFFFu;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float qa = __fmul_rn(lo_f(w[i]), recip), qb = __fmul_rn(hi_f(w[i]), recip);
    const uint32_t lows = __byte_perm(__float_as_uint(qa), __float_as_uint(qb), 0x5410);
    nearest = __vminu2(nearest, lows + 0x80048004u);
    out[i] = pack_bf16x2(qa, qb);
  }
  if ((nearest & 0xFFFFu) < 10u || (nearest >> 16) < 10u) {
    // Some product of this group is close to a rounding boundary (exact ties are common when
    // the tensor absmax has a short mantissa).  Redo the words concerned with the correctly
    // rounded quotient: two residual corrections q += (y - q*scale) * recip with fused
    // multiply-adds (the classic division refinement, exact because recip is the correctly
    // rounded reciprocal), or an IEEE division for tiny operands or a subnormal quotient.
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float ya = lo_f(w[i]), yb = hi_f(w[i]);
      float qa = __fmul_rn(ya, recip), qb = __fmul_rn(yb, recip);
      const uint32_t ta = (__float_as_uint(qa) + 0x8004u) & 0xFFFFu;
      const uint32_t tb = (__float_as_uint(qb) + 0x8004u) & 0xFFFFu;
      if (ta < 9u || tb < 9u) {
        // residuals are exact for |y| >= 2^-100, and the refinement theorem needs a normal quotient
        if (fminf(fabsf(ya), fabsf(yb)) < 7.8886090522101181e-31f || fminf(fabsf(qa), fabsf(qb)) < 2.3509887e-38f) {
          qa = __fdiv_rn(ya, scale);
          qb = __fdiv_rn(yb, scale);
        } else {
          qa = __fmaf_rn(__fmaf_rn(-qa, scale, ya), recip, qa);
          qb = __fmaf_rn(__fmaf_rn(-qb, scale, yb), recip, qb);
          qa = __fmaf_rn(__fmaf_rn(-qa, scale, ya), recip, qa);
          qb = __fmaf_rn(__fmaf_rn(-qb, scale, yb), recip, qb);
        }
        out[i] = pack_bf16x2(qa, qb);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = out[i];
}

// A selected pair whose score is non-zero but below 2^-118 (key = float bits | pair index).
constexpr uint32_t kTinyKey = 0x04800000u - 4u;

// float(bf16(x)): the divisor of the non-RMSNorm path.  On a CUDA device `x / scale` with a bf16
// tensor x and a 0-dim float32 tensor scale (model/quantize.py:179-183 of the reference) casts
// the scale to the common dtype bf16 before dividing in float.
__device__ __forceinline__ float round_to_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Tensor-scale division and quantisation of one group.
//   kMode 1: the divisor is the float32 scale (the reference's RMSNorm kernel divides by it with
//            __fdiv_rn): products with a boundary test, see scale_group32.
//   kMode 2: the divisor has an 8-bit significand (see round_to_bf16), and so has y.  The exact
//            quotient of two such numbers is either representable in 8 bits or at least a
//            relative 2^-17 away from every value with a 9-bit significand, i.e. from every bf16
//            rounding boundary, while y * (1/div) is within 2^-22 of it: the product rounds to
//            the same bf16 as the IEEE quotient, no test needed.  The argument needs a normal
//            quotient; subnormal quotients only matter when such a value takes part in a pair
//            selection, which the keys show (second_min): that group is redone with divisions.
//            The retry reads the group again through `reload` instead of keeping a second copy
//            of it in registers across the quantisation.
template <int kMode, bool kDebug, typename Reload>
__device__ __forceinline__ void scale_quantize_group(uint32_t (&y)[16], float div, float recip, const ScaleTables &tbl,
                                                     GroupOut &o, Reload reload) {
  if (kMode == 1) {
    scale_group32(y, div, recip);
    quantize_group32<kDebug>(y, tbl, o);
  } else if (kMode == 2) {
#pragma unroll 1
    for (int attempt = 0; attempt < 2; ++attempt) {
      if (attempt == 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = pack_bf16x2(__fmul_rn(lo_f(y[i]), recip), __fmul_rn(hi_f(y[i]), recip));
      } else {
        reload(y);
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = pack_bf16x2(__fdiv_rn(lo_f(y[i]), div), __fdiv_rn(hi_f(y[i]), div));
      }
      quantize_group32<kDebug>(y, tbl, o);
      if (o.second_min >= kTinyKey) break;
    }
  } else {
    quantize_group32<kDebug>(y, tbl, o);
  }
}

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

// uint4 index of 16-byte piece j of group g inside a cached row: the pieces of a group are
// permuted so that a quarter-warp reading or writing neighbouring groups hits distinct banks
__device__ __forceinline__ int cache_slot(int g, int j) { return (g << 2) + (j ^ ((g >> 1) & 3)); }

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

}  // namespace prep
}  // namespace sharq
