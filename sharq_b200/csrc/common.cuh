// Shared device helpers for the SharQ sm_100a kernels: scalar formats, the blocked
// scale-factor layout and small utilities.  Everything here is arithmetic the
// reference performs through cutlass::NumericConverter<..., round_to_nearest>
// (kernels/src/fused_sparse_prepare.cu:113-116 of the reference project); on sm_100a
// those converters map to the cvt.rn.satfinite instructions used below.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sharq {

constexpr float kFp4Max = 6.0f;
constexpr float kFp8Max = 448.0f;
constexpr float kScaleEps = 0.001953125f;  // 2^-9

// ---- comparison helpers with the reference's NaN-dropping '?:' semantics
//      (kernels/src/fused_sparse_prepare.cu:27-41)
__device__ __forceinline__ float fp_abs(float x) { return x < 0.0f ? -x : x; }
__device__ __forceinline__ float fp_max(float a, float b) { return a > b ? a : b; }
__device__ __forceinline__ float fp_min(float a, float b) { return a < b ? a : b; }
__device__ __forceinline__ float clamp_val(float x, float lo, float hi) { return fp_max(lo, fp_min(x, hi)); }

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// float -> bf16 bits, round to nearest even.
__device__ __forceinline__ uint32_t float_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// Eight floats -> four bytes of packed e2m1 (element 2i in the low nibble of byte i),
// round to nearest even, saturating at +-6.
__device__ __forceinline__ uint32_t pack_e2m1x8(float f0, float f1, float f2, float f3, float f4, float f5,
                                                float f6, float f7) {
  uint32_t out;
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t"
      "}"
      : "=r"(out)
      : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
  return out;
}

// float (already clamped to [2^-9, 448]) -> UE4M3 code.  For non-negative inputs
// the signed e4m3 conversion produces the same bits as the unsigned format.
__device__ __forceinline__ uint32_t float_to_ue4m3(float f) {
  uint32_t out;
  asm("{\n\t"
      ".reg .b16 h, z;\n\t"
      "mov.b16 z, 0;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 h, %1, %1;\n\t"
      "mov.b32 %0, {h, z};\n\t"
      "}"
      : "=r"(out)
      : "f"(f));
  return out & 0xFFu;
}

// UE4M3 code -> float (exact).
__device__ __forceinline__ float ue4m3_to_float(uint32_t code) {
  uint32_t h2;
  asm("{\n\t"
      ".reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %1;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "}"
      : "=r"(h2)
      : "r"(code & 0xFFu));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
}

// 2 * |value| of an e2m1 code as a small integer: 0,1,2,3,4,6,8,12.
__device__ __forceinline__ int e2m1_twice_magnitude(uint32_t code) {
  return (int)((0xC8643210u >> ((code & 7u) * 4u)) & 0xFu);
}

// e2m1 code -> float.
__device__ __forceinline__ float e2m1_to_float(uint32_t code) {
  float v = 0.5f * (float)e2m1_twice_magnitude(code);
  return (code & 8u) ? -v : v;
}

// Byte offset of the scale of (row, group) in the blocked scale-factor layout:
// 512-byte tiles of 128 rows x 4 scales; the K tiles of one 128-row band are
// contiguous.  groups_per_row is K/16 (dense) or K/32 (sparse main path).
__host__ __device__ __forceinline__ size_t sf_offset(int row, int group, int groups_per_row) {
  size_t tiles_k = (size_t)((groups_per_row + 3) / 4);
  return (size_t)(row / 128) * tiles_k * 512 + (size_t)(group / 4) * 512 + (size_t)(row % 32) * 16 +
         (size_t)((row / 32) % 4) * 4 + (size_t)(group % 4);
}

__host__ __device__ __forceinline__ size_t sf_alloc_bytes(int rows, int k) {
  return (size_t)(rows / 128 + 1) * 128 * (size_t)k / 16;
}
__host__ __device__ __forceinline__ size_t e_bytes(int m, int k) {
  return (size_t)((m + 127) / 128 * 128) * (size_t)((k + 255) / 256 * 256) / 16;
}
__host__ __device__ __forceinline__ size_t a_comp_bytes(int m, int k) {
  return (size_t)m * (size_t)((k + 255) / 256 * 256) / 4;
}

}  // namespace sharq
