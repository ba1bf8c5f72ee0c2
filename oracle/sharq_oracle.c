/*
 * CPU oracle for the SharQ quantized-linear hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain scalar C, the arithmetic of the reference's CUDA
 * kernels so that the sm_100a kernels can be compared byte for byte.  Nothing in
 * the product path may call it: only tests, the smoke check and the bench's
 * cpu_baseline leg load the shared object built from this file.
 *
 * Parity pin: the reference ships no golden vectors for these kernels (its
 * correctness scripts only print metrics).  The scalar converters below are
 * pinned against tables produced by the CUTLASS 4.5.0 host NumericConverter
 * (tests/golden/converter_tables.npz) and the whole-path behaviour is pinned
 * against the reference's SHARQ_SIM fake-quant path on tie-free inputs
 * (tests/golden/sharq_sim_*.npz).  Bit-level parity with the reference's device
 * kernels is otherwise pinned only by the arithmetic written in its .cu files.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -shared -fPIC (see Makefile).
 * -ffp-contract=off keeps every multiply and add separately rounded, which is
 * what the device code produces: each place where nvcc may fuse a multiply-add
 * in the reference has an exact product (bf16*bf16, e2m1*ue4m3), so fused and
 * unfused evaluation agree.
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * reference project root).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define SHARQ_FP4_MAX 6.0f
#define SHARQ_FP8_MAX 448.0f
#define SHARQ_SCALE_EPS 0.001953125f /* 2^-9, kernels/src/fused_sparse_prepare.cu:18-20 */

/* ------------------------------------------------------------------------- */
/* scalar formats                                                             */
/* ------------------------------------------------------------------------- */

static inline float bits_to_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

float sharq_bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

/* float -> bf16, round to nearest even (cutlass::NumericConverter<bfloat16_t,
 * float, round_to_nearest>, used at kernels/src/fused_rmsnorm_sparse_prepare.cu:136,201-203). */
uint16_t sharq_f32_to_bf16(float f) {
  uint32_t u = f32_to_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

/* e2m1 code -> value.  codes 0..7 = 0,0.5,1,1.5,2,3,4,6; bit 3 = sign. */
float sharq_e2m1_to_f32(uint8_t code) {
  static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float v = mag[code & 7];
  return (code & 8) ? -v : v;
}

/* float -> e2m1, round to nearest, ties to the even code, saturating at 6
 * (cutlass::NumericConverter<float_e2m1_t, float, round_to_nearest>, used at
 * kernels/src/fused_sparse_prepare.cu:113,168,194-195).  The sign is kept, so a
 * small negative input gives 0x8 (minus zero). */
uint8_t sharq_f32_to_e2m1(float f) {
  uint8_t sign = (f32_to_bits(f) >> 31) ? 8 : 0;
  float a = fabsf(f);
  uint8_t code;
  if (!(a == a)) {
    code = 7; /* NaN saturates to the largest magnitude */
  } else if (a <= 0.25f) {
    code = 0; /* tie 0.25 -> 0 (even) */
  } else if (a < 0.75f) {
    code = 1;
  } else if (a <= 1.25f) {
    code = 2; /* ties 0.75 and 1.25 -> 1.0 (even) */
  } else if (a < 1.75f) {
    code = 3;
  } else if (a <= 2.5f) {
    code = 4; /* ties 1.75 and 2.5 -> 2.0 */
  } else if (a < 3.5f) {
    code = 5;
  } else if (a <= 5.0f) {
    code = 6; /* ties 3.5 and 5.0 -> 4.0 */
  } else {
    code = 7;
  }
  return (uint8_t)(sign | code);
}

/* UE4M3 (unsigned E4M3, bias 7, subnormals, 0x7E = 448) -> float. */
float sharq_ue4m3_to_f32(uint8_t code) {
  int e = (code >> 3) & 0xF;
  int m = code & 7;
  if (e == 0) return ldexpf((float)m, -9);
  return ldexpf(1.0f + (float)m / 8.0f, e - 7);
}

/* float -> UE4M3, round to nearest even with true subnormals, saturating at 448
 * (cutlass::NumericConverter<float_ue4m3_t, float, round_to_nearest>, used at
 * kernels/src/fused_sparse_prepare.cu:115,158,186).  Callers clamp the input to
 * [2^-9, 448] first, so only that range matters. */
uint8_t sharq_f32_to_ue4m3(float f) {
  if (!(f == f)) return 0x7E;
  if (f <= 0.0f) return 0;
  if (f >= SHARQ_FP8_MAX) return 0x7E;
  int e;
  (void)frexpf(f, &e); /* f = m * 2^e, m in [0.5,1) -> exponent of the leading bit is e-1 */
  int ue = e - 1;
  if (ue < -6) ue = -6; /* subnormal range shares the 2^-6 exponent, quantum 2^-9 */
  /* quantum is 2^(ue-3): f / quantum is exact in float (power-of-two scaling) */
  float q = ldexpf(f, 3 - ue);
  float r = nearbyintf(q); /* default rounding mode: nearest even */
  int ri = (int)r;         /* 0..16 */
  int code;
  if (ue == -6 && ri < 8) {
    code = ri; /* subnormal, exponent field 0 */
  } else {
    if (ri == 16) {
      ri = 8;
      ue += 1;
    }
    code = ((ue + 7) << 3) | (ri - 8);
  }
  if (code > 0x7E) code = 0x7E;
  return (uint8_t)code;
}

/* ------------------------------------------------------------------------- */
/* layouts                                                                    */
/* ------------------------------------------------------------------------- */

/* Byte offset of scale (row r, group g) in the blocked scale-factor layout:
 * 512-byte tiles of 128 rows x 4 scales, K tiles contiguous inside a 128-row
 * band (kernels/src/fused_sparse_prepare.cu:48-57 with the layouts built at
 * :275-278; the same swizzle is restated by the reference's own to_blocked,
 * benchmarks/perf/benchmark_transformer_gemm_shapes.py:100-115). */
size_t sharq_sf_offset(int r, int g, int groups_per_row) {
  size_t tiles_k = (size_t)((groups_per_row + 3) / 4);
  return (size_t)(r / 128) * tiles_k * 512 + (size_t)(g / 4) * 512 + (size_t)(r % 32) * 16 +
         (size_t)((r / 32) % 4) * 4 + (size_t)(g % 4);
}

/* Allocation size of a scale-factor buffer (kernels/src/bindings.cpp:50-60 and
 * kernels/include/sparse_nvfp4.h:145-151): one spare 128-row tile. */
size_t sharq_sf_alloc_bytes(int rows, int k) { return (size_t)(rows / 128 + 1) * 128 * (size_t)k / 16; }

/* Metadata buffer size: rows padded to 128, K padded to 256, 16 logical
 * elements per byte (sizes in the reference come from the CUTLASS compressor
 * utility, kernels/include/sparse_nvfp4.h:107-143). */
size_t sharq_e_bytes(int m, int k) {
  size_t am = (size_t)((m + 127) / 128) * 128;
  size_t ak = (size_t)((k + 255) / 256) * 256;
  return am * ak / 16;
}

/* Compressed A: rows x K/4 bytes with K padded to 256 (same utility). */
size_t sharq_a_comp_bytes(int m, int k) {
  size_t ak = (size_t)((k + 255) / 256) * 256;
  return (size_t)m * ak / 4;
}

static inline float fp_abs(float x) { return x < 0.0f ? -x : x; }
static inline float fp_max(float a, float b) { return a > b ? a : b; }
static inline float fp_min(float a, float b) { return a < b ? a : b; }
static inline float clamp_val(float x, float lo, float hi) { return fp_max(lo, fp_min(x, hi)); }

/* kernels/src/fused_sparse_prepare.cu:59-86: of the four adjacent pairs in an
 * 8-element chunk keep the two with the largest max(|a|,|b|); strict '>' so the
 * earlier pair wins a tie; indices returned ascending; an all-zero chunk keeps
 * pairs 0 and 1. */
static void top2_pair_indices_8(const float *vals, int *idx0, int *idx1) {
  float best0 = -1.0f, best1 = -1.0f;
  int i0 = 0, i1 = 1;
  for (int i = 0; i < 4; ++i) {
    float score = fp_max(fp_abs(vals[2 * i]), fp_abs(vals[2 * i + 1]));
    if (score > best0) {
      best1 = best0;
      i1 = i0;
      best0 = score;
      i0 = i;
    } else if (score > best1) {
      best1 = score;
      i1 = i;
    }
  }
  if (i1 < i0) {
    int t = i0;
    i0 = i1;
    i1 = t;
  }
  *idx0 = i0;
  *idx1 = i1;
}

/* One 32-element group of the fused prepare: kernels/src/fused_sparse_prepare.cu:118-250
 * (identical body at kernels/src/fused_rmsnorm_sparse_prepare.cu:210-324). */
static void prepare_group32(const float *x, int row, int g, int k, int aligned_m, uint8_t *a_comp,
                            uint8_t *e, uint8_t *q_sparse_dense, uint8_t *sfa_sparse,
                            uint8_t *q_res, uint8_t *sf_res) {
  int keep[32];
  float residual[32];
  uint8_t nib[32];
  int sel0[4], sel1[4];
  for (int i = 0; i < 32; ++i) {
    keep[i] = 0;
    residual[i] = x[i];
    nib[i] = 0;
  }
  float sparse_max = 0.0f;
  for (int c = 0; c < 4; ++c) {
    int i0, i1;
    top2_pair_indices_8(x + 8 * c, &i0, &i1);
    sel0[c] = i0;
    sel1[c] = i1;
    int p0 = 8 * c + 2 * i0, p1 = 8 * c + 2 * i1;
    keep[p0] = keep[p0 + 1] = keep[p1] = keep[p1 + 1] = 1;
    sparse_max = fp_max(sparse_max, fp_abs(x[p0]));
    sparse_max = fp_max(sparse_max, fp_abs(x[p0 + 1]));
    sparse_max = fp_max(sparse_max, fp_abs(x[p1]));
    sparse_max = fp_max(sparse_max, fp_abs(x[p1 + 1]));
  }
  float s_f = clamp_val(sparse_max / SHARQ_FP4_MAX, SHARQ_SCALE_EPS, SHARQ_FP8_MAX);
  uint8_t s_code = sharq_f32_to_ue4m3(s_f);
  float s_q = sharq_ue4m3_to_f32(s_code);
  float rs = 1.0f / s_q;
  for (int i = 0; i < 32; ++i) {
    if (!keep[i]) continue;
    float q = clamp_val(x[i] * rs, -SHARQ_FP4_MAX, SHARQ_FP4_MAX);
    uint8_t code = sharq_f32_to_e2m1(q);
    nib[i] = code & 0xF;
    float prod = sharq_e2m1_to_f32(code) * s_q; /* exact: 2-bit x 4-bit significands */
    residual[i] = x[i] - prod;
  }
  uint8_t res_packed[16];
  uint8_t res_scale[2];
  for (int h = 0; h < 2; ++h) {
    float rmax = 0.0f;
    for (int i = 0; i < 16; ++i) rmax = fp_max(rmax, fp_abs(residual[16 * h + i]));
    float r_f = clamp_val(rmax / SHARQ_FP4_MAX, SHARQ_SCALE_EPS, SHARQ_FP8_MAX);
    res_scale[h] = sharq_f32_to_ue4m3(r_f);
    float r_q = sharq_ue4m3_to_f32(res_scale[h]);
    float rr = 1.0f / r_q;
    for (int i = 0; i < 16; i += 2) {
      float q0 = clamp_val(residual[16 * h + i] * rr, -SHARQ_FP4_MAX, SHARQ_FP4_MAX);
      float q1 = clamp_val(residual[16 * h + i + 1] * rr, -SHARQ_FP4_MAX, SHARQ_FP4_MAX);
      res_packed[(16 * h + i) / 2] =
          (uint8_t)((sharq_f32_to_e2m1(q0) & 0xF) | ((sharq_f32_to_e2m1(q1) & 0xF) << 4));
    }
  }
  int g32 = k / 32, g16 = k / 16;
  sfa_sparse[sharq_sf_offset(row, g, g32)] = s_code;
  sf_res[sharq_sf_offset(row, 2 * g, g16)] = res_scale[0];
  sf_res[sharq_sf_offset(row, 2 * g + 1, g16)] = res_scale[1];
  size_t dense_row_bytes = (size_t)k / 2;
  if (q_sparse_dense) {
    uint8_t *p = q_sparse_dense + (size_t)row * dense_row_bytes + (size_t)g * 16;
    for (int i = 0; i < 16; ++i) p[i] = (uint8_t)(nib[2 * i] | (nib[2 * i + 1] << 4));
  }
  if (a_comp && e) {
    size_t comp_row_bytes = (size_t)k / 4;
    uint8_t *ap = a_comp + (size_t)row * comp_row_bytes + (size_t)g * 8;
    uint8_t *ep = e + (size_t)(g / 8) * (size_t)aligned_m * 16 + (size_t)row * 16 + (size_t)(g % 8) * 2;
    uint8_t mn[4];
    for (int c = 0; c < 4; ++c) {
      uint8_t db[4];
      for (int p = 0; p < 4; ++p) db[p] = (uint8_t)(nib[8 * c + 2 * p] | (nib[8 * c + 2 * p + 1] << 4));
      ap[2 * c] = db[sel0[c]];
      ap[2 * c + 1] = db[sel1[c]];
      mn[c] = (uint8_t)(sel0[c] | (sel1[c] << 2));
    }
    ep[0] = (uint8_t)(mn[0] | (mn[1] << 4));
    ep[1] = (uint8_t)(mn[2] | (mn[3] << 4));
  }
  memcpy(q_res + (size_t)row * dense_row_bytes + (size_t)g * 16, res_packed, 16);
}

/* Whole-buffer semantics of sharq_ops.fused_sparse_residual_quantize_x
 * (kernels/src/bindings.cpp:255-289): every output buffer is zero-filled, then
 * the kernel writes the used bytes.  Buffers must have the sizes returned by
 * sharq_a_comp_bytes / sharq_e_bytes / sharq_sf_alloc_bytes / m*k/2.
 * a_comp/e may both be NULL and q_sparse_dense non-NULL for the _debug op
 * (kernels/src/bindings.cpp:357-390). */
void sharq_oracle_prepare(const uint16_t *x_bf16, int m, int k, uint8_t *a_comp, uint8_t *e,
                          uint8_t *q_sparse_dense, uint8_t *sfa_sparse, uint8_t *q_res,
                          uint8_t *sf_res) {
  int aligned_m = (m + 127) / 128 * 128;
  if (a_comp) memset(a_comp, 0, sharq_a_comp_bytes(m, k));
  if (e) memset(e, 0, sharq_e_bytes(m, k));
  if (q_sparse_dense) memset(q_sparse_dense, 0, (size_t)m * k / 2);
  memset(sfa_sparse, 0, sharq_sf_alloc_bytes(m, k));
  memset(q_res, 0, (size_t)m * k / 2);
  memset(sf_res, 0, sharq_sf_alloc_bytes(m, k));
  for (int r = 0; r < m; ++r) {
    for (int g = 0; g < k / 32; ++g) {
      float x[32];
      for (int i = 0; i < 32; ++i) x[i] = sharq_bf16_to_f32(x_bf16[(size_t)r * k + 32 * g + i]);
      prepare_group32(x, r, g, k, aligned_m, a_comp, e, q_sparse_dense, sfa_sparse, q_res, sf_res);
    }
  }
}

/* kernels/src/fused_rmsnorm_sparse_prepare.cu:85-149.  Sum of squares: each
 * 32-element group is summed left to right, then the group sums are added left
 * to right (thread 0's loop at :120-124).  inv_rms uses the device rsqrtf,
 * which is an approximation (<= 2 ulp) that no CPU can reproduce bit for bit;
 * here it is 1/sqrt in double rounded to float.  Callers that need bit parity
 * downstream pass the device's inv_rms into sharq_oracle_rmsnorm_prepare.
 * sum_sq_out (optional) receives the exactly ordered sum for direct checks. */
void sharq_oracle_rmsnorm_row_stats(const uint16_t *x_bf16, const uint16_t *gamma_bf16, float eps,
                                    int m, int k, const float *inv_rms_in, float *inv_rms_out,
                                    float *row_absmax, float *sum_sq_out) {
  for (int r = 0; r < m; ++r) {
    float total = 0.0f;
    for (int g = 0; g < k / 32; ++g) {
      float s = 0.0f;
      for (int i = 0; i < 32; ++i) {
        float v = sharq_bf16_to_f32(x_bf16[(size_t)r * k + 32 * g + i]);
        s += v * v;
      }
      total += s;
    }
    if (sum_sq_out) sum_sq_out[r] = total;
    float arg = total / (float)k + eps;
    float inv = inv_rms_in ? inv_rms_in[r] : (float)(1.0 / sqrt((double)arg));
    if (inv_rms_out) inv_rms_out[r] = inv;
    float mx = 0.0f;
    for (int i = 0; i < k; ++i) {
      float y = sharq_bf16_to_f32(x_bf16[(size_t)r * k + i]) * inv;
      y = y * sharq_bf16_to_f32(gamma_bf16[i]);
      float yb = sharq_bf16_to_f32(sharq_f32_to_bf16(y));
      mx = fp_max(mx, fp_abs(yb));
    }
    row_absmax[r] = mx;
  }
}

/* Tensor scale glue at kernels/src/bindings.cpp:337 and model/quantize.py:43-44:
 * clamp(amax / 2688, min 1e-9).  ATen's CUDA division of a tensor by a host
 * scalar multiplies by the float reciprocal (cuda_mode != 0); on CPU it is a
 * true division (cuda_mode == 0). */
float sharq_oracle_tensor_scale(float amax, int cuda_mode) {
  float s;
  if (cuda_mode) {
    float inv = 1.0f / 2688.0f;
    s = amax * inv;
  } else {
    s = amax / 2688.0f;
  }
  return s < 1.0e-9f ? 1.0e-9f : s; /* NaN propagates like torch.clamp */
}

/* kernels/src/fused_rmsnorm_sparse_prepare.cu:152-325 with the whole-buffer
 * zero-fill of kernels/src/bindings.cpp:318-326. */
void sharq_oracle_rmsnorm_prepare(const uint16_t *x_bf16, const uint16_t *gamma_bf16,
                                  const float *inv_rms, float input_scale, int m, int k,
                                  uint8_t *a_comp, uint8_t *e, uint8_t *q_sparse_dense,
                                  uint8_t *sfa_sparse, uint8_t *q_res, uint8_t *sf_res) {
  int aligned_m = (m + 127) / 128 * 128;
  if (a_comp) memset(a_comp, 0, sharq_a_comp_bytes(m, k));
  if (e) memset(e, 0, sharq_e_bytes(m, k));
  if (q_sparse_dense) memset(q_sparse_dense, 0, (size_t)m * k / 2);
  memset(sfa_sparse, 0, sharq_sf_alloc_bytes(m, k));
  memset(q_res, 0, (size_t)m * k / 2);
  memset(sf_res, 0, sharq_sf_alloc_bytes(m, k));
  float sc = fp_max(input_scale, 1.0e-9f);
  for (int r = 0; r < m; ++r) {
    float inv = inv_rms[r];
    for (int g = 0; g < k / 32; ++g) {
      float x[32];
      for (int i = 0; i < 32; ++i) {
        size_t col = (size_t)32 * g + i;
        float y = sharq_bf16_to_f32(x_bf16[(size_t)r * k + col]) * inv;
        y = y * sharq_bf16_to_f32(gamma_bf16[col]);
        float yb = sharq_bf16_to_f32(sharq_f32_to_bf16(y));
        float scaled = yb / sc;
        x[i] = sharq_bf16_to_f32(sharq_f32_to_bf16(scaled));
      }
      prepare_group32(x, r, g, k, aligned_m, a_comp, e, q_sparse_dense, sfa_sparse, q_res, sf_res);
    }
  }
}

/* Host-side pre-scaling of the non-RMSNorm path, model/quantize.py:179-183:
 * x' = (x / scale).to(bf16) with x a bf16 tensor and scale a 0-dim float32 tensor.
 * cuda_mode == 0: torch on the CPU divides float(x) by the float32 scale.
 * cuda_mode != 0: torch on a CUDA device first casts the scale to the common dtype of the
 * operation, bf16, and divides float(x) by float(bf16(scale)) (pinned by
 * tests/golden/cuda_scale_division.npz, produced on a B200 by
 * tests/golden/make_cuda_scale_division.py). */
void sharq_oracle_scale_bf16(const uint16_t *x_bf16, float scale, size_t n, uint16_t *out_bf16, int cuda_mode) {
  float div = cuda_mode ? sharq_bf16_to_f32(sharq_f32_to_bf16(scale)) : scale;
  for (size_t i = 0; i < n; ++i) out_bf16[i] = sharq_f32_to_bf16(sharq_bf16_to_f32(x_bf16[i]) / div);
}

float sharq_oracle_absmax_bf16(const uint16_t *x_bf16, size_t n) {
  float mx = 0.0f;
  for (size_t i = 0; i < n; ++i) {
    float a = fabsf(sharq_bf16_to_f32(x_bf16[i]));
    if (a > mx || a != a) mx = a;
  }
  return mx;
}

/* kernels/src/shared_weight_nvfp4.cu:20-107 (+ zero-fill at kernels/src/bindings.cpp:405-406):
 * weight rows quantised in 32-element groups; the group scale goes to the
 * sparse-layout buffer and, duplicated into two 16-group slots, to the dense one. */
void sharq_oracle_quantize_w32_shared(const uint16_t *w_bf16, int n, int k, uint8_t *qw,
                                      uint8_t *sfw_sparse, uint8_t *sfw_dense) {
  memset(sfw_sparse, 0, sharq_sf_alloc_bytes(n, k));
  memset(sfw_dense, 0, sharq_sf_alloc_bytes(n, k));
  int g32 = k / 32, g16 = k / 16;
  for (int r = 0; r < n; ++r) {
    for (int g = 0; g < g32; ++g) {
      const uint16_t *p = w_bf16 + (size_t)r * k + 32 * g;
      float maxv = 0.0f;
      for (int i = 0; i < 32; ++i) maxv = fmaxf(maxv, fabsf(sharq_bf16_to_f32(p[i])));
      float scale = fminf(fmaxf(maxv / SHARQ_FP4_MAX, SHARQ_SCALE_EPS), SHARQ_FP8_MAX);
      uint8_t code = sharq_f32_to_ue4m3(scale);
      float inv = 1.0f / sharq_ue4m3_to_f32(code);
      sfw_sparse[sharq_sf_offset(r, g, g32)] = code;
      sfw_dense[sharq_sf_offset(r, 2 * g, g16)] = code;
      sfw_dense[sharq_sf_offset(r, 2 * g + 1, g16)] = code;
      uint8_t *q = qw + (size_t)r * (k / 2) + 16 * g;
      for (int i = 0; i < 32; i += 2) {
        float r0 = fminf(fmaxf(sharq_bf16_to_f32(p[i]) * inv, -SHARQ_FP4_MAX), SHARQ_FP4_MAX);
        float r1 = fminf(fmaxf(sharq_bf16_to_f32(p[i + 1]) * inv, -SHARQ_FP4_MAX), SHARQ_FP4_MAX);
        q[i / 2] = (uint8_t)((sharq_f32_to_e2m1(r0) & 0xF) | ((sharq_f32_to_e2m1(r1) & 0xF) << 4));
      }
    }
  }
}

/* kernels/src/shared_weight_nvfp4.cu:138-162 (+ zero-fill at kernels/src/bindings.cpp:429). */
void sharq_oracle_duplicate_sf32_to_sf16(const uint8_t *sf32, int rows, int k, uint8_t *sf16) {
  memset(sf16, 0, sharq_sf_alloc_bytes(rows, k));
  int g32 = k / 32, g16 = k / 16;
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < g32; ++g) {
      uint8_t c = sf32[sharq_sf_offset(r, g, g32)];
      sf16[sharq_sf_offset(r, 2 * g, g16)] = c;
      sf16[sharq_sf_offset(r, 2 * g + 1, g16)] = c;
    }
}

/* Dense NVFP4 quantisation with identity reorder and no outlier tail:
 * kernels/src/reorder.cu:69-203 (16 elements per thread), :381-555 (32 per
 * thread, two 16-groups) and kernels/src/down.cu:72-233 reduce to the same
 * arithmetic when KE == 0.  The reciprocal there is written `1.0 / x`, a double
 * division rounded to float (reorder.cu:146).  Outputs are allocated with
 * torch::empty in the reference (bindings.cpp:83-84), so only the written bytes
 * are defined; this function leaves the rest untouched. */
void sharq_oracle_quantize_dense_nvfp4(const uint16_t *x_bf16, int rows, int k, uint8_t *q,
                                       uint8_t *sf) {
  int g16 = k / 16;
  for (int r = 0; r < rows; ++r) {
    for (int g = 0; g < g16; ++g) {
      const uint16_t *p = x_bf16 + (size_t)r * k + 16 * g;
      float maxv = 0.0f;
      for (int i = 0; i < 16; ++i) maxv = fp_max(maxv, fp_abs(sharq_bf16_to_f32(p[i])));
      float scale = clamp_val(maxv / SHARQ_FP4_MAX, SHARQ_SCALE_EPS, SHARQ_FP8_MAX);
      uint8_t code = sharq_f32_to_ue4m3(scale);
      float r_scale = (float)(1.0 / (double)sharq_ue4m3_to_f32(code));
      sf[sharq_sf_offset(r, g, g16)] = code;
      uint8_t *qo = q + (size_t)r * (k / 2) + 8 * g;
      for (int i = 0; i < 16; i += 2) {
        float r0 = clamp_val(sharq_bf16_to_f32(p[i]) * r_scale, -SHARQ_FP4_MAX, SHARQ_FP4_MAX);
        float r1 = clamp_val(sharq_bf16_to_f32(p[i + 1]) * r_scale, -SHARQ_FP4_MAX, SHARQ_FP4_MAX);
        qo[i / 2] = (uint8_t)((sharq_f32_to_e2m1(r0) & 0xF) | ((sharq_f32_to_e2m1(r1) & 0xF) << 4));
      }
    }
  }
}

/* The structured-sparse compressor the reference calls for its debug path
 * (kernels/src/bindings.cpp:164-230; algorithm published in NVIDIA CUTLASS,
 * cutlass/transform/kernel/sm90_sparse_gemm_compressor.hpp, version unpinned by
 * the reference, 4.5.0 read here): per 4-byte chunk the bytes that are non-zero
 * after masking both sign bits are kept in order; a single survivor at index 3
 * becomes (0, x) with indices (0,3), a single survivor elsewhere (x, 0) with
 * indices (i,3); an empty chunk gives zeros with indices (0,0). */
void sharq_oracle_compress_sparse_a(const uint8_t *a_dense, int m, int k, uint8_t *a_comp, uint8_t *e) {
  int aligned_m = (m + 127) / 128 * 128;
  memset(a_comp, 0, sharq_a_comp_bytes(m, k));
  memset(e, 0, sharq_e_bytes(m, k));
  for (int r = 0; r < m; ++r) {
    for (int c = 0; c < k / 8; ++c) {
      const uint8_t *d = a_dense + (size_t)r * (k / 2) + 4 * (size_t)c;
      int idx[2] = {0, 0};
      uint8_t val[2] = {0, 0};
      int cnt = 0;
      for (int p = 0; p < 4; ++p) {
        if ((d[p] & 0x77) != 0 && cnt < 2) {
          idx[cnt] = p;
          val[cnt] = d[p];
          cnt++;
        }
      }
      if (cnt == 1 && idx[0] == 3) {
        val[1] = val[0];
        val[0] = 0;
        idx[0] = 0;
        idx[1] = 3;
      } else if (cnt == 1) {
        val[1] = 0;
        idx[1] = 3;
      }
      a_comp[(size_t)r * (k / 4) + 2 * (size_t)c] = val[0];
      a_comp[(size_t)r * (k / 4) + 2 * (size_t)c + 1] = val[1];
      uint8_t nibble = (uint8_t)(idx[0] | (idx[1] << 2));
      int g = c / 4; /* 32-element group */
      size_t off = (size_t)(g / 8) * (size_t)aligned_m * 16 + (size_t)r * 16 + (size_t)(g % 8) * 2 +
                   (size_t)((c % 4) / 2);
      e[off] |= (uint8_t)((c & 1) ? (nibble << 4) : nibble);
    }
  }
}

/* ------------------------------------------------------------------------- */
/* dequantisation (for GEMM checks): the exact real values the tensor core    */
/* multiplies.                                                                */
/* ------------------------------------------------------------------------- */

/* Dense payload [rows, k/2] + blocked scales with `group` (16 or 32) -> float [rows, k]. */
void sharq_oracle_dequant_dense(const uint8_t *q, const uint8_t *sf, int rows, int k, int group,
                                float *out) {
  int gpr = k / group;
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < k; ++c) {
      uint8_t b = q[(size_t)r * (k / 2) + c / 2];
      uint8_t code = (c & 1) ? (b >> 4) : (b & 0xF);
      float s = sharq_ue4m3_to_f32(sf[sharq_sf_offset(r, c / group, gpr)]);
      out[(size_t)r * k + c] = sharq_e2m1_to_f32(code) * s;
    }
}

/* Compressed A + metadata + 32-group scales -> float [m, k] (zeros at dropped
 * positions).  Layouts as written by kernels/src/fused_sparse_prepare.cu:215-242. */
void sharq_oracle_dequant_sparse(const uint8_t *a_comp, const uint8_t *e, const uint8_t *sfa, int m,
                                 int k, float *out) {
  int aligned_m = (m + 127) / 128 * 128;
  int g32 = k / 32;
  memset(out, 0, (size_t)m * k * sizeof(float));
  for (int r = 0; r < m; ++r)
    for (int c = 0; c < k / 8; ++c) {
      int g = c / 4;
      size_t off = (size_t)(g / 8) * (size_t)aligned_m * 16 + (size_t)r * 16 + (size_t)(g % 8) * 2 +
                   (size_t)((c % 4) / 2);
      uint8_t nibble = (c & 1) ? (e[off] >> 4) : (e[off] & 0xF);
      int idx[2] = {nibble & 3, (nibble >> 2) & 3};
      float s = sharq_ue4m3_to_f32(sfa[sharq_sf_offset(r, g, g32)]);
      for (int j = 0; j < 2; ++j) {
        uint8_t b = a_comp[(size_t)r * (k / 4) + 2 * (size_t)c + j];
        size_t base = (size_t)r * k + 8 * (size_t)c + 2 * (size_t)idx[j];
        out[base] += sharq_e2m1_to_f32(b & 0xF) * s;
        out[base + 1] += sharq_e2m1_to_f32(b >> 4) * s;
      }
    }
}
