// Element-wise steps of a decoder layer that sit between the SharQ linears, as single
// kernels for sm_100a.  The reference leaves both to HuggingFace's PyTorch code
// (model/qLlamaLayer.py:137-141 rotary embedding, :183-185 act_fn(gate) * up); as ATen ops on
// strided views they cost more than the quantised GEMMs they connect, so the prefill path
// runs them here.  Every intermediate is rounded to bf16 exactly where the PyTorch
// composition rounds, so results are those of the ATen ops.
//
//   rope_inplace      x*cos + rotate_half(x)*sin on the query and key heads of a merged
//                     qkv activation, in place: bf16(bf16(x*cos) + bf16(rot*sin))
//   swiglu_absmax     h = bf16(bf16(silu(gate)) * up) from a merged gate_up activation, plus
//                     the tensor-wide max|h| the scaled prepare of down_proj needs, so that
//                     prepare does not have to read h a second time for it
//   add_rmsnorm       y = bf16(s * rsqrt(mean(s^2) + eps) * gamma) with s = bf16(x + residual)
//                     (or s = x), products and mean in float: the normalised bf16 activation
//                     that a mixture-of-experts router and its experts both read
//                     (model/qMixtralLayer.py:205-213), in one pass instead of six ATen passes
#include <cuda_bf16.h>

#include <cstdint>

#include "decoder_ops.cuh"

namespace sharq {

namespace {

__device__ __forceinline__ float lo_f(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float exp2f_approx(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

__device__ __forceinline__ float rcp_approx(float v) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}

// one element of the rotary embedding: bf16(bf16(x * c) + bf16(r * s))
__device__ __forceinline__ float rope1(float x, float r, float c, float s) {
  return round_bf16(__fmul_rn(x, c)) + round_bf16(__fmul_rn(r, s));
}

// A thread rotates 8 elements of the first half of a head with their 8 partners in the
// second half (rotate_half pairs element d with d + D/2).
__global__ void __launch_bounds__(256) rope_kernel(__nv_bfloat16 *__restrict__ x, long long rows, long long row_stride,
                                                   int seq_len, int heads, int head_dim,
                                                   const __nv_bfloat16 *__restrict__ cos_t,
                                                   const __nv_bfloat16 *__restrict__ sin_t) {
  const int half = head_dim >> 1;
  const int vecs = half >> 3;  // 16-byte vectors per half head
  const long long total = rows * heads * vecs;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vecs);
    const long long rh = i / vecs;
    const int head = (int)(rh % heads);
    const long long row = rh / heads;
    const int pos = (int)(row % seq_len);
    __nv_bfloat16 *p = x + row * row_stride + (long long)head * head_dim + v * 8;
    const __nv_bfloat16 *c = cos_t + (long long)pos * head_dim + v * 8;
    const __nv_bfloat16 *s = sin_t + (long long)pos * head_dim + v * 8;
    const uint4 a4 = *reinterpret_cast<const uint4 *>(p);
    const uint4 b4 = *reinterpret_cast<const uint4 *>(p + half);
    const uint4 ca4 = __ldg(reinterpret_cast<const uint4 *>(c));
    const uint4 cb4 = __ldg(reinterpret_cast<const uint4 *>(c + half));
    const uint4 sa4 = __ldg(reinterpret_cast<const uint4 *>(s));
    const uint4 sb4 = __ldg(reinterpret_cast<const uint4 *>(s + half));
    const uint32_t a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
    const uint32_t ca[4] = {ca4.x, ca4.y, ca4.z, ca4.w}, cb[4] = {cb4.x, cb4.y, cb4.z, cb4.w};
    const uint32_t sa[4] = {sa4.x, sa4.y, sa4.z, sa4.w}, sb[4] = {sb4.x, sb4.y, sb4.z, sb4.w};
    uint32_t oa[4], ob[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // first half: x*cos + (-partner)*sin ; second half: x*cos + partner*sin
      oa[j] = pack2(rope1(lo_f(a[j]), -lo_f(b[j]), lo_f(ca[j]), lo_f(sa[j])),
                    rope1(hi_f(a[j]), -hi_f(b[j]), hi_f(ca[j]), hi_f(sa[j])));
      ob[j] = pack2(rope1(lo_f(b[j]), lo_f(a[j]), lo_f(cb[j]), lo_f(sb[j])),
                    rope1(hi_f(b[j]), hi_f(a[j]), hi_f(cb[j]), hi_f(sb[j])));
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
    *reinterpret_cast<uint4 *>(p + half) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
  }
}

// silu as ATen computes it for a bf16 tensor: x / (1 + exp(-x)) in float, rounded to bf16.
// The kernel would be bound by the accurate expf and the IEEE division, so the value is first
// formed with the approximate exp2 and reciprocal units: for |x| <= 16 that result is within
// (1.5 |x| + 8) * 2^-24 <= 2^-19 relative (32 float ulps) of the true value (argument
// rounding 1.5 |x|, ex2.approx 4, the addition 1, rcp.approx 2, the product 1), and the
// accurate formula within 3 ulps.  When the fast value lies more than 40 ulps from every bf16
// rounding boundary (float bits ...8000) both round to the same bf16 number; otherwise, and
// for |x| > 16, the accurate formula is evaluated.
__device__ __forceinline__ float silu_accurate(float x) { return x / (1.0f + expf(-x)); }

__device__ __forceinline__ float silu_bf16(float x) {
  const float e = exp2f_approx(-1.4426950408889634f * x);
  const float fast = x * rcp_approx(1.0f + e);
  const uint32_t t = (__float_as_uint(fast) + 0x8000u + 40u) & 0xFFFFu;
  float v = fast;
  if (!(fabsf(x) <= 16.0f && t >= 81u)) v = silu_accurate(x);
  return round_bf16(v);
}

// One CTA walks rows; its 256 threads hold up to four 16-byte vectors of the row each (K <= 8192)
// between the sum of squares and the scaling, so the row is read once.
constexpr int kNormThreads = 256;
constexpr int kNormVecsPerThread = 4;

template <bool kAdd>
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(const __nv_bfloat16 *__restrict__ x,
                                                                   const __nv_bfloat16 *__restrict__ residual,
                                                                   __nv_bfloat16 *__restrict__ sum_out,
                                                                   const __nv_bfloat16 *__restrict__ gamma, float eps,
                                                                   long long rows, int k, __nv_bfloat16 *__restrict__ out) {
  __shared__ float warp_sum[kNormThreads / 32];
  const int vecs = k >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4 *xs = reinterpret_cast<const uint4 *>(x + row * k);
    uint4 v[kNormVecsPerThread];
#pragma unroll
    for (int i = 0; i < kNormVecsPerThread; ++i) {
      const int j = threadIdx.x + i * kNormThreads;
      if (j < vecs) v[i] = __ldg(xs + j);
    }
    if (kAdd) {
      const uint4 *rs = reinterpret_cast<const uint4 *>(residual + row * k);
      uint4 *ss = reinterpret_cast<uint4 *>(sum_out + row * k);
#pragma unroll
      for (int i = 0; i < kNormVecsPerThread; ++i) {
        const int j = threadIdx.x + i * kNormThreads;
        if (j < vecs) {
          const uint4 r = __ldg(rs + j);
          // bf16(x + residual), rounded like the ATen add
          v[i].x = pack2(__fadd_rn(lo_f(v[i].x), lo_f(r.x)), __fadd_rn(hi_f(v[i].x), hi_f(r.x)));
          v[i].y = pack2(__fadd_rn(lo_f(v[i].y), lo_f(r.y)), __fadd_rn(hi_f(v[i].y), hi_f(r.y)));
          v[i].z = pack2(__fadd_rn(lo_f(v[i].z), lo_f(r.z)), __fadd_rn(hi_f(v[i].z), hi_f(r.z)));
          v[i].w = pack2(__fadd_rn(lo_f(v[i].w), lo_f(r.w)), __fadd_rn(hi_f(v[i].w), hi_f(r.w)));
          ss[j] = v[i];
        }
      }
    }
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormVecsPerThread; ++i) {
      const int j = threadIdx.x + i * kNormThreads;
      if (j < vecs) {
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float a = lo_f(w[t]), b = hi_f(w[t]);
          sq = __fmaf_rn(a, a, sq);
          sq = __fmaf_rn(b, b, sq);
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
    __syncthreads();  // warp_sum may still be read by the previous row
    if (lane == 0) warp_sum[warp] = sq;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += warp_sum[w];  // same order in every thread
    const float inv = rsqrtf(total / (float)k + eps);
    const uint4 *gs = reinterpret_cast<const uint4 *>(gamma);
    uint4 *os = reinterpret_cast<uint4 *>(out + row * k);
#pragma unroll
    for (int i = 0; i < kNormVecsPerThread; ++i) {
      const int j = threadIdx.x + i * kNormThreads;
      if (j < vecs) {
        const uint4 g = __ldg(gs + j);
        uint4 y;
        y.x = pack2(__fmul_rn(__fmul_rn(lo_f(v[i].x), inv), lo_f(g.x)), __fmul_rn(__fmul_rn(hi_f(v[i].x), inv), hi_f(g.x)));
        y.y = pack2(__fmul_rn(__fmul_rn(lo_f(v[i].y), inv), lo_f(g.y)), __fmul_rn(__fmul_rn(hi_f(v[i].y), inv), hi_f(g.y)));
        y.z = pack2(__fmul_rn(__fmul_rn(lo_f(v[i].z), inv), lo_f(g.z)), __fmul_rn(__fmul_rn(hi_f(v[i].z), inv), hi_f(g.z)));
        y.w = pack2(__fmul_rn(__fmul_rn(lo_f(v[i].w), inv), lo_f(g.w)), __fmul_rn(__fmul_rn(hi_f(v[i].w), inv), hi_f(g.w)));
        os[j] = y;
      }
    }
  }
}

// CTA-wide maximum of a packed |value| accumulator, raised into *amax_bits (may be null).  All 256 threads call it.
__device__ __forceinline__ void cta_absmax_to(float *warp_max, __nv_bfloat162 mx2, unsigned int *amax_bits) {
  float mx = fmaxf(__bfloat162float(mx2.x), __bfloat162float(mx2.y));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // warp_max may still be read by the previous call
  if (lane == 0) warp_max[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    mx = lane < 8 ? warp_max[lane] : 0.0f;
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    // non-negative floats order like their bit patterns
    if (lane == 0 && amax_bits != nullptr) atomicMax(amax_bits, __float_as_uint(mx));
  }
}

// With unit_group != nullptr (grouped activation of a mixture-of-experts layer: rows sorted by
// group, 256-row units, unit_group[u] < 0 = no rows) a CTA takes chunks of kGroupedChunkRows
// consecutive rows, skips chunks of empty units and raises amax_bits[group of the chunk].
constexpr int kGroupedChunkRows = 64;

__global__ void __launch_bounds__(256) swiglu_absmax_kernel(const __nv_bfloat16 *__restrict__ gate_up, long long rows,
                                                            int ffn, long long row_stride, __nv_bfloat16 *__restrict__ h,
                                                            unsigned int *__restrict__ amax_bits,
                                                            const int *__restrict__ unit_group) {
  __shared__ float warp_max[8];
  const int vecs = ffn >> 3;
  __nv_bfloat162 mx2 = __floats2bfloat162_rn(0.0f, 0.0f);  // running max of |h|, two lanes
  const bool grouped = unit_group != nullptr;
  const long long n_chunks = grouped ? (rows + kGroupedChunkRows - 1) / kGroupedChunkRows : rows;
  // a CTA walks rows (chunks of rows when grouped), its threads the 16-byte vectors of a row, two vectors in flight per thread
  for (long long chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
   const long long row_lo = grouped ? chunk * kGroupedChunkRows : chunk;
   const long long row_hi = grouped ? min(rows, row_lo + kGroupedChunkRows) : chunk + 1;
   const int grp = grouped ? unit_group[row_lo / 256] : 0;
   if (grp < 0) continue;
   for (long long row = row_lo; row < row_hi; ++row) {
    const __nv_bfloat16 *grow = gate_up + row * row_stride;
    __nv_bfloat16 *hrow = h + row * (long long)ffn;
    for (int v0 = threadIdx.x; v0 < vecs; v0 += 2 * blockDim.x) {
      uint4 g4[2], u4[2];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int v = v0 + t * blockDim.x;
        if (v < vecs) {
          g4[t] = __ldg(reinterpret_cast<const uint4 *>(grow + v * 8));
          u4[t] = __ldg(reinterpret_cast<const uint4 *>(grow + ffn + v * 8));
        }
      }
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int v = v0 + t * blockDim.x;
        if (v >= vecs) break;
        const uint32_t gw[4] = {g4[t].x, g4[t].y, g4[t].z, g4[t].w}, uw[4] = {u4[t].x, u4[t].y, u4[t].z, u4[t].w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // the product of two bf16 values is exact in float; the packed conversion rounds it once
          o[j] = pack2(__fmul_rn(silu_bf16(lo_f(gw[j])), lo_f(uw[j])), __fmul_rn(silu_bf16(hi_f(gw[j])), hi_f(uw[j])));
          mx2 = __hmax2(mx2, __habs2(*reinterpret_cast<__nv_bfloat162 *>(&o[j])));
        }
        *reinterpret_cast<uint4 *>(hrow + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
   }
   if (grouped) {  // one reduction per chunk, into the chunk's group
     cta_absmax_to(warp_max, mx2, amax_bits == nullptr ? nullptr : amax_bits + grp);
     mx2 = __floats2bfloat162_rn(0.0f, 0.0f);
   }
  }
  if (!grouped) cta_absmax_to(warp_max, mx2, amax_bits);
}

// Tensor absmax per group of a grouped bf16 activation [rows, width] (see swiglu_absmax_kernel).
__global__ void __launch_bounds__(256) abs_stats_grouped_kernel(const __nv_bfloat16 *__restrict__ x, long long rows, int width,
                                                                unsigned int *__restrict__ amax_bits,
                                                                const int *__restrict__ unit_group,
                                                                const int *__restrict__ src_row) {
  __shared__ float warp_max[8];
  const int vecs = width >> 3;
  const long long n_chunks = (rows + kGroupedChunkRows - 1) / kGroupedChunkRows;
  for (long long chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    const long long row_lo = chunk * kGroupedChunkRows, row_hi = min(rows, row_lo + kGroupedChunkRows);
    const int grp = unit_group[row_lo / 256];
    if (grp < 0) continue;
    __nv_bfloat162 mx2 = __floats2bfloat162_rn(0.0f, 0.0f);
    const long long n16 = (row_hi - row_lo) * vecs;
    for (long long i = threadIdx.x; i < n16; i += blockDim.x) {
      const long long r = row_lo + i / vecs;
      const long long in_row = src_row != nullptr ? src_row[r] : r;  // gathered rows; < 0: a padding row
      if (in_row < 0) continue;
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + in_row * width) + (i % vecs));
      mx2 = __hmax2(mx2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&v.x)));
      mx2 = __hmax2(mx2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&v.y)));
      mx2 = __hmax2(mx2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&v.z)));
      mx2 = __hmax2(mx2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&v.w)));
    }
    cta_absmax_to(warp_max, mx2, amax_bits + grp);
  }
}

// Output of a grouped mixture-of-experts FFN back into token order: token t sums its top_k expert
// outputs y[dest[t, j], :] * w[t, j] in ascending order of the expert index, every product and every
// partial sum rounded to bf16 - the arithmetic of the reference's per-expert loop
// `final.index_add_(0, top_x, y * w[top_x, idx, None])` (model/qMixtralLayer.py:223-231), which
// visits the experts in that order on a zero-initialised buffer.
constexpr int kCombineMaxTopK = 8;
__global__ void __launch_bounds__(256) moe_combine_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ y,
                                                          const int *__restrict__ dest, const long long *__restrict__ selected,
                                                          const __nv_bfloat16 *__restrict__ w, long long tokens, int top_k,
                                                          int width) {
  const int vecs = width >> 3;
  for (long long t = blockIdx.x; t < tokens; t += gridDim.x) {
    // slots of this token in ascending expert order (every thread computes the same tiny sort)
    int order[kCombineMaxTopK];
    for (int j = 0; j < top_k; ++j) order[j] = j;
    for (int a = 1; a < top_k; ++a)
      for (int b = a; b > 0 && selected[t * top_k + order[b]] < selected[t * top_k + order[b - 1]]; --b) {
        const int tmp = order[b];
        order[b] = order[b - 1];
        order[b - 1] = tmp;
      }
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < top_k; ++j) {
        const int slot = order[j];
        const float wj = __bfloat162float(w[t * top_k + slot]);
        const uint4 yv = __ldg(reinterpret_cast<const uint4 *>(y + (long long)dest[t * top_k + slot] * width) + v);
        const uint32_t yw[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[2 * q] = round_bf16(acc[2 * q] + round_bf16(__fmul_rn(lo_f(yw[q]), wj)));
          acc[2 * q + 1] = round_bf16(acc[2 * q + 1] + round_bf16(__fmul_rn(hi_f(yw[q]), wj)));
        }
      }
      *reinterpret_cast<uint4 *>(out + t * width + (long long)v * 8) =
          make_uint4(pack2(acc[0], acc[1]), pack2(acc[2], acc[3]), pack2(acc[4], acc[5]), pack2(acc[6], acc[7]));
    }
  }
}

// Expert output back into the token-major buffer of a mixture-of-experts layer:
// out[rows[i], :] = bf16(out[rows[i], :] + bf16(y[i, :] * w[i])), rounded like the ATen
// `index_add_(0, rows, y * w[:, None])`.  A token reaches an expert at most once, so the rows of
// one call are distinct and no atomics are needed.  An index outside [0, out_rows) is skipped.
__global__ void __launch_bounds__(256) scatter_add_scaled_kernel(__nv_bfloat16 *__restrict__ out,
                                                                 const __nv_bfloat16 *__restrict__ y,
                                                                 const long long *__restrict__ rows,
                                                                 const __nv_bfloat16 *__restrict__ w, long long n_rows,
                                                                 int width, long long out_rows) {
  const int vecs = width >> 3;
  for (long long r = blockIdx.x; r < n_rows; r += gridDim.x) {
    const long long target = rows[r];
    if (target < 0 || target >= out_rows) continue;
    const float wr = __bfloat162float(w[r]);
    const uint4 *src = reinterpret_cast<const uint4 *>(y + r * (long long)width);
    uint4 *dst = reinterpret_cast<uint4 *>(out + target * (long long)width);
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      const uint4 a4 = __ldg(src + v);
      const uint4 o4 = dst[v];
      const uint32_t a[4] = {a4.x, a4.y, a4.z, a4.w}, o[4] = {o4.x, o4.y, o4.z, o4.w};
      uint32_t res[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        res[j] = pack2(lo_f(o[j]) + round_bf16(__fmul_rn(lo_f(a[j]), wr)), hi_f(o[j]) + round_bf16(__fmul_rn(hi_f(a[j]), wr)));
      dst[v] = make_uint4(res[0], res[1], res[2], res[3]);
    }
  }
}

int sm_count() {
  static int sms[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0 && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms[dev] = 148;
  return sms[dev];
}

unsigned grid_for(long long work_items) {
  long long blocks = (work_items + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

}  // namespace

cudaError_t run_rope_inplace(void *x, long long rows, long long row_stride, int seq_len, int heads, int head_dim,
                             const void *cos_t, const void *sin_t, cudaStream_t stream) {
  const long long items = rows * heads * (head_dim / 16);
  rope_kernel<<<grid_for(items), 256, 0, stream>>>(static_cast<__nv_bfloat16 *>(x), rows, row_stride, seq_len, heads,
                                                   head_dim, static_cast<const __nv_bfloat16 *>(cos_t),
                                                   static_cast<const __nv_bfloat16 *>(sin_t));
  return cudaGetLastError();
}

cudaError_t run_scatter_add_scaled(void *out, const void *y, const long long *rows, const void *w, long long n_rows,
                                   int width, long long out_rows, cudaStream_t stream) {
  long long ctas = (long long)sm_count() * 8;
  if (ctas > n_rows) ctas = n_rows;
  if (ctas < 1) return cudaSuccess;
  scatter_add_scaled_kernel<<<(unsigned)ctas, 256, 0, stream>>>(static_cast<__nv_bfloat16 *>(out),
                                                                static_cast<const __nv_bfloat16 *>(y), rows,
                                                                static_cast<const __nv_bfloat16 *>(w), n_rows, width, out_rows);
  return cudaGetLastError();
}

cudaError_t run_add_rmsnorm(const void *x, const void *residual, void *sum_out, const void *gamma, float eps, long long rows,
                            int k, void *out, cudaStream_t stream) {
  if (k <= 0 || (k & 7) != 0 || k > 8 * kNormThreads * kNormVecsPerThread) return cudaErrorInvalidValue;
  long long ctas = (long long)sm_count() * 8;
  if (ctas > rows) ctas = rows;
  if (ctas < 1) return cudaSuccess;
  if (residual != nullptr)
    add_rmsnorm_kernel<true><<<(unsigned)ctas, kNormThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(residual),
        static_cast<__nv_bfloat16 *>(sum_out), static_cast<const __nv_bfloat16 *>(gamma), eps, rows, k,
        static_cast<__nv_bfloat16 *>(out));
  else
    add_rmsnorm_kernel<false><<<(unsigned)ctas, kNormThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(x), nullptr, nullptr, static_cast<const __nv_bfloat16 *>(gamma), eps, rows, k,
        static_cast<__nv_bfloat16 *>(out));
  return cudaGetLastError();
}

cudaError_t run_swiglu_absmax(const void *gate_up, long long rows, int ffn, long long row_stride, void *h,
                              unsigned int *amax_bits, cudaStream_t stream, const int *unit_group, int groups) {
  if (amax_bits != nullptr) {
    cudaError_t err = cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int) * (unit_group != nullptr ? groups : 1), stream);
    if (err != cudaSuccess) return err;
  }
  long long ctas = (long long)sm_count() * 8;
  const long long work = unit_group != nullptr ? (rows + kGroupedChunkRows - 1) / kGroupedChunkRows : rows;
  if (ctas > work) ctas = work;
  swiglu_absmax_kernel<<<(unsigned)ctas, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(gate_up), rows, ffn,
                                                            row_stride, static_cast<__nv_bfloat16 *>(h), amax_bits, unit_group);
  return cudaGetLastError();
}

cudaError_t run_abs_stats_grouped(const void *x, long long rows, int width, unsigned int *amax_bits, const int *unit_group,
                                  int groups, cudaStream_t stream, const int *src_row) {
  cudaError_t err = cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int) * groups, stream);
  if (err != cudaSuccess) return err;
  long long ctas = (long long)sm_count() * 8;
  const long long work = (rows + kGroupedChunkRows - 1) / kGroupedChunkRows;
  if (ctas > work) ctas = work;
  abs_stats_grouped_kernel<<<(unsigned)ctas, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), rows, width, amax_bits,
                                                                unit_group, src_row);
  return cudaGetLastError();
}

cudaError_t run_moe_combine(void *out, const void *y, const int *dest, const long long *selected, const void *w,
                            long long tokens, int top_k, int width, cudaStream_t stream) {
  if (top_k < 1 || top_k > kCombineMaxTopK) return cudaErrorInvalidValue;
  long long ctas = (long long)sm_count() * 8;
  if (ctas > tokens) ctas = tokens;
  if (ctas < 1) return cudaSuccess;
  moe_combine_kernel<<<(unsigned)ctas, 256, 0, stream>>>(static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(y),
                                                          dest, selected, static_cast<const __nv_bfloat16 *>(w), tokens, top_k,
                                                          width);
  return cudaGetLastError();
}

}  // namespace sharq
