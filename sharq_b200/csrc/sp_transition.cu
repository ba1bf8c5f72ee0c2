// Tensor-parallel layer transition in ONE kernel per GPU: everything between a row-parallel
// SharQ linear (o_proj, down_proj) and the next column-parallel one (gate_up, qkv),
//   reduce-scatter of the partial sums  ->  residual add  ->  RMSNorm statistics  ->
//   tensor-wide absmax over all GPUs  ->  4:8 sparse + residual NVFP4 prepare  ->
//   all-gather of the PACKED activation,
// over NVLink / NVSwitch peer memory.  The residual stream stays sharded by rows (tokens): a GPU
// owns M / world rows.  It pulls the fp32 in-switch sum of its rows of every GPU's partial
// product (multimem.ld_reduce), adds its rows of the residual stream, normalises and quantises
// them exactly as the single-GPU RMSNorm prepare does (same per-row inv_rms, same tensor scale,
// hence the same bytes), and pushes the packed result (A_comp, E, both scale buffers, Q_res:
// 0.906 bytes per element instead of 2 for bf16) into every GPU's copy of the prepared
// activation (multimem.st).  Compared with "all-reduce, then every GPU prepares all M rows"
// a GPU receives 1/world + 0.45 of the bf16 activation instead of all of it, and prepares
// M / world rows instead of M.
//
// The reference has no tensor parallelism (its parallel_utils only places whole layers), so
// this kernel has no counterpart there; its arithmetic is that of
// kernels/src/fused_rmsnorm_sparse_prepare.cu:85-325 and bindings.cpp:337 on this GPU's rows.
//
// Synchronisation (state words in symmetric memory, zero-initialised once; everything
// resets itself, so a captured launch can be replayed):
//   A  "partial products delivered": every GPU signals all others when its kernel starts (its GEMM,
//      whose epilogue stored into the peers, precedes it on the stream); all CTAs wait for all GPUs
//      before the first read of the collection buffer.
//   B  tensor absmax: after a grid-wide barrier CTA 0 stores {absmax, launch number} as one
//      8-byte word into every GPU's state; all CTAs wait until all words carry the number.
//   C  "broadcast landed": after its packed rows are stored to all GPUs, a GPU signals all
//      others; CTA 0 waits for all of them before the kernel ends, so the GEMM that follows on
//      the stream reads complete buffers.
// Every wait is bounded (about ten seconds); a wait that runs out sets *error_flag and the
// kernel carries on to its end (the result is then wrong, and the host sees the code).
// Plain peer / multicast loads and stores only: no TMA touches another GPU's memory.
#include <cuda_bf16.h>

#include <cstdint>
#include <cstdlib>

#include "prepare_device.cuh"
#include "sp_transition.cuh"

namespace sharq {

using namespace prep;

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kSmemBudget = 200 * 1024;
constexpr long long kWaitLimitCycles = 20000000000LL;  // about ten seconds: covers the skew between ranks that launch eagerly
long long g_wait_limit_cycles = kWaitLimitCycles;     // host-side setting, see set_sp_transition_wait_limit

// state words (uint32 index)
constexpr int kReady = 0;        // [16] counters
constexpr int kAmax = 16;        // [16] x 2 words {absmax bits, launch number}
constexpr int kDone = 48;        // [16] counters
constexpr int kEpoch = 64;       // launches completed
constexpr int kGridArrive = 65;  // CTA arrivals at the local grid barriers, monotonic
constexpr int kAmaxLocal = 66;   // [2] this GPU's absmax accumulator, by launch parity
constexpr int kStateWords = 80;

struct SpParams {
  const uint8_t *partial;             // this GPU's collection buffer [world][rows, k] bf16 (block s: GPU s's partial
                                      // products of this GPU's rows, stored there by GPU s's GEMM), or null
  const __nv_bfloat16 *residual_in;   // this GPU's rows [rows, k], or null
  __nv_bfloat16 *residual_out;        // this GPU's rows of the new residual stream [rows, k]
  const __nv_bfloat16 *gamma;
  float eps;
  float *inv_rms;                     // [rows] scratch
  float *scale_out;                   // tensor scale, one float on this GPU
  uint8_t *a_comp, *e, *sfa_sparse, *q_res, *sf_res;  // this GPU's copy of the prepared activation (all m rows)
  long long mc_delta;                 // multicast address of that copy minus its local address
  long long peer_delta[kSpMaxRanks];  // GPU r's copy as mapped here minus this GPU's copy (unicast all-gather)
  int unicast;                        // all-gather by plain peer stores instead of multimem.st
  uint32_t *state[kSpMaxRanks];       // state[r]: GPU r's state words as mapped here
  int rank, world;
  int m, k;                           // whole activation
  int row0, rows;                     // this GPU's row block
  int rows_per_cta, chunk_rows;
  long long wait_limit;               // clock cycles a wait may take
  int *error_flag;
};

__device__ __forceinline__ void st_multicast_16(uint8_t *mc_addr, const uint4 &v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void signal_add_release(uint32_t *flag) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long ld_acquire_sys64(const uint32_t *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys64(uint32_t *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Wait until the counter reaches `target` (wrap-safe).  False when the limit ran out.
__device__ __forceinline__ bool wait_counter(const uint32_t *p, uint32_t target, bool gpu_scope, long long limit) {
  const long long t0 = clock64();
  for (;;) {
    const uint32_t v = gpu_scope ? ld_acquire_gpu(p) : ld_acquire_sys(p);
    if ((int32_t)(v - target) >= 0) return true;
    if (clock64() - t0 > limit) return false;
  }
}

// Local grid barrier number `which` (1-based) of this launch; all CTAs arrive, and wait if asked.
__device__ __forceinline__ void grid_barrier(const SpParams &p, uint32_t epoch, int which, bool wait, int code) {
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t *arrive = p.state[p.rank] + kGridArrive;
    __threadfence();
    atomicAdd(arrive, 1u);
    if (wait && !wait_counter(arrive, (epoch * 3u + (uint32_t)which) * gridDim.x, true, p.wait_limit)) atomicExch(p.error_flag, code);
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kThreads, 1) sp_transition_kernel(const SpParams p) {
  const int k = p.k;
  const int groups32 = k >> 5;
  const int groups_padded = ((k + 255) / 256) * 8;
  const int aligned_m = (p.m + 127) / 128 * 128;
  const int row_vecs = k >> 3;
  const int partial_stride = groups32 + 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t *my_state = p.state[p.rank];

  __shared__ ScaleTables tbl;
  __shared__ float warp_red[kWarps];
  __shared__ uint32_t rank_amax[kSpMaxRanks];
  extern __shared__ uint4 sp_smem[];
  uint4 *gamma_s = sp_smem;
  uint4 *cache = sp_smem + row_vecs;
  float *partial = reinterpret_cast<float *>(cache + (size_t)p.chunk_rows * row_vecs);
  float *inv_s = partial + p.chunk_rows * partial_stride;

  const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(my_state + kEpoch);
  const uint32_t tag = epoch + 1u;

  // ---- A: tell every GPU that this GPU's partial sums are complete
  if (blockIdx.x == 0 && (int)threadIdx.x < p.world) {
    __threadfence_system();
    signal_add_release(p.state[threadIdx.x] + kReady + p.rank);
  }
  if (threadIdx.x < 128) {
    const float v = ue4m3_to_float(threadIdx.x);
    tbl.value[threadIdx.x] = v;
    tbl.recip[threadIdx.x] = __frcp_rn(v);
  }
  {
    const uint4 *gsrc = reinterpret_cast<const uint4 *>(p.gamma);
    for (int i = threadIdx.x; i < row_vecs; i += kThreads) gamma_s[cache_slot(i >> 2, i & 3)] = __ldg(gsrc + i);
  }
  // zero what no owner thread writes in THIS GPU's copy: the spare band of the scale buffers,
  // the tail of A_comp, padding rows of the metadata (none when m is a multiple of 128)
  {
    const int worker = blockIdx.x * kThreads + threadIdx.x;
    const int workers = gridDim.x * kThreads;
    const size_t bands = (size_t)aligned_m / 128;
    zero_range(p.sfa_sparse, bands * (size_t)(groups32 / 4) * 512, sf_alloc_bytes(p.m, k), worker, workers);
    zero_range(p.sf_res, bands * (size_t)(k / 16 / 4) * 512, sf_alloc_bytes(p.m, k), worker, workers);
    zero_range(p.a_comp, (size_t)p.m * (k / 4), a_comp_bytes(p.m, k), worker, workers);
  }
  // ---- A: wait for every GPU's partial sums
  if ((int)threadIdx.x < p.world) {
    if (!wait_counter(my_state + kReady + threadIdx.x, tag, false, p.wait_limit)) atomicExch(p.error_flag, 0x301);
  }
  __syncthreads();

  const int row_begin = min(p.rows, (int)blockIdx.x * p.rows_per_cta);  // local row index
  const int row_end = min(p.rows, row_begin + p.rows_per_cta);
  const int rows = row_end - row_begin;
  const int chunks = rows > 0 ? (rows + p.chunk_rows - 1) / p.chunk_rows : 0;
  const int first_chunk_rows = rows - (chunks - 1) * p.chunk_rows;
  auto chunk_first_row = [&](int c) { return c == 0 ? 0 : first_chunk_rows + (c - 1) * p.chunk_rows; };
  auto chunk_size = [&](int c) { return c == 0 ? first_chunk_rows : p.chunk_rows; };

  // ------------------------------------------------------------------ phase 1: reduce, add, statistics
  __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);
  for (int c = 0; c < chunks; ++c) {
    const int c_rows = chunk_size(c), c_row0 = row_begin + chunk_first_row(c);
    if (c > 0) __syncthreads();
    // 1a: sum of the `world` partial blocks (fp32, in rank order, one rounding to bf16 - the arithmetic of the
    // peer-copy all-reduce kernel) + residual add; the new residual rows go to global memory and,
    // group-permuted, into the shared-memory cache.  The blocks were written by other GPUs: L2 loads (.cg).
    const int n_vecs = c_rows * row_vecs;
    const size_t block_vecs = (size_t)p.rows * row_vecs;  // 16-byte vectors per source block
    for (int v0 = threadIdx.x; v0 < n_vecs; v0 += 2 * kThreads) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int v = v0 + u * kThreads;
        if (v >= n_vecs) continue;
        const int rl = v / row_vecs, i = v - rl * row_vecs;
        const size_t vec_l = (size_t)(c_row0 + rl) * row_vecs + i;  // vector index inside this GPU's row block
        uint32_t w[4];
        uint4 rv = make_uint4(0u, 0u, 0u, 0u);
        if (p.residual_in != nullptr) rv = __ldg(reinterpret_cast<const uint4 *>(p.residual_in) + vec_l);
        if (p.partial != nullptr) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          const uint4 *blk = reinterpret_cast<const uint4 *>(p.partial) + vec_l;
          for (int r0 = 0; r0 < p.world; r0 += 4) {  // four source blocks in flight
            uint4 pv[4];
#pragma unroll
            for (int t = 0; t < 4; ++t)
              if (r0 + t < p.world) pv[t] = __ldcg(blk + (size_t)(r0 + t) * block_vecs);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              if (r0 + t < p.world) {
                const uint32_t pw[4] = {pv[t].x, pv[t].y, pv[t].z, pv[t].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  acc[2 * q] += lo_f(pw[q]);
                  acc[2 * q + 1] += hi_f(pw[q]);
                }
              }
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) w[q] = pack_bf16x2(acc[2 * q], acc[2 * q + 1]);
        }
        const uint32_t r4[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (p.partial == nullptr)
            w[q] = r4[q];
          else if (p.residual_in != nullptr)  // bf16(residual + sum), rounded like the ATen add of two bf16 tensors
            w[q] = pack_bf16x2(__fadd_rn(lo_f(r4[q]), lo_f(w[q])), __fadd_rn(hi_f(r4[q]), hi_f(w[q])));
        }
        const uint4 out = make_uint4(w[0], w[1], w[2], w[3]);
        *(reinterpret_cast<uint4 *>(p.residual_out) + vec_l) = out;
        cache[(size_t)rl * row_vecs + cache_slot(i >> 2, i & 3)] = out;
      }
    }
    __syncthreads();
    // 1b: sum of squares of every 32-element group in the reference's order
    for (int t = threadIdx.x; t < c_rows * groups32; t += kThreads) {
      const int rl = t / groups32, g = t - rl * groups32;
      const uint4 *row_cache = cache + (size_t)rl * row_vecs;
      float sq = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 xv = row_cache[cache_slot(g, j)];
        const uint32_t w[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float a = lo_f(w[q]), b2 = hi_f(w[q]);
          sq = __fmaf_rn(a, a, sq);
          sq = __fmaf_rn(b2, b2, sq);
        }
      }
      partial[rl * partial_stride + g] = sq;
    }
    __syncthreads();
    if (threadIdx.x < c_rows) {
      const float4 *pr = reinterpret_cast<const float4 *>(partial + threadIdx.x * partial_stride);
      float total = 0.0f;
      for (int i = 0; i < groups32 / 4; ++i) {
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
    for (int t = threadIdx.x; t < c_rows * groups32; t += kThreads) {
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

  // ---- this GPU's absmax (grid barrier 1), then B: the tensor absmax over all GPUs
  {
    float mx = fmaxf(__bfloat162float(m2.x), __bfloat162float(m2.y));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) warp_red[warp] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
      for (int w = 1; w < kWarps; ++w) mx = fmaxf(mx, warp_red[w]);
      if (mx > 0.0f) atomicMax(my_state + kAmaxLocal + (epoch & 1u), __float_as_uint(mx));
    }
  }
  grid_barrier(p, epoch, 1, true, 0x302);
  if (blockIdx.x == 0 && (int)threadIdx.x < p.world) {
    const uint32_t mine = ld_acquire_gpu(my_state + kAmaxLocal + (epoch & 1u));
    st_release_sys64(p.state[threadIdx.x] + kAmax + 2 * p.rank, ((unsigned long long)tag << 32) | mine);
    if (threadIdx.x == 0) my_state[kAmaxLocal + ((epoch + 1u) & 1u)] = 0u;  // the next launch's accumulator
  }
  if ((int)threadIdx.x < p.world) {
    const long long t0 = clock64();
    unsigned long long v;
    for (;;) {
      v = ld_acquire_sys64(my_state + kAmax + 2 * threadIdx.x);
      if ((uint32_t)(v >> 32) == tag) break;
      if (clock64() - t0 > p.wait_limit) {
        atomicExch(p.error_flag, 0x303);
        break;
      }
    }
    rank_amax[threadIdx.x] = (uint32_t)v;
  }
  __syncthreads();
  uint32_t amax_bits = 0u;
  for (int r = 0; r < p.world; ++r) amax_bits = max(amax_bits, rank_amax[r]);  // non-negative floats order like integers
  const float scale = fmaxf(__fmul_rn(__uint_as_float(amax_bits), 1.0f / 2688.0f), 1.0e-9f);
  const float recip = __frcp_rn(scale);
  if (blockIdx.x == 0 && threadIdx.x == 0) *p.scale_out = scale;

  // ------------------------------------------------------------------ phase 2: quantise into this GPU's copy
  const int tasks_per_row = (groups_padded + 31) >> 5;
  for (int c = chunks - 1; c >= 0; --c) {
    const bool cached = c == chunks - 1;
    const int c_rows = chunk_size(c), c_row0 = row_begin + chunk_first_row(c);
    for (int wt = warp; wt < c_rows * tasks_per_row; wt += kWarps) {
      const int rl = wt / tasks_per_row;
      const int group = (wt - rl * tasks_per_row) * 32 + lane;
      const int row_l = c_row0 + rl;
      const int row = p.row0 + row_l;  // row of the whole activation
      const bool live = group < groups32;
      uint32_t xw[16];
      GroupOut o;
      o.a_comp[0] = o.a_comp[1] = 0;
      o.meta = 0;
      o.sf_sparse = 0;
      o.sf_res = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) o.q_res[i] = o.q_sparse[i] = 0;
      if (live) {
        if (cached) {
          const uint4 *row_cache = cache + (size_t)rl * row_vecs;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v = row_cache[cache_slot(group, j)];
            xw[4 * j + 0] = v.x;
            xw[4 * j + 1] = v.y;
            xw[4 * j + 2] = v.z;
            xw[4 * j + 3] = v.w;
          }
        } else {
          // plain loads: these bytes were written by this CTA in phase 1
          const uint4 *xs = reinterpret_cast<const uint4 *>(p.residual_out + (size_t)row_l * k + (size_t)group * 32);
          const float inv = inv_s[chunk_first_row(c) + rl];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v = xs[j];
            const uint4 gv = gamma_s[cache_slot(group, j)];
            const uint32_t vw[4] = {v.x, v.y, v.z, v.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q)
              xw[4 * j + q] = pack_bf16x2(__fmul_rn(__fmul_rn(lo_f(vw[q]), inv), lo_f(gw[q])),
                                          __fmul_rn(__fmul_rn(hi_f(vw[q]), inv), hi_f(gw[q])));
          }
        }
        scale_quantize_group<1, false>(xw, scale, recip, tbl, o, [](uint32_t (&)[16]) {});  // mode 1 never reloads
        *reinterpret_cast<uint4 *>(p.q_res + (size_t)row * (k / 2) + (size_t)group * 16) =
            make_uint4(o.q_res[0], o.q_res[1], o.q_res[2], o.q_res[3]);
        *reinterpret_cast<uint2 *>(p.a_comp + (size_t)row * (k / 4) + (size_t)group * 8) = make_uint2(o.a_comp[0], o.a_comp[1]);
      }
      const uint32_t mine = o.meta & 0xFFFFu;
      const uint32_t other = __shfl_down_sync(0xffffffffu, mine, 1);
      if ((lane & 1) == 0 && group < groups_padded)
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
  }

  // ------------------------------------------------------------------ phase 3: push this GPU's rows to every GPU.
  // By default with plain peer stores to the other GPUs: a multicast store also comes back to its
  // sender, so every GPU's port receives the whole packed activation, N / (N - 1) times the bytes
  // that it needs (twice at two GPUs); SHARQ_TP_ALLGATHER=multicast selects multimem.st.
  // A separate pass of contiguous 16-byte stores: storing the packed words straight from the
  // quantise phase (16 / 8 / 4-byte multimem.st as they are produced) was measured slower (82 against
  // 63 us per call at two GPUs): the switch wants a warp's multicast stores contiguous.
  grid_barrier(p, epoch, 2, true, 0x304);  // the packed rows are complete in this GPU's copy
  {
    // byte ranges of rows [row0, row0 + rows) in units of 16 bytes; rows is a multiple of 128
    const size_t n_q = (size_t)p.rows * (k / 2) / 16;
    const size_t n_a = (size_t)p.rows * (k / 4) / 16;
    const size_t k_tiles = (size_t)(groups_padded >> 3);
    const size_t n_e = k_tiles * (size_t)p.rows;
    const size_t n_sfa = (size_t)(p.rows / 128) * (size_t)(groups32 / 4) * 32;
    const size_t n_sfr = (size_t)(p.rows / 128) * (size_t)(k / 64) * 32;
    const size_t total = n_q + n_a + n_e + n_sfa + n_sfr;
    const size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
      uint8_t *src;
      size_t j = i;
      if (j < n_q) {
        src = p.q_res + (size_t)p.row0 * (k / 2) + j * 16;
      } else if ((j -= n_q) < n_a) {
        src = p.a_comp + (size_t)p.row0 * (k / 4) + j * 16;
      } else if ((j -= n_a) < n_e) {
        const size_t kt = j / p.rows, r = j - kt * p.rows;
        src = p.e + (kt * aligned_m + p.row0 + r) * 16;
      } else if ((j -= n_e) < n_sfa) {
        src = p.sfa_sparse + (size_t)(p.row0 / 128) * (size_t)(groups32 / 4) * 512 + j * 16;
      } else {
        j -= n_sfa;
        src = p.sf_res + (size_t)(p.row0 / 128) * (size_t)(k / 64) * 512 + j * 16;
      }
      const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(src));
      if (p.unicast) {
        // one plain 16-byte store per peer, destinations staggered over the GPUs; a warp writes 512 contiguous bytes
        for (int t = 1; t < p.world; ++t) {
          int r = p.rank + t;
          if (r >= p.world) r -= p.world;
          *reinterpret_cast<uint4 *>(src + p.peer_delta[r]) = v;
        }
      } else {
        st_multicast_16(src + p.mc_delta, v);
      }
    }
  }
  // ---- C: this GPU's stores are out (grid barrier 3, CTA 0 alone waits), tell everyone, wait for everyone
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    atomicAdd(my_state + kGridArrive, 1u);
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0 && !wait_counter(my_state + kGridArrive, (epoch * 3u + 3u) * gridDim.x, true, p.wait_limit))
      atomicExch(p.error_flag, 0x305);
    __syncthreads();
    if ((int)threadIdx.x < p.world) {
      __threadfence_system();
      signal_add_release(p.state[threadIdx.x] + kDone + p.rank);
      if (!wait_counter(my_state + kDone + threadIdx.x, tag, false, p.wait_limit)) atomicExch(p.error_flag, 0x306);
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t *>(my_state + kEpoch) = tag;
  }
}

}  // namespace

void set_sp_transition_wait_limit(long long cycles) { g_wait_limit_cycles = cycles > 0 ? cycles : kWaitLimitCycles; }

size_t sp_transition_state_bytes() { return (size_t)kStateWords * sizeof(uint32_t); }

size_t sp_transition_workspace_bytes(int rows) { return (size_t)rows * sizeof(float); }

cudaError_t run_sp_transition(const SpTransitionArgs &a, cudaStream_t stream) {
  static bool attr_set[64] = {};
  static int sms_of[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (sms_of[dev] == 0) {
    int coop = 0;
    if ((err = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev)) != cudaSuccess) return err;
    if (!coop) return cudaErrorNotSupported;
    if ((err = cudaDeviceGetAttribute(&sms_of[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return err;
  }
  const int sms = sms_of[dev];
  SpParams p{};
  p.partial = static_cast<const uint8_t *>(a.partial_blocks);
  p.residual_in = static_cast<const __nv_bfloat16 *>(a.residual_in);
  p.residual_out = static_cast<__nv_bfloat16 *>(a.residual_out);
  p.gamma = static_cast<const __nv_bfloat16 *>(a.gamma);
  p.eps = a.eps;
  p.inv_rms = static_cast<float *>(a.workspace);
  p.scale_out = a.scale_out;
  p.a_comp = static_cast<uint8_t *>(a.a_comp);
  p.e = static_cast<uint8_t *>(a.e);
  p.sfa_sparse = static_cast<uint8_t *>(a.sfa_sparse);
  p.q_res = static_cast<uint8_t *>(a.q_res);
  p.sf_res = static_cast<uint8_t *>(a.sf_res);
  p.mc_delta = a.multicast_delta;
  {
    static const bool multicast = [] {
      const char *v = getenv("SHARQ_TP_ALLGATHER");  // tuning hook
      return v != nullptr && v[0] == 'm';
    }();
    p.unicast = multicast ? 0 : 1;
    // the state block lies in the same symmetric allocation as the output buffers, so the distance between
    // two GPUs' mappings of it is the distance between their mappings of every byte of the allocation
    for (int r = 0; r < a.world; ++r)
      p.peer_delta[r] = (long long)(reinterpret_cast<intptr_t>(a.rank_state_ptrs[r]) -
                                    reinterpret_cast<intptr_t>(a.rank_state_ptrs[a.rank]));
  }
  for (int r = 0; r < a.world; ++r) p.state[r] = static_cast<uint32_t *>(a.rank_state_ptrs[r]);
  p.rank = a.rank;
  p.world = a.world;
  p.m = a.m;
  p.k = a.k;
  p.rows = a.m / a.world;
  p.row0 = a.rank * p.rows;
  p.error_flag = a.error_flag;
  p.wait_limit = g_wait_limit_cycles;
  const int groups32 = a.k / 32;
  p.rows_per_cta = (p.rows + sms - 1) / sms;
  const size_t row_bytes = (size_t)a.k * 2 + (size_t)(groups32 + 4) * 4;
  const size_t fixed = (size_t)a.k * 2 + (size_t)p.rows_per_cta * 4;
  if (fixed + row_bytes > (size_t)kSmemBudget) return cudaErrorInvalidValue;
  const size_t capacity = ((size_t)kSmemBudget - fixed) / row_bytes;
  p.chunk_rows = (int)(capacity < (size_t)p.rows_per_cta ? capacity : (size_t)p.rows_per_cta);
  const size_t smem = fixed + (size_t)p.chunk_rows * row_bytes + 16;
  if (!attr_set[dev]) {
    err = cudaFuncSetAttribute(sp_transition_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 16);
    if (err != cudaSuccess) return err;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  // the grid is the same for every launch on a device: the local barrier counters are monotonic
  cfg.gridDim = dim3(sms);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, sp_transition_kernel, p);
}

}  // namespace sharq
