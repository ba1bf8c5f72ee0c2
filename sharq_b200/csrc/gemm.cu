// Block-scaled FP4 GEMMs for sm_100a, hand-written on tcgen05 / TMEM / TMA:
//   dense NVFP4      D = bf16(alpha * (A . B^T) + beta * C)         (one UE4M3 scale per 16 along K)
//   sparse NVFP4     the same with a pair-wise 4:8 compressed A     (one scale per 32 logical K)
//   fused SharQ      sparse main + dense residual against the SAME weight tile, both
//                    accumulated into one TMEM tile, one epilogue (+ optional bias).
// They replace the reference's CUTLASS-generated kernels behind the same buffers:
//   kernels/src/nvfp4.cu:432-455, kernels/src/sparse_nvfp4.cu:436-460 and the two-launch
//   composition at model/qLinearLayer.py:130-154.
//
// One persistent kernel, one CTA per SM (or one CTA pair per SM pair), looping over output
// tiles with the M index fastest so that CTAs working at the same time share weight tiles
// in L2.  K is consumed in stages of 256.  Warp roles:
//   warp 0     TMA producer: per stage three tensor-map loads (weight tile, dense A tile,
//              compressed A tile; 128-byte / 64-byte swizzle) and plain bulk copies of the
//              metadata tile and the scale-factor tiles, all landing on one mbarrier.  It runs
//              ahead across tile boundaries, so the pipeline never drains between tiles.
//   warp 1     MMA issuer: copies metadata and scale factors shared -> tensor memory
//              (tcgen05.cp), then issues 2 sparse (K=128) and 4 dense (K=64) MMAs per stage
//              into the same accumulator; tcgen05.commit releases the stage.
//   warps 2-9  epilogue: pull the whole accumulator into registers with tcgen05.ld, hand the
//              tensor memory back to the MMA warp at once, then alpha/beta/bias, bf16 (packed
//              conversions), a transpose through a small shared-memory tile and coalesced
//              global stores overlap the next tile's MMAs.
// Small M with caller scratch: K is split over the SMs, units add fp32 partial sums into the
// scratch and splitk_finalize_kernel applies the epilogue.
// CTA-pair mode (cta_group::2, cluster of 2): the pair computes a 256 x 256 tile; CTA r owns
// rows [128r,128r+128) (its A operands, scales, metadata, accumulator) and loads weight rows
// [128r,128r+128) of the tile; the tensor cores of both SMs read both halves.  Every CTA
// loads with its own plain TMA copies - there is no multicast load anywhere.  Hand-shake:
// the peer CTA reports each loaded stage on the leader's peer barrier, the leader issues
// the pair's MMAs and commits to the barriers of both CTAs.
// All mbarrier waits are bounded; a timed-out wait sets *error_flag and every role drains
// to the common exit, where tensor memory is released.
#include "common.cuh"
#include "gemm.cuh"
#include "sm100_ptx.cuh"

#include <cstring>
#include <mutex>

namespace sharq {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 256;  // logical K per stage
constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;

// Shared-memory stage and tensor-memory column layout.  In pair mode BN is the pair's tile
// width (256) and each CTA stores half of the weight tile.
template <int BN, bool SPARSE, bool DENSE, bool PAIR>
struct StageLayout {
  static constexpr int kBands = BN / 128;  // 128-row scale-factor bands of the weight tile
  static constexpr int kWRows = PAIR ? BN / 2 : BN;
  static constexpr int kWBytes = kWRows * 128;
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
  static constexpr int kOutStageBytes = kEpiWarps * 32 * 64;  // per epilogue warp 32 rows x 32 bf16 for the tile store
  static constexpr int kMaxSmem = 227 * 1024 - 2048 - kOutStageBytes;
  static constexpr int kStagesFit = kMaxSmem / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  // tensor memory columns
  static constexpr int kColAcc = 0;
  static constexpr int kColE = BN;
  static constexpr int kColSfaSp = kColE + 4;
  static constexpr int kColSfbSp = kColSfaSp + 8;
  static constexpr int kColSfaD = kColSfbSp + 2 * (BN / 32);
  static constexpr int kColSfbD = kColSfaD + 16;
  static constexpr int kColEnd = kColSfbD + 4 * (BN / 32);
  static constexpr int kTmemCols = kColEnd <= 256 ? 256 : 512;
  static constexpr int kSmemBytes =
      kStages * kStageBytes + kOutStageBytes + 1024 /*alignment slack*/ + 512 /*barriers*/;
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
  // Split K (small M): every output tile is computed by k_splits units, each over its share of
  // the K stages; their fp32 partial sums are added into splitk_acc [m, n] (zero-filled by the
  // launcher) with vector reductions and a second kernel applies the epilogue.
  int k_splits;
  float *splitk_acc;
  int staged_store;  // output tiles are transposed through shared memory for coalesced stores (N % 8 == 0)
  // Scatter mode (row-parallel linear under tensor parallelism): the output rows are dealt to their owner GPUs.
  // Row r belongs to GPU o = r / scatter_rows and is stored, through the peer mapping, into d_peer[o] at row
  // scatter_rank * scatter_rows + (r - o * scatter_rows): every GPU collects one [scatter_rows, n] block per
  // source GPU.  scatter_rows is a multiple of 128, so a tile has one owner.  scatter_rows == 0: plain output.
  __nv_bfloat16 *d_peer[kGemmMaxPeers];
  int scatter_rows, scatter_rank;
};

// Grouped launch (mixture-of-experts layers): the rows of the activation are sorted by group
// (expert) in segments padded to whole 256-row units; every unit multiplies with the weight of
// its own group.  unit_group[u] < 0 marks a unit without rows (skipped).
constexpr int kMaxGroups = 16;
struct GroupTable {
  CUtensorMap tm_w[kMaxGroups];
  const uint8_t *sfb_sparse[kMaxGroups];
  const uint8_t *sfb_dense[kMaxGroups];
  const int *unit_group;  // [units along M] on the device
  const float *alpha;     // [groups] on the device: per-group factor (activation scale x weight scale)
};

// Epilogue of 32 accumulator columns held in registers: d = bf16(alpha * acc + beta * c_in),
// then (+ bias) in bf16; rows >= M and columns >= N are masked.  A thread owns one row and
// stores 64 contiguous bytes.
// With `stage` non-null the 64 bytes go to row `stage_row` of a 32-row x 64-byte shared-memory
// tile instead, 16-byte chunk v at position v ^ ((row >> 1) & 3) (no bank conflicts on the way in
// or out); the caller stores the tile and masks rows >= M and columns >= N; requires N % 8 == 0.
// kWide: the tile is 16 rows x 128 bytes (two calls fill a row: chunk_base 0 and 4), chunk c of a
// row at position c ^ (row & 7).
template <bool kWide = false>
__device__ __forceinline__ void epilogue_chunk(const GemmParams &p, const uint32_t *acc, int row, int col0, float alpha,
                                               float beta, bool has_c, uint8_t *stage = nullptr, int stage_row = 0,
                                               int chunk_base = 0) {
  if (stage == nullptr && (row >= p.m || col0 >= p.n)) return;
  if (stage != nullptr && (row >= p.m || col0 >= p.n)) {
    has_c = false;  // masked by the caller's store; C_in must not be read out of range
  }
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
    // two values per conversion instruction (the scalar conversion unit is the slow pipe here)
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 pair = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      o[i] = *reinterpret_cast<uint32_t *>(&pair);
    }
    if (p.bias != nullptr) {
      // bias is added to the bf16 result, as a separate bf16 add would (a bf16 add rounds the
      // exact sum once, which is what the fp32 add + rounding of two bf16 values gives)
      if (full && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
        const uint4 bv = __ldg(reinterpret_cast<const uint4 *>(p.bias + col0 + 8 * v));
        const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 sum = __hadd2(*reinterpret_cast<__nv_bfloat162 *>(&o[i]),
                                       *reinterpret_cast<const __nv_bfloat162 *>(&bw[i]));
          o[i] = *reinterpret_cast<uint32_t *>(&sum);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int cc = col0 + 8 * v + 2 * i;
          const float b0 = cc < p.n ? __bfloat162float(p.bias[cc]) : 0.0f;
          const float b1 = cc + 1 < p.n ? __bfloat162float(p.bias[cc + 1]) : 0.0f;
          const uint32_t lo = float_to_bf16_bits(bf16_bits_to_float(o[i] & 0xFFFFu) + b0);
          const uint32_t hi = float_to_bf16_bits(bf16_bits_to_float(o[i] >> 16) + b1);
          o[i] = lo | (hi << 16);
        }
      }
    }
    if (stage != nullptr) {
      uint8_t *slot = kWide ? stage + stage_row * 128 + (((chunk_base + v) ^ (stage_row & 7)) << 4)
                            : stage + stage_row * 64 + ((v ^ ((stage_row >> 1) & 3)) << 4);
      *reinterpret_cast<uint4 *>(slot) = make_uint4(o[0], o[1], o[2], o[3]);
    } else if (full) {
      *reinterpret_cast<uint4 *>(p.d + off + 8 * v) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (col0 + 8 * v + i < p.n)
          p.d[off + 8 * v + i] = __ushort_as_bfloat16((unsigned short)((o[i >> 1] >> (16 * (i & 1))) & 0xFFFFu));
    }
  }
}

template <int BN, bool SPARSE, bool DENSE, bool PAIR, bool GROUPED, bool WIDE = false>
__device__ __forceinline__ void gemm_body(const CUtensorMap &tm_w, const CUtensorMap &tm_a_dense, const CUtensorMap &tm_a_comp,
                                          const GemmParams &p, const GroupTable *gt) {
  using L = StageLayout<BN, SPARSE, DENSE, PAIR>;
  constexpr int S = L::kStages;
  constexpr int CG = PAIR ? 2 : 1;
  constexpr int kColsPerEpiWarp = BN / 2;  // two warps share each tensor-memory lane quadrant

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + S * L::kStageBytes);
  uint64_t *empty_bar = full_bar + S;
  uint64_t *peer_bar = empty_bar + S;  // pair mode, leader CTA: "the peer has loaded stage s"
  uint64_t *acc_full_bar = peer_bar + S;
  uint64_t *acc_empty_bar = acc_full_bar + 1;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty_bar + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int k_stages = (p.k + kBK - 1) / kBK;
  const int aligned_m = (p.m + 127) / 128 * 128;
  const int a_bands = aligned_m / 128;     // 128-row bands of the activation operands
  const int b_bands = (p.n + 127) / 128;   // 128-row bands of the weight scale factors
  const int tiles_sp = p.k / 128;  // 512-byte scale tiles per 128-row band, 32-group layout
  const int tiles_d = p.k / 64;    // same, 16-group layout
  // work units: a unit is one output tile of a CTA (128 x BN) or of a pair (256 x BN)
  const int m_units = PAIR ? (p.m + 255) / 256 : (p.m + kBM - 1) / kBM;
  const int n_tiles = (p.n + BN - 1) / BN;
  const int k_splits = p.k_splits;
  const int num_units = m_units * n_tiles * k_splits;
  // unit -> (K share, tile); tiles M-fastest
  auto k_begin = [&](int u) { return (int)((long long)k_stages * (u % k_splits) / k_splits); };
  auto k_end = [&](int u) { return (int)((long long)k_stages * (u % k_splits + 1) / k_splits); };
  const int unit0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int unit_stride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 32) {
    // fetch the tensor maps while the barriers and tensor memory are being set up
    if (!GROUPED) ptx::tma_prefetch_desc(&tm_w);
    if (DENSE) ptx::tma_prefetch_desc(&tm_a_dense);
    if (SPARSE) ptx::tma_prefetch_desc(&tm_a_comp);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
      ptx::mbar_init(peer_bar + s, 1);
    }
    ptx::mbar_init(acc_full_bar, 1);
    ptx::mbar_init(acc_empty_bar, PAIR ? 2 * kEpiWarps : kEpiWarps);
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc<CG>(tmem_slot, L::kTmemCols);
    ptx::tmem_relinquish<CG>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (PAIR) ptx::cluster_sync();  // both CTAs' barriers exist before any remote arrive
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t g = 0;  // stages issued so far, across tiles
      bool ok = true;
      for (int u = unit0; u < num_units && ok; u += unit_stride) {
        const int tile = u / k_splits;
        const int grp = GROUPED ? gt->unit_group[tile % m_units] : 0;
        if (GROUPED && grp < 0) continue;
        const CUtensorMap *tw = GROUPED ? &gt->tm_w[grp] : &tm_w;
        const uint8_t *sfb_dense = GROUPED ? gt->sfb_dense[grp] : p.sfb_dense;
        const uint8_t *sfb_sparse = GROUPED ? gt->sfb_sparse[grp] : p.sfb_sparse;
        const int m_tile = PAIR ? 2 * (tile % m_units) + (int)cta_rank : (tile % m_units);
        const int n_tile = tile / m_units;
        const int w_row = n_tile * BN + (PAIR ? (int)cta_rank * (BN / 2) : 0);
        // The metadata and scale-factor copies are plain bulk copies without bounds checks.  A
        // tile may hang over the last 128-row band (the second CTA of a pair when ceil(M/128) is
        // odd, the second weight band of a 256-wide tile when ceil(N/128) is odd): such a band
        // is loaded from the last band that exists.  Its rows / columns are masked on output.
        const int a_band = min(m_tile, a_bands - 1);
        int b_band[L::kBands];
#pragma unroll
        for (int b = 0; b < L::kBands; ++b) b_band[b] = min(n_tile * L::kBands + b, b_bands - 1);
        for (int it = k_begin(u), it_end = k_end(u); it < it_end; ++it, ++g) {
          const int s = (int)(g % S);
          const uint32_t ph = (g / S) & 1u;
          if (!ptx::mbar_wait(empty_bar + s, ph ^ 1u, abort_flag)) {
            *abort_flag = 1;
            atomicExch(p.error_flag, 1);
            ok = false;
            break;
          }
          uint8_t *st = smem + s * L::kStageBytes;
          const int n_sp = SPARSE ? min(2, tiles_sp - 2 * it) : 0;
          const int n_d = DENSE ? min(4, tiles_d - 4 * it) : 0;
          uint32_t tx = L::kWBytes + L::kADenseBytes + L::kACompBytes + L::kEBytes;
          tx += (uint32_t)(n_sp * 512 * (1 + L::kBands) + n_d * 512 * (1 + L::kBands));
          ptx::mbar_arrive_expect_tx(full_bar + s, tx);
          ptx::tma_load_2d(st + L::kOffW, tw, it * 128, w_row, full_bar + s);
          if (DENSE) {
            ptx::tma_load_2d(st + L::kOffADense, &tm_a_dense, it * 128, m_tile * kBM, full_bar + s);
            ptx::bulk_load_1d(st + L::kOffSfaD, p.sfa_dense + ((size_t)a_band * tiles_d + 4 * (size_t)it) * 512,
                              (uint32_t)n_d * 512, full_bar + s);
#pragma unroll
            for (int b = 0; b < L::kBands; ++b)
              ptx::bulk_load_1d(st + L::kOffSfbD + b * 2048,
                                sfb_dense + ((size_t)b_band[b] * tiles_d + 4 * (size_t)it) * 512,
                                (uint32_t)n_d * 512, full_bar + s);
          }
          if (SPARSE) {
            ptx::tma_load_2d(st + L::kOffAComp, &tm_a_comp, it * 64, m_tile * kBM, full_bar + s);
            ptx::bulk_load_1d(st + L::kOffE, p.e + ((size_t)it * aligned_m + (size_t)a_band * 128) * 16, 2048,
                              full_bar + s);
            ptx::bulk_load_1d(st + L::kOffSfaSp, p.sfa_sparse + ((size_t)a_band * tiles_sp + 2 * (size_t)it) * 512,
                              (uint32_t)n_sp * 512, full_bar + s);
#pragma unroll
            for (int b = 0; b < L::kBands; ++b)
              ptx::bulk_load_1d(st + L::kOffSfbSp + b * 1024,
                                sfb_sparse + ((size_t)b_band[b] * tiles_sp + 2 * (size_t)it) * 512,
                                (uint32_t)n_sp * 512, full_bar + s);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      if (PAIR && !leader) {
        // ---------------------------------------------------------- peer CTA: report loaded stages
        uint32_t g = 0;
        bool ok = true;
        for (int u = unit0; u < num_units && ok; u += unit_stride) {
          if (GROUPED && gt->unit_group[(u / k_splits) % m_units] < 0) continue;
          for (int it = k_begin(u), it_end = k_end(u); it < it_end; ++it, ++g) {
            const int s = (int)(g % S);
            if (!ptx::mbar_wait(full_bar + s, (g / S) & 1u, abort_flag)) {
              *abort_flag = 1;
              atomicExch(p.error_flag, 4);
              ok = false;
              break;
            }
            ptx::mbar_arrive_cluster(peer_bar + s, 0);
          }
        }
      } else {
        // ---------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc_d = ptx::make_idesc_nvf4(PAIR ? 256 : kBM, BN, false);
        constexpr uint32_t idesc_s = ptx::make_idesc_nvf4(PAIR ? 256 : kBM, BN, true);
        uint32_t g = 0;
        uint32_t tile_iter = 0;
        bool ok = true;
        for (int u = unit0; u < num_units && ok; u += unit_stride) {
          if (GROUPED && gt->unit_group[(u / k_splits) % m_units] < 0) continue;
          // the epilogue warps must have pulled the previous tile out of tensor memory
          const bool drained = PAIR ? ptx::mbar_wait_cluster(acc_empty_bar, (tile_iter & 1u) ^ 1u, abort_flag)
                                    : ptx::mbar_wait(acc_empty_bar, (tile_iter & 1u) ^ 1u, abort_flag);
          if (!drained) {
            *abort_flag = 1;
            atomicExch(p.error_flag, 5);
            break;
          }
          ptx::tc_fence_after();
          uint32_t accumulate = 0;
          for (int it = k_begin(u), it_end = k_end(u); it < it_end; ++it, ++g) {
            const int s = (int)(g % S);
            const uint32_t ph = (g / S) & 1u;
            bool got = ptx::mbar_wait(full_bar + s, ph, abort_flag);
            if (PAIR && got) got = ptx::mbar_wait_cluster(peer_bar + s, ph, abort_flag);
            if (!got) {
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
              ptx::tmem_cp_128x128b<CG>(tmem_base + L::kColE, ptx::make_smem_desc(st + L::kOffE, 128, 0, 0));
#pragma unroll
              for (int t = 0; t < 2; ++t) {
                if (t < n_sp) {
                  ptx::tmem_cp_32x128b_warpx4<CG>(tmem_base + L::kColSfaSp + 4 * t,
                                                  ptx::make_smem_desc(st + L::kOffSfaSp + t * 512, 128, 0, 0));
#pragma unroll
                  for (int b = 0; b < L::kBands; ++b)
                    ptx::tmem_cp_32x128b_warpx4<CG>(
                        tmem_base + L::kColSfbSp + t * (BN / 32) + 4 * b,
                        ptx::make_smem_desc(st + L::kOffSfbSp + b * 1024 + t * 512, 128, 0, 0));
                }
              }
            }
            if (DENSE) {
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                if (t < n_d) {
                  ptx::tmem_cp_32x128b_warpx4<CG>(tmem_base + L::kColSfaD + 4 * t,
                                                  ptx::make_smem_desc(st + L::kOffSfaD + t * 512, 128, 0, 0));
#pragma unroll
                  for (int b = 0; b < L::kBands; ++b)
                    ptx::tmem_cp_32x128b_warpx4<CG>(
                        tmem_base + L::kColSfbD + t * (BN / 32) + 4 * b,
                        ptx::make_smem_desc(st + L::kOffSfbD + b * 2048 + t * 512, 128, 0, 0));
                }
              }
            }
            if (SPARSE) {
              // compressed A: 64-byte swizzled rows, 32 bytes (128 logical K) per MMA;
              // weight: 128-byte swizzled rows, 64 bytes (128 K) per MMA.
#pragma unroll
              for (int t = 0; t < 2; ++t) {
                if (t < n_sp) {
                  uint64_t da = ptx::make_smem_desc(st + L::kOffAComp + t * 32, 512, 16, 4);
                  uint64_t db = ptx::make_smem_desc(st + L::kOffW + t * 64, 1024, 16, 2);
                  ptx::mma_nvf4_sparse<CG>(tmem_base + L::kColAcc, da, db, idesc_s, tmem_base + L::kColSfaSp + 4 * t,
                                           tmem_base + L::kColSfbSp + t * (BN / 32), tmem_base + L::kColE + 2 * t,
                                           accumulate);
                  accumulate = 1;
                }
              }
            }
            if (DENSE) {
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                if (t < n_d) {
                  uint64_t da = ptx::make_smem_desc(st + L::kOffADense + t * 32, 1024, 16, 2);
                  uint64_t db = ptx::make_smem_desc(st + L::kOffW + t * 32, 1024, 16, 2);
                  ptx::mma_nvf4_dense<CG>(tmem_base + L::kColAcc, da, db, idesc_d, tmem_base + L::kColSfaD + 4 * t,
                                          tmem_base + L::kColSfbD + t * (BN / 32), accumulate);
                  accumulate = 1;
                }
              }
            }
            if (PAIR)
              ptx::tc_commit_multicast2(empty_bar + s, 3);
            else
              ptx::tc_commit<1>(empty_bar + s);
          }
          if (ok) {
            if (PAIR)
              ptx::tc_commit_multicast2(acc_full_bar, 3);
            else
              ptx::tc_commit<1>(acc_full_bar);
          }
          ++tile_iter;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int ew = warp - 2;
    const int quad = warp & 3;  // tensor-memory lane quadrant this warp may read
    const int half = ew >> 2;   // which half of the tile's columns
    const float alpha0 = p.alpha_ptr ? p.alpha * (*p.alpha_ptr) : p.alpha;
    const float beta = p.beta;
    const bool has_c = (p.c_in != nullptr) && (beta != 0.0f);
    // Output path: a lane holds one row of the accumulator, so a direct store instruction would
    // touch 32 different rows with 16 bytes each (32 memory lines per instruction).  Every
    // epilogue warp owns a 32-row x 64-byte shared-memory tile instead: 32 columns at a time are
    // converted into it (swizzled, conflict-free), read back with four lanes per row, and
    // stored as 8 rows x 64 contiguous bytes per instruction.
    uint8_t *stage = p.staged_store ? smem + S * L::kStageBytes + 512 + ew * 2048 : nullptr;
    uint32_t tile_iter = 0;
    for (int u = unit0; u < num_units; u += unit_stride) {
      const int tile = u / k_splits;
      const int grp = GROUPED ? gt->unit_group[tile % m_units] : 0;
      if (GROUPED && grp < 0) continue;
      const float alpha = GROUPED ? alpha0 * gt->alpha[grp] : alpha0;
      const int m_tile = PAIR ? 2 * (tile % m_units) + (int)cta_rank : (tile % m_units);
      const int n_tile = tile / m_units;
      bool ok = ptx::mbar_wait(acc_full_bar, tile_iter & 1u, abort_flag);
      ++tile_iter;
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error_flag, 3);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      uint32_t acc[kColsPerEpiWarp];
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(L::kColAcc + half * kColsPerEpiWarp);
#pragma unroll
      for (int c = 0; c < kColsPerEpiWarp / 32; ++c)
        ptx::tmem_ld_32x32b_x32(taddr + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&acc[32 * c]));
      ptx::tmem_ld_wait();
      // the accumulator is in registers: give tensor memory back before the slow part
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && !leader)
          ptx::mbar_arrive_cluster(acc_empty_bar, 0);
        else
          ptx::mbar_arrive(acc_empty_bar);
      }
      const int row = m_tile * kBM + quad * 32 + lane;
      const int col_base = n_tile * BN + half * kColsPerEpiWarp;
      if (k_splits > 1) {
        // partial sums of this K share: fp32 vector reductions into the accumulation buffer
        if (row < p.m) {
          float *dst = p.splitk_acc + (size_t)row * p.n + col_base;
          const bool vec = (p.n & 3) == 0;
#pragma unroll
          for (int i = 0; i < kColsPerEpiWarp; i += 4) {
            if (vec && col_base + i + 4 <= p.n) {
              ptx::red_add_v4_f32(dst + i, __uint_as_float(acc[i]), __uint_as_float(acc[i + 1]),
                                  __uint_as_float(acc[i + 2]), __uint_as_float(acc[i + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (col_base + i + j < p.n) atomicAdd(dst + i + j, __uint_as_float(acc[i + j]));
            }
          }
        }
        continue;
      }
      if (stage != nullptr) {
        const int row0 = m_tile * kBM + quad * 32;
        __nv_bfloat16 *d_base = p.d;
        if (p.scatter_rows > 0) {
          const int owner = (m_tile * kBM) / p.scatter_rows;
          d_base = p.d_peer[owner] + ((long long)p.scatter_rank - owner) * p.scatter_rows * (long long)p.n;
        }
        if (WIDE) {
          // Scatter mode (rows that go to another GPU): a peer store moves 18 % more bytes per second in 128-byte
          // row pieces than in 64-byte ones (measured 605 against 511 GB/s), so the tile is staged
          // 64 columns at a time in two halves of 16 rows (the lanes of the other half wait) and
          // stored as 4 rows x 128 contiguous bytes per instruction.
#pragma unroll
          for (int c = 0; c < kColsPerEpiWarp / 64; ++c) {
            const int col0 = col_base + 64 * c;
            const int gcol = col0 + (lane & 7) * 8;
#pragma unroll 1
            for (int hrow = 0; hrow < 2; ++hrow) {
              if ((lane >> 4) == hrow) {
                epilogue_chunk<true>(p, &acc[64 * c], row, col0, alpha, beta, false, stage, lane & 15, 0);
                epilogue_chunk<true>(p, &acc[64 * c + 32], row, col0 + 32, alpha, beta, false, stage, lane & 15, 4);
              }
              __syncwarp();
#pragma unroll
              for (int it = 0; it < 4; ++it) {
                const int r = it * 4 + (lane >> 3);
                const uint4 v = *reinterpret_cast<const uint4 *>(stage + r * 128 + (((lane & 7) ^ (r & 7)) << 4));
                const int grow = row0 + 16 * hrow + r;
                if (grow < p.m && gcol < p.n) *reinterpret_cast<uint4 *>(d_base + (size_t)grow * p.n + gcol) = v;
              }
              __syncwarp();
            }
          }
          continue;
        }
#pragma unroll
        for (int c = 0; c < kColsPerEpiWarp / 32; ++c) {
          const int col0 = col_base + 32 * c;
          epilogue_chunk(p, &acc[32 * c], row, col0, alpha, beta, has_c, stage, lane);
          __syncwarp();
          const int gcol = col0 + (lane & 3) * 8;
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int r = it * 8 + (lane >> 2);
            const uint4 v = *reinterpret_cast<const uint4 *>(stage + r * 64 + (((lane & 3) ^ ((r >> 1) & 3)) << 4));
            if (row0 + r < p.m && gcol < p.n)
              *reinterpret_cast<uint4 *>(d_base + (size_t)(row0 + r) * p.n + gcol) = v;
          }
          __syncwarp();
        }
      } else {
#pragma unroll
        for (int c = 0; c < kColsPerEpiWarp / 32; ++c)
          epilogue_chunk(p, &acc[32 * c], row, col_base + 32 * c, alpha, beta, has_c);
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (PAIR) ptx::cluster_sync();  // neither CTA leaves (or frees tensor memory) while its peer may still use it
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<CG>(tmem_base, L::kTmemCols);
  }
}

// WIDE: the scatter-mode epilogue (128-byte row pieces for the peer stores), its own instantiation so
// that the other kernels keep their register allocation.
template <int BN, bool SPARSE, bool DENSE, bool PAIR, bool WIDE = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a_dense,
                const __grid_constant__ CUtensorMap tm_a_comp, const GemmParams p) {
  gemm_body<BN, SPARSE, DENSE, PAIR, false, WIDE>(tm_w, tm_a_dense, tm_a_comp, p, nullptr);
}

// The fused SharQ GEMM of all groups (experts) of a mixture-of-experts layer in one launch, CTA pairs.
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_grouped_kernel(const __grid_constant__ GroupTable groups, const __grid_constant__ CUtensorMap tm_a_dense,
                        const __grid_constant__ CUtensorMap tm_a_comp, const GemmParams p) {
  gemm_body<256, true, true, true, true>(groups.tm_w[0], tm_a_dense, tm_a_comp, p, &groups);
}

// Second kernel of a split-K GEMM: the epilogue on the accumulated fp32 sums, 32 columns per thread.
__global__ void __launch_bounds__(256) splitk_finalize_kernel(const GemmParams p) {
  const int chunks = (p.n + 31) / 32;
  const long long total = (long long)p.m * chunks;
  const float alpha = p.alpha_ptr ? p.alpha * (*p.alpha_ptr) : p.alpha;
  const bool has_c = (p.c_in != nullptr) && (p.beta != 0.0f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / chunks);
    const int col0 = (int)(i % chunks) * 32;
    const float *src = p.splitk_acc + (size_t)row * p.n + col0;
    uint32_t acc[32];
    if ((p.n & 3) == 0 && col0 + 32 <= p.n) {
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const float4 t = __ldcg(reinterpret_cast<const float4 *>(src) + v);
        acc[4 * v] = __float_as_uint(t.x);
        acc[4 * v + 1] = __float_as_uint(t.y);
        acc[4 * v + 2] = __float_as_uint(t.z);
        acc[4 * v + 3] = __float_as_uint(t.w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = col0 + j < p.n ? __float_as_uint(__ldcg(src + j)) : 0u;
    }
    epilogue_chunk(p, acc, row, col0, alpha, p.beta, has_c);
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

struct DeviceInfo {
  bool known = false;
  int sms = 0;
};

// Per-device state: SM count and which kernel instantiations already have their
// shared-memory attribute set.
cudaError_t device_info(int *dev_out, int *sms_out) {
  static DeviceInfo info[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!info[dev].known) {
    e = cudaDeviceGetAttribute(&info[dev].sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    info[dev].known = true;
  }
  *dev_out = dev;
  *sms_out = info[dev].sms;
  return cudaSuccess;
}

template <int BN, bool SPARSE, bool DENSE, bool PAIR, bool WIDE = false>
cudaError_t launch(const GemmArgs &a, cudaStream_t stream) {
  using L = StageLayout<BN, SPARSE, DENSE, PAIR>;
  static bool attr_set[64] = {};
  auto kernel = gemm_kernel<BN, SPARSE, DENSE, PAIR, WIDE>;
  int dev = 0, sms = 0;
  cudaError_t e = device_info(&dev, &sms);
  if (e != cudaSuccess) return e;
  if (!attr_set[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  CUtensorMap tm_w, tm_ad, tm_ac;
  memset(&tm_ad, 0, sizeof(tm_ad));
  memset(&tm_ac, 0, sizeof(tm_ac));
  if (!make_tmap_bytes(&tm_w, a.b, (uint64_t)a.n, (uint64_t)a.k / 2, L::kWRows, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return cudaErrorInvalidValue;
  if (DENSE && !make_tmap_bytes(&tm_ad, a.a_dense, (uint64_t)a.m, (uint64_t)a.k / 2, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return cudaErrorInvalidValue;
  if (SPARSE && !make_tmap_bytes(&tm_ac, a.a_comp, (uint64_t)a.m, (uint64_t)a.k / 4, kBM, 64, CU_TENSOR_MAP_SWIZZLE_64B))
    return cudaErrorInvalidValue;
  GemmParams p{};
  p.staged_store = (a.n % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.scatter_world > 1 ? a.d_peer[0] : a.d) & 15) == 0);
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
  p.scatter_rows = 0;
  if (a.scatter_world > 1) {
    // dealing rows to their owners needs whole 128-row tiles per owner and the coalesced store path
    if (a.scatter_world > kGemmMaxPeers || a.m % (128 * a.scatter_world) != 0 || !p.staged_store || a.c_in != nullptr)
      return cudaErrorInvalidValue;
    for (int r = 0; r < a.scatter_world; ++r) {
      if (a.d_peer[r] == nullptr || (reinterpret_cast<uintptr_t>(a.d_peer[r]) & 15) != 0) return cudaErrorInvalidValue;
      p.d_peer[r] = static_cast<__nv_bfloat16 *>(a.d_peer[r]);
    }
    p.scatter_rows = a.m / a.scatter_world;
    p.scatter_rank = a.scatter_rank;
  }
  const int n_tiles = (a.n + BN - 1) / BN;
  const int m_units = PAIR ? (a.m + 255) / 256 : (a.m + kBM - 1) / kBM;
  int units = m_units * n_tiles;
  // Split K when one row of tiles cannot fill the GPU (M <= 128 is weight-bandwidth-bound: the
  // weights must stream through as many SMs as possible) and the caller gave scratch.
  p.k_splits = 1;
  p.splitk_acc = nullptr;
  const int k_stages = (a.k + kBK - 1) / kBK;
  if (!PAIR && m_units == 1 && a.scatter_world <= 1 && a.workspace != nullptr &&
      a.workspace_bytes >= (size_t)a.m * a.n * sizeof(float)) {
    int splits = sms / units;
    if (splits > k_stages / 2) splits = k_stages / 2;  // at least two K stages per unit
    // the fp32 reductions cost M x N x splits atomics: measured worth it for M <= 64 (qkv
    // 16.2 -> 13.3 us, down 39.9 -> 17.3 us at M = 16) and for long K (down at M = 128:
    // 41.0 -> 22.9 us), not for M = 128 with K = 4096 (17.8 -> 19.0 us)
    if (splits >= 2 && (a.m <= 64 || k_stages >= 32)) {
      p.k_splits = splits;
      p.splitk_acc = static_cast<float *>(a.workspace);
      units *= splits;
      e = cudaMemsetAsync(a.workspace, 0, (size_t)a.m * a.n * sizeof(float), stream);
      if (e != cudaSuccess) return e;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  if (PAIR) {
    const int clusters = units < sms / 2 ? units : sms / 2;
    cfg.gridDim = dim3(2 * clusters);
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  } else {
    cfg.gridDim = dim3(units < sms ? units : sms);
  }
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = L::kSmemBytes;
  cfg.stream = stream;
  e = cudaLaunchKernelEx(&cfg, kernel, tm_w, tm_ad, tm_ac, p);
  if (e != cudaSuccess || p.k_splits == 1) return e;
  const long long chunks = (long long)a.m * ((a.n + 31) / 32);
  long long blocks = (chunks + 255) / 256;
  if (blocks > 4LL * sms) blocks = 4LL * sms;
  splitk_finalize_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t run_gemm_grouped(const GroupedGemmArgs &a, cudaStream_t stream) {
  using L = StageLayout<256, true, true, true>;
  static bool attr_set[64] = {};
  if (a.groups < 1 || a.groups > kMaxGroups || a.m <= 0 || a.m % 256 != 0 || a.n <= 0 || a.k <= 0 || a.k % 128 != 0)
    return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaError_t e = device_info(&dev, &sms);
  if (e != cudaSuccess) return e;
  if (!attr_set[dev]) {
    e = cudaFuncSetAttribute(gemm_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  GroupTable gt;
  memset(&gt, 0, sizeof(gt));
  for (int g = 0; g < a.groups; ++g) {
    if (!make_tmap_bytes(&gt.tm_w[g], a.b[g], (uint64_t)a.n, (uint64_t)a.k / 2, L::kWRows, 128, CU_TENSOR_MAP_SWIZZLE_128B))
      return cudaErrorInvalidValue;
    gt.sfb_sparse[g] = static_cast<const uint8_t *>(a.sfb_sparse[g]);
    gt.sfb_dense[g] = static_cast<const uint8_t *>(a.sfb_dense[g]);
  }
  gt.unit_group = a.unit_group;
  gt.alpha = a.alpha_vec;
  CUtensorMap tm_ad, tm_ac;
  if (!make_tmap_bytes(&tm_ad, a.a_dense, (uint64_t)a.m, (uint64_t)a.k / 2, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return cudaErrorInvalidValue;
  if (!make_tmap_bytes(&tm_ac, a.a_comp, (uint64_t)a.m, (uint64_t)a.k / 4, kBM, 64, CU_TENSOR_MAP_SWIZZLE_64B))
    return cudaErrorInvalidValue;
  GemmParams p{};
  p.staged_store = (a.n % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.d) & 15) == 0);
  p.e = static_cast<const uint8_t *>(a.e);
  p.sfa_sparse = static_cast<const uint8_t *>(a.sfa_sparse);
  p.sfa_dense = static_cast<const uint8_t *>(a.sfa_dense);
  p.d = static_cast<__nv_bfloat16 *>(a.d);
  p.alpha = a.alpha;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.error_flag = a.error_flag;
  p.k_splits = 1;
  const int units = (a.m / 256) * ((a.n + 255) / 256);
  const int clusters = units < sms / 2 ? units : sms / 2;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = L::kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_grouped_kernel, gt, tm_ad, tm_ac, p);
}

cudaError_t run_gemm(const GemmArgs &a, cudaStream_t stream) {
  const bool sparse = a.a_comp != nullptr;
  const bool dense = a.a_dense != nullptr;
  if (!sparse && !dense) return cudaErrorInvalidValue;
  // tile_n: 0 = automatic, 128 / 256 = single-CTA tiles of that width, 512 = CTA pairs (256 x 256)
  int tile_n = a.tile_n;
  if (tile_n == 0) {
    int dev = 0, sms = 0;
    cudaError_t e = device_info(&dev, &sms);
    if (e != cudaSuccess) return e;
    const int pair_units = ((a.m + 255) / 256) * ((a.n + 255) / 256);
    if (a.m <= 128 || a.n <= 128) {
      tile_n = a.n > 128 ? 256 : 128;
    } else if (pair_units * 4 <= sms || a.k <= 512) {
      // 256 x 256 pair tiles would keep at most half of the SMs busy, or the K loop is too
      // short to hide the drain of a 256-wide accumulator: 128 x 128 tiles (measured at the
      // 8-way tensor-parallel shapes: 14.6 vs 18.8 us for N = 768, 12.7 vs 16.7 us for K = 512)
      tile_n = 128;
    } else {
      tile_n = 512;
    }
  }
  const bool pair = tile_n == 512;
  const bool scatter = a.scatter_world > 1;  // validated by launch(): fused GEMM, staged stores, whole tiles per owner
  if (pair) {
    if (sparse && dense) return scatter ? launch<256, true, true, true, true>(a, stream) : launch<256, true, true, true>(a, stream);
    if (sparse) return launch<256, true, false, true>(a, stream);
    return launch<256, false, true, true>(a, stream);
  }
  const int bn = tile_n == 128 ? 128 : 256;
  if (bn == 256) {
    if (sparse && dense) return scatter ? launch<256, true, true, false, true>(a, stream) : launch<256, true, true, false>(a, stream);
    if (sparse) return launch<256, true, false, false>(a, stream);
    return launch<256, false, true, false>(a, stream);
  }
  if (sparse && dense) return scatter ? launch<128, true, true, false, true>(a, stream) : launch<128, true, true, false>(a, stream);
  if (sparse) return launch<128, true, false, false>(a, stream);
  return launch<128, false, true, false>(a, stream);
}

}  // namespace sharq
