// Sum of the partial outputs of a row-parallel SharQ linear over the GPUs of one NVSwitch
// domain, in place, in one kernel per GPU: every rank reduces its 1/world slice of the
// buffer INSIDE the switch (multimem.ld_reduce on the multicast address adds the same
// 16 bytes of every rank's copy, accumulating in fp32) and writes the rounded result back to
// every rank's copy with one multicast store (multimem.st).  Each GPU therefore receives the
// buffer once (its own slice reduced, the other slices broadcast) and sends 1/world of it.
//
// The reference has no tensor parallelism, so this kernel has no counterpart there.
//
// Synchronisation: CTA b of every rank meets CTA b of all other ranks at a flag barrier
// before reading (all partial sums are complete: a rank's kernel only starts after its GEMM
// on the same stream) and again after storing (all copies are complete, and nobody still
// reads this rank's copy).  A flag is one 32-bit counter in the RECEIVER's memory per (CTA,
// sender): the sender adds 1 with a one-way system-scope release reduction through the peer
// mapping, the receiver waits until the counter reaches the number of barriers it has been
// through, which it keeps in its own memory next to the flags.  All state is in device
// memory, so a captured launch can be replayed.  Every spin is bounded: when the limit
// passes the kernel records an error code and goes on (the result is then wrong, and the
// host sees the code), it never hangs.
#include <cuda_bf16.h>

#include <cstdint>

#include "allreduce.cuh"

namespace sharq {

namespace {

constexpr int kThreads = 512;
constexpr int kUnroll = 4;
constexpr long long kSpinLimitCycles = 4000000000LL;  // about two seconds
long long g_spin_limit_cycles = kSpinLimitCycles;     // host-side setting, see set_allreduce_wait_limit

struct AllReduceParams {
  uint8_t *data[kAllReduceMaxRanks];      // peer-copy variant: rank p's buffer as mapped here
  uint8_t *mc;                            // multicast address of the data
  uint32_t *flags[kAllReduceMaxRanks];    // flags[p]: rank p's flag words as mapped here
  int rank, world;
  size_t slice_bytes;                     // bytes / world, multiple of 16
  long long spin_limit;                   // clock cycles a flag wait may take
  int *error_flag;
};

__device__ __forceinline__ void ld_reduce_bf16x8(const uint8_t *mc_addr, uint32_t (&v)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "l"(mc_addr)
               : "memory");
}

__device__ __forceinline__ void st_multicast_16(uint8_t *mc_addr, const uint32_t (&v)[4]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3])
               : "memory");
}

__device__ __forceinline__ void signal_add_release(uint32_t *flag) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
}

__device__ __forceinline__ uint32_t load_acquire(const uint32_t *flag) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}

// All ranks' CTAs with this block index meet for the `epoch`-th time.  Threads 0..world-1
// each talk to one rank.
__device__ __forceinline__ void cross_rank_barrier(const AllReduceParams &p, uint32_t epoch, int code) {
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    signal_add_release(p.flags[peer] + (size_t)blockIdx.x * p.world + p.rank);
    const uint32_t *recv = p.flags[p.rank] + (size_t)blockIdx.x * p.world + peer;
    const long long t0 = clock64();
    while ((int32_t)(load_acquire(recv) - epoch) < 0) {
      if (clock64() - t0 > p.spin_limit) {
        atomicExch(p.error_flag, code);
        break;
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ uint4 ld_sys_16(const uint8_t *addr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}

__device__ __forceinline__ void st_sys_16(uint8_t *addr, const uint4 &v) {
  asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void add_bf16x2(float (&acc)[8], const uint4 &v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __uint_as_float(w[i] << 16);
    acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// The same all-reduce with plain peer loads and stores instead of the switch's multicast
// object: rank r sums slice r of every rank's copy in rank order (fp32) and writes the bf16
// result into every copy.  With two ranks this moves fewer bytes per link than the in-switch
// form (a multicast store also loops back to its sender); it is used for world == 2.
__global__ void __launch_bounds__(kThreads) allreduce_peer_kernel(const AllReduceParams p) {
  uint32_t *my_epoch = p.flags[p.rank] + (size_t)kAllReduceMaxCtas * kAllReduceMaxRanks + blockIdx.x;
  const uint32_t epoch = *my_epoch;
  cross_rank_barrier(p, epoch + 1, 0x200 + 1);
  const size_t base = (size_t)p.rank * p.slice_bytes;
  const size_t stride = (size_t)gridDim.x * kThreads * 16;
  for (size_t off = ((size_t)blockIdx.x * kThreads + threadIdx.x) * 16; off < p.slice_bytes; off += kUnroll * stride) {
    uint4 v[kUnroll][kAllReducePeerMaxRanks];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (off + u * stride < p.slice_bytes)
#pragma unroll
        for (int r = 0; r < kAllReducePeerMaxRanks; ++r)
          if (r < p.world) v[u][r] = ld_sys_16(p.data[r] + base + off + u * stride);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (off + u * stride < p.slice_bytes) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kAllReducePeerMaxRanks; ++r)
          if (r < p.world) add_bf16x2(acc, v[u][r]);
        uint4 out;
        uint32_t *o = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 pair = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
          o[i] = *reinterpret_cast<uint32_t *>(&pair);
        }
#pragma unroll
        for (int r = 0; r < kAllReducePeerMaxRanks; ++r)
          if (r < p.world) st_sys_16(p.data[r] + base + off + u * stride, out);
      }
    }
  }
  cross_rank_barrier(p, epoch + 2, 0x200 + 2);
  if (threadIdx.x == 0) *my_epoch = epoch + 2;
}

__global__ void __launch_bounds__(kThreads) allreduce_multimem_kernel(const AllReduceParams p) {
  // barriers this CTA index has been through so far (same on every rank)
  uint32_t *my_epoch = p.flags[p.rank] + (size_t)kAllReduceMaxCtas * kAllReduceMaxRanks + blockIdx.x;
  const uint32_t epoch = *my_epoch;
  cross_rank_barrier(p, epoch + 1, 0x100 + 1);
  uint8_t *base = p.mc + (size_t)p.rank * p.slice_bytes;
  const size_t stride = (size_t)gridDim.x * kThreads * 16;
  for (size_t off = ((size_t)blockIdx.x * kThreads + threadIdx.x) * 16; off < p.slice_bytes; off += kUnroll * stride) {
    uint32_t v[kUnroll][4];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (off + u * stride < p.slice_bytes) ld_reduce_bf16x8(base + off + u * stride, v[u]);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (off + u * stride < p.slice_bytes) st_multicast_16(base + off + u * stride, v[u]);
  }
  cross_rank_barrier(p, epoch + 2, 0x100 + 2);
  if (threadIdx.x == 0) *my_epoch = epoch + 2;
}

}  // namespace

void set_allreduce_wait_limit(long long cycles) { g_spin_limit_cycles = cycles > 0 ? cycles : kSpinLimitCycles; }

size_t allreduce_flag_bytes() {
  return ((size_t)kAllReduceMaxCtas * kAllReduceMaxRanks + kAllReduceMaxCtas) * sizeof(uint32_t);
}

cudaError_t run_allreduce(void *multicast_data, void *const *rank_data_ptrs, void *const *rank_flag_ptrs, int rank,
                          int world, size_t bytes, int max_ctas, int *error_flag, cudaStream_t stream) {
  AllReduceParams p{};
  const bool peer = multicast_data == nullptr;
  if (peer && (rank_data_ptrs == nullptr || world > kAllReducePeerMaxRanks)) return cudaErrorInvalidValue;
  if (peer)
    for (int i = 0; i < world; ++i) p.data[i] = static_cast<uint8_t *>(rank_data_ptrs[i]);
  p.mc = static_cast<uint8_t *>(multicast_data);
  for (int i = 0; i < world; ++i) p.flags[i] = static_cast<uint32_t *>(rank_flag_ptrs[i]);
  p.rank = rank;
  p.world = world;
  p.slice_bytes = bytes / world;
  p.spin_limit = g_spin_limit_cycles;
  p.error_flag = error_flag;
  // about 128 KB of the slice per CTA, between 16 and the limit: measured best for a 16.8 MB
  // buffer (16 CTAs at 8 ranks: 54.9 us against 59.3 with 96; 64 CTAs at 2 ranks: 58.6 us
  // against 89.3 with 16); the kernel is bound by round trips through the switch, not by SMs
  const size_t per_cta = (size_t)128 * 1024;
  size_t ctas = (p.slice_bytes + per_cta - 1) / per_cta;
  if (ctas < 16) ctas = 16;
  const size_t fit = (p.slice_bytes + (size_t)kThreads * 16 - 1) / ((size_t)kThreads * 16);  // no idle CTAs on tiny buffers
  if (ctas > fit) ctas = fit;
  if (max_ctas <= 0 || max_ctas > kAllReduceMaxCtas) max_ctas = kAllReduceDefaultCtas;
  if (ctas > (size_t)max_ctas) ctas = max_ctas;
  if (ctas < 1) ctas = 1;
  if (peer)
    allreduce_peer_kernel<<<(unsigned)ctas, kThreads, 0, stream>>>(p);
  else
    allreduce_multimem_kernel<<<(unsigned)ctas, kThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace sharq
