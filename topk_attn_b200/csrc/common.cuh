// Device helpers shared by the sm_100a kernels: mbarrier / TMA wrappers with bounded waits,
// order-preserving score keys, small warp utilities.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace ra {

constexpr int kHeadDim = 128;          // the reference's only head size
constexpr int kRowBytes = kHeadDim * 2;
constexpr int kConsumerGroups = 2;     // most warp groups of the scan kernel (each on its own tile)
constexpr int kConsumerWarps = 8 * kConsumerGroups;
constexpr int kConsumerThreads = 32 * kConsumerWarps;
constexpr int kThreads = kConsumerThreads + 32;   // + one TMA producer warp
constexpr int kMergeThreads = 256;     // threads per CTA of the candidate-merge kernel
constexpr int kMaxWarps = 32;
constexpr int kRendezvous = 4;         // most scan iterations between list-overflow checks
constexpr int kTileRows = 128;         // K rows (tokens x kv heads) per pipeline stage
constexpr int kStageBytes = kTileRows * kRowBytes;   // 32 KiB
constexpr int kMaxStages = 6;
constexpr int kMaxLists = 8;           // candidate lists (kv heads x queries) per CTA
constexpr unsigned long long kWaitLimitNs = 1000000000ull;   // bounded mbarrier wait: 1 s

// status word bits written by kernels that abandon a bounded wait
constexpr unsigned kStatusTimeout = 1u;
constexpr unsigned kStatusBadId = 2u;      // a winner id outside the value cache was skipped
constexpr unsigned kStatusOverflow = 4u;   // a candidate list overflowed its capacity

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Order-preserving map float -> uint32 (larger float = larger key; +NaN sorts highest, the
// order torch.topk uses) and back.
__device__ __forceinline__ uint32_t score_key(float s) {
  uint32_t u = __float_as_uint(s);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_score(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}
__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t addr, unsigned parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(addr), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Wait on an mbarrier phase for at most limit_ns (default kWaitLimitNs) of wall time.  Returns false when the limit
// ran out or when another thread of the CTA already gave up (*abort != 0); in both cases *abort is
// set, the caller records that in the status word and carries on so that every barrier stays
// matched and the kernel ends promptly.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort,
                                          unsigned long long limit_ns = kWaitLimitNs) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_try_wait(addr, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
    if (mbar_try_wait(addr, parity)) return true;
    if (*abort) return false;
    if (global_timer_ns() - t0 > limit_ns) {
      *abort = 1;
      return false;
    }
  }
}

// Tiled TMA load of a 4-D box into shared memory, completion on an mbarrier.
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3)
      : "memory");
}
// The same load with an L2 eviction hint: rows that are read exactly once (a K stream) are marked
// evict-first so that they do not push out data the next kernel re-reads (stored scores, V rows).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_4d_hint(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                 int c0, int c1, int c2, int c3, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
      ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "r"(addr));
  return r;
}
__device__ __forceinline__ uint4 ldg128_nc(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// d += a(16x16, row) * b(16x8, col), fp16 inputs, fp32 accumulate
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// A 128-token x 128-dim fp16 tile loaded by TMA as two [128 tokens][64 dims] halves of 16 KiB with
// the 128-byte swizzle: byte offset of (token row, 16-byte chunk c8 in 0..15 of the 256-byte row).
constexpr int kSwzHalfBytes = 128 * 128;
__device__ __forceinline__ uint32_t swz128(int token, int c8) {
  return (uint32_t)((c8 >> 3) * kSwzHalfBytes + token * 128 + (((c8 & 7) ^ (token & 7)) << 4));
}
__device__ __forceinline__ float2 h2f2(uint32_t u) {
  __half2 h = *reinterpret_cast<__half2*>(&u);
  return __half22float2(h);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Phase-timing switches of the scan kernel exist only in RA_TUNING builds of the library.
#ifdef RA_TUNING
#define RA_DEBUG(P, bit) ((P).debug & (bit))
#else
#define RA_DEBUG(P, bit) 0
#endif

// Phase stamps (RA_TUNING builds only): thread 0 of CTA 0 writes the wall clock into 64-bit slot
// 4 + slot of the 256-byte status block, for reading back after the launch.
#ifdef RA_TUNING
#define RA_STAMP(status, slot)                                                              \
  do {                                                                                      \
    if (blockIdx.x == 0 && threadIdx.x == 0)                                                \
      reinterpret_cast<unsigned long long*>(status)[4 + (slot)] = ra::global_timer_ns();    \
  } while (0)
#else
#define RA_STAMP(status, slot) \
  do {                         \
  } while (0)
#endif

// host-side count of kernel launches (read through ra_launch_count)
extern std::atomic<unsigned long long> g_launch_count;
inline void note_launch() { g_launch_count.fetch_add(1, std::memory_order_relaxed); }

}  // namespace ra
