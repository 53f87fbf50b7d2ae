// Parameters of the peer-store exchange kernels of the sequence-sharded path.
#pragma once
#include "common.cuh"

namespace ra {

constexpr int kMaxPeers = 32;      // ranks of one exchange (one node)
constexpr int kPushThreads = 256;

struct PushParams {
  const uint4* src;            // local piece, 16-byte aligned
  size_t n16;                  // its size in 16-byte units
  uint4* dst[kMaxPeers];       // the piece's slot in every rank's receive buffer (own slot may equal src)
  unsigned* flag[kMaxPeers];   // this rank's flag word on every rank
  int npeers;
  const unsigned* epoch;       // device word holding the current step's epoch
  unsigned* done;              // device word, zero between launches: CTAs that have finished
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Exchange steps fused into a consumer or producer kernel (all pointers optional).
struct ExchangeHooks {
  // before the kernel reads what the peers stored: wait until each of wait_n flags has reached the
  // epoch, at most limit_ns each
  const unsigned* wait_flags;
  int wait_n;
  const unsigned* epoch;
  unsigned long long limit_ns;
  // after the kernel has written its rows: the same rows go to every peer, then this rank's flag
  float* peer_rows[kMaxPeers];     // row r of this rank's slot on peer p: peer_rows[p] + r * pitch
  unsigned* peer_flag[kMaxPeers];
  int npeers;
  unsigned* done;                  // zero between launches: CTAs that have finished
  int advance;                     // the last CTA to finish adds one to the epoch word
  unsigned* epoch_rw;
};

// Called by the first threads of a CTA before it touches exchanged data; ends with a CTA barrier.
__device__ __forceinline__ void exchange_wait_in_kernel(const ExchangeHooks& X, unsigned* status) {
  if (X.wait_flags == nullptr) return;
  if ((int)threadIdx.x < X.wait_n) {
    const unsigned want = *X.epoch;
    const unsigned long long t0 = global_timer_ns();
    while ((int)(ld_acquire_sys(X.wait_flags + threadIdx.x) - want) < 0) {
      if (global_timer_ns() - t0 > X.limit_ns) {
        atomicOr(status, kStatusTimeout);
        break;
      }
    }
  }
  __syncthreads();
}

// Called by all threads of every CTA after its stores to peer memory: the last CTA of the grid
// publishes the flags (and advances the epoch when asked to).
__device__ __forceinline__ void exchange_publish_in_kernel(const ExchangeHooks& X) {
  if (X.done == nullptr) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned arrived = atomicAdd(X.done, 1u);
    if (arrived == gridDim.x - 1) {
      *X.done = 0u;
      __threadfence_system();
      const unsigned e = *X.epoch;
      for (int p = 0; p < X.npeers; ++p) st_release_sys(X.peer_flag[p], e);
      if (X.advance) *X.epoch_rw = e + 1u;
    }
  }
}

cudaError_t launch_exchange_push(const PushParams& P, int grid, cudaStream_t stream);
cudaError_t launch_exchange_wait(const unsigned* flags, int n, unsigned* epoch, int advance,
                                 unsigned long long limit_ns, unsigned* status, cudaStream_t stream);

}  // namespace ra
