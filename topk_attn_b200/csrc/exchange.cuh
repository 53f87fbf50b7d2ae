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
    // a wait that ran out in an earlier kernel left its sticky bit: do not wait a full limit again
    const bool gave_up = (*reinterpret_cast<volatile unsigned*>(status) & kStatusTimeout) != 0;
    while ((int)(ld_acquire_sys(X.wait_flags + threadIdx.x) - want) < 0) {
      if (gave_up || global_timer_ns() - t0 > X.limit_ns) {
        atomicOr(status, kStatusTimeout);
        break;
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Publish step shared by the push kernel and the kernels with the exchange fused in; called by all
// threads of every CTA after its stores to peer memory.  Every CTA orders its stores at device
// scope and counts itself; the last CTA to arrive issues ONE system-scope fence (cumulative: it
// covers the stores of all CTAs it synchronised with through the counter) and then writes this
// rank's flag on every peer with relaxed system-scope stores, one lane per peer.  System-scope
// fences and release stores cost microseconds each here, so there is exactly one per launch.
__device__ __forceinline__ void exchange_publish(unsigned* done, const unsigned* epoch,
                                                 unsigned* const* peer_flag, int npeers,
                                                 unsigned* epoch_rw) {
  __shared__ unsigned s_last, s_epoch;
  __syncthreads();   // orders every thread's stores before thread 0's (cumulative) fence
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(done, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) {
    *done = 0u;   // ready for the next launch (kernel boundaries order it)
    __threadfence_system();
    s_epoch = *epoch;
  }
  __syncthreads();
  if ((int)threadIdx.x < npeers) st_relaxed_sys(peer_flag[threadIdx.x], s_epoch);
  if (epoch_rw && threadIdx.x == 0) *epoch_rw = s_epoch + 1u;
}

__device__ __forceinline__ void exchange_publish_in_kernel(const ExchangeHooks& X) {
  if (X.done == nullptr) return;
  exchange_publish(X.done, X.epoch, X.peer_flag, X.npeers, X.advance ? X.epoch_rw : nullptr);
}

cudaError_t launch_stream_read(const void* src, size_t bytes, unsigned* sink, int grid, cudaStream_t stream);
cudaError_t launch_exchange_push(const PushParams& P, int grid, cudaStream_t stream);
cudaError_t launch_exchange_wait(const unsigned* flags, int n, unsigned* epoch, int advance,
                                 unsigned long long limit_ns, unsigned* status, cudaStream_t stream);

}  // namespace ra
