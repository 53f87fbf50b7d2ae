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

cudaError_t launch_exchange_push(const PushParams& P, int grid, cudaStream_t stream);
cudaError_t launch_exchange_wait(const unsigned* flags, int n, unsigned* epoch, int advance,
                                 unsigned long long limit_ns, unsigned* status, cudaStream_t stream);

}  // namespace ra
