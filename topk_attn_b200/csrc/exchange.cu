// Exchange step of the sequence-sharded path without a collective library: every rank stores its
// piece (its k proposals per head, later its partial output) straight into a slot of every peer's
// receive buffer with ordinary stores over peer-mapped memory, then raises a flag on each peer; the
// consumer waits for the flags of all ranks before its next kernel reads the slots.
//
//   exchange_push_kernel   copies `bytes` from a local buffer to the same slot on each peer and,
//                          after the last CTA has finished, writes the current epoch to this
//                          rank's flag on every peer (release at system scope).
//   exchange_wait_kernel   one thread per flag: waits until it holds the current epoch (acquire at
//                          system scope).  Every wait is bounded by wall time; a wait that runs out
//                          sets the timeout bit of the status word and the kernel returns, so the
//                          context stays usable and the host learns of it from ra_check_status().
//
// The epoch lives in device memory and is advanced by the last wait of a step, so a captured CUDA
// graph of the step can be replayed without changing any kernel argument.  Only plain loads and
// stores touch peer memory (no switch-side replication, no bulk-tensor copies).  The reference is
// single-device;
// the in-GPU mechanism this generalises is the cluster-wide max/sum exchange through distributed
// shared memory of baseline_1.cu:549-598.
#include "exchange.cuh"

namespace ra {

__global__ void __launch_bounds__(kPushThreads)
exchange_push_kernel(const __grid_constant__ PushParams P) {
  const size_t stride = (size_t)gridDim.x * kPushThreads;
  bool any_remote = false;
  for (int p = 0; p < P.npeers; ++p) any_remote |= (P.dst[p] != P.src);
  if (any_remote) {
    for (size_t i0 = (size_t)blockIdx.x * kPushThreads + threadIdx.x; i0 < P.n16; i0 += 4 * stride) {
      uint4 v[4];   // four loads in flight per thread, then the stores to every peer
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = (i0 + u * stride < P.n16) ? P.src[i0 + u * stride] : make_uint4(0, 0, 0, 0);
#pragma unroll 1
      for (int p = 0; p < P.npeers; ++p) {
        if (P.dst[p] == P.src) continue;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i0 + u * stride < P.n16) P.dst[p][i0 + u * stride] = v[u];
      }
    }
  }
  exchange_publish(P.done, P.epoch, P.flag, P.npeers, nullptr);
}

__global__ void __launch_bounds__(kMaxPeers)
exchange_wait_kernel(const unsigned* flags, int n, unsigned* epoch, int advance,
                     unsigned long long limit_ns, unsigned* status) {
  const unsigned want = *epoch;
  if ((int)threadIdx.x < n) {
    const unsigned long long t0 = global_timer_ns();
    // a wait that ran out in an earlier kernel left its sticky bit: do not wait a full limit again
    const bool gave_up = (*reinterpret_cast<volatile unsigned*>(status) & kStatusTimeout) != 0;
    // flags only grow; compare as a signed distance so that a wrapped counter still works
    while ((int)(ld_acquire_sys(flags + threadIdx.x) - want) < 0) {
      if (gave_up || global_timer_ns() - t0 > limit_ns) {
        atomicOr(status, kStatusTimeout);
        break;
      }
    }
  }
  __syncthreads();
  if (advance && threadIdx.x == 0) *epoch = want + 1u;
}

// Read-only stream over a buffer (a measuring aid for benchmarks: what this GPU delivers to a
// kernel that only reads, next to the copy figure the roofline is quoted against).  Eight 16-byte
// loads in flight per thread; the folded words go to `sink` so that nothing is optimised away.
__global__ void __launch_bounds__(512)
stream_read_kernel(const uint4* __restrict__ src, size_t n16, unsigned* sink) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  unsigned acc = 0u;
  for (size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < n16; i0 += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      v[u] = (i0 + u * stride < n16) ? ldg128_nc(src + i0 + u * stride) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int u = 0; u < 8; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  if (acc == 0x9e3779b9u) sink[0] = acc;   // practically never: keeps the loads alive
}

cudaError_t launch_stream_read(const void* src, size_t bytes, unsigned* sink, int grid, cudaStream_t stream) {
  note_launch();
  stream_read_kernel<<<grid, 512, 0, stream>>>(static_cast<const uint4*>(src), bytes / 16, sink);
  return cudaGetLastError();
}

cudaError_t launch_exchange_push(const PushParams& P, int grid, cudaStream_t stream) {
  note_launch();
  exchange_push_kernel<<<grid, kPushThreads, 0, stream>>>(P);
  return cudaGetLastError();
}

cudaError_t launch_exchange_wait(const unsigned* flags, int n, unsigned* epoch, int advance,
                                 unsigned long long limit_ns, unsigned* status, cudaStream_t stream) {
  note_launch();
  exchange_wait_kernel<<<1, kMaxPeers, 0, stream>>>(flags, n, epoch, advance, limit_ns, status);
  return cudaGetLastError();
}

}  // namespace ra
