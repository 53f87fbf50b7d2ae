// Parameters of select_sharded_kernel: the selection of the sequence-sharded step in which the
// ranks exchange histograms of their score keys instead of candidates.
#pragma once
#include "exchange.cuh"
#include "select_common.cuh"

namespace ra {

constexpr int kShardRounds = 3;   // 11 + 11 + 10 bits of a key

struct ShardHist {
  uint32_t* hist_peer[kMaxPeers];   // rank p's receive buffer [kShardRounds][world][rows][kHistBins]
  unsigned* flag_peer[kMaxPeers];   // rank p's flag words    [kShardRounds][world][rows]
  int world, rank;
  const unsigned* epoch;            // device word holding the current step's epoch
  unsigned long long limit_ns;      // bound of every wait
};

struct SelectShardedParams {
  SelectStoredParams s;   // s.m.out_partial = this rank's slot of its own partial buffer
  ShardHist x;
  ExchangeHooks part;     // push of the partial rows (peer_rows, peer_flag, npeers, done), or done == NULL
};

size_t select_sharded_fixed_smem_bytes();
cudaError_t launch_select_sharded(const SelectShardedParams& P, int rows, size_t smem, cudaStream_t stream);

}  // namespace ra
