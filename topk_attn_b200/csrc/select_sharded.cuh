// Parameters of select_sharded_kernel: the selection of the sequence-sharded step in which the
// ranks exchange histograms of their score keys instead of candidates.
#pragma once
#include "exchange.cuh"
#include "select_common.cuh"

namespace ra {

constexpr int kShardRounds = 3;    // 11 + 11 + 10 bits of a key
constexpr int kPartWords = 132;    // a partial row: 128 sums, weight, maximum, 2 words of padding

// Every rank owns one receive buffer of 8-byte words (32 bits of payload under a 32-bit epoch tag):
//   histograms [kShardRounds][world][rows][kHistBins], then partial rows [world][rows][kPartWords].
struct ShardHist {
  unsigned long long* buf_peer[kMaxPeers];   // rank p's receive buffer as mapped here
  int world, rank;
  const unsigned* epoch;            // device word holding the current step's epoch
  unsigned* epoch_rw;               // the same word: the last CTA adds one
  unsigned* done;                   // zero between launches: CTAs that have finished
  unsigned long long limit_ns;      // bound of every wait
};

struct SelectShardedParams {
  SelectStoredParams s;   // s.m.out = the final fp16 output of this rank
  ShardHist x;
};

size_t select_sharded_fixed_smem_bytes();
cudaError_t launch_select_sharded(const SelectShardedParams& P, int rows, size_t smem, cudaStream_t stream);

}  // namespace ra
