// Parameters of the candidate-merge kernel.
#pragma once
#include "cluster_merge.cuh"
#include "exchange.cuh"

namespace ra {

struct MergeParams {
  MergeArgs m;              // m.topk winners out of m_total candidates per (batch row, head)
  const float* cand_score;  // candidate c of row r: [ (c / part_len) * part_stride +
  const int* cand_idx;      //                       r * row_stride + c % part_len ]
  long long part_stride, row_stride;
  int part_len;
  int m_total;
  int cap;                  // ceil(m_total / cluster)
  int group;                // query heads per kv head
  int own_part;             // >= 0: ids are read for the candidates of this part only (the others
                            // count as -1: never owned); -1: every id is read
  int ids_global;           // single-CTA form: ids are read from cand_idx for the winners only
  ExchangeHooks x;          // single-CTA form: wait for the candidates / push the partial rows
};

size_t merge_attend_smem_bytes(int per, int cap);
cudaError_t launch_merge_attend(const MergeParams& P, int rows, size_t smem, cudaStream_t stream);
// one CTA per row, for candidate lists that fit in its shared memory
size_t merge_attend_cta_smem_bytes(int m_total, int topk, bool ids_global);
cudaError_t launch_merge_attend_cta(const MergeParams& P, int rows, size_t smem, cudaStream_t stream);
// out[r, :] = sum_p w_p o_p / sum_p w_p l_p with w_p = exp(m_p - max m); partials are
// [parts][rows][130] = 128 un-normalised sums, their weight l, their maximum m.
cudaError_t launch_lse_combine(const float* partials, int parts, int rows, __half* out,
                               cudaStream_t stream, const ExchangeHooks* x = nullptr,
                               unsigned* status = nullptr);

}  // namespace ra
