// Parameters of the candidate-merge kernel.
#pragma once
#include "cluster_merge.cuh"

namespace ra {

struct MergeParams {
  MergeArgs m;              // m.topk winners out of m_total candidates per (batch row, head)
  const float* cand_score;  // [B*Hq, m_total]
  const int* cand_idx;      // [B*Hq, m_total]
  int m_total;
  int cap;                  // ceil(m_total / cluster)
  int group;                // query heads per kv head
};

size_t merge_attend_smem_bytes(int per, int cap);
cudaError_t launch_merge_attend(const MergeParams& P, int rows, size_t smem, cudaStream_t stream);

}  // namespace ra
