// Parameters of the short-segment selection kernel.
#pragma once
#include "common.cuh"

namespace ra {

constexpr int kDenseThreads = 256;
constexpr int kDenseMaxSeg = 4096;   // longer segments stream through the scan kernel
constexpr int kDenseMaxCluster = 8;

struct DenseSelectParams {
  const __half* q;        // [batch, hq, 128]
  const __half* k;        // key cache, strides in elements
  long long batch_stride, token_stride, head_stride;
  int batch, hq, hkv, group;
  int bshare;             // batch rows scored per K row (one shared cache), bshare * group <= NQ
  int nq_valid;           // bshare * group
  int seg_len, segments, topk;
  int cluster, per;       // CTAs per (segment, kv head, batch group); rows scored by each
  int index_base;         // added to the token ids written
  int* out_idx;           // [batch, hq, segments * topk], unordered inside a segment
  float* out_score;       // same shape: q.K of the listed ids
  unsigned* status;       // status block of the caller's workspace
};

size_t dense_select_smem_bytes(int nq, int seg_len, int topk);
cudaError_t launch_dense_select(const DenseSelectParams& P, int nq, cudaStream_t stream);

}  // namespace ra
