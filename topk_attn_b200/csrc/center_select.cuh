// Parameters of the centroid-table selection kernel.
#pragma once
#include "common.cuh"

namespace ra {

constexpr int kCenterThreads = 512;
constexpr int kCenterMaxCsz = 8192;   // centroid scores of one head kept in shared memory
constexpr int kCenterMaxCluster = 8;

struct CenterSelectParams {
  const __half* q;        // [rows, 128], rows = batch * heads
  const __half* centers;  // [heads, csz, 128]
  int heads, csz, topc, clen;
  int cluster;            // CTAs per row; each scores `per` centroids (a multiple of 4)
  int per;
  int vec_members;        // clen % 4 == 0 and out_members 16-byte aligned: 128-bit id stores
  int* out_cluster_ids;   // optional [rows, topc], descending score (ties: lower id first)
  float* out_scores;      // optional [rows, topc], same order
  int* out_members;       // optional [rows, topc * clen]: id * clen + 0 .. clen-1 per winner
  // fused attention over the member tokens of the winners (center_attend_kernel only)
  const __half* k;        // key / value caches, strides in elements; one kv head per query head
  const __half* v;
  __half* out;            // [rows, 128]
  long long batch_stride, token_stride, head_stride;
  int n_tokens;
  float scale_log2e;
  unsigned* status;
};

size_t center_select_smem_bytes(int csz, int topc);
cudaError_t launch_center_select(const CenterSelectParams& P, int rows, cudaStream_t stream);
// selection, expansion and attention over the member tokens in one launch
cudaError_t launch_center_attend(const CenterSelectParams& P, int rows, cudaStream_t stream);

}  // namespace ra
