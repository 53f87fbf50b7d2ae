// Parameters of the gathered-attention kernel.
#pragma once
#include "cluster_merge.cuh"

namespace ra {

struct GatherParams {
  MergeArgs m;               // m.topk == n_entries, m.select_all == 1
  const __half* q;           // [B,Hq,128]
  const __half* k;           // key cache, strides as m.v_*
  const int* src_idx;        // ids (expand_clen == 0) or cluster ids (expand_clen > 0)
  const float* src_score;    // scores of the cluster ids (rank order of the expansion); optional
  long long src_batch_stride, src_head_stride;  // elements; batch stride 0 = shared by the batch
  int n_src;                 // ids per (row, head) in src_idx
  int expand_clen;           // > 0: id j expands to tokens id*clen .. id*clen + clen - 1
  int n_entries;             // n_src or n_src * expand_clen
  int* out_token_ids;        // optional [B,Hq,n_entries]: the expanded ids in rank order
  int cap;                   // ceil(n_entries / cluster)
  int group;                 // query heads per kv head
};

size_t gather_attend_smem_bytes(int per, int cap, int n_src);
cudaError_t launch_kv_append(__half* kc, __half* vc, const __half* nk, const __half* nv,
                             __half* centers, int batch, int hkv, int pos, long long bstride,
                             long long tstride, long long hstride, int num_centers, int cluster_len,
                             cudaStream_t stream);
size_t gather_flash_smem_bytes(int n_src);
cudaError_t launch_gather_flash(const GatherParams& P, int rows, size_t smem, cudaStream_t stream);
cudaError_t launch_rank_sort(const float* score, const int* idx, int rows, int n, int* out_idx,
                             float* out_score, cudaStream_t stream);
cudaError_t launch_gather_attend(const GatherParams& P, int rows, size_t smem, cudaStream_t stream);

}  // namespace ra
