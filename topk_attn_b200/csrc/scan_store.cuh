// Parameters of the two kernels that select the top-k when several queries share a K row and k is
// large: scan_store_kernel streams K once, scores every row for all its queries on the tensor cores
// and stores the ordered 32-bit score keys; select_stored_kernel finds the exact k best of the
// stored keys of every (batch row, query head) and attends over them.
#pragma once
#include "cluster_merge.cuh"

namespace ra {

constexpr int kHistBins = 2048;        // coarse histogram of the score keys: their top 11 bits
constexpr int kHistShift = 21;
constexpr int kSelThreads = 1024;      // threads per CTA of select_stored_kernel
constexpr int kSelMaxCluster = 8;

struct StoreParams {
  CUtensorMap kmap;          // 4-D map over the key cache: 64-dim boxes, 128-byte swizzle
  const __half* q;           // [B,Hq,128]
  unsigned* status;
  uint32_t* keys_ws;         // [B*Hq][n_pad]: ordered key of q.K per token
  uint32_t* hist_ws;         // [B*Hq][nparts][kHistBins]: this part's count per coarse bin
  int batch, hq, hkv, n_tokens;
  int n_pad;                 // row pitch of keys_ws (a multiple of 128)
  int group;                 // hq / hkv
  int bshare;                // batch rows scored together on one shared cache
  int nq_valid;              // bshare * group <= 8 queries per K row
  int kv_per_batch;
  int nstages, groups;       // TMA pipeline depth, consumer warp groups (1 or 2)
  int nparts, part_len;      // CTAs per (batch group, kv head) and their share of the token axis
};

struct SelectStoredParams {
  MergeArgs m;               // m.topk winners per row, dealt over m.cluster CTAs
  const uint32_t* keys_ws;
  const uint32_t* hist_ws;
  int n_tokens, n_pad, nparts;
  int chunk;                 // tokens per CTA of a row's cluster (a multiple of 128)
  int cap;                   // capacity of a CTA's candidate list
  int group;
};

size_t scan_store_smem_bytes(int nq_valid, int nstages);
cudaError_t launch_scan_store(const StoreParams& P, int grid, size_t smem, cudaStream_t stream);
size_t select_stored_fixed_smem_bytes(int per, int det_words);
cudaError_t launch_select_stored(const SelectStoredParams& P, int rows, size_t smem,
                                 cudaStream_t stream);

}  // namespace ra
