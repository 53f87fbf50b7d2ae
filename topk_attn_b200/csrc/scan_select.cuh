// Parameters shared by the scan+select kernel and its host launcher.
#pragma once
#include "cluster_merge.cuh"

namespace ra {

struct ScanParams {
  CUtensorMap kmap;          // 4-D map over the key cache (or the centroid table)
  MergeArgs m;               // selection / output arguments (list_off is set per cluster)
  const __half* q;           // [B,Hq,128]
  unsigned* status;          // one word, bit 0 = a bounded wait gave up
  const int* part_ids;       // optional [B,Hq,nparts]: which slice of length part_len each part is
  // two-level retrieval with a small centroid table: instead of part_ids every CTA scores the
  // coarse_csz centroids of its head itself and takes the cluster of rank `part`
  const __half* coarse_centers;   // [Hq, coarse_csz, 128]
  int coarse_csz;                 // <= kMaxCoarse
  int* coarse_ids_out;            // optional [B,Hq,nparts]: the chosen cluster ids in rank order
  int batch, hq, hkv, n_tokens;
  int group;                 // hq / hkv
  int bshare;                // batch rows that share one cache and are scored together
  int nq_valid;              // bshare * group, queries that share a K row
  int qsplit;                // clusters the queries of a row are dealt over
  int nq_cta;                // nq_valid / qsplit, queries scored per K row by one cluster (<= NQ)
  int kv_per_batch;          // 1: every batch row has its own cache
  int cap;                   // capacity of a candidate list (>= topk + 2 tiles)
  int nstages;               // TMA pipeline depth (a multiple of groups)
  int groups;                // consumer warp groups: 1 or 2
  int rendezvous;            // scan iterations between list-overflow checks
  int parts_in_cluster;      // 1: the nparts parts of a (batch row, head) are the CTAs of one cluster
  int nparts;                // parts (segments x splits) per (batch row, head)
  int part_len;              // tokens per part
  int head_major;            // 1: table is [H, N, 128] (centroids); one head per CTA
  int swizzled;              // 1: tiles are two 64-dim halves with the 128-byte swizzle (tensor-core scoring)
  unsigned long long wait_limit_ns;   // bound of every wait on a pipeline barrier
  int debug;                 // RA_TUNING builds only: bits switch parts of the kernel off (phase timing)
};

constexpr int kMaxCoarse = 256;   // centroids per head the scan kernel's prologue ranks itself

size_t scan_smem_bytes(int nl, int cap, int nstages);
size_t merge_scratch_bytes(int nl, int per, int det_words);
cudaError_t launch_scan_select(const ScanParams& P, int hg, int nq, int grid, size_t smem,
                               cudaStream_t stream);

}  // namespace ra
