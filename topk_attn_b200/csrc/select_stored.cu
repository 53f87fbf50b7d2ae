// Exact top-k of the score keys that scan_store_kernel left in the workspace, then softmax.V over
// the winners.  One cluster of CTAs per (batch row, query head); CTA c owns a contiguous range of
// the token axis.
//
//   1. The per-part coarse histograms (top 11 bits of the keys) are summed and give the bin that
//      holds the k-th largest key: every key in a higher bin is a winner, the k-th lies in this bin.
//   2. If that bin and the bins above hold more keys than a CTA's candidate list, the bin is
//      refined 8 bits at a time by passes over the stored keys (histograms summed across the
//      cluster through distributed shared memory).  Typical inputs need no such pass.
//   3. One pass over the stored keys (mostly L2 hits: they were just written) collects the keys at
//      or above the lower edge of the bin into a candidate list in shared memory.
//   4. The common cluster code finds the exact k-th key among the candidates, deals the winners
//      over the CTAs and mixes their V rows.
// If even a single key value has more copies than the list can hold (ties at the k-th key on a
// grand scale), the copies are taken in ascending token order up to the number needed.
//
// The selection stage of retrieval_attention_kernel<K> (retrieval_attn/retrieval_attention.cu:335:
// a full radix sort of all scores to keep K of them) and of gemv_topk_kernel (gemv_topk.cu:353-361).
#include "select_common.cuh"

namespace ra {

__global__ void __launch_bounds__(kSelThreads, 1)
select_stored_kernel(const __grid_constant__ SelectStoredParams P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.m.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = blockIdx.x / C;   // (batch row, query head)
  const int bq = row / P.m.hq_total, hq = row % P.m.hq_total;
  const int k = P.m.topk, cap = P.cap;

  const size_t scratch_bytes = select_scratch_bytes(1, P.m.per, P.m.det_words);
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem + scratch_bytes);
  int* idxs = reinterpret_cast<int*>(keys + cap);
  int* cnt = idxs + cap;
  int* hist0 = cnt + 4;                                        // [kHistBins]
  SelCtrl* sc = reinterpret_cast<SelCtrl*>(hist0 + kHistBins);

  RA_STAMP(P.m.status, 0);
  // ---- 1. the coarse bin of the k-th key
  {
    const uint32_t* hrow = P.hist_ws + (size_t)row * P.nparts * kHistBins;
    for (int bin = tid; bin < kHistBins; bin += kSelThreads) {
      int s = 0;
      for (int p = 0; p < P.nparts; ++p) s += (int)hrow[(size_t)p * kHistBins + bin];
      hist0[bin] = s;
    }
    if (tid == 0) {
      cnt[0] = 0;
      sc->bin = 0; sc->n_above = 0; sc->rem = k; sc->n_in = 0;
      sc->n_eq_local = 0;
    }
    __syncthreads();
    find_coarse_bin(hist0, k, sc, tid);
  }
  uint32_t lo_key = (uint32_t)sc->bin << kHistShift;   // lower edge of the bin of the k-th key
  int shift = kHistShift;                              // the bin spans 2^shift keys
  int n_above = sc->n_above, rem = sc->rem, n_in = sc->n_in;

  const int lo = min(P.n_tokens, crank * P.chunk), hi = min(P.n_tokens, lo + P.chunk);
  const uint32_t* krow = P.keys_ws + (size_t)row * P.n_pad;

  RA_STAMP(P.m.status, 1);
  // ---- 2. refine the bin while it holds too much for the candidate list
  int buf = 0, last_local = 0;
  while (n_above + n_in > cap && shift > 0) {
    const int new_shift = max(0, shift - 8);
    if (tid < 256) sc->hist[buf][tid] = 0;
    __syncthreads();
    const uint32_t span = 1u << shift;
    for (int base = lo; base < hi; base += kSelThreads * 4 * kSelUnroll) {
      uint4 kk[kSelUnroll];
#pragma unroll
      for (int u = 0; u < kSelUnroll; ++u) {
        const int i = base + (u * kSelThreads + tid) * 4;
        kk[u] = i < hi ? ldg128_nc(krow + i) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < kSelUnroll; ++u) {
        const int i = base + (u * kSelThreads + tid) * 4;
        const uint32_t kv[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t rel = kv[e] - lo_key;   // wraps to a huge value below the bin
          if (i + e < hi && rel < span) atomicAdd(&sc->hist[buf][rel >> new_shift], 1);
        }
      }
    }
    cluster.sync();
    if (tid < 256) {
      int s = 0;
      for (int c = 0; c < C; ++c) s += cluster.map_shared_rank(&sc->hist[buf][0], c)[tid];
      sc->ghist[tid] = s;
    }
    __syncthreads();
    if (warp == 0) {
      int d, nr;
      warp_find_digit(sc->ghist, rem, lane, d, nr);
      if (lane == 0) {
        sc->bin = d;
        sc->rem = nr;
      }
    }
    __syncthreads();
    const int d = sc->bin;
    n_above += rem - sc->rem;
    rem = sc->rem;
    n_in = sc->ghist[d];
    last_local = sc->hist[buf][d];
    lo_key += (uint32_t)d << new_shift;
    shift = new_shift;
    buf ^= 1;   // a peer may still read this round's buffer; it is zeroed again two rounds on
  }

  // ---- ties on a grand scale: more copies of the k-th key than the list holds.  Copies are taken
  // in ascending token order: the CTAs before this one take theirs first.
  const bool tie_mode = n_above + n_in > cap;   // only possible with shift == 0
  int tie_take = 0;
  if (tie_mode) {
    if (tid == 0) sc->n_eq_local = last_local;
    cluster.sync();
    int before = 0;
    for (int c = 0; c < crank; ++c) before += *cluster.map_shared_rank(&sc->n_eq_local, c);
    tie_take = max(0, min(last_local, rem - before));
  }

  RA_STAMP(P.m.status, 2);
  // ---- 3. candidates: every key at or above the lower edge of the bin
  if (!tie_mode)
    collect_candidates(krow, lo, hi, lo_key, keys, idxs, cnt, cap, P.m.status, tid, lane);
  else
    collect_candidates_ties(krow, lo, hi, lo_key, tie_take, keys, idxs, cnt, cap, sc, P.m.status, tid, warp, lane);
  __syncthreads();

  RA_STAMP(P.m.status, 3);
  // ---- 4. exact k-th key over the cluster's candidates, winners dealt, V rows mixed
  MergeArgs A = P.m;
  A.list_off = 0;
  auto dest = [&](int) {
    ListDest d;
    d.valid = true;
    d.bq = bq;
    d.hq = hq;
    d.hkv = hq / P.group;
    return d;
  };
  cluster_select_attend<1>(cluster, smem, keys, idxs, cnt, cap, A, dest, lo, max(hi - lo, 1), lo_key, shift,
                           n_above);
}

size_t select_stored_fixed_smem_bytes(int per, int det_words) {
  return select_scratch_bytes(1, per, det_words) + 16 + (size_t)kHistBins * 4 + sizeof(SelCtrl) + 128;
}

cudaError_t launch_select_stored(const SelectStoredParams& P, int rows, size_t smem,
                                 cudaStream_t stream) {
  auto kern = select_stored_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * P.m.cluster), 1, 1);
  cfg.blockDim = dim3(kSelThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)P.m.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  note_launch();
  return cudaLaunchKernelEx(&cfg, kern, P);
}

}  // namespace ra
