// Sequence-sharded selection by exchanged histograms: every rank has scored its own shard
// (scan_store_kernel) and holds the score keys of its tokens; the ranks find the exact global k-th
// key together by a radix select whose histograms -- never the keys or candidates themselves --
// cross the links, and each rank then attends over the winners among its own tokens.
//
// One cluster of CTAs per (batch row, query head) on every rank, all ranks in step per row:
//   round 0   the coarse histogram (top 11 bits, counted during the scan) of this rank goes to
//             every rank; the sum over ranks gives the bin of the global k-th key;
//   round 1+  while that bin holds more keys than are still wanted from it, the bin is split by
//             its next 11 (then 10) bits: one pass over the stored keys of this rank, the counts
//             summed over the cluster through distributed shared memory, exchanged and summed over
//             the ranks.  Distinct scores end after round 1; only copies or near-copies of the k-th
//             score need round 2;
//   then      keys above the k-th key win; of its copies each rank takes its share in rank order
//             (lower ranks hold lower token ids), inside a rank in token order.  The winners' V
//             rows are mixed into an un-normalised partial, which goes to every rank for the
//             log-sum-exp combine.
// An exchange is plain stores into the sender's slot of every rank's receive buffer, one
// system-scope fence, then the sender's flag word for that (round, row) on every rank; a receiver
// polls its own flag words, every wait bounded in time (status bit on giving up).  Since all
// ranks see the same sums they take the same number of rounds.
//
// The reference is single-device; the result is defined as equal to the single-device operator on
// the concatenated cache (retrieval_attn/test_ra.py:88-160 generalised to a global top-k).
#include "select_sharded.cuh"

namespace ra {

namespace {

struct ShardCtrl {
  int own_above;   // this rank's keys above the current interval
  int red[32];
};

// Sum over the block of v; result to every thread.  Two barriers.
__device__ __forceinline__ int block_sum(int v, int* red, int tid) {
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  int s = red[lane];
#pragma unroll
  for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  return s;
}

}  // namespace

__global__ void __launch_bounds__(kSelThreads, 1)
select_sharded_kernel(const __grid_constant__ SelectShardedParams P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  cg::cluster_group cluster = cg::this_cluster();
  const SelectStoredParams& S = P.s;
  const ShardHist& X = P.x;
  const int C = S.m.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = blockIdx.x / C;   // (batch row, query head)
  const int rows = gridDim.x / C;
  const int bq = row / S.m.hq_total, hq = row % S.m.hq_total;
  const int k = S.m.topk, cap = S.cap;
  const int G = X.world, me = X.rank;

  const size_t scratch_bytes = select_scratch_bytes(1, S.m.per, S.m.det_words);
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem + scratch_bytes);
  int* idxs = reinterpret_cast<int*>(keys + cap);
  int* cnt = idxs + cap;
  int* hist_all = cnt + 4;                   // [kHistBins] sum over the ranks
  int* hist_own = hist_all + kHistBins;      // [kHistBins] this rank
  int* hist_cta = hist_own + kHistBins;      // [kHistBins] this CTA's token range (read by the peers)
  SelCtrl* sc = reinterpret_cast<SelCtrl*>(hist_cta + kHistBins);
  ShardCtrl* hc = reinterpret_cast<ShardCtrl*>(sc + 1);

  const unsigned epoch = *X.epoch;
  const uint32_t* my_hist = X.hist_peer[me];      // this rank's receive buffer [round][rank][row][bin]
  const unsigned* my_flag = X.flag_peer[me];      // [round][rank][row]
  const int slice = kHistBins / C, b0 = crank * slice;
  auto slot_of = [&](int round, int r) { return ((size_t)(round * G + r) * rows + row) * kHistBins; };
  auto flag_of = [&](int round, int r) { return (size_t)(round * G + r) * rows + row; };

  // Publish this row's round: called by all threads of every CTA of the cluster after their stores
  // into the peers' slots.  One system-scope fence for the row, then its flag on every rank.
  auto publish_round = [&](int round) {
    cluster_barrier(cluster, C);   // every CTA's slice is stored (and nobody still reads hist_cta)
    if (crank == 0 && warp == 0) {
      __threadfence_system();   // one fence instruction for the warp, cumulative over the barrier
      if (lane < G) st_relaxed_sys(X.flag_peer[lane] + flag_of(round, me), epoch);
    }
  };
  // Wait for every rank's flag of this (round, row), then sum the ranks' histograms.
  auto gather_round = [&](int round) {
    if (tid < G) {
      const unsigned long long t0 = global_timer_ns();
      while ((int)(ld_acquire_sys(my_flag + flag_of(round, tid)) - epoch) < 0) {
        if (global_timer_ns() - t0 > X.limit_ns) {
          atomicOr(S.m.status, kStatusTimeout);
          break;
        }
      }
    }
    __syncthreads();
    for (int bin = tid; bin < kHistBins; bin += kSelThreads) {
      int s = 0, own = 0;
      for (int r = 0; r < G; ++r) {
        const int c = (int)__ldcg(my_hist + slot_of(round, r) + bin);
        s += c;
        if (r == me) own = c;
      }
      hist_all[bin] = s;
      hist_own[bin] = own;
    }
    __syncthreads();
  };

  RA_STAMP(S.m.status, 0);
  // ---- round 0: the coarse histograms counted by the scan
  {
    const uint32_t* hrow = S.hist_ws + (size_t)row * S.nparts * kHistBins;
    for (int bin = b0 + tid; bin < b0 + slice; bin += kSelThreads) {
      uint32_t s = 0;
      for (int p = 0; p < S.nparts; ++p) s += hrow[(size_t)p * kHistBins + bin];
      for (int r = 0; r < G; ++r) X.hist_peer[r][slot_of(0, me) + bin] = s;
    }
    if (tid == 0) {
      cnt[0] = 0;
      sc->bin = -1; sc->n_above = 0; sc->rem = k; sc->n_in = 0;
      sc->n_eq_local = 0;
      hc->own_above = 0;
    }
    publish_round(0);
    gather_round(0);
    find_coarse_bin(hist_all, k, sc, tid);
  }
  RA_STAMP(S.m.status, 1);
  const int lo = min(S.n_tokens, crank * S.chunk), hi = min(S.n_tokens, lo + S.chunk);
  const uint32_t* krow = S.keys_ws + (size_t)row * S.n_pad;

  uint32_t lo_key = 0u;
  int shift = 32, rem = k, n_in = 0, own_above = 0, own_in = 0, last_local = 0, last_bin = 0, last_round = 0;
  bool everything = sc->bin < 0;   // fewer than k keys on all ranks together: every key wins
  if (!everything) {
    const int bin = sc->bin;
    lo_key = (uint32_t)bin << kHistShift;
    shift = kHistShift;
    rem = sc->rem;
    n_in = sc->n_in;
    int part = 0;
    for (int b = bin + 1 + tid; b < kHistBins; b += kSelThreads) part += hist_own[b];
    own_above = block_sum(part, hc->red, tid);
    own_in = hist_own[bin];
    last_bin = bin;
  }

  // ---- further rounds: split the bin while it holds more keys than are wanted from it
  int round = 1;
  while (!everything && shift > 0 && n_in != rem) {
    const int new_shift = max(0, shift - 11);
    __syncthreads();
    for (int bin = tid; bin < kHistBins; bin += kSelThreads) hist_cta[bin] = 0;
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
          if (i + e < hi && rel < span) atomicAdd(&hist_cta[rel >> new_shift], 1);
        }
      }
    }
    cluster_barrier(cluster, C);
    for (int bin = b0 + tid; bin < b0 + slice; bin += kSelThreads) {
      int s = 0;
      for (int c = 0; c < C; ++c) s += cluster.map_shared_rank(hist_cta, c)[bin];
      for (int r = 0; r < G; ++r) X.hist_peer[r][slot_of(round, me) + bin] = (uint32_t)s;
    }
    publish_round(round);
    gather_round(round);
    if (tid == 0) sc->bin = -1;
    __syncthreads();
    find_coarse_bin(hist_all, rem, sc, tid);
    const int d = max(sc->bin, 0);
    rem = sc->rem;
    n_in = sc->n_in;
    int part = 0;
    for (int b = d + 1 + tid; b < kHistBins; b += kSelThreads) part += hist_own[b];
    own_above += block_sum(part, hc->red, tid);
    own_in = hist_own[d];
    last_local = hist_cta[d];
    last_bin = d;
    last_round = round;
    lo_key += (uint32_t)d << new_shift;
    shift = new_shift;
    ++round;
  }
  RA_STAMP(S.m.status, 2);

  // ---- this rank's winners: keys >= lo_key when the whole bin wins, else keys > lo_key and this
  // rank's share of the copies of lo_key (the ranks before it take theirs first)
  const bool whole_bin = everything || n_in == rem;
  int quota = own_in;
  if (!whole_bin) {
    int before = 0;
    for (int r = 0; r < me; ++r) before += (int)__ldcg(my_hist + slot_of(last_round, r) + last_bin);
    quota = max(0, min(own_in, rem - before));
  }
  const int own_total = everything ? min(S.n_tokens, k) : min(own_above + quota, k);
  const bool tie_mode = !whole_bin && own_above + own_in > cap;   // copies beyond the list's capacity
  int tie_take = 0;
  if (tie_mode) {
    if (tid == 0) sc->n_eq_local = last_local;
    cluster_barrier(cluster, C);
    int before = 0;
    for (int c = 0; c < crank; ++c) before += *cluster.map_shared_rank(&sc->n_eq_local, c);
    tie_take = max(0, min(last_local, quota - before));
  }
  if (!tie_mode)
    collect_candidates(krow, lo, hi, lo_key, keys, idxs, cnt, cap, S.m.status, tid, lane);
  else
    collect_candidates_ties(krow, lo, hi, lo_key, tie_take, keys, idxs, cnt, cap, sc, S.m.status, tid, warp, lane);
  __syncthreads();
  RA_STAMP(S.m.status, 3);

  // ---- winners dealt over the cluster's CTAs, their V rows mixed into this rank's partial
  MergeArgs A = S.m;
  A.list_off = 0;
  A.topk = own_total;
  A.deal_per = max(1, min(A.per, ceil_div(max(own_total, 1), C)));
  auto dest = [&](int) {
    ListDest d;
    d.valid = true;
    d.bq = bq;
    d.hq = hq;
    d.hkv = hq / S.group;
    return d;
  };
  // With the whole bin winning the threshold passed on is the key just below the bin (nothing in
  // the list equals it); with copies to share it is the k-th key itself and `quota` copies are taken.
  uint32_t thr = lo_key;
  int above = own_above;
  if (whole_bin) {
    if (lo_key > 0u) {
      thr = lo_key - 1u;
      above = own_total;
    } else {
      above = own_total - 0x40000000;   // every copy of key 0 wins as well
    }
  }
  cluster_select_attend<1>(cluster, smem, keys, idxs, cnt, cap, A, dest, lo, max(hi - lo, 1), thr, 0, above);

  // ---- the partial row goes to every rank (the cluster's CTAs each wrote some of its elements;
  // the cluster barrier that ends the common code ordered those stores)
  if (P.part.done != nullptr) {
    if (crank == 0) {
      const float* src = S.m.out_partial + (size_t)row * (kHeadDim + 2);
      for (int i = tid; i < (kHeadDim + 2) * P.part.npeers; i += kSelThreads) {
        const int peer = i / (kHeadDim + 2), j = i - peer * (kHeadDim + 2);
        float* dst = P.part.peer_rows[peer] + (size_t)row * (kHeadDim + 2);
        if (dst != src) dst[j] = __ldcg(src + j);
      }
    }
    exchange_publish_in_kernel(P.part);
  }
  RA_STAMP(S.m.status, 9);
}

size_t select_sharded_fixed_smem_bytes(int per, int det_words) {
  return select_scratch_bytes(1, per, det_words) + 16 + (size_t)3 * kHistBins * 4 + sizeof(SelCtrl) +
         sizeof(ShardCtrl) + 128;
}

cudaError_t launch_select_sharded(const SelectShardedParams& P, int rows, size_t smem, cudaStream_t stream) {
  auto kern = select_sharded_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * P.s.m.cluster), 1, 1);
  cfg.blockDim = dim3(kSelThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)P.s.m.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  note_launch();
  return cudaLaunchKernelEx(&cfg, kern, P);
}

}  // namespace ra
