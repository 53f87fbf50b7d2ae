// Sequence-sharded selection by exchanged histograms: every rank has scored its own shard
// (scan_store_kernel) and holds the score keys of its tokens; the ranks find the exact global k-th
// key together by a radix select whose histograms -- never the keys or candidates themselves --
// cross the links, and each rank then attends over the winners among its own tokens.
//
// One cluster of CTAs per (batch row, query head) on every rank, all ranks in step per row; CTA c
// owns a contiguous range of the shard's token axis:
//   round 0   the coarse histogram (top 11 bits, counted during the scan) of this rank goes to
//             every rank; the sum over ranks gives the bin of the global k-th key;
//   collect   the keys of this CTA's range at or above the lower edge of that bin go into a list
//             in shared memory, in ascending token order (when the bin and everything above it
//             are too many for a list the collection waits until the k-th key is known);
//   round 1+  while the bin holds more keys than are still wanted from it, it is split by its next
//             11 (then 10) bits: counts over the list, summed over the cluster through distributed
//             shared memory, exchanged and summed over the ranks.  Distinct scores end after
//             round 1; only copies or near-copies of the k-th score need round 2;
//   winners   keys above the k-th key win; of its copies each rank takes its share in rank order
//             (lower ranks hold lower token ids), inside a rank in token order.  Every CTA mixes
//             the V rows of its own winners, in token order, so that the same inputs always give
//             the same bits; the CTAs' sums are merged through their maxima into the rank's
//             un-normalised partial, which goes to every rank for the log-sum-exp combine.
//   combine   the cluster waits for the row's partials of all ranks and writes the final output
//             (the log-sum-exp merge of baseline_1.cu:549-598 across devices).
// Everything that crosses the links travels as 8-byte words, each carrying 32 bits of payload and
// the step's epoch as a tag, written with plain system-scope stores into the sender's slot of
// every rank's receive buffer.  A receiver polls the words themselves in its own memory until
// they carry the current epoch (an aligned 8-byte store arrives whole), so there are no separate
// flags and no fences; every wait is bounded in time (status bit on giving up).  Since all ranks
// see the same sums they take the same decisions and the same number of rounds.  The last CTA to
// finish adds one to the epoch word.
//
// The reference is single-device; the result is defined as equal to the single-device operator on
// the concatenated cache (retrieval_attn/test_ra.py:88-160 generalised to a global top-k).
#include "select_sharded.cuh"

namespace ra {

namespace {

struct ShardCtrl {
  int red[32];
  int wt[kSelUnroll][32];      // ordered collection: hits of every warp per segment of an iteration
  int wbase[kSelUnroll][32];
  int utot[kSelUnroll];
  int ftot[32];                // ordered prefix over list flags
  int n_eq_cta;                // copies of the k-th key in this CTA's list (read by the peers)
  int n_win;                   // winners of this CTA (read by the peers)
  uint32_t max_key;            // best winner of this CTA (read by the peers)
  float l_part;                // read by the peers
  float lred[32];
  float o_part[kHeadDim];      // read by the peers
  float red_o[32][kHeadDim];
};

__device__ __forceinline__ void st_tagged(unsigned long long* p, unsigned epoch, uint32_t payload) {
  const unsigned long long v = ((unsigned long long)epoch << 32) | payload;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// One look at a tagged word (several of these in a row are in flight together).
__device__ __forceinline__ unsigned long long ld_word(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p));
  return v;
}
// Payload of a tagged word once it carries `epoch`, given a first look `v` at it; polls on until it
// does and gives up after limit_ns (status bit, payload of whatever is there).
// `gave_up` (per thread; starts out as the sticky timeout bit left by earlier kernels) is set when
// a wait runs out, and nothing waits once it is set: a rank that lost its peers finishes in one
// time limit, not one per word.
__device__ __forceinline__ uint32_t await_tagged(unsigned long long v, const unsigned long long* p,
                                                 unsigned epoch, unsigned long long limit_ns,
                                                 unsigned* status, bool& gave_up) {
  if ((unsigned)(v >> 32) != epoch && !gave_up) {
    const unsigned long long t0 = global_timer_ns();
    do {
      v = ld_word(p);
      if (global_timer_ns() - t0 > limit_ns) {
        atomicOr(status, kStatusTimeout);
        gave_up = true;
        break;
      }
    } while ((unsigned)(v >> 32) != epoch);
  }
  return (uint32_t)v;
}
__device__ __forceinline__ uint32_t ld_tagged(const unsigned long long* p, unsigned epoch,
                                              unsigned long long limit_ns, unsigned* status, bool& gave_up) {
  return await_tagged(ld_word(p), p, epoch, limit_ns, status, gave_up);
}

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

// Exclusive prefix of a flag in thread order over the block, and the block's total.  Two barriers.
__device__ __forceinline__ int block_flag_prefix(bool flag, int* ftot, int tid, int& total) {
  const int lane = tid & 31, warp = tid >> 5;
  const unsigned bal = __ballot_sync(0xffffffffu, flag);
  __syncthreads();
  if (lane == 0) ftot[warp] = __popc(bal);
  __syncthreads();
  int before = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < 32; ++w) {
    const int c = ftot[w];
    before += w < warp ? c : 0;
    tot += c;
  }
  total = tot;
  return before + __popc(bal & ((1u << lane) - 1u));
}

// Keys of the token range [lo, hi) that are >= lo_key into the list, in ascending token order
// (`take` == nullptr), or -- when a single key value has more copies than a list can hold -- keys
// above lo_key and the first *take copies of lo_key.  Returns the list length to every thread.
__device__ __forceinline__ int ordered_collect(const uint32_t* krow, int lo, int hi, uint32_t lo_key,
                                               const int* take, uint32_t* keys, int* idxs, int cap,
                                               ShardCtrl* hc, unsigned* status, int tid) {
  const int lane = tid & 31, warp = tid >> 5;
  int count = 0;
  if (take == nullptr) {
    constexpr int U = kSelUnroll;
    // one iteration covers U segments of 4 * kSelThreads tokens; list order is (segment, thread, element)
    for (int base = lo; base < hi; base += kSelThreads * 4 * U) {   // same trip count for all threads
      uint4 kk[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + (u * kSelThreads + tid) * 4;
        kk[u] = i < hi ? ldg128_nc(krow + i) : make_uint4(0u, 0u, 0u, 0u);
      }
      // per-segment hit counts of this thread (at most 4 each), packed: 4 bits per segment in cpk,
      // and 8 bits per segment in two registers for the warp scans (a warp holds at most 128 hits
      // of one segment, so the packed fields never carry into each other)
      static_assert(U == 8, "two registers of four 8-bit fields");
      uint32_t cpk = 0u, lo4 = 0u, hi4 = 0u;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + (u * kSelThreads + tid) * 4;
        const uint32_t kv[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
        uint32_t c = 0u;
#pragma unroll
        for (int e = 0; e < 4; ++e) c += (i + e < hi && kv[e] >= lo_key);
        cpk |= c << (4 * u);
        if (u < 4) lo4 |= c << (8 * u); else hi4 |= c << (8 * (u - 4));
      }
      if (__ballot_sync(0xffffffffu, cpk != 0u)) {
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const uint32_t a = __shfl_up_sync(0xffffffffu, lo4, off);
          const uint32_t b = __shfl_up_sync(0xffffffffu, hi4, off);
          if (lane >= off) {
            lo4 += a;
            hi4 += b;
          }
        }
      }
      auto incl_of = [&](int u) { return (int)(((u < 4 ? lo4 : hi4) >> (8 * (u & 3))) & 255u); };
      if (lane == 31) {
#pragma unroll
        for (int u = 0; u < U; ++u) hc->wt[u][warp] = incl_of(u);
      }
      __syncthreads();
      if (warp < U) {
        const int v = hc->wt[warp][lane];
        int inc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int n = __shfl_up_sync(0xffffffffu, inc, off);
          if (lane >= off) inc += n;
        }
        hc->wbase[warp][lane] = inc - v;
        if (lane == 31) hc->utot[warp] = inc;
      }
      __syncthreads();
      int ubase = count;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = (int)((cpk >> (4 * u)) & 15u);
        if (c) {
          int pos = ubase + hc->wbase[u][warp] + incl_of(u) - c;
          const int i = base + (u * kSelThreads + tid) * 4;
          const uint32_t kv[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (i + e < hi && kv[e] >= lo_key) {
              if (pos < cap) {
                keys[pos] = kv[e];
                idxs[pos] = i + e;
              } else {
                atomicOr(status, kStatusOverflow);
              }
              ++pos;
            }
          }
        }
        ubase += hc->utot[u];
      }
      count = ubase;
      __syncthreads();   // the totals are read before the next iteration overwrites them
    }
  } else {
    const int tie_take = *take;
    int tie_base = 0;   // copies of lo_key seen so far in this CTA
    for (int base = lo; base < hi; base += kSelThreads * 4) {   // thread order is token order
      const int i = base + tid * 4;
      uint4 kk = make_uint4(0u, 0u, 0u, 0u);
      if (i < hi) kk = ldg128_nc(krow + i);
      const uint32_t kv[4] = {kk.x, kk.y, kk.z, kk.w};
      bool pass[4];
      // copies of lo_key: per-thread count, ordered prefix over threads
      int mine_eq = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) mine_eq += (i + e < hi && kv[e] == lo_key);
      int incl = mine_eq;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
      }
      __syncthreads();
      if (lane == 31) hc->ftot[warp] = incl;
      __syncthreads();
      int wb = 0, tot = 0;
#pragma unroll
      for (int w = 0; w < 32; ++w) {
        const int cw = hc->ftot[w];
        wb += w < warp ? cw : 0;
        tot += cw;
      }
      int o = tie_base + wb + incl - mine_eq;
      int mine_pass = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pass[e] = i + e < hi && kv[e] > lo_key;
        if (i + e < hi && kv[e] == lo_key) {
          pass[e] = o < tie_take;
          ++o;
        }
        mine_pass += pass[e];
      }
      tie_base += tot;
      // positions of the passing keys: the same ordered prefix
      int pincl = mine_pass;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, pincl, off);
        if (lane >= off) pincl += n;
      }
      __syncthreads();
      if (lane == 31) hc->ftot[warp] = pincl;
      __syncthreads();
      int pb = 0, ptot = 0;
#pragma unroll
      for (int w = 0; w < 32; ++w) {
        const int cw = hc->ftot[w];
        pb += w < warp ? cw : 0;
        ptot += cw;
      }
      int p = count + pb + pincl - mine_pass;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (pass[e]) {
          if (p < cap) {
            keys[p] = kv[e];
            idxs[p] = i + e;
          } else {
            atomicOr(status, kStatusOverflow);
          }
          ++p;
        }
      }
      count += ptot;
    }
  }
  __syncthreads();
  return min(count, cap);
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
  const MergeArgs& A = S.m;
  const int C = A.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = blockIdx.x / C;   // (batch row, query head)
  const int rows = gridDim.x / C;
  const int bq = row / A.hq_total, hq = row % A.hq_total, hkv = hq / S.group;
  const int k = A.topk, cap = S.cap;
  const int G = X.world, me = X.rank;

  uint32_t* keys = reinterpret_cast<uint32_t*>(smem);
  int* idxs = reinterpret_cast<int*>(keys + cap);
  int* hist_all = idxs + cap;                // [kHistBins] sum over the ranks
  int* hist_own = hist_all + kHistBins;      // [kHistBins] this rank
  int* hist_cta = hist_own + kHistBins;      // [kHistBins] this CTA's token range (read by the peers)
  SelCtrl* sc = reinterpret_cast<SelCtrl*>(hist_cta + kHistBins);
  ShardCtrl* hc = reinterpret_cast<ShardCtrl*>(sc + 1);

  const unsigned epoch = *X.epoch;
  bool gave_up = (*A.status & kStatusTimeout) != 0;   // an earlier kernel's wait ran out: do not wait
  // this rank's receive buffer: histograms [round][rank][row][bin], then partials [rank][row][132]
  const unsigned long long* my_buf = X.buf_peer[me];
  const int slice = kHistBins / C, b0 = crank * slice;
  auto slot_of = [&](int round, int r) { return ((size_t)(round * G + r) * rows + row) * kHistBins; };
  const size_t part_base = (size_t)kShardRounds * G * rows * kHistBins;
  auto part_of = [&](int r) { return part_base + ((size_t)r * rows + row) * kPartWords; };

  // Every rank's histogram of this (round, row), summed; each word is polled until it has arrived.
  auto gather_round = [&](int round) {
    // a thread's words of up to 4 ranks x 2 bins are looked at together (one round trip), then
    // the ones that have not arrived yet are polled
    constexpr int NB = kHistBins / kSelThreads, RC = 4;
    int s[NB], own[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) s[j] = own[j] = 0;
    for (int r0 = 0; r0 < G; r0 += RC) {
      unsigned long long v[RC][NB];
#pragma unroll
      for (int i = 0; i < RC; ++i)
#pragma unroll
        for (int j = 0; j < NB; ++j)
          if (r0 + i < G) v[i][j] = ld_word(my_buf + slot_of(round, r0 + i) + tid + j * kSelThreads);
#pragma unroll
      for (int i = 0; i < RC; ++i)
#pragma unroll
        for (int j = 0; j < NB; ++j)
          if (r0 + i < G) {
            const int c = (int)await_tagged(v[i][j], my_buf + slot_of(round, r0 + i) + tid + j * kSelThreads,
                                            epoch, X.limit_ns, A.status, gave_up);
            s[j] += c;
            if (r0 + i == me) own[j] = c;
          }
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      hist_all[tid + j * kSelThreads] = s[j];
      hist_own[tid + j * kSelThreads] = own[j];
    }
    __syncthreads();
  };

  RA_STAMP(A.status, 0);
  // ---- round 0: the coarse histograms counted by the scan
  {
    const uint32_t* hrow = S.hist_ws + (size_t)row * S.nparts * kHistBins;
    for (int bin = b0 + tid; bin < b0 + slice; bin += kSelThreads) {
      uint32_t s = 0;
      for (int p = 0; p < S.nparts; ++p) s += hrow[(size_t)p * kHistBins + bin];
      for (int r = 0; r < G; ++r) st_tagged(X.buf_peer[r] + slot_of(0, me) + bin, epoch, s);
    }
    if (tid == 0) {
      sc->bin = -1; sc->n_above = 0; sc->rem = k; sc->n_in = 0;
      hc->n_eq_cta = 0;
    }
    __syncthreads();
    gather_round(0);
    find_coarse_bin(hist_all, k, sc, tid);
  }
  RA_STAMP(A.status, 1);
  const int lo = min(S.n_tokens, crank * S.chunk), hi = min(S.n_tokens, lo + S.chunk);
  const uint32_t* krow = S.keys_ws + (size_t)row * S.n_pad;

  uint32_t lo_key = 0u;
  int shift = 32, rem = k, n_in = 0, own_in = 0, last_bin = 0, last_round = 0;
  const bool everything = sc->bin < 0;   // fewer than k keys on all ranks together: every key wins
  bool listed = everything;              // the list is filled before the further rounds
  if (!everything) {
    const int bin = sc->bin;
    lo_key = (uint32_t)bin << kHistShift;
    shift = kHistShift;
    rem = sc->rem;
    n_in = sc->n_in;
    own_in = hist_own[bin];
    last_bin = bin;
    // all candidates of the row fit in any one list: collect now, split the bin over the list
    listed = sc->n_above + n_in <= cap;
  }
  int n_list = 0;
  if (listed) n_list = ordered_collect(krow, lo, hi, lo_key, nullptr, keys, idxs, cap, hc, A.status, tid);
  RA_STAMP(A.status, 2);

  // ---- further rounds: split the bin while it holds more keys than are wanted from it
  int round = 1;
  while (!everything && shift > 0 && n_in != rem) {
    const int new_shift = max(0, shift - 11);
    if (round > 1) cluster_barrier(cluster, C);   // nobody still reads this CTA's counts of the last round
    __syncthreads();
    for (int bin = tid; bin < kHistBins; bin += kSelThreads) hist_cta[bin] = 0;
    __syncthreads();
    const uint32_t span = 1u << shift;
    if (listed) {
      for (int e = tid; e < n_list; e += kSelThreads) {
        const uint32_t rel = keys[e] - lo_key;
        if (rel < span) atomicAdd(&hist_cta[rel >> new_shift], 1);
      }
    } else {
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
    }
    cluster_barrier(cluster, C);
    for (int bin = b0 + tid; bin < b0 + slice; bin += kSelThreads) {
      int s = 0;
      for (int c = 0; c < C; ++c) s += cluster.map_shared_rank(hist_cta, c)[bin];
      for (int r = 0; r < G; ++r) st_tagged(X.buf_peer[r] + slot_of(round, me) + bin, epoch, (uint32_t)s);
    }
    gather_round(round);
    if (tid == 0) sc->bin = -1;
    __syncthreads();
    find_coarse_bin(hist_all, rem, sc, tid);
    const int d = max(sc->bin, 0);
    rem = sc->rem;
    n_in = sc->n_in;
    own_in = hist_own[d];
    last_bin = d;
    last_round = round;
    lo_key += (uint32_t)d << new_shift;
    shift = new_shift;
    ++round;
  }
  RA_STAMP(A.status, 3);

  // ---- this rank's winners: keys >= lo_key when the whole bin wins, else keys > lo_key and this
  // rank's share of the copies of lo_key (the ranks before it take theirs first)
  const bool whole_bin = everything || n_in == rem;
  int quota = own_in;
  if (!whole_bin) {
    int before = 0;
    for (int r = 0; r < me; ++r) before += (int)ld_tagged(my_buf + slot_of(last_round, r) + last_bin, epoch, X.limit_ns, A.status, gave_up);
    quota = max(0, min(own_in, rem - before));
  }
  // this CTA's share of the rank's copies, in CTA (= token) order
  int cta_take = 0x7fffffff;
  if (!whole_bin && quota < own_in) {
    int cta_eq;
    if (listed) {
      int mine = 0;
      for (int e = tid; e < n_list; e += kSelThreads) mine += keys[e] == lo_key;
      cta_eq = block_sum(mine, hc->red, tid);
    } else {
      cta_eq = hist_cta[last_bin];   // the last round counted the single values of this CTA's range
    }
    if (tid == 0) hc->n_eq_cta = cta_eq;
    cluster_barrier(cluster, C);
    int before = 0;
    for (int c = 0; c < crank; ++c) before += *cluster.map_shared_rank(&hc->n_eq_cta, c);
    cta_take = max(0, min(cta_eq, quota - before));
  }
  if (!listed)
    n_list = ordered_collect(krow, lo, hi, lo_key, (whole_bin || cta_take == 0x7fffffff) ? nullptr : &cta_take,
                             keys, idxs, cap, hc, A.status, tid);

  // ---- winners compacted to the front of the list, still in token order
  int n_win = 0;
  uint32_t best = 0u;
  {
    int eq_seen = 0;
    for (int base = 0; base < n_list; base += kSelThreads) {   // same trip count for all threads
      const int e = base + tid;
      const uint32_t key = e < n_list ? keys[e] : 0u;
      const int id = e < n_list ? idxs[e] : 0;
      bool win = e < n_list && (whole_bin ? key >= lo_key : key > lo_key);
      if (!whole_bin && cta_take > 0) {
        const bool eq = e < n_list && key == lo_key;
        int eq_tot;
        const int ord = eq_seen + block_flag_prefix(eq, hc->ftot, tid, eq_tot);
        if (eq && ord < cta_take) win = true;
        eq_seen += eq_tot;
      }
      int tot;
      const int pos = n_win + block_flag_prefix(win, hc->ftot, tid, tot);
      // every thread holds its entry in registers: positions at or below the ones just read are free
      if (win) {
        keys[pos] = key;
        idxs[pos] = id;
        best = max(best, key);
      }
      n_win += tot;
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, off));
    __syncthreads();
    if (lane == 0) hc->red[warp] = (int)best;
    __syncthreads();
    best = (uint32_t)hc->red[lane];
#pragma unroll
    for (int off = 16; off; off >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, off));
  }
  RA_STAMP(A.status, 4);

  // ---- V rows of this CTA's winners mixed by half-warps, weights against the CTA's best score
  {
    const float smax = key_score(best);
    const __half* vb = A.v + (size_t)bq * A.v_batch_stride + (size_t)hkv * A.v_head_stride + (lane & 15) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    float lsum = 0.f;
    constexpr int UN = 4, NW = kSelThreads / 32;
    for (int e0 = warp * 2 + (lane >> 4); e0 < n_win; e0 += 2 * NW * UN) {
      uint4 vv[UN];
      float w[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int e = e0 + 2 * NW * u;
        const int id = (e < n_win) ? idxs[e] : -1;
        if (e < n_win && (unsigned)id >= (unsigned)A.n_tokens) atomicOr(A.status, kStatusBadId);
        if ((unsigned)id < (unsigned)A.n_tokens) {
          w[u] = fast_exp2((key_score(keys[e]) - smax) * A.scale_log2e);
          vv[u] = ldg128_nc(vb + (size_t)id * A.v_token_stride);
        } else {
          w[u] = 0.f;
          vv[u] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const uint32_t ww[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = h2f2(ww[i]);
          acc[2 * i] = fmaf(w[u], f.x, acc[2 * i]);
          acc[2 * i + 1] = fmaf(w[u], f.y, acc[2 * i + 1]);
        }
        lsum += w[u];
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 16);
    if (lane < 16) {
#pragma unroll
      for (int i = 0; i < 8; ++i) hc->red_o[warp][lane * 8 + i] = acc[i];
    }
    if (lane == 0) hc->lred[warp] = lsum;
    __syncthreads();
    if (tid < kHeadDim) {
      float o = 0.f;
      for (int w = 0; w < NW; ++w) o += hc->red_o[w][tid];
      hc->o_part[tid] = o;
      if (tid == 0) {
        float ls = 0.f;
        for (int w = 0; w < NW; ++w) ls += hc->lred[w];
        hc->l_part = ls;
        hc->max_key = best;
        hc->n_win = n_win;
      }
    }
  }
  RA_STAMP(A.status, 5);
  cluster_barrier(cluster, C);

  // ---- the CTAs' sums merged through their maxima: CTA c finishes the dimensions d % C == c and
  // sends them to every rank
  {
    uint32_t mk = 0u;
    int total_win = 0, win_before = 0;
    for (int c = 0; c < C; ++c) {
      const int nw = *cluster.map_shared_rank(&hc->n_win, c);
      if (nw > 0) mk = max(mk, *cluster.map_shared_rank(&hc->max_key, c));
      win_before += c < crank ? nw : 0;
      total_win += nw;
    }
    const float smax = key_score(mk);
    if (tid < kHeadDim && tid % C == crank) {
      float o = 0.f, lt = 0.f;
      for (int c = 0; c < C; ++c) {
        if (*cluster.map_shared_rank(&hc->n_win, c) == 0) continue;
        const float wc = fast_exp2((key_score(*cluster.map_shared_rank(&hc->max_key, c)) - smax) * A.scale_log2e);
        o = fmaf(wc, cluster.map_shared_rank(&hc->o_part[0], c)[tid], o);
        lt = fmaf(wc, *cluster.map_shared_rank(&hc->l_part, c), lt);
      }
      // a rank without winners for this row weighs nothing in the combine
      const float mscaled = total_win > 0 ? smax * A.sm_scale : -INFINITY;
      for (int r = 0; r < G; ++r) {
        unsigned long long* dst = X.buf_peer[r] + part_of(me);
        st_tagged(dst + tid, epoch, __float_as_uint(o));
        if (tid == 0) {
          st_tagged(dst + kHeadDim, epoch, __float_as_uint(lt));
          st_tagged(dst + kHeadDim + 1, epoch, __float_as_uint(mscaled));
        }
      }
    }
    if (A.sel_idx) {
      const size_t dst = (size_t)row * A.list_pitch + win_before;
      for (int e = tid; e < n_win; e += kSelThreads) {
        if (win_before + e < A.list_pitch) {
          A.sel_idx[dst + e] = idxs[e] + A.index_base;
          if (A.sel_score) A.sel_score[dst + e] = key_score(keys[e]);
        }
      }
    }
  }
  RA_STAMP(A.status, 6);

  // ---- combine: out = sum_r w_r o_r / sum_r w_r l_r with w_r = exp(m_r - max m) over the ranks'
  // partials of this row, in rank order (the same bits on every rank).  Every thread fetches its
  // share of the words into shared memory (the candidate list is no longer needed), all at once.
  {
    __syncthreads();   // the list has been written out if it was asked for
    float* prow = reinterpret_cast<float*>(keys);   // [G][kPartWords]
    const int nwords = G * kPartWords;
    for (int w0 = tid; w0 < nwords; w0 += kSelThreads * 4) {
      unsigned long long v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int w = w0 + i * kSelThreads;
        if (w < nwords) v[i] = ld_word(my_buf + part_base + ((size_t)(w / kPartWords) * rows + row) * kPartWords + w % kPartWords);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int w = w0 + i * kSelThreads;
        if (w < nwords && w % kPartWords < kHeadDim + 2)
          prow[w] = __uint_as_float(await_tagged(
              v[i], my_buf + part_base + ((size_t)(w / kPartWords) * rows + row) * kPartWords + w % kPartWords, epoch,
              X.limit_ns, A.status, gave_up));
      }
    }
    __syncthreads();
    if (tid < kHeadDim && tid % C == crank) {
      float m = -INFINITY;
      for (int r = 0; r < G; ++r) m = fmaxf(m, prow[r * kPartWords + kHeadDim + 1]);
      float o = 0.f, l = 0.f;
      for (int r = 0; r < G; ++r) {
        const float lp = prow[r * kPartWords + kHeadDim];
        const float w = (lp > 0.f) ? __expf(prow[r * kPartWords + kHeadDim + 1] - m) : 0.f;
        o = fmaf(w, prow[r * kPartWords + tid], o);
        l = fmaf(w, lp, l);
      }
      A.out[(size_t)row * kHeadDim + tid] = __float2half_rn(o / l);
    }
  }
  cluster_barrier(cluster, C);  // nobody leaves while a peer may still read its shared memory

  // ---- the step ends: the last CTA to finish advances the epoch (every CTA read it long ago)
  if (tid == 0) {
    if (atomicAdd(X.done, 1u) == gridDim.x - 1) {
      *X.done = 0u;
      *X.epoch_rw = epoch + 1u;
    }
  }
  RA_STAMP(A.status, 7);
}

size_t select_sharded_fixed_smem_bytes() {
  return (size_t)3 * kHistBins * 4 + sizeof(SelCtrl) + sizeof(ShardCtrl) + 256;
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
