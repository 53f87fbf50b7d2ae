// Cluster-wide exact k-select over per-CTA candidate lists held in shared memory, followed by
// either writing the winners out or softmax.V over them.  Shared by the scan kernel (lists
// filled while streaming K) and the merge kernel (lists loaded from global candidate buffers).
//
// All CTAs of the cluster run the same code.  Histograms, counts, winners and partial outputs
// cross CTAs through distributed shared memory between hardware cluster barriers; there are no
// polled flags (the reference hands scores to a consumer CTA that spins on a counter,
// retrieval_attn/retrieval_attention.cu:381-394, and reduces max/sum with 2(C-1) cluster
// barriers, baseline_1.cu:549-588).
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace ra {

namespace cg = cooperative_groups;

constexpr int kMaxDetWords = 8192;       // most bitmap words of one window of the ordered deal
constexpr int kTagByPosition = 0x7fffffff;   // tag_lo value: a candidate's tag is its list position

struct MergeScratch {
  int hist[2][kMaxLists][256];
  int ghist[kMaxLists][256];
  uint32_t prefix[kMaxLists];
  int remaining[kMaxLists];
  uint32_t counts[kMaxLists][4];  // n_gt, n_eq, best key — read by the other CTAs
  int off_win[kMaxLists], take_eq[kMaxLists], total_sel[kMaxLists];
  uint32_t maxkey[kMaxLists];
  // ordered deal: warp totals of the block scan and the tag up to which copies of the k-th key are
  // taken (the bitmap itself -- one bit per candidate tag of the current window and an exclusive
  // popcount prefix per word -- follows the dealt winners, MergeArgs::det_words words of each)
  int wsum[kMaxWarps + 2];
  int cut_tag, cut_found;
  float red[kMaxWarps][kHeadDim];
  float lred[kMaxWarps];
  float o_part[kMaxLists][kHeadDim];  // read by the other CTAs
  float l_part[kMaxLists];            // read by the other CTAs
};

// Shared memory the cluster code needs in every CTA: its scratch block, the dealt winners of nl
// lists (per = ceil(topk / cluster) slots each) and the bitmap window of the ordered deal.
__host__ __device__ inline size_t select_scratch_bytes(int nl, int per, int det_words) {
  return ((sizeof(MergeScratch) + (size_t)nl * per * 8 + 127) & ~size_t(127)) + (size_t)det_words * 8;
}
// Bitmap words that cover `range` candidate tags in one window (fewer words: several windows).
__host__ __device__ inline int det_words_for(int range) {
  const int w = (range + 31) / 32;
  return w < 32 ? 32 : (w > kMaxDetWords ? kMaxDetWords : ((w + 31) & ~31));
}

enum OutMode : int {
  kOutNone = 0,     // only the winner lists are written
  kOutFinal = 1,    // normalised fp16 output
  kOutPartial = 2,  // un-normalised fp32 sum, its weight, and the common maximum
};

struct MergeArgs {
  int topk;        // winners per list
  int per;         // ceil(topk / cluster): winner slots per CTA (shared-memory layout)
  int deal_per;    // winners dealt to each CTA in turn; 0 = per.  Smaller when a caller lowers topk
                   // for one row at run time and wants its fewer winners spread over all CTAs.
  int cluster;
  int out_mode;
  int hq_total;    // query heads (row pitch of the outputs)
  int list_pitch;  // winners slots per (batch row, head) in sel_idx/sel_score
  int list_off;    // offset of this cluster's winners inside that pitch
  int index_base;
  int own_lo, own_hi;  // only winners with own_lo <= id < own_hi are mixed (id before index_base)
  int id_shift;        // subtracted from an id to address V (ids of another shard's frame)
  int det_words;       // bitmap words of the ordered deal's window (0 with select_all + local_deal)
  int per_cta_select;  // 1: every CTA keeps the topk best of its own list (per == topk); the cluster
                       // only shares the maximum and merges the attention over all CTAs' winners
  int select_all;      // 1: every candidate is a winner (topk == number of candidates)
  int local_deal;      // with select_all: CTA c already holds winners c*per .. c*per+cnt-1, keep them
  int expand_clen;     // > 0 with expand_out: winners are cluster ids, written out expanded
  int* expand_out;     // [B,Hq,topk*expand_clen] member tokens id*clen+i, clusters in rank order
  int* expand_ids;     // optional [B,Hq,topk]: the winners themselves in rank order
  int n_tokens;        // rows of V; ids outside [0, n_tokens) after the shift are never read
  unsigned* status;    // device status word (bit kStatusBadId is set on such an id)
  int* sel_idx;        // optional
  float* sel_score;    // optional
  const __half* v;
  long long v_batch_stride, v_token_stride, v_head_stride;
  __half* out;          // kOutFinal
  float* out_lse;       // optional (max*scale, sum)
  float* out_partial;   // kOutPartial: [B,Hq,130] = 128 sums, weight, max*scale
  float scale_log2e, sm_scale;
};

// Visit keys[0..n) with all threads of the CTA, eight independent loads in flight per thread (the
// lists may live in global memory, where one load at a time would cost a full L2 round trip each).
template <typename F>
__device__ __forceinline__ void for_each_key(const uint32_t* keys, int n, int tid, int nthr, F f) {
  for (int base = 0; base < n; base += nthr * 8) {
    uint32_t kk[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int i = base + e * nthr + tid;
      kk[e] = (i < n) ? keys[i] : 0u;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int i = base + e * nthr + tid;
      if (i < n) f(kk[e], i);
    }
  }
}

// Barrier over the cluster; a cluster of one CTA needs only the CTA barrier.
__device__ __forceinline__ void cluster_barrier(cg::cluster_group& cluster, int C) {
  if (C > 1) cluster.sync(); else __syncthreads();
}

// One list's destination: batch row, query head, kv head, and whether it is in use.
struct ListDest {
  int bq, hq, hkv;
  bool valid;
};

// Among 256 bins find the one holding the `remaining`-th largest element (bins ordered by
// digit, larger digit = larger key).  Executed by one full warp.  If the bins hold fewer than
// `remaining` elements bin 0 is returned.  new_remaining = 1-based rank inside that bin.
__device__ __forceinline__ void warp_find_digit(const int* hist, int remaining, int lane,
                                                int& digit, int& new_remaining) {
  int c[8];
  int s = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    c[i] = hist[255 - 8 * lane - i];
    s += c[i];
  }
  int incl = s;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  const int excl = incl - s;
  const bool cross = (excl < remaining) && (remaining <= incl);
  const unsigned bal = __ballot_sync(0xffffffffu, cross);
  const int src = bal ? (__ffs(bal) - 1) : 31;
  int d = 0, nr = 1;
  if (lane == src) {
    int run = excl;
    bool found = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (!found && run + c[i] >= remaining) {
        d = 255 - 8 * lane - i;
        nr = remaining - run;
        found = true;
      }
      if (!found) run += c[i];
    }
    if (!found) {  // fewer elements than asked for: everything is kept
      d = 0;
      nr = max(1, remaining - (run - c[7]));
    }
  }
  digit = __shfl_sync(0xffffffffu, d, src);
  new_remaining = __shfl_sync(0xffffffffu, nr, src);
}

// Exclusive prefix of the popcounts of bits[0..nw) into wpre[0..nw); returns their total.  Called
// by all nthr threads of the CTA (nthr a multiple of 32); wsum holds kMaxWarps + 2 ints.  Ends
// with the CTA synchronised.
__device__ __forceinline__ int bitmap_prefix(const uint32_t* bits, int* wpre, int* wsum, int nw,
                                             int tid, int nthr) {
  const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
  const int wpt = (nw + nthr - 1) / nthr;
  const int w0 = min(nw, tid * wpt), w1 = min(nw, w0 + wpt);
  int s = 0;
  for (int w = w0; w < w1; ++w) s += __popc(bits[w]);
  int incl = s;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int v = lane < nwarps ? wsum[lane] : 0;
    int inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += n;
    }
    wsum[lane] = inc - v;
    if (lane == 31) wsum[kMaxWarps] = inc;
  }
  __syncthreads();
  int run = wsum[warp] + incl - s;
  for (int w = w0; w < w1; ++w) {
    wpre[w] = run;
    run += __popc(bits[w]);
  }
  const int total = wsum[kMaxWarps];
  __syncthreads();
  return total;
}

// keys/idxs: NL lists of capacity `cap` in this CTA's shared memory with cnt[l] entries each.
// scratch: shared memory of at least sizeof(MergeScratch) + NL*per*8 bytes, at the same
// offset in every CTA of the cluster.  dest(l) gives the ListDest of list l.
//
// The winners are dealt in a fixed order, so that the same candidates always give the same lists and
// the same output bits: every candidate has a tag that is unique inside its CTA and lies in
// [0, tag_range) -- its id minus tag_lo (CTA c of a cluster holds an ascending range of ids), or
// its position in the list when tag_lo == kTagByPosition.  Winners are ordered by (CTA rank,
// tag); among copies of the k-th key the first ones in that order are taken.
//
// A caller that already knows that the k-th key lies in [sel_base, sel_base + 2^sel_shift) and that
// sel_above candidates of the whole cluster lie above that interval passes the three values: the
// radix select then only counts the keys inside the interval (fewer passes, well spread bins).
template <int NL, typename DestFn>
__device__ void cluster_select_attend(cg::cluster_group& cluster, unsigned char* scratch,
                                      const uint32_t* keys, const int* idxs, const int* cnt,
                                      int cap, const MergeArgs& A, DestFn dest,
                                      int tag_lo = kTagByPosition, int tag_range = 0,
                                      uint32_t sel_base = 0u, int sel_shift = 32, int sel_above = 0) {
  MergeScratch* ms = reinterpret_cast<MergeScratch*>(scratch);
  const int per = A.per, k = A.topk, C = A.cluster;
  const int dper = A.deal_per > 0 ? A.deal_per : per;
  uint32_t* sel_key = reinterpret_cast<uint32_t*>(scratch + sizeof(MergeScratch));
  int* sel_idx = reinterpret_cast<int*>(sel_key + (size_t)NL * per);
  uint32_t* det_bits = reinterpret_cast<uint32_t*>(scratch + select_scratch_bytes(NL, per, 0));
  int* det_pre = reinterpret_cast<int*>(det_bits + A.det_words);
  const int det_window = A.det_words * 32;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nthr = blockDim.x, nwarps = nthr >> 5;
  const int crank = (int)cluster.block_rank();

  RA_STAMP(A.status, 3);
  for (int i = tid; i < 2 * kMaxLists * 256; i += nthr) (&ms->hist[0][0][0])[i] = 0;
  // winner slots start out empty; a slot nobody fills is skipped by the mixing loop
  for (int i = tid; i < NL * per; i += nthr) sel_idx[i] = -1;
  if (tid < kMaxLists) {
    ms->prefix[tid] = 0u;
    ms->remaining[tid] = k - sel_above;
    ms->counts[tid][0] = 0u;
    ms->counts[tid][1] = 0u;
    ms->counts[tid][2] = 0u;
  }
  __syncthreads();

  // radix select inside [sel_base, sel_base + 2^sel_shift), most significant digit first, up to 8
  // bits per pass; one cluster barrier per pass.  `prefix` holds the digits found so far of
  // (k-th key - sel_base), `mask` the bits they cover (and the bits above the interval, which are
  // zero for every key inside it).
  int buf = 0;
  if (A.select_all) {
    if (tid < kMaxLists) ms->remaining[tid] = 0;  // threshold key 0: everything is above it
    __syncthreads();
  }
  int cur = A.select_all ? 0 : sel_shift;
  uint32_t mask = cur >= 32 ? 0u : ~((1u << cur) - 1u);
#pragma unroll 1
  while (cur > 0) {
    const int ns = max(0, cur - 8);
    const uint32_t dmask = (1u << (cur - ns)) - 1u;
#pragma unroll
    for (int l = 0; l < NL; ++l) {
      const int n = min(cnt[l], cap);
      const uint32_t pre = ms->prefix[l];
      const uint32_t* kl = keys + (size_t)l * cap;
      for_each_key(kl, n, tid, nthr, [&](uint32_t key, int) {
        const uint32_t rel = key - sel_base;
        if (key >= sel_base && (rel & mask) == pre) atomicAdd(&ms->hist[buf][l][(rel >> ns) & dmask], 1);
      });
    }
    if (A.per_cta_select) __syncthreads(); else cluster_barrier(cluster, C);
    for (int item = tid; item < NL * 256; item += nthr) {
      const int l = item >> 8, bin = item & 255;
      int sum = 0;
      if (A.per_cta_select) {
        sum = ms->hist[buf][l][bin];
      } else {
        for (int c = 0; c < C; ++c) {
          const int* rh = cluster.map_shared_rank(&ms->hist[buf][l][0], c);
          sum += rh[bin];
        }
      }
      ms->ghist[l][bin] = sum;
      ms->hist[buf ^ 1][l][bin] = 0;  // peers finished reading it before the barrier above
    }
    __syncthreads();
    for (int l = warp; l < NL; l += nwarps) {
      int d, nr;
      warp_find_digit(ms->ghist[l], ms->remaining[l], lane, d, nr);
      if (lane == 0) {
        ms->prefix[l] |= (uint32_t)d << ns;
        ms->remaining[l] = nr;
      }
    }
    __syncthreads();
    mask = ns > 0 ? ~((1u << ns) - 1u) : 0xffffffffu;
    cur = ns;
    buf ^= 1;
  }
  if (tid < kMaxLists) ms->prefix[tid] += sel_base;   // from here on: the k-th key itself
  __syncthreads();

  RA_STAMP(A.status, 4);
  // my candidates above / equal to the k-th key, and my best key
#pragma unroll
  for (int l = 0; l < NL; ++l) {
    const int n = min(cnt[l], cap);
    const uint32_t kth = ms->prefix[l];
    const uint32_t* kl = keys + (size_t)l * cap;
    int ngt = 0, neq = 0;
    uint32_t mx = 0u;
    for_each_key(kl, n, tid, nthr, [&](uint32_t key, int) {
      ngt += key > kth;
      neq += key == kth;
      mx = max(mx, key);
    });
#pragma unroll
    for (int off = 16; off; off >>= 1) {
      ngt += __shfl_xor_sync(0xffffffffu, ngt, off);
      neq += __shfl_xor_sync(0xffffffffu, neq, off);
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    if (lane == 0) {
      atomicAdd(&ms->counts[l][0], (uint32_t)ngt);
      atomicAdd(&ms->counts[l][1], (uint32_t)neq);
      atomicMax(&ms->counts[l][2], mx);
    }
  }
  cluster_barrier(cluster, C);
  if (tid < NL) {
    const int l = tid;
    const int need_eq = ms->remaining[l];
    // copies of the k-th key are taken in CTA order; winners of CTA c start at the sum of the
    // winners of the CTAs before it
    int total = 0, eq_before = 0, my_take = 0, off_win = 0;
    uint32_t mx = 0u;
    for (int c = 0; c < C; ++c) {
      const uint32_t* rc = cluster.map_shared_rank(&ms->counts[l][0], c);
      const int g = (int)rc[0], e = (int)rc[1];
      mx = max(mx, rc[2]);
      if (A.per_cta_select) {
        // own selection: only the maximum is common
        if (c == crank) {
          my_take = max(0, min(e, need_eq));
          total = g + my_take;
        }
        continue;
      }
      const int take = max(0, min(e, need_eq - eq_before));
      if (c < crank) off_win += g + take;
      if (c == crank) my_take = take;
      total += g + take;
      eq_before += e;
    }
    ms->off_win[l] = off_win;
    ms->take_eq[l] = my_take;
    ms->total_sel[l] = min(k, total);
    ms->maxkey[l] = mx;
  }
  __syncthreads();
  RA_STAMP(A.status, 5);
  if (A.select_all && A.local_deal) {
    // nothing to deal: the lists were filled evenly and every entry wins
#pragma unroll
    for (int l = 0; l < NL; ++l) {
      const int n = min(min(cnt[l], cap), per);
      for (int i = tid; i < n; i += nthr) {
        sel_key[(size_t)l * per + i] = keys[(size_t)l * cap + i];
        sel_idx[(size_t)l * per + i] = idxs[(size_t)l * cap + i];
      }
    }
    __syncthreads();
  } else {
  // deal the winners evenly and in order: global position p goes to CTA p / dper, slot p % dper
  const int trange = (tag_lo == kTagByPosition) ? cap : max(tag_range, 1);
#pragma unroll 1
  for (int l = 0; l < NL; ++l) {
    const int n = min(cnt[l], cap);
    const uint32_t kth = ms->prefix[l];
    const uint32_t* kl = keys + (size_t)l * cap;
    const int* il = idxs + (size_t)l * cap;
    const int off_win = ms->off_win[l], take_eq = ms->take_eq[l];
    const int n_eq = (int)ms->counts[l][1];
    auto tag_of = [&](int i) { return tag_lo == kTagByPosition ? i : il[i] - tag_lo; };
    // tag up to which this CTA takes copies of the k-th key
    int cut = take_eq >= n_eq ? 0x7fffffff : -1;
    if (take_eq > 0 && take_eq < n_eq) {   // uniform over the CTA
      if (tid == 0) ms->cut_found = 0;
      int seen = 0;
      for (int wlo = 0; wlo < trange; wlo += det_window) {
        for (int w = tid; w < A.det_words; w += nthr) det_bits[w] = 0u;
        __syncthreads();
        for_each_key(kl, n, tid, nthr, [&](uint32_t key, int i) {
          const unsigned t = (unsigned)(tag_of(i) - wlo);
          if (key == kth && t < (unsigned)det_window) atomicOr(&det_bits[t >> 5], 1u << (t & 31));
        });
        __syncthreads();
        const int total = bitmap_prefix(det_bits, det_pre, ms->wsum, A.det_words, tid, nthr);
        if (seen + total >= take_eq) {
          const int need = take_eq - seen;   // 1-based rank inside this window
          for (int w = tid; w < A.det_words; w += nthr) {
            const int before = det_pre[w];
            const uint32_t word = det_bits[w];
            if (before < need && need <= before + __popc(word)) {
              ms->cut_tag = wlo + 32 * w + (int)__fns(word, 0, need - before);
              ms->cut_found = 1;
            }
          }
        }
        seen += total;
        __syncthreads();
        if (ms->cut_found) break;
      }
      cut = ms->cut_tag;
      __syncthreads();
    }
    int base = 0;
    for (int wlo = 0; wlo < trange; wlo += det_window) {
      for (int w = tid; w < A.det_words; w += nthr) det_bits[w] = 0u;
      __syncthreads();
      for_each_key(kl, n, tid, nthr, [&](uint32_t key, int i) {
        const int tg = tag_of(i);
        const unsigned t = (unsigned)(tg - wlo);
        if ((key > kth || (key == kth && tg <= cut)) && t < (unsigned)det_window)
          atomicOr(&det_bits[t >> 5], 1u << (t & 31));
      });
      __syncthreads();
      const int total = bitmap_prefix(det_bits, det_pre, ms->wsum, A.det_words, tid, nthr);
      for_each_key(kl, n, tid, nthr, [&](uint32_t key, int i) {
        const int tg = tag_of(i);
        const unsigned t = (unsigned)(tg - wlo);
        if ((key > kth || (key == kth && tg <= cut)) && t < (unsigned)det_window) {
          const int p = off_win + base + det_pre[t >> 5] + __popc(det_bits[t >> 5] & ((1u << (t & 31)) - 1u));
          if (p < k) {
            const int dst = A.per_cta_select ? crank : p / dper;
            const int slot = A.per_cta_select ? p : p - dst * dper;
            uint32_t* rk = cluster.map_shared_rank(sel_key, dst);
            int* ri = cluster.map_shared_rank(sel_idx, dst);
            rk[(size_t)l * per + slot] = key;
            ri[(size_t)l * per + slot] = il[i];
          }
        }
      });
      base += total;
      __syncthreads();
    }
  }
  cluster_barrier(cluster, C);
  }

  RA_STAMP(A.status, 6);
  // Centroid retrieval: the winners are cluster ids.  Rank every local winner among all k winners
  // of its list (descending score, ties by id; the peers' winners are read through distributed
  // shared memory) and write the clusters' member tokens in that order.
  if (A.expand_clen > 0 && A.expand_out) {
#pragma unroll 1
    for (int l = 0; l < NL; ++l) {
      const ListDest ld = dest(l);
      if (!ld.valid) continue;
      const int total = ms->total_sel[l];
      const int n_l = max(0, min(dper, total - crank * dper));
      const size_t rowi = (size_t)ld.bq * A.hq_total + ld.hq;
      for (int e = warp; e < n_l; e += nwarps) {
        const uint32_t mk = sel_key[(size_t)l * per + e];
        const int mi = sel_idx[(size_t)l * per + e];
        int rank = 0;
        for (int j = lane; j < total; j += 32) {
          const int c = j / dper, slot = j - c * dper;
          const uint32_t ok = cluster.map_shared_rank(sel_key, c)[(size_t)l * per + slot];
          const int oi = cluster.map_shared_rank(sel_idx, c)[(size_t)l * per + slot];
          rank += (ok > mk) || (ok == mk && oi < mi);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, off);
        if (A.expand_ids && lane == 0) A.expand_ids[rowi * k + rank] = mi + A.index_base;
        int* dst = A.expand_out + (rowi * k + rank) * A.expand_clen;
        const int t0 = mi * A.expand_clen;
        for (int i = lane; i < A.expand_clen; i += 32) dst[i] = t0 + i;
      }
    }
    cluster_barrier(cluster, C);  // nobody leaves or reuses its winner slots while a peer still ranks against them
    if (A.out_mode == kOutNone && !A.sel_idx) return;
  }

#pragma unroll 1
  for (int l = 0; l < NL; ++l) {
    const ListDest ld = dest(l);
    if (!ld.valid) continue;  // uniform over the CTA
    const int n_l = A.per_cta_select ? ms->total_sel[l] : max(0, min(dper, ms->total_sel[l] - crank * dper));
    const uint32_t* sk = sel_key + (size_t)l * per;
    const int* si = sel_idx + (size_t)l * per;
    if (A.sel_idx) {
      const size_t dst = ((size_t)ld.bq * A.hq_total + ld.hq) * A.list_pitch + A.list_off +
                         (A.per_cta_select ? (size_t)0 : (size_t)crank * dper);
      for (int e = tid; e < n_l; e += nthr) {
        A.sel_idx[dst + e] = si[e] + A.index_base;
        if (A.sel_score) A.sel_score[dst + e] = key_score(sk[e]);
      }
      // a part with fewer than k keys pads its slots with entries that can never win
      const int slots = A.per_cta_select ? k : max(0, min(dper, k - crank * dper));
      for (int e = n_l + tid; e < slots; e += nthr) {
        A.sel_idx[dst + e] = -1;
        if (A.sel_score) A.sel_score[dst + e] = -INFINITY;
      }
    }
    if (A.out_mode == kOutNone) continue;
    // softmax weights against the cluster-wide best score; V rows mixed by half-warps
    const float smax = key_score(ms->maxkey[l]);
    const __half* vb = A.v + (size_t)ld.bq * A.v_batch_stride + (size_t)ld.hkv * A.v_head_stride +
                       (lane & 15) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    float lsum = 0.f;
    constexpr int UN = 8;
    for (int e0 = warp * 2 + (lane >> 4); e0 < n_l; e0 += 2 * nwarps * UN) {
      uint4 vv[UN];
      float w[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int e = e0 + 2 * nwarps * u;
        const int id = (e < n_l) ? si[e] : -1;
        const int local = id - A.id_shift;
        const bool mine = id >= A.own_lo && id < A.own_hi;
        if (mine && (unsigned)local >= (unsigned)A.n_tokens) atomicOr(A.status, kStatusBadId);
        if (mine && (unsigned)local < (unsigned)A.n_tokens) {
          w[u] = fast_exp2((key_score(sk[e]) - smax) * A.scale_log2e);
          vv[u] = ldg128_nc(vb + (size_t)local * A.v_token_stride);
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
      for (int i = 0; i < 8; ++i) ms->red[warp][lane * 8 + i] = acc[i];
    }
    if (lane == 0) ms->lred[warp] = lsum;
    __syncthreads();
    if (tid < kHeadDim) {
      float o = 0.f;
      for (int w = 0; w < nwarps; ++w) o += ms->red[w][tid];
      ms->o_part[l][tid] = o;
      if (tid == 0) {
        float ls = 0.f;
        for (int w = 0; w < nwarps; ++w) ls += ms->lred[w];
        ms->l_part[l] = ls;
      }
    }
    __syncthreads();
  }

  RA_STAMP(A.status, 7);
  if (A.out_mode != kOutNone) {
    cluster_barrier(cluster, C);
    // CTA c finishes the dimensions d with d % C == c (any cluster size)
    for (int item = tid; item < NL * kHeadDim; item += nthr) {
      const int l = item / kHeadDim, d = item % kHeadDim;
      if (d % C != crank) continue;
      const ListDest ld = dest(l);
      if (!ld.valid) continue;
      float o = 0.f, lt = 0.f;
      for (int c = 0; c < C; ++c) {
        const float* ro = cluster.map_shared_rank(&ms->o_part[l][0], c);
        const float* rl = cluster.map_shared_rank(&ms->l_part[0], c);
        o += ro[d];
        lt += rl[l];
      }
      const size_t row = (size_t)ld.bq * A.hq_total + ld.hq;
      // a list without winners (a shard that holds none of a row's top-k) weighs nothing
      const float mscaled = ms->total_sel[l] > 0 ? key_score(ms->maxkey[l]) * A.sm_scale : -INFINITY;
      if (A.out_mode == kOutFinal) {
        A.out[row * kHeadDim + d] = __float2half_rn(o / lt);
        if (A.out_lse && d == 0) {
          A.out_lse[row * 2 + 0] = mscaled;
          A.out_lse[row * 2 + 1] = lt;
        }
      } else {
        float* dstp = A.out_partial + row * (kHeadDim + 2);
        dstp[d] = o;
        if (d == 0) {
          dstp[kHeadDim] = lt;
          dstp[kHeadDim + 1] = mscaled;
        }
      }
    }
    cluster_barrier(cluster, C);  // nobody leaves while a peer may still read its shared memory
  }
  RA_STAMP(A.status, 8);
}

}  // namespace ra
