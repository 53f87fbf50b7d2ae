// Pieces shared by the kernels that select among the score keys scan_store_kernel left in the
// workspace: the search for the coarse bin of the k-th key and the two passes that collect the
// candidates of a CTA's token range into its shared-memory list.
#pragma once
#include "scan_store.cuh"

namespace ra {

constexpr int kSelUnroll = 8;   // 128-bit loads in flight per thread when passing over stored keys

struct SelCtrl {
  int hist[2][256];
  int ghist[256];
  int wtot[32];
  int bin, n_above, rem, n_in;   // result of a search step
  int n_eq_local;                // copies of the k-th key in this CTA's range (read by the peers)
  int scan_tot;
};

// 2048 bins, larger bin = larger key: find the bin holding the k-th largest element.  Called by
// all kSelThreads threads; results in sc->bin, n_above (elements in higher bins), rem (1-based
// rank of the k-th inside the bin, from its top) and n_in (elements in the bin).
__device__ inline void find_coarse_bin(const int* hist, int k, SelCtrl* sc, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  // warp w owns the 64 bins 2047-64w .. 1984-64w, lane l the two bins 2047-64w-2l, -2l-1
  const int top = kHistBins - 1 - 64 * warp - 2 * lane;
  const int c0 = hist[top], c1 = hist[top - 1];
  int s = c0 + c1;
#pragma unroll
  for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) sc->wtot[warp] = s;
  __syncthreads();
  int tot = sc->wtot[lane];
  int incl = tot;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  const unsigned cross = __ballot_sync(0xffffffffu, incl - tot < k && k <= incl);
  const int wsel = cross ? (__ffs(cross) - 1) : 31;
  const int above_w = __shfl_sync(0xffffffffu, incl - tot, wsel);
  if (warp == wsel) {
    const int pair = c0 + c1;
    int pin = pair;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, pin, off);
      if (lane >= off) pin += n;
    }
    const int above = above_w + pin - pair;
    if (above < k && k <= above + pair) {
      if (k <= above + c0) {
        sc->bin = top; sc->n_above = above; sc->rem = k - above; sc->n_in = c0;
      } else {
        sc->bin = top - 1; sc->n_above = above + c0; sc->rem = k - above - c0; sc->n_in = c1;
      }
    }
  }
  __syncthreads();
}


// Candidates of the token range [lo, hi) of one row: every stored key >= lo_key goes into the list
// (keys/idxs, capacity cap, count in cnt[0]) with its token position.  Several 128-bit loads are
// in flight per thread (the pass is bound by L2 latency otherwise); the rare hits of a warp are
// appended with one shared-memory atomic per iteration.  Called by all kSelThreads threads.
__device__ __forceinline__ void collect_candidates(const uint32_t* krow, int lo, int hi, uint32_t lo_key,
                                                   uint32_t* keys, int* idxs, int* cnt, int cap,
                                                   unsigned* status, int tid, int lane) {
  // several 128-bit loads in flight per thread (the pass is bound by L2 latency otherwise); the
  // rare hits of a warp are appended with one shared-memory atomic per iteration
  constexpr int U = kSelUnroll;
  for (int base = lo; base < hi; base += kSelThreads * 4 * U) {   // same trip count for all threads
    uint4 kk[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + (u * kSelThreads + tid) * 4;
      kk[u] = i < hi ? ldg128_nc(krow + i) : make_uint4(0u, 0u, 0u, 0u);
    }
    int mine = 0;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + (u * kSelThreads + tid) * 4;
      const uint32_t kv[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) mine += (i + e < hi && kv[e] >= lo_key);
    }
    if (__ballot_sync(0xffffffffu, mine > 0)) {
      int incl = mine;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
      }
      int basepos = 0;
      if (lane == 31) basepos = atomicAdd(&cnt[0], incl);
      basepos = __shfl_sync(0xffffffffu, basepos, 31);
      int pos = basepos + incl - mine;
      if (mine) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
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
      }
    }
  }
}

// The same when a single key value has more copies than the list can hold: keys above lo_key, and
// the first tie_take copies of lo_key in ascending token order (thread order is token order).
__device__ __forceinline__ void collect_candidates_ties(const uint32_t* krow, int lo, int hi, uint32_t lo_key,
                                                        int tie_take, uint32_t* keys, int* idxs, int* cnt,
                                                        int cap, SelCtrl* sc, unsigned* status, int tid,
                                                        int warp, int lane) {
  const unsigned lt_mask = (1u << lane) - 1u;
  int tie_base = 0;   // copies of the k-th key seen so far in this CTA
  for (int base = lo; base < hi; base += kSelThreads * 4) {   // same trip count for all threads
    const int i = base + tid * 4;
    uint4 kk = make_uint4(0u, 0u, 0u, 0u);
    if (i < hi) kk = *reinterpret_cast<const uint4*>(krow + i);
    const uint32_t kv[4] = {kk.x, kk.y, kk.z, kk.w};
    bool pass[4];
    // ordinal of each copy in token order: thread order is token order
    int mine = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) mine += (i + e < hi && kv[e] == lo_key);
    int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += n;
    }
    if (lane == 31) sc->wtot[warp] = incl;
    __syncthreads();
    int wbase = 0;
    for (int w = 0; w < warp; ++w) wbase += sc->wtot[w];
    if (tid == kSelThreads - 1) sc->scan_tot = wbase + incl;
    int ord = tie_base + wbase + incl - mine;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      pass[e] = i + e < hi && kv[e] > lo_key;
      if (i + e < hi && kv[e] == lo_key) {
        pass[e] = ord < tie_take;
        ++ord;
      }
    }
    __syncthreads();
    tie_base += sc->scan_tot;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const unsigned bal = __ballot_sync(0xffffffffu, pass[e]);
      if (bal) {
        const int leader = __ffs(bal) - 1;
        int basepos = 0;
        if (lane == leader) basepos = atomicAdd(&cnt[0], __popc(bal));
        basepos = __shfl_sync(0xffffffffu, basepos, leader);
        if (pass[e]) {
          const int pos = basepos + __popc(bal & lt_mask);
          if (pos < cap) {
            keys[pos] = kv[e];
            idxs[pos] = i + e;
          } else {
            atomicOr(status, kStatusOverflow);
          }
        }
      }
    }
  }
}

}  // namespace ra
