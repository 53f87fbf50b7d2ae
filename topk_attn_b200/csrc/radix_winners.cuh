// Exact top-c of n ordered keys held in shared memory, by one CTA: a radix descent over 64-bit
// composites (key, inverted index).  Composites are distinct, so the descent always ends on an
// exact cut, and among equal keys the lower index wins.
#pragma once
#include "common.cuh"

namespace ra {

constexpr int kWinnerWords = 256;   // one bit per key: up to 8192 keys

struct WinnerCtrl {
  unsigned bits[kWinnerWords];
  int wpre[kWinnerWords];
  int wtot[kWinnerWords / 32];
  unsigned hist[256];
  unsigned wmin[32], wmax[32];
  unsigned long long base;   // lower edge of the active interval of composites
  unsigned long long range;  // its width - 1
  int need;                  // winners still to take from the active interval
  int done;
  int nwin, nown;
};

__device__ __forceinline__ unsigned long long composite(uint32_t key, int idx) {
  return ((unsigned long long)key << 32) | (uint32_t)~idx;
}

// All NT threads of the CTA call this (NT a multiple of 32, at least 256); the keys must be
// visible to the CTA.  On return winners[0 .. topc) hold the indices of the topc largest
// composites in no particular order, ctrl.nwin == topc, and the CTA is synchronised.  A caller
// that selects again with the same ctrl synchronises the CTA once more before the next call.
// n is at most 32 * kWinnerWords.
template <int NT>
__device__ void select_winners(const uint32_t* keys, int n, int topc, WinnerCtrl& ctrl, int* winners) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    ctrl.nwin = 0;
    ctrl.done = 0;
  }
  // ---- range of the keys ----
  {
    uint32_t mn = 0xffffffffu, mx = 0u;
    for (int i = tid; i < n; i += NT) {
      const uint32_t k = keys[i];
      mn = min(mn, k);
      mx = max(mx, k);
    }
    mn = __reduce_min_sync(0xffffffffu, mn);
    mx = __reduce_max_sync(0xffffffffu, mx);
    if (lane == 0) {
      ctrl.wmin[warp] = mn;
      ctrl.wmax[warp] = mx;
    }
    if (tid < 256) ctrl.hist[tid] = 0u;
    __syncthreads();
    if (tid == 0) {
      for (int w = 0; w < NT / 32; ++w) {
        mn = min(mn, ctrl.wmin[w]);
        mx = max(mx, ctrl.wmax[w]);
      }
      ctrl.base = (unsigned long long)mn << 32;
      ctrl.range = (((unsigned long long)mx << 32) | 0xffffffffull) - ctrl.base;
      ctrl.need = topc;
    }
    __syncthreads();
  }

  // ---- radix descent to the topc-th largest composite: at most 8 digits of 8 bits ----
  unsigned long long base = ctrl.base, range = ctrl.range;
  for (int it = 0; it < 9; ++it) {
    const int bits = 64 - __clzll(range | 1ull);
    const int shift = max(0, bits - 8);
    for (int i = tid; i < n; i += NT) {
      const unsigned long long c = composite(keys[i], i);
      if (c >= base && c - base <= range) atomicAdd(&ctrl.hist[(unsigned)((c - base) >> shift)], 1u);
    }
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins 255-8l .. 248-8l; walk from the top until `need` composites are covered
      const unsigned need = (unsigned)ctrl.need;   // read by every lane before the shuffles below
      unsigned cnt[8], s = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        cnt[j] = ctrl.hist[255 - 8 * lane - j];
        s += cnt[j];
      }
      unsigned incl = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      unsigned above = incl - s;
      if (above < need && need <= incl) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (above < need && need <= above + cnt[j]) {
            const int b = 255 - 8 * lane - j;
            ctrl.base = base + ((unsigned long long)b << shift);
            ctrl.range = shift ? ((1ull << shift) - 1ull) : 0ull;
            ctrl.need = (int)(need - above);
            ctrl.done = (cnt[j] == need - above) ? 1 : 0;   // the whole bin wins: exact cut
            above = need;                                    // stop the walk
          } else {
            above += cnt[j];
          }
        }
      }
    }
    __syncthreads();
    base = ctrl.base;
    range = ctrl.range;
    const int done = ctrl.done;
    if (tid < 256) ctrl.hist[tid] = 0u;
    __syncthreads();
    if (done) break;
  }
  // every composite >= base is a winner, and there are exactly topc of them; they are listed in
  // ascending index order (one bit per key, popcount prefix), so the list is the same on every run
  const int nwords = (n + 31) >> 5;
  for (int w = tid; w < nwords; w += NT) ctrl.bits[w] = 0u;
  __syncthreads();
  for (int i = tid; i < n; i += NT)
    if (composite(keys[i], i) >= base) atomicOr(&ctrl.bits[i >> 5], 1u << (i & 31));
  __syncthreads();
  {
    // exclusive popcount prefix over at most kWinnerWords words: warp w scans words 32w .. 32w+31
    const int w = tid;
    const unsigned word = w < nwords ? ctrl.bits[w] : 0u;
    const int c = __popc(word);
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (w < kWinnerWords) ctrl.wpre[w] = incl - c;
    if (lane == 31 && warp < kWinnerWords / 32) ctrl.wtot[warp] = incl;
    __syncthreads();
    if (tid == 0) {
      int run = 0;
      for (int j = 0; j < kWinnerWords / 32; ++j) {
        const int t = ctrl.wtot[j];
        ctrl.wtot[j] = run;
        run += t;
      }
      ctrl.nwin = min(run, topc);
    }
    __syncthreads();
  }
  for (int i = tid; i < n; i += NT)
    if (composite(keys[i], i) >= base) {
      const int w = i >> 5;
      const int slot = ctrl.wtot[w >> 5] + ctrl.wpre[w] + __popc(ctrl.bits[w] & ((1u << (i & 31)) - 1u));
      if (slot < topc) winners[slot] = i;
    }
  __syncthreads();
}

}  // namespace ra
