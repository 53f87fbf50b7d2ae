// Fused K scan + exact top-k (+ softmax.V) for single-token decode on sm_100a.
//
// One thread-block cluster owns one "part": a token range of one (batch group, kv-head
// group).  Its CTAs split the range; every CTA streams its slab of the fp16 key cache through
// a multi-stage TMA pipeline (cp.async.bulk.tensor, 128 rows = 32 KiB per stage), scores the
// rows with fp32 accumulation on the CUDA cores (8 lanes per 256-byte row, warp-shuffle
// reduction) and appends every score above a running threshold to a candidate list in shared
// memory.  When a list is about to overflow the CTA raises the threshold to the exact k-th
// candidate with a radix select and drops the rest.  After the scan the cluster finds the
// exact global k-th score with a radix select whose histograms are summed across CTAs through
// distributed shared memory, deals the k winners evenly over the CTAs, and either writes them
// out (candidate mode) or mixes their V rows and reduces the partial outputs through
// distributed shared memory (fused mode).  Nothing is written to global memory in between.
//
// This replaces, with a different decomposition, retrieval_attention_kernel<K>
// (retrieval_attn/retrieval_attention.cu:254-472: per-chunk scoring, full radix sort, DSMEM
// hand-off to a fifth CTA that spins on a counter) and gemv_topk_kernel (gemv_topk.cu:173-380).
// All inter-CTA hand-offs here are hardware cluster barriers; the only polled wait is the
// bounded mbarrier wait on TMA completion.
#include "scan_select.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace ra {

struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  int cnt[kMaxLists];
  uint32_t thr[kMaxLists];
  int hist[kMaxLists][256];
  // per-list state of a cut (see compact_lists)
  uint32_t kmax[kMaxLists], base[kMaxLists], prefix[kMaxLists], mask[kMaxLists];
  int shift[kMaxLists], remaining[kMaxLists], state[kMaxLists];
  int wpos, eqc;
  uint32_t tie_pre;   // radix descent over the inverted ids of the copies of a cut's k-th key
  int tie_rem;
  int timeout;
  int coarse_id;              // two-level retrieval: the cluster this part scans
  float coarse[kMaxCoarse];   // its head's centroid scores
};
enum CutState : int { kCutIdle = 0, kCutRun = 1, kCutInclusive = 2, kCutExact = 3 };

// Barrier among the consumer warps only (the producer warp never joins it).
__device__ __forceinline__ void consumer_sync(int nct) {
  asm volatile("bar.sync 1, %0;" ::"r"(nct) : "memory");
}

// Cut back every list whose bit is set in `need`: raise its threshold so that at least k and at most
// `accept` candidates stay.  All candidates of a list lie above its old threshold, so the radix
// select works on (key - old threshold) and starts at the highest bit that actually differs; a
// list is done as soon as keeping the whole current bin leaves few enough candidates, and only
// runs down to an exact k-th key (ties taken one by one) when it has to.  The lists go through
// the passes together (one set of barriers for all of them, their loads overlap); only the
// in-place filtering is done list by list.  Called by all consumer threads.
template <int NL>
__device__ void compact_lists(uint32_t* keys, int* idxs, Ctrl* ctrl, int need, int k, int cap,
                              int accept, int tid, int nct) {
  const int lane = tid & 31, warp = tid >> 5, nwarps = nct >> 5;
  if (tid < NL) ctrl->kmax[tid] = 0u;
  consumer_sync(nct);
#pragma unroll
  for (int l = 0; l < NL; ++l) {
    if (!((need >> l) & 1)) continue;
    const int n = min(ctrl->cnt[l], cap);
    uint32_t mx = 0u;
    for_each_key(keys + (size_t)l * cap, n, tid, nct, [&](uint32_t key, int) { mx = max(mx, key); });
#pragma unroll
    for (int off = 16; off; off >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) atomicMax(&ctrl->kmax[l], mx);
  }
  consumer_sync(nct);
  if (tid < NL) {
    const int l = tid;
    const bool on = (need >> l) & 1;
    const uint32_t base = ctrl->thr[l] + 1u;  // smallest key the list can hold
    const uint32_t range = ctrl->kmax[l] - base;
    ctrl->base[l] = base;
    ctrl->shift[l] = max(0, 32 - __clz((int)(range | 1u)) - 8);
    ctrl->prefix[l] = 0u;
    ctrl->mask[l] = 0u;
    ctrl->remaining[l] = k;
    ctrl->state[l] = on ? kCutRun : kCutIdle;
  }
  consumer_sync(nct);
#pragma unroll 1
  for (;;) {
    for (int i = tid; i < NL * 256; i += nct) (&ctrl->hist[0][0])[i] = 0;
    consumer_sync(nct);
    bool any = false;
#pragma unroll
    for (int l = 0; l < NL; ++l) {
      if (ctrl->state[l] != kCutRun) continue;
      any = true;
      const int n = min(ctrl->cnt[l], cap);
      const uint32_t base = ctrl->base[l], prefix = ctrl->prefix[l], mask = ctrl->mask[l];
      const int shift = ctrl->shift[l];
      for_each_key(keys + (size_t)l * cap, n, tid, nct, [&](uint32_t key, int) {
        const uint32_t rel = key - base;
        if ((rel & mask) == prefix) atomicAdd(&ctrl->hist[l][(rel >> shift) & 255], 1);
      });
    }
    if (!any) break;  // the states were settled before the barrier above: same for every thread
    consumer_sync(nct);
    for (int l = warp; l < NL; l += nwarps) {
      if (ctrl->state[l] != kCutRun) continue;
      int d, nr;
      warp_find_digit(ctrl->hist[l], ctrl->remaining[l], lane, d, nr);
      if (lane == 0) {
        const int shift = ctrl->shift[l];
        ctrl->prefix[l] |= (uint32_t)d << shift;
        ctrl->mask[l] = 0xffffffffu << shift;
        ctrl->remaining[l] = nr;
        const int kept = (k - nr) + ctrl->hist[l][d];  // candidates at or above the bin's start
        if (kept <= accept) ctrl->state[l] = kCutInclusive;
        else if (shift == 0) ctrl->state[l] = kCutExact;
        else ctrl->shift[l] = max(0, shift - 8);
      }
    }
    consumer_sync(nct);
  }
  // inclusive: keep every key >= base + prefix; exact: keys above the k-th and `remaining` ties
#pragma unroll 1
  for (int l = 0; l < NL; ++l) {
    const int st = ctrl->state[l];
    if (st != kCutInclusive && st != kCutExact) continue;  // uniform
    const bool inclusive = st == kCutInclusive;
    const uint32_t kth = ctrl->base[l] + ctrl->prefix[l];
    const int need_eq = ctrl->remaining[l];
    const int n = min(ctrl->cnt[l], cap);
    uint32_t* kl = keys + (size_t)l * cap;
    int* il = idxs + (size_t)l * cap;
    if (tid == 0) {
      ctrl->wpos = 0;
      ctrl->eqc = 0;
    }
    consumer_sync(nct);
    // Exact cut: of the copies of the k-th key the need_eq with the lowest ids stay (later tokens
    // never beat an equal earlier one, so the final selection prefers low ids as well).  They are
    // the need_eq largest inverted ids, found by a radix descent over the copies.
    uint32_t inv_cut = 0u;
    if (!inclusive) {
      int ties = 0;
      for_each_key(kl, n, tid, nct, [&](uint32_t key, int) { ties += key == kth; });
#pragma unroll
      for (int off = 16; off; off >>= 1) ties += __shfl_xor_sync(0xffffffffu, ties, off);
      if (lane == 0 && ties) atomicAdd(&ctrl->eqc, ties);
      consumer_sync(nct);
      if (ctrl->eqc > need_eq) {   // the same for every thread
        uint32_t pre = 0u, msk = 0u;
        int remain = need_eq;
#pragma unroll 1
        for (int sh = 24; sh >= 0; sh -= 8) {
          for (int i = tid; i < 256; i += nct) ctrl->hist[l][i] = 0;
          consumer_sync(nct);
          for_each_key(kl, n, tid, nct, [&](uint32_t key, int i) {
            const uint32_t inv = ~(uint32_t)il[i];
            if (key == kth && (inv & msk) == pre) atomicAdd(&ctrl->hist[l][(inv >> sh) & 255], 1);
          });
          consumer_sync(nct);
          if (warp == 0) {
            int d, nr;
            warp_find_digit(ctrl->hist[l], remain, lane, d, nr);
            if (lane == 0) {
              ctrl->tie_pre = pre | ((uint32_t)d << sh);
              ctrl->tie_rem = nr;
            }
          }
          consumer_sync(nct);
          pre = ctrl->tie_pre;
          remain = ctrl->tie_rem;
          msk |= 255u << sh;
        }
        inv_cut = pre;
      }
    }
    constexpr int E = 8;
#pragma unroll 1
    for (int cb = 0; cb < n; cb += nct * E) {
      uint32_t kk[E];
      int ii[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int i = cb + e * nct + tid;
        kk[e] = (i < n) ? kl[i] : 0u;
        ii[e] = (i < n) ? il[i] : 0;
      }
      consumer_sync(nct);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int i = cb + e * nct + tid;
        if (i < n) {
          const bool keep = inclusive ? (kk[e] >= kth)
                                      : (kk[e] > kth || (kk[e] == kth && ~(uint32_t)ii[e] >= inv_cut));
          if (keep) {
            const int p = atomicAdd(&ctrl->wpos, 1);
            kl[p] = kk[e];
            il[p] = ii[e];
          }
        }
      }
      consumer_sync(nct);
    }
    if (tid == 0) {
      ctrl->cnt[l] = ctrl->wpos;
      ctrl->thr[l] = inclusive ? kth - 1u : kth;
    }
    consumer_sync(nct);
  }
}

// acc0 += k.lo * q.lo, acc1 += k.hi * q.hi for one packed pair of fp16 values; products of
// two fp16 numbers are exact in fp32, so both forms give the same sums.
template <bool MIXED>
__device__ __forceinline__ void fma_pair(float& acc0, float& acc1, uint32_t kw, uint32_t qw) {
  if constexpr (MIXED) {
    asm("{\n\t.reg .b16 kl, kh, ql, qh;\n\t"
        "mov.b32 {kl, kh}, %2;\n\t"
        "mov.b32 {ql, qh}, %3;\n\t"
        "fma.rn.f32.f16 %0, kl, ql, %0;\n\t"
        "fma.rn.f32.f16 %1, kh, qh, %1;\n\t}"
        : "+f"(acc0), "+f"(acc1)
        : "r"(kw), "r"(qw));
  } else {
    const float2 kf = h2f2(kw), qf = h2f2(qw);
    acc0 = fmaf(kf.x, qf.x, acc0);
    acc1 = fmaf(kf.y, qf.y, acc1);
  }
}

template <int HG, int NQ, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
scan_select_kernel(const __grid_constant__ ScanParams P) {
  constexpr int NL = HG * NQ;
  constexpr bool MIXED = (MODE == 1);
  static_assert(NL <= kMaxLists, "too many candidate lists per CTA");
  static_assert(MODE != 2 || HG == 1, "tensor-core scoring takes one kv head per CTA");
  constexpr int T = kTileRows / HG;     // tokens per tile
  constexpr int NV = (NQ + 1) / 2;      // scores a lane keeps per tile
  const int G = P.groups;      // consumer warp groups (1 or 2), each on its own tile
  const int R = P.rendezvous;  // iterations between overflow checks
  const int nct = 256 * G;     // consumer threads
  // a cut may leave a little more than k candidates (an eighth of the free room, at least 256):
  // one histogram pass over the actual key range usually gets that close, and the fewer
  // candidates stay the longer it takes until the next cut
  const int room = max(0, P.cap - R * G * (kTileRows / HG) - P.m.topk);
  const int accept = P.m.topk + min(room / 2, max(256, room / 8));
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.m.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cap = P.cap, k = P.m.topk;

  unsigned char* stages = smem;
  // candidate lists and control block behind the stages
  unsigned char* after_stages = smem + (size_t)P.nstages * kStageBytes;
  uint32_t* keys = reinterpret_cast<uint32_t*>(after_stages);
  int* idxs = reinterpret_cast<int*>(keys + (size_t)NL * cap);
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(idxs + (size_t)NL * cap);

  RA_STAMP(P.status, 0);
  // which part of which (batch group, kv-head group) this cluster owns
  // (or, with parts_in_cluster, which part this CTA owns: the cluster holds all parts of a row)
  const bool pic = P.parts_in_cluster != 0;
  int cid = blockIdx.x / C;
  const int part = pic ? crank : cid % P.nparts;
  if (!pic) cid /= P.nparts;
  // the queries that share a K row may be dealt over several clusters (each re-reads the rows,
  // mostly from L2, and keeps fewer candidate lists): this cluster scores queries q0 .. q0+nq_cta-1
  const int q0 = (cid % P.qsplit) * P.nq_cta;
  cid /= P.qsplit;
  const int hgroups = P.hkv / HG;
  const int h0 = (cid % hgroups) * HG;
  const int b0 = (cid / hgroups) * P.bshare;
  const int kv_b = P.kv_per_batch ? b0 : 0;

  // a part is normally the part-th slice of the token axis; with part_ids it is the cluster whose
  // id the (batch row, head) chose at that rank (two-level retrieval, one head and query per CTA)
  int part_slice = part;
  if (P.part_ids) part_slice = P.part_ids[((size_t)b0 * P.hq + (size_t)h0 * P.group) * P.nparts + part];
  if (P.coarse_centers) {
    // Coarse stage in the prologue (gemv_topk.cu:218-262: score the head's centroids, keep the best
    // few): half-warp per centroid row, the arithmetic of center_select_kernel, then every
    // centroid counts the ones ahead of it in (score descending, id ascending) order; the one with
    // `part` ahead of it is this part's cluster.
    const int row = b0 * P.hq + h0 * P.group;
    const int hw = tid >> 4, l16 = tid & 15;
    float qf[8];
    {
      const uint4 qraw = *reinterpret_cast<const uint4*>(P.q + (size_t)row * kHeadDim + l16 * 8);
      const float2 a = h2f2(qraw.x), b = h2f2(qraw.y), c = h2f2(qraw.z), d = h2f2(qraw.w);
      qf[0] = a.x; qf[1] = a.y; qf[2] = b.x; qf[3] = b.y;
      qf[4] = c.x; qf[5] = c.y; qf[6] = d.x; qf[7] = d.y;
    }
    const __half* table = P.coarse_centers + (size_t)(h0 * P.group) * P.coarse_csz * kHeadDim + l16 * 8;
    const int nhw = (int)blockDim.x >> 4;
    for (int r0 = 0; r0 < P.coarse_csz; r0 += nhw) {   // same trip count for all threads
      const int r = r0 + hw;
      const uint4 kv = r < P.coarse_csz ? ldg128_nc(table + (size_t)r * kHeadDim) : make_uint4(0, 0, 0, 0);
      const float2 a = h2f2(kv.x), b = h2f2(kv.y), c = h2f2(kv.z), d = h2f2(kv.w);
      float sc = a.x * qf[0];
      sc = fmaf(a.y, qf[1], sc); sc = fmaf(b.x, qf[2], sc); sc = fmaf(b.y, qf[3], sc);
      sc = fmaf(c.x, qf[4], sc); sc = fmaf(c.y, qf[5], sc); sc = fmaf(d.x, qf[6], sc);
      sc = fmaf(d.y, qf[7], sc);
      sc += __shfl_xor_sync(0xffffffffu, sc, 8);
      sc += __shfl_xor_sync(0xffffffffu, sc, 4);
      sc += __shfl_xor_sync(0xffffffffu, sc, 2);
      sc += __shfl_xor_sync(0xffffffffu, sc, 1);
      if (l16 == 0 && r < P.coarse_csz) ctrl->coarse[r] = sc;
    }
    __syncthreads();
    for (int r = tid; r < P.coarse_csz; r += blockDim.x) {
      const uint32_t me = score_key(ctrl->coarse[r]);
      int ahead = 0;
      for (int j = 0; j < P.coarse_csz; ++j) {
        const uint32_t o = score_key(ctrl->coarse[j]);
        ahead += (o > me) || (o == me && j < r);
      }
      if (ahead == part) ctrl->coarse_id = r;
    }
    __syncthreads();
    part_slice = ctrl->coarse_id;
    if ((pic || crank == 0) && tid == 0 && P.coarse_ids_out)   // one writer per part
      P.coarse_ids_out[(size_t)row * P.nparts + part] = part_slice;
  }
  const int part_lo = part_slice * P.part_len;
  const int part_hi = min(P.n_tokens, part_lo + P.part_len);
  const int ntiles_part = ceil_div(max(part_hi - part_lo, 0), T);
  const int tpc = pic ? ntiles_part : ceil_div(ntiles_part, C);
  const int tile_b = pic ? 0 : crank * tpc;
  const int my_ntiles = max(0, min(ntiles_part, tile_b + tpc) - tile_b);
  const int tok_begin = part_lo + tile_b * T;
  const int S = P.nstages;

  if (tid == 0) {
    tma_prefetch_desc(&P.kmap);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&ctrl->full[s], 1);
      mbar_init(&ctrl->empty[s], 8);  // the 8 warps of the group that consumed the stage
    }
    ctrl->timeout = 0;
    fence_barrier_init();
  }
  if (tid < kMaxLists) {
    ctrl->cnt[tid] = 0;
    ctrl->thr[tid] = 0u;
  }
  __syncthreads();

  if (warp == 8 * G) {
    // ------------------------------------------------------------ producer warp
    if (lane == 0) {
      // Every consumer group has its own ring of S/G stages, so a warp waits on every phase of
      // the barriers it uses (a warp that skipped a phase could not tell parities apart).
      const int SG = S / G;
      for (int it = 0; it < my_ntiles; ++it) {
        const int jt = it / G;
        const int s = (jt % SG) * G + (it % G);
        if (jt >= SG && !mbar_wait(&ctrl->empty[s], (unsigned)(((jt / SG) - 1) & 1), &ctrl->timeout,
                                   P.wait_limit_ns))
          atomicOr(P.status, kStatusTimeout);
        // tuning builds: leave the last tile out, so that its consumers' wait runs out (a test of
        // the bounded wait; nothing is read or written out of place)
        if (RA_DEBUG(P, 32) && it == my_ntiles - 1) continue;
        const int tok = tok_begin + it * T;
        unsigned char* dst = stages + (size_t)s * kStageBytes;
        mbar_expect_tx(&ctrl->full[s], kStageBytes);
        if constexpr (MODE == 2) {
          // two 64-dim halves with the 128-byte swizzle (operands of ldmatrix)
          if (P.head_major) {
            tma_load_4d(dst, &P.kmap, &ctrl->full[s], 0, tok, h0, kv_b);
            tma_load_4d(dst + kSwzHalfBytes, &P.kmap, &ctrl->full[s], 64, tok, h0, kv_b);
          } else {
            tma_load_4d(dst, &P.kmap, &ctrl->full[s], 0, h0, tok, kv_b);
            tma_load_4d(dst + kSwzHalfBytes, &P.kmap, &ctrl->full[s], 64, h0, tok, kv_b);
          }
        } else {
          if (P.head_major)
            tma_load_4d(dst, &P.kmap, &ctrl->full[s], 0, tok, h0, kv_b);
          else
            tma_load_4d(dst, &P.kmap, &ctrl->full[s], 0, h0, tok, kv_b);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ consumer warps
    // Group g takes tiles g, g+G, ...; inside a tile a warp owns (kv head hh, 16 consecutive
    // tokens): 4 passes of 4 rows, 8 lanes per 256-byte row.
    const int grp = warp >> 3, w8 = warp & 7;
    const int hh = w8 % HG;
    const int tw = w8 / HG;
    const int r = lane >> 3, j = lane & 7;
    const int b2 = (j >> 2) & 1, b1 = (j >> 1) & 1, b0l = j & 1;
    const int my_p = j >> 1;  // pass whose score this lane ends up with
    const int my_qpar = b0l;  // parity of the queries it ends up with

    // query fragments: dims [8j,8j+8) and [64+8j,64+8j+8) of each query, packed fp16
    uint32_t qh[NQ][8];
#pragma unroll
    for (int qi = 0; qi < NQ; ++qi) {
      if (qi < P.nq_cta && q0 + qi < P.nq_valid) {
        const int bq = b0 + (q0 + qi) / P.group;
        const int hq = (h0 + hh) * P.group + (q0 + qi) % P.group;
        const __half* qp = P.q + ((size_t)bq * P.hq + hq) * kHeadDim;
        const uint4 a = *reinterpret_cast<const uint4*>(qp + 8 * j);
        const uint4 b = *reinterpret_cast<const uint4*>(qp + 64 + 8 * j);
        qh[qi][0] = a.x; qh[qi][1] = a.y; qh[qi][2] = a.z; qh[qi][3] = a.w;
        qh[qi][4] = b.x; qh[qi][5] = b.y; qh[qi][6] = b.z; qh[qi][7] = b.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) qh[qi][i] = 0u;
      }
    }

    // the lists this lane appends to and their thresholds
    int my_list[NV];
    uint32_t my_thr[NV];
    bool my_valid[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int qi = 2 * v + my_qpar;
      my_valid[v] = (NQ == 1) ? (b0l == 0) : (qi < P.nq_cta && q0 + qi < P.nq_valid && qi < NQ);
      my_list[v] = hh * NQ + ((NQ == 1) ? 0 : min(qi, NQ - 1));
      my_thr[v] = 0u;
    }
    const unsigned grp_mask = my_qpar ? 0xAAAAAAAAu : 0x55555555u;
    const unsigned lt_mask = (1u << lane) - 1u;

    const uint32_t stage0 = smem_u32(stages);
    const uint32_t row_off = (uint32_t)(((tw * 16 + r) * HG + hh) * kRowBytes + j * 16);

    // Tensor-core scoring (MODE 2): the queries that share a K row (GQA group and/or batch rows
    // on one cache, <= 8) are the N dimension of an m16n8k16 product whose M dimension is this
    // warp's 16 tokens.  Lane (g, t) holds B fragments of query g and ends up with the scores
    // of tokens g, g+8 for queries 2t, 2t+1.
    const int mg = lane >> 2, mt = lane & 3;
    uint32_t qb[8][2];
    uint32_t thr2[2] = {0u, 0u};
    const int a_tok = w8 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
    const int a_c8 = lane >> 4;
    if constexpr (MODE == 2) {
      if (mg < P.nq_cta && q0 + mg < P.nq_valid) {
        const int bq = b0 + (q0 + mg) / P.group;
        const int hq = h0 * P.group + (q0 + mg) % P.group;
        const __half* qp = P.q + ((size_t)bq * P.hq + hq) * kHeadDim;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          qb[kk][0] = *reinterpret_cast<const uint32_t*>(qp + 16 * kk + 2 * mt);
          qb[kk][1] = *reinterpret_cast<const uint32_t*>(qp + 16 * kk + 8 + 2 * mt);
        }
      } else {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) qb[kk][0] = qb[kk][1] = 0u;
      }
    }
    const int iters = ceil_div(my_ntiles, G);
    const int SG = S / G;  // stages in this group's ring

#pragma unroll 1
    for (int jt = 0; jt < iters; ++jt) {
      const int it = jt * G + grp;
      if (it < my_ntiles) {
        const int s = (jt % SG) * G + grp;
        if (!mbar_wait(&ctrl->full[s], (unsigned)((jt / SG) & 1), &ctrl->timeout, P.wait_limit_ns)) {
          if (lane == 0) atomicOr(P.status, kStatusTimeout);
        }
        if constexpr (MODE == 2) {
          const uint32_t tbase = stage0 + (uint32_t)s * kStageBytes;
          float c[4] = {0.f, 0.f, 0.f, 0.f};
          if (!RA_DEBUG(P, 1)) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              uint32_t a[4];
              ldmatrix_x4(a, tbase + swz128(a_tok, 2 * kk + a_c8));
              mma_16816(c, a, qb[kk][0], qb[kk][1]);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctrl->empty[s]);
          const int tok_lo = tok_begin + it * T + w8 * 16 + mg;
          const unsigned tmask = 0x11111111u << mt;  // the lanes that share my two queries
#pragma unroll
          for (int jv = 0; jv < 4; ++jv) {
            const int qi = 2 * mt + (jv & 1);
            const int tok = tok_lo + 8 * (jv >> 1);
            const uint32_t key = score_key(c[jv]);
            const bool pass = qi < P.nq_cta && q0 + qi < P.nq_valid && tok < part_hi &&
                              key > thr2[jv & 1] && !RA_DEBUG(P, 4);
            const unsigned bal = __ballot_sync(0xffffffffu, pass);
            if (bal) {
              const unsigned mym = bal & tmask;
              const int leader = mym ? (__ffs(mym) - 1) : 0;
              int basepos = 0;
              if (pass && lane == leader) basepos = atomicAdd(&ctrl->cnt[qi], __popc(mym));
              basepos = __shfl_sync(0xffffffffu, basepos, leader);
              if (pass) {
                const int pos = basepos + __popc(mym & lt_mask);
                if (pos < cap) {
                  keys[(size_t)qi * cap + pos] = key;
                  idxs[(size_t)qi * cap + pos] = tok;
                } else {
                  atomicOr(P.status, kStatusOverflow);
                }
              }
            }
          }
        } else {
        const uint32_t base = stage0 + (uint32_t)s * kStageBytes + row_off;
        float part_sum[NQ][4];
        if (!RA_DEBUG(P, 1)) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const uint32_t addr = base + (uint32_t)(p * 4 * HG * kRowBytes);
            const uint4 a = lds128(addr);
            const uint4 b = lds128(addr + 128);
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int qi = 0; qi < NQ; ++qi) {
              float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
              for (int i = 0; i < 8; i += 2) {
                fma_pair<MIXED>(a0, a1, w[i], qh[qi][i]);
                fma_pair<MIXED>(a2, a3, w[i + 1], qh[qi][i + 1]);
              }
              part_sum[qi][p] = (a0 + a1) + (a2 + a3);
            }
          }
        } else {
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi)
#pragma unroll
            for (int p = 0; p < 4; ++p) part_sum[qi][p] = 0.f;
        }
        // the stage is free as soon as this warp's loads have returned
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctrl->empty[s]);

        // transposing butterfly over the 8 lanes of a row: after three exchange steps each lane
        // holds the complete dot product of pass (j >> 1) for the queries of parity (j & 1)
        float mine[NV];
        float red2[NQ];
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          const float s0 = b2 ? part_sum[qi][0] : part_sum[qi][2];
          const float s1 = b2 ? part_sum[qi][1] : part_sum[qi][3];
          float k0 = b2 ? part_sum[qi][2] : part_sum[qi][0];
          float k1 = b2 ? part_sum[qi][3] : part_sum[qi][1];
          k0 += __shfl_xor_sync(0xffffffffu, s0, 4);
          k1 += __shfl_xor_sync(0xffffffffu, s1, 4);
          const float s2 = b1 ? k0 : k1;
          float kk = b1 ? k1 : k0;
          kk += __shfl_xor_sync(0xffffffffu, s2, 2);
          red2[qi] = kk;
        }
        if constexpr (NQ == 1) {
          mine[0] = red2[0] + __shfl_xor_sync(0xffffffffu, red2[0], 1);
        } else {
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            const float snd = b0l ? red2[2 * v] : red2[2 * v + 1];
            float kept = b0l ? red2[2 * v + 1] : red2[2 * v];
            kept += __shfl_xor_sync(0xffffffffu, snd, 1);
            mine[v] = kept;
          }
        }
        // append the scores above the threshold
        const int tok = tok_begin + it * T + tw * 16 + my_p * 4 + r;
        const bool in_range = tok < part_hi;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const uint32_t key = score_key(mine[v]);
          const bool pass = my_valid[v] && in_range && key > my_thr[v] && !RA_DEBUG(P, 4);
          const unsigned bal = __ballot_sync(0xffffffffu, pass);
          if (bal) {
            const unsigned mym = bal & grp_mask;
            const int leader = mym ? (__ffs(mym) - 1) : 0;
            int basepos = 0;
            if (pass && lane == leader) basepos = atomicAdd(&ctrl->cnt[my_list[v]], __popc(mym));
            basepos = __shfl_sync(0xffffffffu, basepos, leader);
            if (pass) {
              const int pos = basepos + __popc(mym & lt_mask);
              if (pos < cap) {
                keys[(size_t)my_list[v] * cap + pos] = key;
                idxs[(size_t)my_list[v] * cap + pos] = tok;
              } else {
                atomicOr(P.status, kStatusOverflow);
              }
            }
          }
        }
        }  // scoring on the CUDA cores
      }
      // Every R iterations all consumer warps meet; a list that could overflow before the next
      // meeting is cut back to its k best.  The counters are settled between the two barriers,
      // so every thread takes the same decision.
      if ((jt + 1) % R == 0) {
        consumer_sync(nct);
        int need = 0;
#pragma unroll
        for (int l = 0; l < NL; ++l)
          if (ctrl->cnt[l] > cap - R * G * T && !RA_DEBUG(P, 8)) need |= 1 << l;
        consumer_sync(nct);
        if (need) {
          compact_lists<NL>(keys, idxs, ctrl, need, k, cap, accept, tid, nct);
#pragma unroll
          for (int v = 0; v < NV; ++v) my_thr[v] = ctrl->thr[my_list[v]];
          if constexpr (MODE == 2) {
            thr2[0] = ctrl->thr[min(2 * mt, NL - 1)];
            thr2[1] = ctrl->thr[min(2 * mt + 1, NL - 1)];
          }
        }
      }
    }
  }
  __syncthreads();

  RA_STAMP(P.status, 1);
  if (RA_DEBUG(P, 16)) return;  // tuning aid: time the scan without the merge
  // ------------------------------------------------------------------ cluster merge
  // The pipeline stages are free now and become the merge scratch.
  MergeArgs A = P.m;
  A.list_off = part * k;
  auto dest = [&](int l) {
    ListDest d;
    const int lh = l / NQ, qi = l % NQ;
    d.valid = qi < P.nq_cta && q0 + qi < P.nq_valid;
    d.bq = b0 + (q0 + qi) / P.group;
    d.hkv = h0 + lh;
    d.hq = (h0 + lh) * P.group + (q0 + qi) % P.group;
    return d;
  };
  cluster_select_attend<NL>(cluster, stages, keys, idxs, ctrl->cnt, cap, A, dest, tok_begin,
                            max(my_ntiles, 1) * T);
}

size_t scan_smem_bytes(int nl, int cap, int nstages) {
  return (size_t)nstages * kStageBytes + (size_t)nl * cap * 8 + sizeof(Ctrl) + 128;
}
size_t merge_scratch_bytes(int nl, int per, int det_words) { return select_scratch_bytes(nl, per, det_words); }

// ---------------------------------------------------------------------------- launcher
template <int HG, int NQ>
static cudaError_t launch_one(const ScanParams& P, int grid, size_t smem, cudaStream_t stream) {
  auto kern = scan_select_kernel<HG, NQ, 1>;
#ifdef RA_TUNING
  if (P.debug & 2) kern = scan_select_kernel<HG, NQ, 0>;
#endif
  if constexpr (HG == 1 && NQ > 1) {
    if (P.swizzled) kern = scan_select_kernel<1, NQ, 2>;
  }
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  if (P.m.cluster > 8) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(32 * (8 * P.groups + 1), 1, 1);
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

cudaError_t launch_scan_select(const ScanParams& P, int hg, int nq, int grid, size_t smem,
                               cudaStream_t stream) {
#define RA_CASE(H, Q) \
  if (hg == H && nq == Q) return launch_one<H, Q>(P, grid, smem, stream);
  RA_CASE(1, 1) RA_CASE(2, 1) RA_CASE(4, 1) RA_CASE(8, 1)
  RA_CASE(1, 2) RA_CASE(2, 2) RA_CASE(4, 2)
  RA_CASE(1, 4) RA_CASE(2, 4)
  RA_CASE(1, 8)
#undef RA_CASE
  return cudaErrorInvalidValue;
}

}  // namespace ra

namespace ra {

template <int HG, int NQ>
static int max_clusters_one(int cluster, size_t smem, int threads) {
  auto kern = scan_select_kernel<HG, NQ, 1>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (cluster > 8 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)cluster * 64, 1, 1);
  cfg.blockDim = dim3((unsigned)threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

// Clusters of this shape that can be resident at once on the current device (cached).
int scan_max_active_clusters(int hg, int nq, int cluster, size_t smem, int threads) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, int, size_t>, int> cache;
  const auto key = std::make_tuple(hg, nq, cluster * 4096 + threads, (smem + 4095) / 4096);
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  int n = 0;
#define RA_CASE(H, Q) \
  if (hg == H && nq == Q) n = max_clusters_one<H, Q>(cluster, smem, threads);
  RA_CASE(1, 1) RA_CASE(2, 1) RA_CASE(4, 1) RA_CASE(8, 1)
  RA_CASE(1, 2) RA_CASE(2, 2) RA_CASE(4, 2)
  RA_CASE(1, 4) RA_CASE(2, 4)
  RA_CASE(1, 8)
#undef RA_CASE
  std::lock_guard<std::mutex> g(mu);
  cache[key] = n;
  return n;
}

}  // namespace ra
