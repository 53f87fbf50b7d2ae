// Second-stage kernel: exact k-select over candidate (score, id) lists held in global memory,
// then softmax.V over the winners.  Used when one head's context was scanned by several
// clusters (each wrote its own k candidates), for the legacy per-chunk selection (every chunk's
// k winners are all attended) and, with an ownership window, for the sequence-sharded path
// (candidates of all ranks are merged; each rank mixes only the V rows it holds and emits an
// un-normalised partial).  The role of retrieval_reduce_kernel
// (retrieval_attn/retrieval_attention.cu:1243-1339) generalised with a selection step.
#include "merge_attend.cuh"

#include <cstring>

namespace ra {

__global__ void __launch_bounds__(kMergeThreads, 1)
merge_attend_kernel(const __grid_constant__ MergeParams P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.m.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x;
  const int row = blockIdx.x / C;  // (batch row, query head)
  const int bq = row / P.m.hq_total, hq = row % P.m.hq_total;

  const size_t scratch_bytes = select_scratch_bytes(1, P.m.per, P.m.det_words);
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem + scratch_bytes);
  int* idxs = reinterpret_cast<int*>(keys + P.cap);
  int* cnt = idxs + P.cap;

  const int chunk = ceil_div(P.m_total, C);
  const int lo = crank * chunk;
  const int n = max(0, min(P.m_total, lo + chunk) - lo);
  for (int i = tid; i < n; i += kMergeThreads) {
    const int c = lo + i;
    const int part = c / P.part_len, off = c - part * P.part_len;
    const size_t src = (size_t)part * P.part_stride + (size_t)row * P.row_stride + off;
    keys[i] = score_key(P.cand_score[src]);
    idxs[i] = (P.own_part < 0 || part == P.own_part) ? P.cand_idx[src] : -1;
  }
  if (tid == 0) cnt[0] = n;
  __syncthreads();

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
  cluster_select_attend<1>(cluster, smem, keys, idxs, cnt, P.cap, A, dest);
}

size_t merge_attend_smem_bytes(int per, int cap) {
  return select_scratch_bytes(1, per, det_words_for(cap)) + (size_t)cap * 8 + 16 + 128;
}

cudaError_t launch_merge_attend(const MergeParams& P, int rows, size_t smem, cudaStream_t stream) {
  auto kern = merge_attend_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  if (P.m.cluster > 8) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * P.m.cluster), 1, 1);
  cfg.blockDim = dim3(kMergeThreads, 1, 1);
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

// One CTA of 128 threads per output row.  The (maximum, weight) pairs of all parts are fetched by
// as many threads at once, one warp turns them into the common maximum and the parts' weights,
// then thread d sums dimension d over the parts with eight loads in flight (one load at a time
// would cost a full L2 round trip per part).
constexpr int kCombineMaxParts = 1024;

__global__ void __launch_bounds__(kHeadDim)
lse_combine_kernel(const float* __restrict__ partials, int parts, int rows, __half* __restrict__ out,
                   const ExchangeHooks X, unsigned* status) {
  __shared__ float wt[kCombineMaxParts];
  __shared__ float wsum4[4];
  exchange_wait_in_kernel(X, status);   // every rank's partial has landed (bounded wait)
  const int row = blockIdx.x, d = threadIdx.x, lane = d & 31;
  const size_t pitch = (size_t)rows * (kHeadDim + 2);
  const float* base = partials + (size_t)row * (kHeadDim + 2);
  float o = 0.f;
  if (parts <= kCombineMaxParts) {
    float m = -INFINITY;
    for (int p = d; p < parts; p += kHeadDim) m = fmaxf(m, __ldcg(base + (size_t)p * pitch + kHeadDim + 1));
#pragma unroll
    for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (lane == 0) wt[d >> 5] = m;
    __syncthreads();
    m = fmaxf(fmaxf(wt[0], wt[1]), fmaxf(wt[2], wt[3]));
    __syncthreads();
    float l = 0.f;
    for (int p = d; p < parts; p += kHeadDim) {
      const float lp = __ldcg(base + (size_t)p * pitch + kHeadDim);
      const float w = (lp > 0.f) ? __expf(__ldcg(base + (size_t)p * pitch + kHeadDim + 1) - m) : 0.f;
      wt[p] = w;
      l = fmaf(w, lp, l);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    if (lane == 0) wsum4[d >> 5] = l;
    __syncthreads();
    const float total = (wsum4[0] + wsum4[1]) + (wsum4[2] + wsum4[3]);   // fixed order: same bits every run
    for (int p0 = 0; p0 < parts; p0 += 8) {
      float x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) x[u] = (p0 + u < parts) ? __ldcg(base + (size_t)(p0 + u) * pitch + d) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (p0 + u < parts) o = fmaf(wt[p0 + u], x[u], o);
    }
    out[(size_t)row * kHeadDim + d] = __float2half_rn(o / total);
  } else {
    float m = -INFINITY;
    for (int p = 0; p < parts; ++p) m = fmaxf(m, base[(size_t)p * pitch + kHeadDim + 1]);
    float l = 0.f;
    for (int p = 0; p < parts; ++p) {
      const float* src = base + (size_t)p * pitch;
      const float lp = src[kHeadDim];
      const float w = (lp > 0.f) ? __expf(src[kHeadDim + 1] - m) : 0.f;
      o = fmaf(w, src[d], o);
      l = fmaf(w, lp, l);
    }
    out[(size_t)row * kHeadDim + d] = __float2half_rn(o / l);
  }
  exchange_publish_in_kernel(X);        // ends the step: the last CTA advances the epoch
}

cudaError_t launch_lse_combine(const float* partials, int parts, int rows, __half* out,
                               cudaStream_t stream, const ExchangeHooks* x, unsigned* status) {
  ExchangeHooks hooks;
  memset(&hooks, 0, sizeof hooks);
  if (x) hooks = *x;
  note_launch();
  lse_combine_kernel<<<rows, kHeadDim, 0, stream>>>(partials, parts, rows, out, hooks, status);
  return cudaGetLastError();
}

}  // namespace ra

namespace ra {

// Single-CTA form of the candidate merge for lists that fit in one CTA's shared memory (up to
// about 22 000 candidates per row): no cluster barriers, 1024 threads.  The exact k-th key is
// found by a radix select over (key - smallest key), which starts at the highest bit that differs
// and spreads the histogram atomics over the bins; winners are compacted, written out if asked for,
// and their V rows mixed by all 32 warps.
constexpr int kMergeCtaThreads = 1024;

struct MergeCtaCtrl {
  int hist[256];
  uint32_t kmin, kmax;
  int digit, remaining, wpos, eqc, cut;
  int own_first, own_last;   // range of winner slots whose ids this rank owns
  int wsum[kMaxWarps + 2];
  float lred[32];
};

__global__ void __launch_bounds__(kMergeCtaThreads, 1)
merge_attend_cta_kernel(const __grid_constant__ MergeParams P) {
  extern __shared__ __align__(16) unsigned char smem_m[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = blockIdx.x;
  const int bq = row / P.m.hq_total, hq = row % P.m.hq_total;
  const int hkv = hq / P.group;
  const int n = P.m_total, k = P.m.topk;
  // candidate ids stay in global memory when keys and ids together would not fit (they are only
  // needed for the k winners)
  const bool ids_global = P.ids_global != 0;
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem_m);
  int* idxs = reinterpret_cast<int*>(keys + n);
  uint32_t* wkey = reinterpret_cast<uint32_t*>(idxs + (ids_global ? 0 : n));  // winners
  int* widx = reinterpret_cast<int*>(wkey + k);
  float* red = reinterpret_cast<float*>(widx + k);         // [32][128]
  MergeCtaCtrl* ctrl = reinterpret_cast<MergeCtaCtrl*>(red + 32 * kHeadDim);
  uint32_t* bits = reinterpret_cast<uint32_t*>(ctrl + 1);   // one bit per candidate
  int* wpre = reinterpret_cast<int*>(bits + ((n + 31) >> 5));
  auto src_of = [&](int c) {
    const int part = c / P.part_len, off = c - part * P.part_len;
    return (size_t)part * P.part_stride + (size_t)row * P.row_stride + off;
  };
  // whether the id of candidate c may be read (with own_part only this rank's own proposals carry ids)
  auto readable = [&](int c) { return P.own_part < 0 || c / P.part_len == P.own_part; };

  if (tid == 0) {
    ctrl->kmin = 0xffffffffu;
    ctrl->kmax = 0u;
    ctrl->wpos = 0;
    ctrl->eqc = 0;
    ctrl->own_first = 0x7fffffff;
    ctrl->own_last = -1;
  }
  RA_STAMP(P.m.status, 0);
  exchange_wait_in_kernel(P.x, P.m.status);   // the peers' candidates have landed (bounded wait)
  __syncthreads();
  RA_STAMP(P.m.status, 1);
  uint32_t mn = 0xffffffffu, mx = 0u;
  // several loads in flight per thread: the lists come from L2 or from a peer's stores.  Lists
  // whose length and strides are multiples of four elements are read 16 bytes at a time.
  const bool vec = (P.part_len % 4 == 0) && (P.part_stride % 4 == 0) && (P.row_stride % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(P.cand_score) | reinterpret_cast<uintptr_t>(P.cand_idx)) & 15u) == 0;
  if (vec) {
    constexpr int LU = 4;
    for (int c0 = 0; c0 < n; c0 += kMergeCtaThreads * LU * 4) {
      float4 sc[LU];
      int4 id[LU];
#pragma unroll
      for (int u = 0; u < LU; ++u) {
        const int c = c0 + (u * kMergeCtaThreads + tid) * 4;
        sc[u] = c < n ? *reinterpret_cast<const float4*>(P.cand_score + src_of(c)) : make_float4(0.f, 0.f, 0.f, 0.f);
        id[u] = (c < n && !ids_global && readable(c)) ? *reinterpret_cast<const int4*>(P.cand_idx + src_of(c))
                                                      : make_int4(-1, -1, -1, -1);
      }
#pragma unroll
      for (int u = 0; u < LU; ++u) {
        const int c = c0 + (u * kMergeCtaThreads + tid) * 4;
        if (c < n) {
          const uint4 kq = make_uint4(score_key(sc[u].x), score_key(sc[u].y), score_key(sc[u].z),
                                      score_key(sc[u].w));
          *reinterpret_cast<uint4*>(keys + c) = kq;
          if (!ids_global) *reinterpret_cast<int4*>(idxs + c) = id[u];
          mn = min(min(mn, kq.x), min(min(kq.y, kq.z), kq.w));
          mx = max(max(mx, kq.x), max(max(kq.y, kq.z), kq.w));
        }
      }
    }
  } else {
    constexpr int LU = 8;
    for (int c0 = 0; c0 < n; c0 += kMergeCtaThreads * LU) {
      float sc[LU];
      int id[LU];
#pragma unroll
      for (int u = 0; u < LU; ++u) {
        const int c = c0 + u * kMergeCtaThreads + tid;
        sc[u] = c < n ? P.cand_score[src_of(c)] : 0.f;
        id[u] = (c < n && !ids_global && readable(c)) ? P.cand_idx[src_of(c)] : -1;
      }
#pragma unroll
      for (int u = 0; u < LU; ++u) {
        const int c = c0 + u * kMergeCtaThreads + tid;
        if (c < n) {
          const uint32_t key = score_key(sc[u]);
          keys[c] = key;
          if (!ids_global) idxs[c] = id[u];
          mn = min(mn, key);
          mx = max(mx, key);
        }
      }
    }
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) {
    mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  if (lane == 0) {
    atomicMin(&ctrl->kmin, mn);
    atomicMax(&ctrl->kmax, mx);
  }
  __syncthreads();
  RA_STAMP(P.m.status, 2);
  const uint32_t base = ctrl->kmin, maxkey = ctrl->kmax;
  int shift = max(0, 32 - __clz((int)((maxkey - base) | 1u)) - 8);
  uint32_t prefix = 0u, mask = 0u;
  int remaining = min(k, n);
#pragma unroll 1
  for (;;) {
    if (tid < 256) ctrl->hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += kMergeCtaThreads) {
      const uint32_t rel = keys[i] - base;
      if ((rel & mask) == prefix) atomicAdd(&ctrl->hist[(rel >> shift) & 255], 1);
    }
    __syncthreads();
    if (tid < 32) {
      int d, nr;
      warp_find_digit(ctrl->hist, remaining, lane, d, nr);
      if (lane == 0) {
        ctrl->digit = d;
        ctrl->remaining = nr;
      }
    }
    __syncthreads();
    prefix |= (uint32_t)ctrl->digit << shift;
    mask = 0xffffffffu << shift;
    remaining = ctrl->remaining;
    if (shift == 0) break;
    shift = max(0, shift - 8);
  }
  RA_STAMP(P.m.status, 3);
  const uint32_t kth = base + prefix;
  const int need_eq = remaining;
  // Winners in a fixed order, so that every rank that merges the same candidates picks the same keys
  // and the same input always gives the same output bits: candidates are ranked by their position
  // in the candidate array (ranks in order, each rank's list in the order it was written); of the
  // copies of the k-th key the first need_eq are taken.
  const int nwords = (n + 31) >> 5;
  // the last pass ran at shift 0: the chosen bin of its histogram holds the copies of the k-th key
  const int n_eq = ctrl->hist[ctrl->digit];
  int cut = need_eq >= n_eq ? 0x7fffffff : -1;
  if (need_eq > 0 && need_eq < n_eq) {
    for (int w = tid; w < nwords; w += kMergeCtaThreads) bits[w] = 0u;
    __syncthreads();
    for (int i = tid; i < n; i += kMergeCtaThreads)
      if (keys[i] == kth) atomicOr(&bits[i >> 5], 1u << (i & 31));
    __syncthreads();
    bitmap_prefix(bits, wpre, ctrl->wsum, nwords, tid, kMergeCtaThreads);
    for (int w = tid; w < nwords; w += kMergeCtaThreads) {
      const int before = wpre[w];
      const uint32_t word = bits[w];
      if (before < need_eq && need_eq <= before + __popc(word))
        ctrl->cut = 32 * w + (int)__fns(word, 0, need_eq - before);
    }
    __syncthreads();
    cut = ctrl->cut;
  }
  for (int w = tid; w < nwords; w += kMergeCtaThreads) bits[w] = 0u;
  __syncthreads();
  for (int i = tid; i < n; i += kMergeCtaThreads) {
    const uint32_t key = keys[i];
    if (key > kth || (key == kth && i <= cut)) atomicOr(&bits[i >> 5], 1u << (i & 31));
  }
  __syncthreads();
  const int total_win = bitmap_prefix(bits, wpre, ctrl->wsum, nwords, tid, kMergeCtaThreads);
  int my_first = 0x7fffffff, my_last = -1;
  for (int i = tid; i < n; i += kMergeCtaThreads) {
    const uint32_t key = keys[i];
    if (key > kth || (key == kth && i <= cut)) {
      const int p = wpre[i >> 5] + __popc(bits[i >> 5] & ((1u << (i & 31)) - 1u));
      if (p < k) {
        const int id = ids_global ? (readable(i) ? P.cand_idx[src_of(i)] : -1) : idxs[i];
        wkey[p] = key;
        widx[p] = id;
        // first and last winner slot this rank owns: the mixing loop only walks that range
        if (id >= P.m.own_lo && id < P.m.own_hi) {
          my_first = min(my_first, p);
          my_last = max(my_last, p);
        }
      }
    }
  }
  my_first = __reduce_min_sync(0xffffffffu, my_first);
  my_last = __reduce_max_sync(0xffffffffu, my_last);
  if (lane == 0 && my_last >= 0) {
    atomicMin(&ctrl->own_first, my_first);
    atomicMax(&ctrl->own_last, my_last);
  }
  if (tid == 0) ctrl->wpos = total_win;
  __syncthreads();
  RA_STAMP(P.m.status, 4);
  const int nw = min(ctrl->wpos, k);
  if (P.m.sel_idx) {
    const size_t dst = (size_t)row * P.m.list_pitch + P.m.list_off;
    for (int e = tid; e < k; e += kMergeCtaThreads) {
      P.m.sel_idx[dst + e] = (e < nw) ? widx[e] + P.m.index_base : -1;
      if (P.m.sel_score) P.m.sel_score[dst + e] = (e < nw) ? key_score(wkey[e]) : -INFINITY;
    }
  }
  if (P.m.out_mode == kOutNone) return;

  const float smax = key_score(maxkey);
  const __half* vb = P.m.v + (size_t)bq * P.m.v_batch_stride + (size_t)hkv * P.m.v_head_stride +
                     (lane & 15) * 8;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  float lsum = 0.f;
  constexpr int UN = 8;
  constexpr int kRows = 2 * (kMergeCtaThreads / 32);
  // only the slots between the first and the last winner this rank owns can contribute (in the
  // sharded step that is one contiguous run: the winners proposed by this rank itself)
  const int e_begin = min(ctrl->own_first, nw), e_end = min(nw, ctrl->own_last + 1);
  for (int e0 = e_begin + warp * 2 + (lane >> 4); e0 < e_end; e0 += kRows * UN) {
    uint4 vv[UN];
    float w[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int e = e0 + kRows * u;
      const int id = (e < e_end) ? widx[e] : -1;
      const int local = id - P.m.id_shift;
      const bool mine = id >= P.m.own_lo && id < P.m.own_hi;
      if (mine && (unsigned)local >= (unsigned)P.m.n_tokens) atomicOr(P.m.status, kStatusBadId);
      if (mine && (unsigned)local < (unsigned)P.m.n_tokens) {
        w[u] = fast_exp2((key_score(wkey[e]) - smax) * P.m.scale_log2e);
        vv[u] = ldg128_nc(vb + (size_t)local * P.m.v_token_stride);
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
    for (int i = 0; i < 8; ++i) red[warp * kHeadDim + lane * 8 + i] = acc[i];
  }
  if (lane == 0) ctrl->lred[warp] = lsum;
  __syncthreads();
  if (tid < kHeadDim) {
    float o = 0.f, lt = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) {
      o += red[w * kHeadDim + tid];
      lt += ctrl->lred[w];
    }
    const float mscaled = smax * P.m.sm_scale;
    if (P.m.out_mode == kOutFinal) {
      P.m.out[(size_t)row * kHeadDim + tid] = __float2half_rn(o / lt);
      if (P.m.out_lse && tid == 0) {
        P.m.out_lse[(size_t)row * 2 + 0] = mscaled;
        P.m.out_lse[(size_t)row * 2 + 1] = lt;
      }
    } else {
      // this rank's partial row, and the same row into this rank's slot on every peer
      const size_t roff = (size_t)row * (kHeadDim + 2);
      float* dstp = P.m.out_partial + roff;
      dstp[tid] = o;
      if (tid == 0) {
        dstp[kHeadDim] = lt;
        dstp[kHeadDim + 1] = mscaled;
      }
      for (int p = 0; p < P.x.npeers; ++p) {
        float* pr = P.x.peer_rows[p];
        if (pr == nullptr || pr == P.m.out_partial) continue;
        pr[roff + tid] = o;
        if (tid == 0) {
          pr[roff + kHeadDim] = lt;
          pr[roff + kHeadDim + 1] = mscaled;
        }
      }
    }
  }
  RA_STAMP(P.m.status, 5);
  exchange_publish_in_kernel(P.x);
  RA_STAMP(P.m.status, 6);
}

size_t merge_attend_cta_smem_bytes(int m_total, int topk, bool ids_global) {
  return (size_t)m_total * (ids_global ? 4 : 8) + (size_t)topk * 8 + 32 * kHeadDim * 4 +
         sizeof(MergeCtaCtrl) + (size_t)((m_total + 31) / 32) * 8 + 64;
}

cudaError_t launch_merge_attend_cta(const MergeParams& P, int rows, size_t smem, cudaStream_t stream) {
  auto kern = merge_attend_cta_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  note_launch();
  kern<<<rows, kMergeCtaThreads, smem, stream>>>(P);
  return cudaGetLastError();
}

}  // namespace ra
