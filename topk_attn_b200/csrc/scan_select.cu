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
  int cnt[kMaxLists];
  uint32_t thr[kMaxLists];
  int hist[256];
  int digit, remaining, wpos, eqc;
  int need[2];  // lists to cut back after the next tile barrier (bit per list)
  int timeout;
};

// Raise the threshold of list `l` to its exact k-th largest key and keep only the k best.
// Called by all threads of the CTA.
__device__ void compact_list(uint32_t* keys, int* idxs, Ctrl* ctrl, int l, int k, int tid) {
  const int n = ctrl->cnt[l];
  const int lane = tid & 31;
  uint32_t prefix = 0, mask = 0;
  int remaining = k;
#pragma unroll 1
  for (int shift = 24; shift >= 0; shift -= 8) {
    ctrl->hist[tid] = 0;  // kThreads == 256 bins
    __syncthreads();
    for (int i = tid; i < n; i += kThreads) {
      const uint32_t key = keys[i];
      if ((key & mask) == prefix) atomicAdd(&ctrl->hist[(key >> shift) & 255], 1);
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
    mask |= 255u << shift;
    remaining = ctrl->remaining;
  }
  const uint32_t kth = prefix;
  const int need_eq = remaining;
  if (tid == 0) {
    ctrl->wpos = 0;
    ctrl->eqc = 0;
  }
  __syncthreads();
  constexpr int E = 8;
#pragma unroll 1
  for (int base = 0; base < n; base += kThreads * E) {
    uint32_t kk[E];
    int ii[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int i = base + e * kThreads + tid;
      kk[e] = (i < n) ? keys[i] : 0u;
      ii[e] = (i < n) ? idxs[i] : 0;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int i = base + e * kThreads + tid;
      if (i < n) {
        bool keep = kk[e] > kth;
        if (!keep && kk[e] == kth) keep = atomicAdd(&ctrl->eqc, 1) < need_eq;
        if (keep) {
          const int p = atomicAdd(&ctrl->wpos, 1);
          keys[p] = kk[e];
          idxs[p] = ii[e];
        }
      }
    }
    __syncthreads();
  }
  if (tid == 0) {
    ctrl->cnt[l] = ctrl->wpos;
    ctrl->thr[l] = kth;
  }
  __syncthreads();
}

template <int HG, int NQ>
__global__ void __launch_bounds__(kThreads, 1)
scan_select_kernel(const __grid_constant__ ScanParams P) {
  constexpr int NL = HG * NQ;
  static_assert(NL <= kMaxLists, "too many candidate lists per CTA");
  constexpr int T = kTileRows / HG;   // tokens per tile
  constexpr int NV = (NQ + 1) / 2;    // scores a lane keeps per tile
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.m.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cap = P.cap, k = P.m.topk;

  unsigned char* stages = smem;
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem + (size_t)P.nstages * kStageBytes);
  int* idxs = reinterpret_cast<int*>(keys + (size_t)NL * cap);
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(idxs + (size_t)NL * cap);

  // which part of which (batch group, kv-head group) this cluster owns
  int cid = blockIdx.x / C;
  const int part = cid % P.nparts;
  cid /= P.nparts;
  const int hgroups = P.hkv / HG;
  const int h0 = (cid % hgroups) * HG;
  const int b0 = (cid / hgroups) * P.bshare;
  const int kv_b = P.kv_per_batch ? b0 : 0;

  const int part_lo = part * P.part_len;
  const int part_hi = min(P.n_tokens, part_lo + P.part_len);
  const int ntiles_part = ceil_div(max(part_hi - part_lo, 0), T);
  const int tpc = ceil_div(ntiles_part, C);
  const int tile_b = crank * tpc;
  const int my_ntiles = max(0, min(ntiles_part, tile_b + tpc) - tile_b);
  const int tok_begin = part_lo + tile_b * T;

  if (tid == 0) {
    tma_prefetch_desc(&P.kmap);
    for (int s = 0; s < kMaxStages; ++s) mbar_init(&ctrl->full[s], 1);
    ctrl->timeout = 0;
    ctrl->need[0] = 0;
    ctrl->need[1] = 0;
    fence_barrier_init();
  }
  if (tid < kMaxLists) {
    ctrl->cnt[tid] = 0;
    ctrl->thr[tid] = 0u;
  }
  __syncthreads();

  auto issue = [&](int it) {
    const int s = it % P.nstages;
    const int tok = tok_begin + it * T;
    mbar_expect_tx(&ctrl->full[s], kStageBytes);
    if (P.head_major)
      tma_load_4d(stages + (size_t)s * kStageBytes, &P.kmap, &ctrl->full[s], 0, tok, h0, kv_b);
    else
      tma_load_4d(stages + (size_t)s * kStageBytes, &P.kmap, &ctrl->full[s], 0, h0, tok, kv_b);
  };
  if (tid == 0) {
    const int pre = min(P.nstages, my_ntiles);
    for (int it = 0; it < pre; ++it) issue(it);
  }

  // row ownership inside a tile: warp -> (kv head hh, 16 consecutive tokens), 4 passes of
  // 4 rows, 8 lanes per row
  const int hh = warp % HG;
  const int tw = warp / HG;
  const int r = lane >> 3, j = lane & 7;
  const int my_p = j & 3;      // pass whose score this lane keeps
  const int my_qpar = j >> 2;  // parity of the queries this lane keeps

  // query fragments: dims [8j,8j+8) and [64+8j,64+8j+8) of each query, fp32
  float qf[NQ][16];
#pragma unroll
  for (int qi = 0; qi < NQ; ++qi) {
    if (qi < P.nq_valid) {
      const int bq = b0 + qi / P.group;
      const int hq = (h0 + hh) * P.group + qi % P.group;
      const __half* qp = P.q + ((size_t)bq * P.hq + hq) * kHeadDim;
      const uint4 a = *reinterpret_cast<const uint4*>(qp + 8 * j);
      const uint4 b = *reinterpret_cast<const uint4*>(qp + 64 + 8 * j);
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = h2f2(w[i]);
        qf[qi][2 * i] = f.x;
        qf[qi][2 * i + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) qf[qi][i] = 0.f;
    }
  }

  // the lists this lane appends to and their thresholds
  int my_list[NV];
  uint32_t my_thr[NV];
  bool my_valid[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int qi = 2 * v + my_qpar;
    my_valid[v] = (NQ == 1) ? (j < 4) : (qi < P.nq_valid && qi < NQ);
    my_list[v] = hh * NQ + ((NQ == 1) ? 0 : min(qi, NQ - 1));
    my_thr[v] = 0u;
  }
  const unsigned grp_mask = my_qpar ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
  const unsigned lt_mask = (1u << lane) - 1u;

  const uint32_t stage0 = smem_u32(stages);
  const uint32_t row_off = (uint32_t)(((tw * 16 + r) * HG + hh) * kRowBytes + j * 16);

#pragma unroll 1
  for (int it = 0; it < my_ntiles; ++it) {
    const int s = it % P.nstages;
    if (!mbar_wait(&ctrl->full[s], (unsigned)((it / P.nstages) & 1))) {
      if (lane == 0) {
        ctrl->timeout = 1;
        atomicOr(P.status, kStatusTimeout);
      }
    }
    const uint32_t base = stage0 + (uint32_t)s * kStageBytes + row_off;
    float mine[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) mine[v] = 0.f;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const uint32_t addr = base + (uint32_t)(p * 4 * HG * kRowBytes);
      const uint4 a = lds128(addr);
      const uint4 b = lds128(addr + 128);
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      float kf[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = h2f2(w[i]);
        kf[2 * i] = f.x;
        kf[2 * i + 1] = f.y;
      }
#pragma unroll
      for (int qi = 0; qi < NQ; ++qi) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          a0 = fmaf(kf[i], qf[qi][i], a0);
          a1 = fmaf(kf[i + 1], qf[qi][i + 1], a1);
        }
        float acc = a0 + a1;
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        if (p == my_p && (qi & 1) == my_qpar) mine[qi >> 1] = acc;
      }
    }
    // append the scores above the threshold
    const int tok = tok_begin + it * T + tw * 16 + my_p * 4 + r;
    const bool in_range = tok < part_hi;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const uint32_t key = score_key(mine[v]);
      const bool pass = my_valid[v] && in_range && key > my_thr[v];
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
          }
        }
      }
    }
    __syncthreads();  // everyone is done with this stage
    if (tid == 0 && it + P.nstages < my_ntiles) issue(it + P.nstages);
    // Lists that could overflow are cut back to their k best.  The decision was taken by
    // thread 0 after the previous barrier, so every thread sees the same one; it leaves room
    // for the two tiles that may be appended before the cut happens.
    const int need = ctrl->need[it & 1];
    if (need) {
#pragma unroll
      for (int l = 0; l < NL; ++l)
        if ((need >> l) & 1)
          compact_list(keys + (size_t)l * cap, idxs + (size_t)l * cap, ctrl, l, k, tid);
#pragma unroll
      for (int v = 0; v < NV; ++v) my_thr[v] = ctrl->thr[my_list[v]];
    }
    if (tid == 0) {
      int m = 0;
#pragma unroll
      for (int l = 0; l < NL; ++l)
        if (ctrl->cnt[l] > cap - 2 * T) m |= 1 << l;
      ctrl->need[(it + 1) & 1] = m;
    }
  }
  __syncthreads();

  // ------------------------------------------------------------------ cluster merge
  // The pipeline stages are free now and become the merge scratch.
  MergeArgs A = P.m;
  A.list_off = part * k;
  auto dest = [&](int l) {
    ListDest d;
    const int lh = l / NQ, qi = l % NQ;
    d.valid = qi < P.nq_valid;
    d.bq = b0 + qi / P.group;
    d.hkv = h0 + lh;
    d.hq = (h0 + lh) * P.group + qi % P.group;
    return d;
  };
  cluster_select_attend<NL>(cluster, stages, keys, idxs, ctrl->cnt, cap, A, dest);
}

size_t scan_smem_bytes(int nl, int cap, int nstages) {
  return (size_t)nstages * kStageBytes + (size_t)nl * cap * 8 + sizeof(Ctrl) + 128;
}
size_t merge_scratch_bytes(int nl, int per) { return sizeof(MergeScratch) + (size_t)nl * per * 8; }

// ---------------------------------------------------------------------------- launcher
template <int HG, int NQ>
static cudaError_t launch_one(const ScanParams& P, int grid, size_t smem, cudaStream_t stream) {
  auto kern = scan_select_kernel<HG, NQ>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  if (P.m.cluster > 8) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)P.m.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
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
static int max_clusters_one(int cluster, size_t smem) {
  auto kern = scan_select_kernel<HG, NQ>;
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
  cfg.blockDim = dim3(kThreads, 1, 1);
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
int scan_max_active_clusters(int hg, int nq, int cluster, size_t smem) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, int, size_t>, int> cache;
  const auto key = std::make_tuple(hg, nq, cluster, (smem + 4095) / 4096);
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  int n = 0;
#define RA_CASE(H, Q) \
  if (hg == H && nq == Q) n = max_clusters_one<H, Q>(cluster, smem);
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
