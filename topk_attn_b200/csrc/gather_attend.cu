// Attention over a given list of key ids: scores q.K[id] (fp32), softmax, mix of V[id].  One
// cluster per (batch row, query head); the CTAs split the list, score their share with
// half-warp-per-row 128-bit gathers, then share maximum, weights and partial outputs through the
// common cluster code.  With expand_clen > 0 the list holds cluster ids which expand to their
// contiguous member tokens, in descending order of the cluster scores.
//
// The role of MHAFlashDecodeKernel (baseline_1.cu:324-610: index-gathered decode, KV split over
// the CTAs of a cluster, DSMEM max/sum combine, fp16 atomicAdd into a pre-zeroed output) and of
// the expansion loop of center_only_topk/gemv_topk.cu:271-279.  The output is written once, no
// atomics, no pre-zeroing.
#include "gather_attend.cuh"

namespace ra {

__global__ void __launch_bounds__(kMergeThreads, 1)
gather_attend_kernel(const __grid_constant__ GatherParams P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.m.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = blockIdx.x / C;
  const int bq = row / P.m.hq_total, hq = row % P.m.hq_total;
  const int hkv = hq / P.group;

  const size_t scratch_bytes = select_scratch_bytes(1, P.m.per, 0);
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem + scratch_bytes);
  int* idxs = reinterpret_cast<int*>(keys + P.cap);
  int* cnt = idxs + P.cap;
  int* src = cnt + 4;  // n_src ids in rank order

  // source ids of this (row, head); in expansion mode ordered by descending score
  const int* gsrc = P.src_idx + (size_t)bq * P.src_batch_stride + (size_t)hq * P.src_head_stride;
  if (P.expand_clen > 0 && P.src_score) {
    const float* gsc = P.src_score + (size_t)bq * P.src_batch_stride + (size_t)hq * P.src_head_stride;
    for (int i = tid; i < P.n_src; i += kMergeThreads) {
      const float si = gsc[i];
      const int ii = gsrc[i];
      int rank = 0;
      for (int j = 0; j < P.n_src; ++j) {
        const float sj = gsc[j];
        rank += (sj > si) || (sj == si && gsrc[j] < ii);
      }
      src[rank] = ii;
    }
  } else {
    for (int i = tid; i < P.n_src; i += kMergeThreads) src[i] = gsrc[i];
  }
  __syncthreads();

  const int chunk = ceil_div(P.n_entries, C);
  const int lo = crank * chunk;
  const int n = max(0, min(P.n_entries, lo + chunk) - lo);
  auto token_of = [&](int e) {
    return P.expand_clen > 0 ? src[e / P.expand_clen] * P.expand_clen + e % P.expand_clen : src[e];
  };
  if (P.out_token_ids) {
    int* dst = P.out_token_ids + (size_t)row * P.n_entries + lo;
    for (int i = tid; i < n; i += kMergeThreads) dst[i] = token_of(lo + i);
  }

  if (P.m.out_mode == kOutNone) return;  // expansion only; uniform over the whole grid

  // scores of my share: a half-warp per K row, 16 bytes per lane
  const int half = lane >> 4, l16 = lane & 15;
  float qf[8];
  {
    const uint4 a = *reinterpret_cast<const uint4*>(P.q + (size_t)row * kHeadDim + 8 * l16);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = h2f2(w[i]);
      qf[2 * i] = f.x;
      qf[2 * i + 1] = f.y;
    }
  }
  const __half* kb = P.k + (size_t)bq * P.m.v_batch_stride + (size_t)hkv * P.m.v_head_stride + l16 * 8;
  constexpr int UN = 8;
  constexpr int kRowsPerIter = 2 * (kMergeThreads / 32);
  // the trip count is the same for every lane: the shuffles below need the whole warp
  for (int base = 0; base < n; base += kRowsPerIter * UN) {
    const int e0 = base + warp * 2 + half;
    uint4 kk[UN];
    int tok[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int e = e0 + kRowsPerIter * u;
      tok[u] = (e < n) ? token_of(lo + e) : -1;
      const bool ok = (unsigned)tok[u] < (unsigned)P.m.n_tokens;
      if (e < n && !ok) atomicOr(P.m.status, kStatusBadId);
      kk[u] = ok ? ldg128_nc(kb + (size_t)tok[u] * P.m.v_token_stride) : make_uint4(0u, 0u, 0u, 0u);
      if (!ok) tok[u] = -1;
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const uint32_t w[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = h2f2(w[i]);
        acc = fmaf(f.x, qf[2 * i], acc);
        acc = fmaf(f.y, qf[2 * i + 1], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 8);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      const int e = e0 + kRowsPerIter * u;
      if (l16 == 0 && e < n) {
        // an id outside the cache keeps its slot (so positions stay dense) but can never weigh in
        keys[e] = tok[u] >= 0 ? score_key(acc) : 1u;
        idxs[e] = tok[u];
      }
    }
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
    d.hkv = hkv;
    return d;
  };
  cluster_select_attend<1>(cluster, smem, keys, idxs, cnt, P.cap, A, dest);
}

// Attention over the id list in one pass: every half-warp streams K and V rows of its ids
// together, keeps a running maximum / weight / weighted sum (online softmax in the log2 domain),
// and the partials are merged through their log-sum-exp inside the warp, across the warps in
// shared memory and across the CTAs of the cluster in distributed shared memory.
struct GatherPartial {
  float m, l;
  float o[kHeadDim];
};

// UN: K and V rows in flight per half-warp.  GIVEN: the list carries the raw scores q.K of its ids
// (src_score, expand_clen == 0), so only the V rows are read.
template <int UN, bool GIVEN>
__global__ void __launch_bounds__(kMergeThreads, 1)
gather_flash_kernel(const __grid_constant__ GatherParams P) {
  extern __shared__ __align__(16) unsigned char smem_g[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.m.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kW = kMergeThreads / 32;
  const int row = blockIdx.x / C;
  const int bq = row / P.m.hq_total, hq = row % P.m.hq_total;
  const int hkv = hq / P.group;
  GatherPartial* wpart = reinterpret_cast<GatherPartial*>(smem_g);  // [kW] per-warp partials
  GatherPartial* cpart = wpart + kW;                                // this CTA's partial (peers read)
  int* src = reinterpret_cast<int*>(cpart + 1);

  const int* gsrc = P.src_idx + (size_t)bq * P.src_batch_stride + (size_t)hq * P.src_head_stride;
  const float* gsc = nullptr;
  if (P.src_score)
    gsc = P.src_score + (size_t)bq * P.src_batch_stride + (size_t)hq * P.src_head_stride;
  if (!GIVEN && P.expand_clen > 0 && gsc) {
    for (int i = tid; i < P.n_src; i += kMergeThreads) {
      const float si = gsc[i];
      const int ii = gsrc[i];
      int rank = 0;
      for (int j = 0; j < P.n_src; ++j) {
        const float sj = gsc[j];
        rank += (sj > si) || (sj == si && gsrc[j] < ii);
      }
      src[rank] = ii;
    }
  } else {
    for (int i = tid; i < P.n_src; i += kMergeThreads) src[i] = gsrc[i];
  }
  __syncthreads();

  const int chunk = ceil_div(P.n_entries, C);
  const int lo = crank * chunk;
  const int n = max(0, min(P.n_entries, lo + chunk) - lo);
  auto token_of = [&](int e) {
    return P.expand_clen > 0 ? src[e / P.expand_clen] * P.expand_clen + e % P.expand_clen : src[e];
  };
  if (P.out_token_ids) {
    int* dst = P.out_token_ids + (size_t)row * P.n_entries + lo;
    for (int i = tid; i < n; i += kMergeThreads) dst[i] = token_of(lo + i);
  }

  const int half = lane >> 4, l16 = lane & 15;
  float qf[8];
  {
    const uint4 a = *reinterpret_cast<const uint4*>(P.q + (size_t)row * kHeadDim + 8 * l16);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = h2f2(w[i]);
      qf[2 * i] = f.x * P.m.scale_log2e;
      qf[2 * i + 1] = f.y * P.m.scale_log2e;
    }
  }
  const size_t head_off = (size_t)bq * P.m.v_batch_stride + (size_t)hkv * P.m.v_head_stride + l16 * 8;
  const __half* kb = P.k + head_off;
  const __half* vb = P.m.v + head_off;
  constexpr int kRowsPerIter = 2 * kW;
  float m_run = -INFINITY, l_run = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  // the trip count is the same for every lane: the shuffles below need the whole warp
  for (int base = 0; base < n; base += kRowsPerIter * UN) {
    uint4 kk[GIVEN ? 1 : UN], vv[UN];
    float given[GIVEN ? UN : 1];
    bool ok[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int e = base + warp * 2 + half + kRowsPerIter * u;
      const int raw = (e < n) ? token_of(lo + e) : -1;
      const int tok = raw - P.m.id_shift;
      ok[u] = raw >= 0 && (unsigned)tok < (unsigned)P.m.n_tokens;
      // an empty slot (-1) is skipped silently; any other id outside the cache is reported
      if (e < n && raw >= 0 && !ok[u] && l16 == 0) atomicOr(P.m.status, kStatusBadId);
      const size_t off = ok[u] ? (size_t)tok * P.m.v_token_stride : 0;
      if constexpr (GIVEN) {
        given[u] = ok[u] ? gsc[lo + e] * P.m.scale_log2e : 0.f;
      } else {
        kk[u] = ok[u] ? ldg128_nc(kb + off) : make_uint4(0u, 0u, 0u, 0u);
      }
      vv[u] = ok[u] ? ldg128_nc(vb + off) : make_uint4(0u, 0u, 0u, 0u);
    }
    float x[UN];
    float bm = -INFINITY;
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      float a = 0.f;
      if constexpr (GIVEN) {
        a = given[u];
      } else {
        const uint32_t w[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = h2f2(w[i]);
          a = fmaf(f.x, qf[2 * i], a);
          a = fmaf(f.y, qf[2 * i + 1], a);
        }
        a += __shfl_xor_sync(0xffffffffu, a, 8);
        a += __shfl_xor_sync(0xffffffffu, a, 4);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        a += __shfl_xor_sync(0xffffffffu, a, 1);
      }
      x[u] = ok[u] ? a : -INFINITY;
      bm = fmaxf(bm, x[u]);
    }
    const float m_new = fmaxf(m_run, bm);
    if (m_new > -INFINITY) {
      const float alpha = fast_exp2(m_run - m_new);
      l_run *= alpha;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= alpha;
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const float pw = fast_exp2(x[u] - m_new);
        l_run += pw;
        const uint32_t w[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = h2f2(w[i]);
          acc[2 * i] = fmaf(pw, f.x, acc[2 * i]);
          acc[2 * i + 1] = fmaf(pw, f.y, acc[2 * i + 1]);
        }
      }
      m_run = m_new;
    }
  }
  // the two half-warps
  {
    const float m_o = __shfl_xor_sync(0xffffffffu, m_run, 16);
    const float l_o = __shfl_xor_sync(0xffffffffu, l_run, 16);
    const float m_n = fmaxf(m_run, m_o);
    const float a_me = (m_run > -INFINITY) ? fast_exp2(m_run - m_n) : 0.f;
    const float a_ot = (m_o > -INFINITY) ? fast_exp2(m_o - m_n) : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float o_o = __shfl_xor_sync(0xffffffffu, acc[i], 16);
      acc[i] = acc[i] * a_me + o_o * a_ot;
    }
    l_run = l_run * a_me + l_o * a_ot;
    m_run = m_n;
  }
  if (lane < 16) {
#pragma unroll
    for (int i = 0; i < 8; ++i) wpart[warp].o[lane * 8 + i] = acc[i];
    if (lane == 0) {
      wpart[warp].m = m_run;
      wpart[warp].l = l_run;
    }
  }
  __syncthreads();
  if (tid < kHeadDim) {
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kW; ++w) m = fmaxf(m, wpart[w].m);
    float o = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kW; ++w) {
      const float f = (wpart[w].m > -INFINITY) ? fast_exp2(wpart[w].m - m) : 0.f;
      o = fmaf(f, wpart[w].o[tid], o);
      l = fmaf(f, wpart[w].l, l);
    }
    cpart->o[tid] = o;
    if (tid == 0) {
      cpart->m = m;
      cpart->l = l;
    }
  }
  cluster.sync();
  const int dper = kHeadDim / C;
  if (tid < dper) {
    const int d = crank * dper + tid;
    float m = -INFINITY;
    for (int c = 0; c < C; ++c) m = fmaxf(m, cluster.map_shared_rank(cpart, c)->m);
    float o = 0.f, l = 0.f;
    for (int c = 0; c < C; ++c) {
      const GatherPartial* rp = cluster.map_shared_rank(cpart, c);
      const float f = (rp->m > -INFINITY) ? fast_exp2(rp->m - m) : 0.f;
      o = fmaf(f, rp->o[d], o);
      l = fmaf(f, rp->l, l);
    }
    P.m.out[(size_t)row * kHeadDim + d] = __float2half_rn(o / l);
    if (P.m.out_lse && d == 0) {
      P.m.out_lse[(size_t)row * 2 + 0] = m * 0.6931471805599453f;  // natural-log domain
      P.m.out_lse[(size_t)row * 2 + 1] = l;
    }
  }
  cluster.sync();  // nobody leaves while a peer may still read its partial
}

size_t gather_flash_smem_bytes(int n_src) {
  return (kMergeThreads / 32 + 1) * sizeof(GatherPartial) + (size_t)n_src * 4 + 16;
}

cudaError_t launch_gather_flash(const GatherParams& P, int rows, size_t smem, cudaStream_t stream) {
  // long lists: eight rows in flight hide the DRAM latency; short ones: four, more CTAs per SM
  const int un = ceil_div(P.n_entries, P.m.cluster) >= 512 ? 8 : 4;
  const bool given = P.expand_clen == 0 && P.src_score != nullptr;
  auto kern = given ? (un == 8 ? gather_flash_kernel<8, true> : gather_flash_kernel<4, true>)
                    : (un == 8 ? gather_flash_kernel<8, false> : gather_flash_kernel<4, false>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
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

// Orders the n (score, id) pairs of every row by descending score (ties: ascending id), the rank
// order in which the reference lists its chosen clusters (gemv_topk.cu:103-104, partial_sort).
__global__ void __launch_bounds__(256)
rank_sort_kernel(const float* __restrict__ score, const int* __restrict__ idx, int n,
                 int* __restrict__ out_idx, float* __restrict__ out_score) {
  extern __shared__ float sh[];
  float* ss = sh;
  int* si = reinterpret_cast<int*>(sh + n);
  const size_t row = blockIdx.x;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    ss[i] = score[row * n + i];
    si[i] = idx[row * n + i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float a = ss[i];
    const int ia = si[i];
    int rank = 0;
    for (int j = 0; j < n; ++j) rank += (ss[j] > a) || (ss[j] == a && si[j] < ia);
    out_idx[row * n + rank] = ia;
    if (out_score) out_score[row * n + rank] = a;
  }
}

cudaError_t launch_rank_sort(const float* score, const int* idx, int rows, int n, int* out_idx,
                             float* out_score, cudaStream_t stream) {
  note_launch();
  rank_sort_kernel<<<rows, 256, (size_t)n * 8, stream>>>(score, idx, n, out_idx, out_score);
  return cudaGetLastError();
}

// Decode-loop step before the attention: write the new token's K and V rows into the caches at
// `pos` and fold the key into the running mean of its cluster's centroid.
__global__ void __launch_bounds__(kHeadDim)
kv_append_kernel(__half* __restrict__ kc, __half* __restrict__ vc, const __half* __restrict__ nk,
                 const __half* __restrict__ nv, __half* __restrict__ centers, int hkv, int pos,
                 long long bstride, long long tstride, long long hstride, int num_centers,
                 int cluster_len) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const size_t src = ((size_t)b * hkv + h) * kHeadDim + d;
  const size_t dst = (size_t)b * bstride + (size_t)pos * tstride + (size_t)h * hstride + d;
  const __half kval = nk[src];
  kc[dst] = kval;
  vc[dst] = nv[src];
  if (centers && b == 0) {
    const int c = pos / cluster_len, seen = pos % cluster_len;
    if (c < num_centers) {
      __half* cp = centers + ((size_t)h * num_centers + c) * kHeadDim + d;
      const float old = seen ? __half2float(*cp) : 0.f;
      *cp = __float2half_rn((old * seen + __half2float(kval)) / (float)(seen + 1));
    }
  }
}

cudaError_t launch_kv_append(__half* kc, __half* vc, const __half* nk, const __half* nv,
                             __half* centers, int batch, int hkv, int pos, long long bstride,
                             long long tstride, long long hstride, int num_centers, int cluster_len,
                             cudaStream_t stream) {
  note_launch();
  kv_append_kernel<<<dim3(hkv, batch), kHeadDim, 0, stream>>>(kc, vc, nk, nv, centers, hkv, pos, bstride,
                                                           tstride, hstride, num_centers, cluster_len);
  return cudaGetLastError();
}

size_t gather_attend_smem_bytes(int per, int cap, int n_src) {
  return select_scratch_bytes(1, per, 0) + (size_t)cap * 8 + 16 +
         (size_t)n_src * 4 + 128;
}

cudaError_t launch_gather_attend(const GatherParams& P, int rows, size_t smem, cudaStream_t stream) {
  auto kern = gather_attend_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
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

}  // namespace ra
