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
#include "gather_flash.cuh"

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

// UN: K and V rows in flight per half-warp.  GIVEN: the list carries the raw scores q.K of its ids
// (src_score, expand_clen == 0), so only the V rows are read.
template <int UN, bool GIVEN>
__global__ void __launch_bounds__(kMergeThreads, 1)
gather_flash_kernel(const __grid_constant__ GatherParams P) {
  extern __shared__ __align__(16) unsigned char smem_g[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.m.cluster;
  const int crank = (int)cluster.block_rank();
  const int tid = threadIdx.x;
  const int row = blockIdx.x / C;
  const int bq = row / P.m.hq_total, hq = row % P.m.hq_total;
  const int hkv = hq / P.group;
  GatherPartial* part = reinterpret_cast<GatherPartial*>(smem_g);
  int* src = reinterpret_cast<int*>(smem_g + flash_partials_bytes<kMergeThreads>());

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
  auto score_of = [&](int e) { return gsc[e]; };
  if (P.out_token_ids) {
    int* dst = P.out_token_ids + (size_t)row * P.n_entries + lo;
    for (int i = tid; i < n; i += kMergeThreads) dst[i] = token_of(lo + i);
  }
  const size_t head_off = (size_t)bq * P.m.v_batch_stride + (size_t)hkv * P.m.v_head_stride;
  flash_over_entries<UN, GIVEN, kMergeThreads>(
      cluster, C, crank, part, P.q + (size_t)row * kHeadDim, GIVEN ? P.m.v + head_off : P.k + head_off,
      P.m.v + head_off, P.m.v_token_stride, P.m.n_tokens, P.m.id_shift, lo, n, P.m.scale_log2e,
      P.m.status, P.m.out + (size_t)row * kHeadDim,
      P.m.out_lse ? P.m.out_lse + (size_t)row * 2 : nullptr, token_of, score_of);
}

size_t gather_flash_smem_bytes(int n_src) {
  return flash_partials_bytes<kMergeThreads>() + (size_t)n_src * 4 + 16;
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
