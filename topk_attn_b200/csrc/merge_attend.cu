// Second-stage kernel: exact k-select over candidate (score, id) lists held in global memory,
// then softmax.V over the winners.  Used when one head's context was scanned by several
// clusters (each wrote its own k candidates), for the legacy per-chunk selection (every chunk's
// k winners are all attended) and, with an ownership window, for the sequence-sharded path
// (candidates of all ranks are merged; each rank mixes only the V rows it holds and emits an
// un-normalised partial).  The role of retrieval_reduce_kernel
// (retrieval_attn/retrieval_attention.cu:1243-1339) generalised with a selection step.
#include "merge_attend.cuh"

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

  const size_t scratch_bytes = (sizeof(MergeScratch) + (size_t)P.m.per * 8 + 127) & ~size_t(127);
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
    idxs[i] = P.cand_idx[src];
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
  return ((sizeof(MergeScratch) + (size_t)per * 8 + 127) & ~size_t(127)) + (size_t)cap * 8 + 16 + 128;
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
  return cudaLaunchKernelEx(&cfg, kern, P);
}

__global__ void __launch_bounds__(kHeadDim)
lse_combine_kernel(const float* __restrict__ partials, int parts, int rows, __half* __restrict__ out) {
  const int row = blockIdx.x, d = threadIdx.x;
  float m = -INFINITY;
  for (int p = 0; p < parts; ++p)
    m = fmaxf(m, partials[((size_t)p * rows + row) * (kHeadDim + 2) + kHeadDim + 1]);
  float o = 0.f, l = 0.f;
  for (int p = 0; p < parts; ++p) {
    const float* src = partials + ((size_t)p * rows + row) * (kHeadDim + 2);
    const float lp = src[kHeadDim];
    const float w = (lp > 0.f) ? __expf(src[kHeadDim + 1] - m) : 0.f;
    o = fmaf(w, src[d], o);
    l = fmaf(w, lp, l);
  }
  out[(size_t)row * kHeadDim + d] = __float2half_rn(o / l);
}

cudaError_t launch_lse_combine(const float* partials, int parts, int rows, __half* out,
                               cudaStream_t stream) {
  lse_combine_kernel<<<rows, kHeadDim, 0, stream>>>(partials, parts, rows, out);
  return cudaGetLastError();
}

}  // namespace ra
