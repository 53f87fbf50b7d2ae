// Exact top-k per (query, segment) for segments short enough that all their scores fit in shared
// memory: score every key once, keep the scores, select afterwards.  No thresholds, candidate
// lists or cuts -- those pay off on long scans, while on a segment of a few thousand keys they are
// fixed cost.
//
// The role of the reference's per-chunk kernels (retrieval_attention_kernel<K>,
// retrieval_attn/retrieval_attention.cu:254-472: 4 chunks of 2048 keys, top-K of each) and of
// gemv_topk_kernel (gemv_topk.cu:173-380) on short inputs.  One cluster of CTAs per (segment, kv
// head, group of batch rows that share the cache): each CTA scores a slice of the segment's K rows
// for all NQ queries at once (half-warp per row, one 128-bit load per lane, NQ dot products) and
// stores the scores into the shared memory of every CTA of the cluster.  After one cluster barrier
// the CTAs divide the NQ score vectors among themselves; each runs the radix descent of
// radix_winners.cuh on its vectors and writes the winners' ids and scores.
#include <cooperative_groups.h>

#include "dense_select.cuh"
#include "radix_winners.cuh"

namespace cg = cooperative_groups;

namespace ra {

template <int NQ>
__global__ void __launch_bounds__(kDenseThreads, 4)   // 64 registers: four CTAs per SM
dense_select_kernel(const __grid_constant__ DenseSelectParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.cluster;
  const int crank = C > 1 ? (int)cluster.block_rank() : 0;
  const int tid = threadIdx.x;
  const int hw = tid >> 4, l16 = tid & 15;
  const int item = blockIdx.x / C;
  const int seg = item % P.segments;
  const int hk = (item / P.segments) % P.hkv;
  const int b0 = (item / (P.segments * P.hkv)) * P.bshare;
  const int n = P.seg_len;
  const int n_pad = (n + 3) & ~3;

  uint32_t* keys = reinterpret_cast<uint32_t*>(smem_raw);          // [NQ][n_pad]
  int* winners = reinterpret_cast<int*>(keys + (size_t)NQ * n_pad);  // [topk]
  __shared__ WinnerCtrl ctrl;

  // ---- the queries of this K row: list qi is batch row b0 + qi / group, head hk*group + qi % group
  float qf[NQ][8];
#pragma unroll
  for (int qi = 0; qi < NQ; ++qi) {
    const int qv = min(qi, P.nq_valid - 1);   // padding lists repeat the last query, never written
    const int b = b0 + qv / P.group, h = hk * P.group + qv % P.group;
    const uint4 raw = *reinterpret_cast<const uint4*>(P.q + ((size_t)b * P.hq + h) * kHeadDim + l16 * 8);
    const float2 a = h2f2(raw.x), bb = h2f2(raw.y), c = h2f2(raw.z), d = h2f2(raw.w);
    qf[qi][0] = a.x; qf[qi][1] = a.y; qf[qi][2] = bb.x; qf[qi][3] = bb.y;
    qf[qi][4] = c.x; qf[qi][5] = c.y; qf[qi][6] = d.x; qf[qi][7] = d.y;
  }
  if (C > 1) cluster.sync();   // every CTA of the cluster is running before its memory is written

  // ---- scores of this CTA's slice, stored into every CTA of the cluster ----
  const int lo = crank * P.per, hi = min(n, lo + P.per);
  const __half* rows = P.k + (size_t)b0 * P.batch_stride + (size_t)hk * P.head_stride +
                       (size_t)seg * n * P.token_stride + l16 * 8;
  constexpr int U = NQ >= 4 ? 4 : 8;   // rows in flight per half-warp
  constexpr int kRowsPerIter = (kDenseThreads / 16) * U;
  for (int r0 = lo; r0 < hi; r0 += kRowsPerIter) {   // same trip count for all threads
    uint4 kv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * (kDenseThreads / 16) + hw;
      kv[u] = r < hi ? ldg128_nc(rows + (size_t)r * P.token_stride) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * (kDenseThreads / 16) + hw;
      const float2 a = h2f2(kv[u].x), b = h2f2(kv[u].y), c = h2f2(kv[u].z), d = h2f2(kv[u].w);
      float s[NQ];
#pragma unroll
      for (int qi = 0; qi < NQ; ++qi) {
        float t = a.x * qf[qi][0];
        t = fmaf(a.y, qf[qi][1], t); t = fmaf(b.x, qf[qi][2], t); t = fmaf(b.y, qf[qi][3], t);
        t = fmaf(c.x, qf[qi][4], t); t = fmaf(c.y, qf[qi][5], t); t = fmaf(d.x, qf[qi][6], t);
        t = fmaf(d.y, qf[qi][7], t);
        s[qi] = t;
      }
      // Transposing reduction over the 16 lanes of the row: each exchange halves the number of
      // queries a lane carries, so lane l ends with the full sum of query l / (16 / NQ).
      float tot;
      if constexpr (NQ == 4) {
        const bool up8 = l16 & 8, up4 = l16 & 4;
        float a0 = up8 ? s[2] : s[0], a1 = up8 ? s[3] : s[1];
        const float b0 = up8 ? s[0] : s[2], b1 = up8 ? s[1] : s[3];
        a0 += __shfl_xor_sync(0xffffffffu, b0, 8);
        a1 += __shfl_xor_sync(0xffffffffu, b1, 8);
        tot = up4 ? a1 : a0;
        const float give = up4 ? a0 : a1;
        tot += __shfl_xor_sync(0xffffffffu, give, 4);
      } else if constexpr (NQ == 2) {
        const bool up8 = l16 & 8;
        tot = up8 ? s[1] : s[0];
        const float give = up8 ? s[0] : s[1];
        tot += __shfl_xor_sync(0xffffffffu, give, 8);
        tot += __shfl_xor_sync(0xffffffffu, tot, 4);
      } else {
        tot = s[0];
        tot += __shfl_xor_sync(0xffffffffu, tot, 8);
        tot += __shfl_xor_sync(0xffffffffu, tot, 4);
      }
      tot += __shfl_xor_sync(0xffffffffu, tot, 2);
      tot += __shfl_xor_sync(0xffffffffu, tot, 1);
      // the 16 / NQ lanes that hold a query's sum deal its C stores among themselves
      if (r < hi) {
        constexpr int kLanesPerQuery = 16 / NQ;
        const int qi = l16 / kLanesPerQuery;
        uint32_t* dst = &keys[(size_t)qi * n_pad + r];
        const uint32_t key = score_key(tot);
        if (C > 1) {
          for (int c2 = l16 % kLanesPerQuery; c2 < C; c2 += kLanesPerQuery)
            *cluster.map_shared_rank(dst, c2) = key;
        } else if (l16 % kLanesPerQuery == 0) {
          *dst = key;
        }
      }
    }
  }
  if (C > 1) cluster.sync(); else __syncthreads();
  // from here on a CTA touches its own shared memory only

  // ---- CTA c selects on score vectors c, c + C, ...; the winners of a vector are written in the
  // order the descent found them (lists are unordered inside a segment) ----
  const int id0 = P.index_base + seg * n;
  for (int l = crank; l < P.nq_valid; l += C) {   // CTA-uniform
    const uint32_t* kl = keys + (size_t)l * n_pad;
    select_winners<kDenseThreads>(kl, n, P.topk, ctrl, winners);
    const int nwin = min(ctrl.nwin, P.topk);
    const int b = b0 + l / P.group, h = hk * P.group + l % P.group;
    const size_t obase = ((size_t)b * P.hq + h) * P.segments * P.topk + (size_t)seg * P.topk;
    for (int w = tid; w < nwin; w += kDenseThreads) {
      const int id = winners[w];
      P.out_idx[obase + w] = id0 + id;
      P.out_score[obase + w] = key_score(kl[id]);
    }
    __syncthreads();   // winners and ctrl are reused by the next vector
  }
}

size_t dense_select_smem_bytes(int nq, int seg_len, int topk) {
  return (size_t)nq * ((seg_len + 3) & ~3) * 4 + (size_t)topk * 4;
}

cudaError_t launch_dense_select(const DenseSelectParams& P, int nq, cudaStream_t stream) {
  void (*kern)(const DenseSelectParams) = nullptr;
  if (nq == 1) kern = dense_select_kernel<1>;
  if (nq == 2) kern = dense_select_kernel<2>;
  if (nq == 4) kern = dense_select_kernel<4>;
  if (!kern) return cudaErrorInvalidValue;
  const size_t smem = dense_select_smem_bytes(nq, P.seg_len, P.topk);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  const int items = P.segments * P.hkv * (P.batch / P.bshare);
  cfg.gridDim = dim3((unsigned)(items * P.cluster), 1, 1);
  cfg.blockDim = dim3(kDenseThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)P.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  note_launch();
  return cudaLaunchKernelEx(&cfg, kern, P);
}

}  // namespace ra
