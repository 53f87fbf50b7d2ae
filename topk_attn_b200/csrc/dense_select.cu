// Exact top-k per (query, segment) for segments short enough that all their scores fit in shared
// memory: score every key once, keep the scores, select afterwards.  No thresholds, candidate
// lists or cuts -- those pay off on long scans, while on a segment of a few thousand keys they are
// fixed cost.
//
// The role of the reference's per-chunk kernels (retrieval_attention_kernel<K>,
// retrieval_attn/retrieval_attention.cu:254-472: 4 chunks of 2048 keys, top-K of each) and of
// gemv_topk_kernel (gemv_topk.cu:173-380) on short inputs.  One cluster of CTAs per (segment, kv
// head, group of batch rows that share the cache): each CTA scores a slice of the segment's K rows
// for all queries of the row at once (tensor cores, 16 rows per warp and step, up to 8 queries) and
// stores the scores into the shared memory of every CTA of the cluster.  After one cluster barrier
// the CTAs divide the NQ score vectors among themselves; each runs the radix descent of
// radix_winners.cuh on its vectors and writes the winners' ids and scores.
#include <cooperative_groups.h>

#include "dense_select.cuh"
#include "radix_winners.cuh"

namespace cg = cooperative_groups;

namespace ra {

// Scoring on the tensor cores without staging K in shared memory: a warp takes 16 K rows per step
// as the M dimension of mma.sync.m16n8k16 and the (up to 8) queries as N.  Lane (g, t) reads rows g
// and g+8 straight from global memory in 16-byte pieces -- piece j of a row is bytes
// 64j + 16t .. +15, so the four lanes of a row read 64 contiguous bytes per load -- and feeds the
// words of a piece to the A fragments of two k-steps.  The k index of the product is only a
// summation index, so any assignment of the 128 dims to k slots is valid as long as the query
// fragments use the same one: lane (g, t) holds the matching 16-byte pieces of query g.
__global__ void __launch_bounds__(kDenseThreads, 2)
dense_select_kernel(const __grid_constant__ DenseSelectParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.cluster;
  const int crank = C > 1 ? (int)cluster.block_rank() : 0;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int item = blockIdx.x / C;
  const int seg = item % P.segments;
  const int hk = (item / P.segments) % P.hkv;
  const int b0 = (item / (P.segments * P.hkv)) * P.bshare;
  const int n = P.seg_len;
  const int n_pad = (n + 3) & ~3;
  const int NQ = P.nq_valid;

  uint32_t* keys = reinterpret_cast<uint32_t*>(smem_raw);          // [NQ][n_pad]
  int* winners = reinterpret_cast<int*>(keys + (size_t)NQ * n_pad);  // [topk]
  __shared__ WinnerCtrl ctrl;

  // ---- query g of this K row: batch row b0 + g / group, head hk*group + g % group
  uint4 qreg[4];
  if (g < NQ) {
    const int b = b0 + g / P.group, h = hk * P.group + g % P.group;
    const __half* qp = P.q + ((size_t)b * P.hq + h) * kHeadDim + 8 * t;
#pragma unroll
    for (int j = 0; j < 4; ++j) qreg[j] = *reinterpret_cast<const uint4*>(qp + 32 * j);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) qreg[j] = make_uint4(0u, 0u, 0u, 0u);
  }
  RA_STAMP(P.status, 0);
  if (C > 1) cluster.sync();   // every CTA of the cluster is running before its memory is written
  RA_STAMP(P.status, 1);

  // ---- scores of this CTA's slice, stored into every CTA of the cluster ----
  const int lo = crank * P.per, hi = min(n, lo + P.per);
  const __half* rows = P.k + (size_t)b0 * P.batch_stride + (size_t)hk * P.head_stride +
                       (size_t)seg * n * P.token_stride + 8 * t;
  constexpr int kWarps = kDenseThreads / 32;
  constexpr int GRP = 2;   // groups of 16 rows in flight per warp
  for (int r0 = lo + warp * 16; r0 < hi; r0 += kWarps * 16 * GRP) {
    uint4 a_lo[GRP][4], a_hi[GRP][4];
#pragma unroll
    for (int gi = 0; gi < GRP; ++gi) {
      const int ra = r0 + gi * kWarps * 16 + g, rb = ra + 8;
      const __half* pa = rows + (size_t)ra * P.token_stride;
      const __half* pb = rows + (size_t)rb * P.token_stride;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a_lo[gi][j] = ra < hi ? ldg128_nc(pa + 32 * j) : make_uint4(0u, 0u, 0u, 0u);
        a_hi[gi][j] = rb < hi ? ldg128_nc(pb + 32 * j) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int gi = 0; gi < GRP; ++gi) {
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t a0[4] = {a_lo[gi][j].x, a_hi[gi][j].x, a_lo[gi][j].y, a_hi[gi][j].y};
        const uint32_t a1[4] = {a_lo[gi][j].z, a_hi[gi][j].z, a_lo[gi][j].w, a_hi[gi][j].w};
        mma_16816(c, a0, qreg[j].x, qreg[j].y);
        mma_16816(c, a1, qreg[j].z, qreg[j].w);
      }
      // lane (g, t) holds the scores of rows g, g+8 for the queries 2t, 2t+1
      const int ra = r0 + gi * kWarps * 16 + g;
#pragma unroll
      for (int jv = 0; jv < 4; ++jv) {
        const int qi = 2 * t + (jv & 1);
        const int r = ra + 8 * (jv >> 1);
        if (qi < NQ && r < hi) {
          uint32_t* dst = &keys[(size_t)qi * n_pad + r];
          const uint32_t key = score_key(c[jv]);
          if (C > 1) {
            for (int c2 = 0; c2 < C; ++c2) *cluster.map_shared_rank(dst, c2) = key;
          } else {
            *dst = key;
          }
        }
      }
    }
  }
  RA_STAMP(P.status, 2);
  if (C > 1) cluster.sync(); else __syncthreads();
  RA_STAMP(P.status, 3);
  // from here on a CTA touches its own shared memory only

  // ---- CTA c selects on score vectors c, c + C, ...; the winners of a vector are written in
  // ascending token order (lists are unordered inside a segment for the caller, but a fixed order
  // makes the attention that follows reproducible) ----
  const int id0 = P.index_base + seg * n;
  for (int l = crank; l < NQ; l += C) {   // CTA-uniform
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
  RA_STAMP(P.status, 4);
}

size_t dense_select_smem_bytes(int nq, int seg_len, int topk) {
  return (size_t)nq * ((seg_len + 3) & ~3) * 4 + (size_t)topk * 4;
}

cudaError_t launch_dense_select(const DenseSelectParams& P, int nq, cudaStream_t stream) {
  (void)nq;
  if (P.nq_valid < 1 || P.nq_valid > 8) return cudaErrorInvalidValue;
  auto kern = dense_select_kernel;
  const size_t smem = dense_select_smem_bytes(P.nq_valid, P.seg_len, P.topk);
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
