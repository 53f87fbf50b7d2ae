// Exact top-C of q.centroid per (batch row, head) for centroid tables small enough that one
// head's scores fit in shared memory (csz <= 8192), written in rank order together with the
// member token ids of the winners.
//
// The role of the reference's centroid pipeline (center_only_topk/gemv_topk.cu:157-457: GEMV over
// the [H,CSZ,D] table, radix top-k, expansion of each winner to its CLEN member tokens :271-279)
// and of the coarse stage of the two-level selection (gemv_topk.cu:218-262).  One cluster of CTAs
// per row: every CTA scores a slice of the table with half-warp-per-row 128-bit loads and stores
// each score into the shared memory of all CTAs of the cluster, so after one cluster barrier every
// CTA holds the whole score vector.  Each CTA then finds the C-th largest (score, id) pair by a
// radix descent over 64-bit composites (score key, inverted id) -- distinct values, so the
// descent always ends on an exact cut --, ranks the C winners among themselves and writes the
// outputs of the winners that lie in its own slice.  No global scratch, one launch.
#include <cooperative_groups.h>

#include "center_select.cuh"
#include "gather_flash.cuh"
#include "radix_winners.cuh"

namespace cg = cooperative_groups;

namespace ra {

__global__ void __launch_bounds__(kCenterThreads)
center_select_kernel(const __grid_constant__ CenterSelectParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.cluster;
  const int crank = C > 1 ? (int)cluster.block_rank() : 0;
  const int tid = threadIdx.x;
  const int hw = tid >> 4, l16 = tid & 15;
  const int row = blockIdx.x / C;
  const int h = row % P.heads;
  const int n = P.csz;
  const int n_pad = (n + 3) & ~3;

  uint32_t* keys = reinterpret_cast<uint32_t*>(smem_raw);          // [n_pad]
  int* winners = reinterpret_cast<int*>(keys + n_pad);             // [topc]
  int2* own = reinterpret_cast<int2*>(winners + ((P.topc + 1) & ~1));  // [topc] (rank, id)
  __shared__ WinnerCtrl ctrl;
  if (tid == 0) ctrl.nown = 0;

  // ---- scores of this CTA's slice, pushed into every CTA of the cluster ----
  const uint4 qraw = *reinterpret_cast<const uint4*>(P.q + (size_t)row * kHeadDim + l16 * 8);
  float qf[8];
  {
    const float2 a = h2f2(qraw.x), b = h2f2(qraw.y), c = h2f2(qraw.z), d = h2f2(qraw.w);
    qf[0] = a.x; qf[1] = a.y; qf[2] = b.x; qf[3] = b.y;
    qf[4] = c.x; qf[5] = c.y; qf[6] = d.x; qf[7] = d.y;
  }
  if (C > 1) cluster.sync();   // every CTA of the cluster is running before its memory is written
  const int lo = crank * P.per, hi = min(n, lo + P.per);
  const __half* table = P.centers + (size_t)h * n * kHeadDim + l16 * 8;
  constexpr int U = 8;         // rows in flight per half-warp
  for (int r0 = lo; r0 < hi; r0 += (kCenterThreads / 16) * U) {   // same trip count for all threads
    uint4 kv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * (kCenterThreads / 16) + hw;
      kv[u] = r < hi ? ldg128_nc(table + (size_t)r * kHeadDim) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * (kCenterThreads / 16) + hw;
      const float2 a = h2f2(kv[u].x), b = h2f2(kv[u].y), c = h2f2(kv[u].z), d = h2f2(kv[u].w);
      float s = a.x * qf[0];
      s = fmaf(a.y, qf[1], s); s = fmaf(b.x, qf[2], s); s = fmaf(b.y, qf[3], s);
      s = fmaf(c.x, qf[4], s); s = fmaf(c.y, qf[5], s); s = fmaf(d.x, qf[6], s);
      s = fmaf(d.y, qf[7], s);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if (l16 == 0 && r < hi) {
        const uint32_t key = score_key(s);
        if (C > 1) {
          for (int c2 = 0; c2 < C; ++c2) *cluster.map_shared_rank(&keys[r], c2) = key;
        } else {
          keys[r] = key;
        }
      }
    }
  }
  if (C > 1) cluster.sync(); else __syncthreads();
  // from here on a CTA touches its own shared memory only

  select_winners<kCenterThreads>(keys, n, P.topc, ctrl, winners);
  // ---- ranks and outputs of the winners in this CTA's slice ----
  const int nwin = min(ctrl.nwin, P.topc);
  // eight lanes per winner count the winners ahead of it
  for (int w0 = 0; w0 < nwin; w0 += kCenterThreads / 8) {   // same trip count for all threads
    const int w = w0 + (tid >> 3), sub = tid & 7;
    const bool valid = w < nwin;
    const int id = valid ? winners[w] : 0;
    const bool mine = valid && id >= lo && id < hi;
    int ahead = 0;
    if (mine) {
      const unsigned long long me = composite(keys[id], id);
      for (int j = sub; j < nwin; j += 8) {
        const int oj = winners[j];
        ahead += composite(keys[oj], oj) > me;
      }
    }
    ahead += __shfl_xor_sync(0xffffffffu, ahead, 4);
    ahead += __shfl_xor_sync(0xffffffffu, ahead, 2);
    ahead += __shfl_xor_sync(0xffffffffu, ahead, 1);
    if (mine && sub == 0) {
      const size_t o = (size_t)row * P.topc + ahead;
      if (P.out_cluster_ids) P.out_cluster_ids[o] = id;
      if (P.out_scores) P.out_scores[o] = key_score(keys[id]);
      own[atomicAdd(&ctrl.nown, 1)] = make_int2(ahead, id);
    }
  }
  if (!P.out_members) return;
  __syncthreads();
  const int nown = ctrl.nown;
  int* members = P.out_members + (size_t)row * P.topc * P.clen;
  if (P.vec_members) {
    const int q4 = P.clen >> 2;
    for (int x = tid; x < nown * q4; x += kCenterThreads) {
      const int2 wi = own[x / q4];
      const int t = (x % q4) * 4, first = wi.y * P.clen + t;
      *reinterpret_cast<int4*>(members + (size_t)wi.x * P.clen + t) =
          make_int4(first, first + 1, first + 2, first + 3);
    }
  } else {
    for (int x = tid; x < nown * P.clen; x += kCenterThreads) {
      const int2 wi = own[x / P.clen];
      const int t = x % P.clen;
      members[(size_t)wi.x * P.clen + t] = wi.y * P.clen + t;
    }
  }
}

// Centroid retrieval in one launch: the scores and the exact top-C as above, then every CTA of the
// cluster takes an equal share of the winners' member tokens (clusters in rank order, members in
// token order) and attends over them; the partial outputs meet through distributed shared memory.
// The cluster ids and member ids never leave shared memory unless the caller asks for them.  The role
// of the fused centroid pipelines of center_only_topk/baselines.cu:546-973 (selection, index
// hand-over through DSMEM :736-751, gathered decode).
template <int UN>
__global__ void __launch_bounds__(kCenterThreads)
center_attend_kernel(const __grid_constant__ CenterSelectParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = P.cluster;
  const int crank = C > 1 ? (int)cluster.block_rank() : 0;
  const int tid = threadIdx.x;
  const int hw = tid >> 4, l16 = tid & 15;
  const int row = blockIdx.x / C;
  const int b = row / P.heads, h = row % P.heads;
  const int n = P.csz;
  const int n_pad = (n + 3) & ~3;

  GatherPartial* part = reinterpret_cast<GatherPartial*>(smem_raw);
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem_raw + flash_partials_bytes<kCenterThreads>());  // [n_pad]
  int* winners = reinterpret_cast<int*>(keys + n_pad);   // [topc], ascending id
  int* ranked = winners + P.topc;                        // [topc], descending score
  __shared__ WinnerCtrl ctrl;

  const uint4 qraw = *reinterpret_cast<const uint4*>(P.q + (size_t)row * kHeadDim + l16 * 8);
  float qf[8];
  {
    const float2 a = h2f2(qraw.x), bb = h2f2(qraw.y), c = h2f2(qraw.z), d = h2f2(qraw.w);
    qf[0] = a.x; qf[1] = a.y; qf[2] = bb.x; qf[3] = bb.y;
    qf[4] = c.x; qf[5] = c.y; qf[6] = d.x; qf[7] = d.y;
  }
  RA_STAMP(P.status, 0);
  if (C > 1) cluster.sync();   // every CTA of the cluster is running before its memory is written
  RA_STAMP(P.status, 1);
  const int lo = crank * P.per, hi = min(n, lo + P.per);
  const __half* table = P.centers + (size_t)h * n * kHeadDim + l16 * 8;
  constexpr int U = 8;
  for (int r0 = lo; r0 < hi; r0 += (kCenterThreads / 16) * U) {   // same trip count for all threads
    uint4 kv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * (kCenterThreads / 16) + hw;
      kv[u] = r < hi ? ldg128_nc(table + (size_t)r * kHeadDim) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u * (kCenterThreads / 16) + hw;
      const float2 a = h2f2(kv[u].x), bb = h2f2(kv[u].y), c = h2f2(kv[u].z), d = h2f2(kv[u].w);
      float s = a.x * qf[0];
      s = fmaf(a.y, qf[1], s); s = fmaf(bb.x, qf[2], s); s = fmaf(bb.y, qf[3], s);
      s = fmaf(c.x, qf[4], s); s = fmaf(c.y, qf[5], s); s = fmaf(d.x, qf[6], s);
      s = fmaf(d.y, qf[7], s);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if (l16 == 0 && r < hi) {
        const uint32_t key = score_key(s);
        if (C > 1) {
          for (int c2 = 0; c2 < C; ++c2) *cluster.map_shared_rank(&keys[r], c2) = key;
        } else {
          keys[r] = key;
        }
      }
    }
  }
  RA_STAMP(P.status, 2);
  if (C > 1) cluster.sync(); else __syncthreads();
  RA_STAMP(P.status, 3);

  select_winners<kCenterThreads>(keys, n, P.topc, ctrl, winners);
  RA_STAMP(P.status, 4);
  const int nwin = min(ctrl.nwin, P.topc);
  // every CTA ranks all winners: eight lanes per winner count the winners ahead of it
  for (int w0 = 0; w0 < nwin; w0 += kCenterThreads / 8) {   // same trip count for all threads
    const int w = w0 + (tid >> 3), sub = tid & 7;
    const bool valid = w < nwin;
    const int id = valid ? winners[w] : 0;
    int ahead = 0;
    if (valid) {
      const unsigned long long me = composite(keys[id], id);
      for (int j = sub; j < nwin; j += 8) {
        const int oj = winners[j];
        ahead += composite(keys[oj], oj) > me;
      }
    }
    ahead += __shfl_xor_sync(0xffffffffu, ahead, 4);
    ahead += __shfl_xor_sync(0xffffffffu, ahead, 2);
    ahead += __shfl_xor_sync(0xffffffffu, ahead, 1);
    if (valid && sub == 0) ranked[ahead] = id;
  }
  __syncthreads();
  if (crank == 0) {
    for (int r = tid; r < nwin; r += kCenterThreads) {
      if (P.out_cluster_ids) P.out_cluster_ids[(size_t)row * P.topc + r] = ranked[r];
      if (P.out_scores) P.out_scores[(size_t)row * P.topc + r] = key_score(keys[ranked[r]]);
    }
  }
  // this CTA's share of the member tokens
  const int n_entries = nwin * P.clen;
  const int chunk = ceil_div(n_entries, C);
  const int elo = crank * chunk;
  const int en = max(0, min(n_entries, elo + chunk) - elo);
  auto token_of = [&](int e) { return ranked[e / P.clen] * P.clen + e % P.clen; };
  auto score_of = [&](int) { return 0.f; };
  if (P.out_members) {
    int* dst = P.out_members + (size_t)row * P.topc * P.clen + elo;
    for (int i = tid; i < en; i += kCenterThreads) dst[i] = token_of(elo + i);
  }
  const size_t head_off = (size_t)b * P.batch_stride + (size_t)h * P.head_stride;
  RA_STAMP(P.status, 5);
  flash_over_entries<UN, false, kCenterThreads>(cluster, C, crank, part, P.q + (size_t)row * kHeadDim,
                                                P.k + head_off, P.v + head_off, P.token_stride,
                                                P.n_tokens, 0, elo, en, P.scale_log2e, P.status,
                                                P.out + (size_t)row * kHeadDim, nullptr, token_of,
                                                score_of);
  RA_STAMP(P.status, 6);
}

size_t center_attend_smem_bytes(int csz, int topc) {
  return flash_partials_bytes<kCenterThreads>() + (size_t)((csz + 3) & ~3) * 4 + (size_t)topc * 8 + 16;
}

cudaError_t launch_center_attend(const CenterSelectParams& P, int rows, cudaStream_t stream) {
  // long shares: eight rows in flight per half-warp hide the DRAM latency; short ones: four
  const int share = ceil_div(P.topc * P.clen, P.cluster);
  auto kern = share >= 256 ? center_attend_kernel<8> : center_attend_kernel<4>;
  const size_t smem = center_attend_smem_bytes(P.csz, P.topc);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * P.cluster), 1, 1);
  cfg.blockDim = dim3(kCenterThreads, 1, 1);
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

size_t center_select_smem_bytes(int csz, int topc) {
  return (size_t)((csz + 3) & ~3) * 4 + (size_t)((topc + 1) & ~1) * 4 + (size_t)topc * 8;
}

cudaError_t launch_center_select(const CenterSelectParams& P, int rows, cudaStream_t stream) {
  auto kern = center_select_kernel;
  const size_t smem = center_select_smem_bytes(P.csz, P.topc);
  static const cudaError_t attr_status = cudaFuncSetAttribute(
      kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
      (int)center_select_smem_bytes(kCenterMaxCsz, kCenterMaxCsz));
  if (attr_status != cudaSuccess) return attr_status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * P.cluster), 1, 1);
  cfg.blockDim = dim3(kCenterThreads, 1, 1);
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
