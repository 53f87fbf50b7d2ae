// K scan for rows that several queries share (a GQA group and/or batch rows on one cache, up to
// 8 queries per row) when k is too large for per-CTA candidate lists: every CTA streams its slab
// of the fp16 key cache through a TMA pipeline (cp.async.bulk.tensor, two 64-dim halves with the
// 128-byte swizzle per 128-token stage), scores 16 tokens per warp against all queries with
// mma.sync.m16n8k16 (tokens as M, queries as N, fp32 accumulation), and
//   * stores the order-preserving 32-bit key of every score to the workspace (4 bytes per token
//     and query, 1/16 of the bytes read for four queries), and
//   * counts the keys' top 11 bits in a shared-memory histogram, written out once per CTA.
// There are no thresholds, candidate lists or cuts in the stream; select_stored_kernel finishes the
// selection from the histogram and the stored keys.
//
// The scoring stage of retrieval_attention_pipelined_kernel<K>
// (retrieval_attn/retrieval_attention.cu:654-896: K read once for the whole batch) and of
// gemv_topk_kernel (gemv_topk.cu:173-380), with the selection moved behind the stream.
#include "scan_store.cuh"

namespace ra {

struct StoreCtrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  int timeout;
};

__global__ void __launch_bounds__(kThreads, 1)
scan_store_kernel(const __grid_constant__ StoreParams P) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* stages =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int S = P.nstages, G = P.groups, SG = S / G;
  uint32_t* hist = reinterpret_cast<uint32_t*>(stages + (size_t)S * kStageBytes);  // [nq_valid][kHistBins]
  StoreCtrl* ctrl = reinterpret_cast<StoreCtrl*>(hist + (size_t)P.nq_valid * kHistBins);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int part = blockIdx.x % P.nparts;
  const int cid = blockIdx.x / P.nparts;
  const int h0 = cid % P.hkv;
  const int b0 = (cid / P.hkv) * P.bshare;
  const int kv_b = P.kv_per_batch ? b0 : 0;
  const int part_lo = part * P.part_len;
  const int part_hi = min(P.n_tokens, part_lo + P.part_len);
  const int ntiles = ceil_div(max(part_hi - part_lo, 0), kTileRows);

  if (tid == 0) {
    tma_prefetch_desc(&P.kmap);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&ctrl->full[s], 1);
      mbar_init(&ctrl->empty[s], 8);  // the 8 warps of the group that consumed the stage
    }
    ctrl->timeout = 0;
    fence_barrier_init();
  }
  for (int i = tid; i < P.nq_valid * kHistBins; i += blockDim.x) hist[i] = 0u;
  __syncthreads();

  if (warp == 8 * G) {
    // ------------------------------------------------------------ producer warp
    if (lane == 0) {
      // every consumer group has its own ring of S/G stages and waits on every phase of it; K is
      // read once, so its lines may leave L2 first and the stored scores stay for the selection
      const uint64_t once = l2_policy_evict_first();
      for (int it = 0; it < ntiles; ++it) {
        const int jt = it / G;
        const int s = (jt % SG) * G + (it % G);
        if (jt >= SG && !mbar_wait(&ctrl->empty[s], (unsigned)(((jt / SG) - 1) & 1), &ctrl->timeout))
          atomicOr(P.status, kStatusTimeout);
        const int tok = part_lo + it * kTileRows;
        unsigned char* dst = stages + (size_t)s * kStageBytes;
        mbar_expect_tx(&ctrl->full[s], kStageBytes);
        tma_load_4d_hint(dst, &P.kmap, &ctrl->full[s], 0, h0, tok, kv_b, once);
        tma_load_4d_hint(dst + kSwzHalfBytes, &P.kmap, &ctrl->full[s], 64, h0, tok, kv_b, once);
      }
    }
  } else {
    // ------------------------------------------------------------ consumer warps
    // Group g takes tiles g, g+G, ...; warp w8 of a group owns tokens 16*w8 .. 16*w8+15 of a tile.
    // Lane (mg, mt) holds the B fragments of query mg and ends up with the scores of tokens
    // mg, mg+8 for the queries 2mt, 2mt+1.
    const int grp = warp >> 3, w8 = warp & 7;
    const int mg = lane >> 2, mt = lane & 3;
    uint32_t qb[8][2];
    if (mg < P.nq_valid) {
      const int bq = b0 + mg / P.group;
      const int hq = h0 * P.group + mg % P.group;
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
    // where this lane's two queries keep their keys and counts
    uint32_t* krow[2];
    uint32_t* hrow[2];
    bool qok[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int qi = 2 * mt + e;
      qok[e] = qi < P.nq_valid;
      const int qv = qok[e] ? qi : 0;
      const int bq = b0 + qv / P.group;
      const int hq = h0 * P.group + qv % P.group;
      krow[e] = P.keys_ws + ((size_t)bq * P.hq + hq) * P.n_pad;
      hrow[e] = hist + (size_t)qv * kHistBins;
    }
    const int a_tok = w8 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
    const int a_c8 = lane >> 4;
    const uint32_t stage0 = smem_u32(stages);
    const int iters = ceil_div(ntiles, G);

#pragma unroll 1
    for (int jt = 0; jt < iters; ++jt) {
      const int it = jt * G + grp;
      if (it >= ntiles) break;
      const int s = (jt % SG) * G + grp;
      if (!mbar_wait(&ctrl->full[s], (unsigned)((jt / SG) & 1), &ctrl->timeout)) {
        if (lane == 0) atomicOr(P.status, kStatusTimeout);
      }
      const uint32_t tbase = stage0 + (uint32_t)s * kStageBytes;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, tbase + swz128(a_tok, 2 * kk + a_c8));
        mma_16816(c, a, qb[kk][0], qb[kk][1]);
      }
      // the stage is free as soon as this warp's fragments are in registers
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctrl->empty[s]);
      const int tok_lo = part_lo + it * kTileRows + w8 * 16 + mg;
#pragma unroll
      for (int jv = 0; jv < 4; ++jv) {
        const int e = jv & 1;
        const int tok = tok_lo + 8 * (jv >> 1);
        if (qok[e] && tok < part_hi) {
          const uint32_t key = score_key(c[jv]);
          krow[e][tok] = key;
          atomicAdd(&hrow[e][key >> kHistShift], 1u);
        }
      }
    }
  }
  __syncthreads();
  // this part's counts, one row of bins per query
  for (int i = tid; i < P.nq_valid * kHistBins; i += blockDim.x) {
    const int qi = i / kHistBins, bin = i - qi * kHistBins;
    const int bq = b0 + qi / P.group;
    const int hq = h0 * P.group + qi % P.group;
    P.hist_ws[(((size_t)bq * P.hq + hq) * P.nparts + part) * kHistBins + bin] = hist[i];
  }
}

size_t scan_store_smem_bytes(int nq_valid, int nstages) {
  return (size_t)nstages * kStageBytes + (size_t)nq_valid * kHistBins * 4 + sizeof(StoreCtrl) + 1024;
}

cudaError_t launch_scan_store(const StoreParams& P, int grid, size_t smem, cudaStream_t stream) {
  auto kern = scan_store_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  note_launch();
  kern<<<grid, 32 * (8 * P.groups + 1), smem, stream>>>(P);
  return cudaGetLastError();
}

}  // namespace ra
