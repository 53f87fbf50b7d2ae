// Dense split-KV decode attention ("flash decoding") for sm_100a.
//
// Work item = (batch row, kv head, split of the token axis).  A persistent grid of one CTA per SM
// walks the items; one producer warp streams K and V tiles of 128 tokens with TMA
// (cp.async.bulk.tensor, 128-byte swizzle, 64 KiB per stage) across item boundaries, eight consumer
// warps take 16 tokens of every tile.  The query heads that share a kv head (GQA group, <= 8) form
// the M dimension of a small dense product, so the two products of a tile run on the tensor cores:
// S = Q K^T and O += P V as m16n8k16 MMAs with fp32 accumulation and an online softmax in between.
// Every item writes one un-normalised partial (sums, weight, maximum); a log-sum-exp combine over
// the splits produces the output.
//
// The role of MHAFlashDecodeKernel (flash_decoding.cu:100-388, corrected in baseline_1.cu:324-610:
// KV split over the CTAs of a cluster, online softmax with ex2.approx, DSMEM max/sum combine, fp16
// atomicAdd into a pre-zeroed output) for the dense case, with the combine as its own step.
#include "flash_decode.cuh"

namespace ra {

struct FdCtrl {
  uint64_t full[kFdMaxStages];
  uint64_t empty[kFdMaxStages];
  float m[kFdConsumerWarps][kFdMaxGroup];
  float l[kFdConsumerWarps][kFdMaxGroup];
  int timeout;
};

__device__ __forceinline__ void fd_consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"r"(32 * kFdConsumerWarps) : "memory");
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t fd_swz(int token, int c8) { return swz128(token, c8); }

__global__ void __launch_bounds__(kFdThreads, 1)
flash_decode_kernel(const __grid_constant__ FlashParams P) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stages = smem;
  float* sm_o = reinterpret_cast<float*>(smem + (size_t)P.nstages * kFdStageBytes);  // [8][G][128]
  FdCtrl* ctrl = reinterpret_cast<FdCtrl*>(sm_o + kFdConsumerWarps * kFdMaxGroup * kHeadDim);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = P.nstages;
  const int G = P.group;
  const int tiles_per_item = ceil_div(P.split_len, kFdTile);

  if (tid == 0) {
    tma_prefetch_desc(&P.kmap);
    tma_prefetch_desc(&P.vmap);
    for (int s = 0; s < kFdMaxStages; ++s) {
      mbar_init(&ctrl->full[s], 1);
      mbar_init(&ctrl->empty[s], kFdConsumerWarps);
    }
    ctrl->timeout = 0;
    fence_barrier_init();
  }
  __syncthreads();

  // item -> (split, kv head, batch row), batch row fastest so that rows sharing one cache run
  // next to each other and meet in L2
  auto decode = [&](int item, int& b, int& h, int& sp) {
    b = item % P.batch;
    const int r = item / P.batch;
    h = r % P.hkv;
    sp = r / P.hkv;
  };

  if (warp == kFdConsumerWarps) {
    // ---------------------------------------------------------------- producer warp
    if (lane == 0) {
      int n = 0;  // running tile count over all my items
      for (int item = blockIdx.x; item < P.num_items; item += gridDim.x) {
        int b, h, sp;
        decode(item, b, h, sp);
        const int kvb = P.kv_per_batch ? b : 0;
        for (int t = 0; t < tiles_per_item; ++t, ++n) {
          const int s = n % S;
          if (n >= S && !mbar_wait(&ctrl->empty[s], (unsigned)(((n / S) - 1) & 1), &ctrl->timeout))
            atomicOr(P.status, kStatusTimeout);
          const int tok = sp * P.split_len + t * kFdTile;
          unsigned char* dst = stages + (size_t)s * kFdStageBytes;
          mbar_expect_tx(&ctrl->full[s], kFdStageBytes);
          tma_load_4d(dst, &P.kmap, &ctrl->full[s], 0, h, tok, kvb);
          tma_load_4d(dst + kFdHalfBytes, &P.kmap, &ctrl->full[s], 64, h, tok, kvb);
          tma_load_4d(dst + 2 * kFdHalfBytes, &P.vmap, &ctrl->full[s], 0, h, tok, kvb);
          tma_load_4d(dst + 3 * kFdHalfBytes, &P.vmap, &ctrl->full[s], 64, h, tok, kvb);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- consumer warps
    const int g = lane >> 2, t = lane & 3;
    const int r0 = warp * 16;  // my 16 tokens inside a tile
    const uint32_t stage0 = smem_u32(stages);
    // per-lane pieces of the ldmatrix addresses
    const int mi = lane >> 3, lr = lane & 7;
    const int k_tok = r0 + (mi >> 1) * 8 + lr;  // K: matrices 0,1 tokens 0-7; 2,3 tokens 8-15
    const int k_c8 = mi & 1;                    //    chunk 2kk + (mi & 1)
    const int v_tok = r0 + (mi & 1) * 8 + lr;   // V: matrices 0,2 tokens 0-7; 1,3 tokens 8-15
    const int v_c8 = mi >> 1;                   //    chunk n + (mi >> 1)
    int n = 0;
    for (int item = blockIdx.x; item < P.num_items; item += gridDim.x) {
      int b, h, sp;
      decode(item, b, h, sp);
      // A fragments of Q: rows 0..G-1 are the query heads of this kv head, rows >= G are zero
      uint32_t qa[8][4];
      {
        const __half* qp = P.q + ((size_t)b * P.hq + (size_t)h * G + g) * kHeadDim;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          qa[kk][0] = (g < G) ? *reinterpret_cast<const uint32_t*>(qp + 16 * kk + 2 * t) : 0u;
          qa[kk][2] = (g < G) ? *reinterpret_cast<const uint32_t*>(qp + 16 * kk + 8 + 2 * t) : 0u;
          qa[kk][1] = 0u;
          qa[kk][3] = 0u;
        }
      }
      float o[16][4];
#pragma unroll
      for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      float m_run = -INFINITY, l_run = 0.f;  // row g (rows g+8 are padding)
      const int split_hi = min(P.n_tokens, (sp + 1) * P.split_len);

      for (int tt = 0; tt < tiles_per_item; ++tt, ++n) {
        const int s = n % S;
        if (!mbar_wait(&ctrl->full[s], (unsigned)((n / S) & 1), &ctrl->timeout)) {
          if (lane == 0) atomicOr(P.status, kStatusTimeout);
        }
        const uint32_t kbase = stage0 + (uint32_t)s * kFdStageBytes;
        const uint32_t vbase = kbase + 2 * kFdHalfBytes;
        // S = Q K^T for my 16 tokens: two n-tiles of 8 tokens
        float sc0[4] = {0.f, 0.f, 0.f, 0.f}, sc1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          uint32_t kb[4];
          ldmatrix_x4(kb, kbase + fd_swz(k_tok, 2 * kk + k_c8));
          mma_16816(sc0, qa[kk], kb[0], kb[1]);
          mma_16816(sc1, qa[kk], kb[2], kb[3]);
        }
        // scale to the log2 domain, mask the tokens past the end of the split
        const int tok0 = sp * P.split_len + tt * kFdTile + r0 + 2 * t;
        float x[4];
        x[0] = (tok0 < split_hi) ? sc0[0] * P.scale_log2e : -INFINITY;
        x[1] = (tok0 + 1 < split_hi) ? sc0[1] * P.scale_log2e : -INFINITY;
        x[2] = (tok0 + 8 < split_hi) ? sc1[0] * P.scale_log2e : -INFINITY;
        x[3] = (tok0 + 9 < split_hi) ? sc1[1] * P.scale_log2e : -INFINITY;
        float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // all masked so far
        const float alpha = fast_exp2(m_run - m_use);            // exp2(-inf) = 0 on the first tile
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = fast_exp2(x[i] - m_use);
        float ps = (p[0] + p[1]) + (p[2] + p[3]);
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = l_run * alpha + ps;
        m_run = m_new;
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            o[i][0] *= alpha;
            o[i][1] *= alpha;
          }
        }
        // O += P V
        uint32_t pa[4];
        pa[0] = pack_half2(p[0], p[1]);
        pa[1] = 0u;
        pa[2] = pack_half2(p[2], p[3]);
        pa[3] = 0u;
#pragma unroll
        for (int nn = 0; nn < 16; nn += 2) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vbase + fd_swz(v_tok, nn + v_c8));
          mma_16816(o[nn], pa, vb[0], vb[1]);
          mma_16816(o[nn + 1], pa, vb[2], vb[3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctrl->empty[s]);
      }

      // ---- item epilogue: merge the eight warps' partial (maximum, weight, sums) in shared memory
      if (t == 0 && g < G) {
        ctrl->m[warp][g] = m_run;
        ctrl->l[warp][g] = l_run;
      }
      fd_consumer_sync();
      if (g < G) {
        float m_cta = -INFINITY;
#pragma unroll
        for (int w = 0; w < kFdConsumerWarps; ++w) m_cta = fmaxf(m_cta, ctrl->m[w][g]);
        const float f = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_cta);
        float* dst = sm_o + ((size_t)warp * kFdMaxGroup + g) * kHeadDim + 2 * t;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          dst[8 * i] = o[i][0] * f;
          dst[8 * i + 1] = o[i][1] * f;
        }
      }
      fd_consumer_sync();
      {
        const size_t rows = (size_t)P.batch * P.hq;
        for (int idx = tid; idx < G * kHeadDim; idx += 32 * kFdConsumerWarps) {
          const int qh = idx / kHeadDim, d = idx % kHeadDim;
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < kFdConsumerWarps; ++w)
            sum += sm_o[((size_t)w * kFdMaxGroup + qh) * kHeadDim + d];
          float* out = P.partials + ((size_t)sp * rows + (size_t)b * P.hq + (size_t)h * G + qh) *
                                        (kHeadDim + 2);
          out[d] = sum;
          if (d == 0) {
            float m_cta = -INFINITY;
#pragma unroll
            for (int w = 0; w < kFdConsumerWarps; ++w) m_cta = fmaxf(m_cta, ctrl->m[w][qh]);
            float l_cta = 0.f;
#pragma unroll
            for (int w = 0; w < kFdConsumerWarps; ++w) {
              const float mw = ctrl->m[w][qh];
              l_cta += (mw == -INFINITY) ? 0.f : ctrl->l[w][qh] * fast_exp2(mw - m_cta);
            }
            out[kHeadDim] = l_cta;
            out[kHeadDim + 1] = m_cta * 0.6931471805599453f;  // back to the natural-log domain
          }
        }
      }
      fd_consumer_sync();  // the buffers are reused by the next item
    }
  }
}

size_t flash_decode_smem_bytes(int nstages) {
  return (size_t)nstages * kFdStageBytes + (size_t)kFdConsumerWarps * kFdMaxGroup * kHeadDim * 4 +
         sizeof(FdCtrl) + 1024;
}

cudaError_t launch_flash_decode(const FlashParams& P, int grid, size_t smem, cudaStream_t stream) {
  auto kern = flash_decode_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  note_launch();
  kern<<<grid, kFdThreads, smem, stream>>>(P);
  return cudaGetLastError();
}

}  // namespace ra
