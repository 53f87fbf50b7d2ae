// Attention over a list of key ids in one pass, shared by the kernels that end in a gathered
// attention: every half-warp streams the K and V rows of its entries together, keeps a running
// maximum / weight / weighted sum (online softmax in the log2 domain), and the partials are merged
// through their log-sum-exp inside the warp, across the warps in shared memory and across the CTAs
// of the cluster in distributed shared memory.
#pragma once
#include <cooperative_groups.h>

#include "cluster_merge.cuh"

namespace ra {

struct GatherPartial {
  float m, l;
  float o[kHeadDim];
};

// Shared memory of flash_over_entries for a CTA of NT threads: NT/32 warp partials and the CTA's own.
template <int NT>
__host__ __device__ constexpr size_t flash_partials_bytes() { return (NT / 32 + 1) * sizeof(GatherPartial); }

// All NT threads of every CTA of the cluster call this.  Entries lo .. lo+n-1 of the row's list are
// this CTA's; token_of(e) gives the key id of entry e (-1: empty slot, skipped), score_of(e) its
// raw q.K when GIVEN (then only V rows are read).  UN: rows in flight per half-warp.  `part` points
// to flash_partials_bytes<NT>() bytes at the same offset in every CTA.  The row's output (and its
// (max, sum) pair when out_lse is given) is written once, no atomics.
template <int UN, bool GIVEN, int NT, typename TokenFn, typename ScoreFn>
__device__ __forceinline__ void flash_over_entries(cg::cluster_group& cluster, int C, int crank,
                                                   GatherPartial* part, const __half* q_row,
                                                   const __half* kb, const __half* vb,
                                                   long long token_stride, int n_tokens, int id_shift,
                                                   int lo, int n, float scale_log2e, unsigned* status,
                                                   __half* out_row, float* out_lse_row,
                                                   TokenFn token_of, ScoreFn score_of) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kW = NT / 32;
  GatherPartial* wpart = part;        // [kW] per-warp partials
  GatherPartial* cpart = part + kW;   // this CTA's partial (peers read)
  const int half = lane >> 4, l16 = lane & 15;
  float qf[8];
  {
    const uint4 a = *reinterpret_cast<const uint4*>(q_row + 8 * l16);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = h2f2(w[i]);
      qf[2 * i] = f.x * scale_log2e;
      qf[2 * i + 1] = f.y * scale_log2e;
    }
  }
  kb += l16 * 8;
  vb += l16 * 8;
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
      const int tok = raw - id_shift;
      ok[u] = raw >= 0 && (unsigned)tok < (unsigned)n_tokens;
      // an empty slot (-1) is skipped silently; any other id outside the cache is reported
      if (e < n && raw >= 0 && !ok[u] && l16 == 0) atomicOr(status, kStatusBadId);
      const size_t off = ok[u] ? (size_t)tok * token_stride : 0;
      if constexpr (GIVEN) {
        given[u] = ok[u] ? score_of(lo + e) * scale_log2e : 0.f;
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
  cluster_barrier(cluster, C);
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
    out_row[d] = __float2half_rn(o / l);
    if (out_lse_row && d == 0) {
      out_lse_row[0] = m * 0.6931471805599453f;  // natural-log domain
      out_lse_row[1] = l;
    }
  }
  cluster_barrier(cluster, C);  // nobody leaves while a peer may still read its partial
}

}  // namespace ra
