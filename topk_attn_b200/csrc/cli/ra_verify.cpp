// Stand-alone C++ driver over the C ABI, in the style of the reference's benchmark programs
// (`make topk`, gemv_topk.cu:388-500; center_only_topk/gemv_topk.cu:465-610): it generates the same
// kind of clustered data on the host (centroids uniform in [-0.5,0.5], members = centroid +
// N(0,0.05), seed 12345), runs the selection on the GPU, times it with CUDA events, and with
// --verify compares the selected ids per (head, cluster rank) slice with a double-precision CPU
// reference, order ignored, reporting recall — the reference's own acceptance check
// (verify_gpu_vs_cpu, gemv_topk.cu:138-170).
//
//   ra_verify topk   [--verify [heads]] [--iters N]    two-level: 32 clusters of 1280 -> top 5 -> top 512
//   ra_verify center [--verify [heads]] [--iters N]    centroid-only: 1024 clusters of 128 -> top 64
//   ra_verify fd     [--verify [heads]] [--iters N]    attention over 2560 random ids per head
//                                                      (flash_decoding.cu:32-37,413-421)
//   ra_verify s1     [--verify [heads]] [--iters N]    two-level selection, then gathered attention:
//                                                      two calls per step (baseline_1.cu:663-701)
//   ra_verify s2     [--verify [heads]] [--iters N]    the pipeline as one call, then once more as two
//                                                      calls, printing max |fused - unfused| over the
//                                                      outputs (`make s2`, baseline_2.cu:1166-1181)
//   ra_verify s3     [--verify [heads]] [--iters N]    the same pipeline as one call
//                                                      (baseline_3.cu:595, the fused version)
//
// For fd/s1/s3 --verify recomputes softmax(q.K/sqrt(D)).V over the ids the GPU used in double
// precision and accepts |diff| <= 1e-3 + 1e-2 |ref|; s1/s3 also check the ids as `topk` does.
//
// Host code only: every device operation goes through topk_attn_b200.h.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "topk_attn_b200.h"

#define CK(x)                                                                      \
  do {                                                                             \
    cudaError_t e_ = (x);                                                          \
    if (e_ != cudaSuccess) {                                                       \
      fprintf(stderr, "%s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(e_));   \
      return 2;                                                                    \
    }                                                                              \
  } while (0)
#define RA(x)                                                                                  \
  do {                                                                                         \
    int s_ = (x);                                                                              \
    if (s_ != RA_OK) {                                                                         \
      fprintf(stderr, "%s:%d %s (%s)\n", __FILE__, __LINE__, ra_strerror(s_), ra_last_cuda_error()); \
      return 2;                                                                                \
    }                                                                                          \
  } while (0)

namespace {

struct Problem {
  int H = 32, D = 128, CSZ, CLEN, TOPC, TOPK;  // TOPK = 0: centroid-only (whole clusters)
  std::vector<__half> q, centers, kv, v;
  bool attend = false;
  int N() const { return CSZ * CLEN; }
  int out_per_head() const { return TOPC * (TOPK ? TOPK : CLEN); }
};

void generate(Problem& p) {
  std::mt19937 rng(12345);
  std::normal_distribution<float> noise(0.0f, 0.05f);
  std::uniform_real_distribution<float> uni(-0.5f, 0.5f);
  p.centers.resize((size_t)p.H * p.CSZ * p.D);
  p.kv.resize((size_t)p.N() * p.H * p.D);
  p.q.resize((size_t)p.H * p.D);
  for (auto& c : p.centers) c = __float2half(uni(rng));
  for (int c = 0; c < p.CSZ; ++c)
    for (int t = 0; t < p.CLEN; ++t)
      for (int h = 0; h < p.H; ++h) {
        const size_t kb = (((size_t)c * p.CLEN + t) * p.H + h) * p.D;
        const size_t cb = ((size_t)h * p.CSZ + c) * p.D;
        for (int d = 0; d < p.D; ++d)
          p.kv[kb + d] = __float2half(__half2float(p.centers[cb + d]) + noise(rng));
      }
  for (auto& x : p.q) x = __float2half(uni(rng));
  if (p.attend) {
    p.v.resize(p.kv.size());
    for (auto& x : p.v) x = __float2half(uni(rng));
  }
}

// double-precision selection on the host: top clusters by centroid score, then (two-level) the
// best TOPK tokens of each chosen cluster; one slice per cluster rank
void cpu_reference(const Problem& p, int heads, std::vector<int>& out) {
  const int per = p.TOPK ? p.TOPK : p.CLEN;
  out.assign((size_t)p.H * p.out_per_head(), -1);
  std::vector<double> cs(p.CSZ);
  std::vector<int> order(p.CSZ);
  std::vector<std::pair<double, int>> ts(p.CLEN);
  for (int h = 0; h < heads; ++h) {
    for (int c = 0; c < p.CSZ; ++c) {
      double acc = 0;
      for (int d = 0; d < p.D; ++d)
        acc += (double)__half2float(p.q[(size_t)h * p.D + d]) *
               (double)__half2float(p.centers[((size_t)h * p.CSZ + c) * p.D + d]);
      cs[c] = acc;
      order[c] = c;
    }
    std::partial_sort(order.begin(), order.begin() + p.TOPC, order.end(),
                      [&](int a, int b) { return cs[a] > cs[b] || (cs[a] == cs[b] && a < b); });
    for (int r = 0; r < p.TOPC; ++r) {
      const int c = order[r];
      int* dst = &out[(size_t)h * p.out_per_head() + (size_t)r * per];
      if (!p.TOPK) {
        for (int i = 0; i < p.CLEN; ++i) dst[i] = c * p.CLEN + i;
        continue;
      }
      for (int t = 0; t < p.CLEN; ++t) {
        double acc = 0;
        const size_t kb = (((size_t)c * p.CLEN + t) * p.H + h) * p.D;
        for (int d = 0; d < p.D; ++d)
          acc += (double)__half2float(p.q[(size_t)h * p.D + d]) * (double)__half2float(p.kv[kb + d]);
        ts[t] = {acc, t};
      }
      std::partial_sort(ts.begin(), ts.begin() + p.TOPK, ts.end(),
                        [](const auto& a, const auto& b) { return a.first > b.first; });
      for (int i = 0; i < p.TOPK; ++i) dst[i] = c * p.CLEN + ts[i].second;
    }
  }
}

bool compare(const Problem& p, int heads, const std::vector<int>& cpu, const std::vector<int>& gpu,
             double& recall) {
  const int per = p.TOPK ? p.TOPK : p.CLEN;
  bool ok = true;
  double sum = 0;
  std::vector<int> a(per), b(per), inter;
  for (int h = 0; h < heads; ++h)
    for (int r = 0; r < p.TOPC; ++r) {
      const size_t off = (size_t)h * p.out_per_head() + (size_t)r * per;
      std::copy(cpu.begin() + off, cpu.begin() + off + per, a.begin());
      std::copy(gpu.begin() + off, gpu.begin() + off + per, b.begin());
      std::sort(a.begin(), a.end());
      std::sort(b.begin(), b.end());
      inter.clear();
      std::set_intersection(a.begin(), a.end(), b.begin(), b.end(), std::back_inserter(inter));
      sum += (double)inter.size() / per;
      if ((int)inter.size() != per) ok = false;
    }
  recall = sum / ((double)heads * p.TOPC);
  return ok;
}

// softmax(scale * q.K[ids]) . V[ids] in double precision over the ids the GPU attended
bool check_attention(const Problem& p, int heads, const std::vector<int>& ids, int n_ids, float scale,
                     const std::vector<__half>& out, double& worst) {
  bool ok = true;
  worst = 0;
  std::vector<double> sc(n_ids), acc(p.D);
  for (int h = 0; h < heads; ++h) {
    double mx = -1e300;
    for (int i = 0; i < n_ids; ++i) {
      const size_t kb = ((size_t)ids[(size_t)h * n_ids + i] * p.H + h) * p.D;
      double a = 0;
      for (int d = 0; d < p.D; ++d)
        a += (double)__half2float(p.q[(size_t)h * p.D + d]) * (double)__half2float(p.kv[kb + d]);
      sc[i] = a * scale;
      mx = std::max(mx, sc[i]);
    }
    double sum = 0;
    std::fill(acc.begin(), acc.end(), 0.0);
    for (int i = 0; i < n_ids; ++i) {
      const double w = std::exp(sc[i] - mx);
      const size_t vb = ((size_t)ids[(size_t)h * n_ids + i] * p.H + h) * p.D;
      sum += w;
      for (int d = 0; d < p.D; ++d) acc[d] += w * (double)__half2float(p.v[vb + d]);
    }
    for (int d = 0; d < p.D; ++d) {
      const double ref = acc[d] / sum, got = __half2float(out[(size_t)h * p.D + d]);
      const double err = std::fabs(ref - got);
      worst = std::max(worst, err);
      if (err > 1e-3 + 1e-2 * std::fabs(ref)) ok = false;
    }
  }
  return ok;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) {
    fprintf(stderr, "usage: %s topk|center|fd|s1|s2|s3 [--verify [heads]] [--iters N]\n", argv[0]);
    return 1;
  }
  Problem p;
  const std::string mode = argv[1];
  const bool random_ids = mode == "fd";
  if (mode == "topk" || mode == "s1" || mode == "s2" || mode == "s3" || mode == "fd") {
    p.CSZ = 32; p.CLEN = 1280; p.TOPC = 5; p.TOPK = 512;       // gemv_topk.cu:21-28
    p.attend = mode != "topk";
  } else if (mode == "center") {
    p.CSZ = 1024; p.CLEN = 128; p.TOPC = 64; p.TOPK = 0;       // center_only_topk/gemv_topk.cu:31-37
  } else {
    fprintf(stderr, "unknown mode %s\n", mode.c_str());
    return 1;
  }
  bool verify = false;
  int heads = p.H, iters = 50;
  for (int i = 2; i < argc; ++i) {
    if (!strcmp(argv[i], "--verify")) {
      verify = true;
      if (i + 1 < argc && argv[i + 1][0] != '-') heads = std::min(p.H, atoi(argv[++i]));
    } else if (!strcmp(argv[i], "--iters") && i + 1 < argc) {
      iters = atoi(argv[++i]);
    }
  }
  generate(p);
  const int n_ids = p.out_per_head();
  const float scale = p.attend ? 1.0f / std::sqrt((float)p.D) : 1.0f;

  __half *d_q, *d_centers, *d_kv, *d_v = nullptr, *d_out = nullptr;
  int *d_ids, *d_clusters;
  const size_t out_elems = (size_t)p.H * n_ids;
  CK(cudaMalloc(&d_q, p.q.size() * 2));
  CK(cudaMalloc(&d_centers, p.centers.size() * 2));
  CK(cudaMalloc(&d_kv, p.kv.size() * 2));
  CK(cudaMalloc(&d_ids, out_elems * 4));
  CK(cudaMalloc(&d_clusters, (size_t)p.H * p.TOPC * 4));
  CK(cudaMemcpy(d_q, p.q.data(), p.q.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_centers, p.centers.data(), p.centers.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_kv, p.kv.data(), p.kv.size() * 2, cudaMemcpyHostToDevice));
  if (p.attend) {
    CK(cudaMalloc(&d_v, p.v.size() * 2));
    CK(cudaMalloc(&d_out, p.q.size() * 2));
    CK(cudaMemcpy(d_v, p.v.data(), p.v.size() * 2, cudaMemcpyHostToDevice));
  }
  std::vector<int> host_ids;
  if (random_ids) {  // distinct random tokens per head, as the reference's flash_decoding program draws
    std::mt19937 rng(777);
    std::vector<int> perm(p.N());
    host_ids.resize(out_elems);
    for (int h = 0; h < p.H; ++h) {
      for (int i = 0; i < p.N(); ++i) perm[i] = i;
      std::shuffle(perm.begin(), perm.end(), rng);
      std::copy(perm.begin(), perm.begin() + n_ids, host_ids.begin() + (size_t)h * n_ids);
    }
    CK(cudaMemcpy(d_ids, host_ids.data(), out_elems * 4, cudaMemcpyHostToDevice));
  }
  const size_t ws_bytes = std::max<size_t>(
      256, p.TOPK ? ra_two_level_workspace_bytes(1, p.H, p.CSZ, p.TOPC, p.TOPK)
                  : ra_center_workspace_bytes(1, p.H, p.CSZ, p.TOPC));
  void* ws;
  CK(cudaMalloc(&ws, ws_bytes));
  CK(cudaMemset(ws, 0, ws_bytes));
  cudaStream_t stream;
  CK(cudaStreamCreate(&stream));

  ra_two_level_params tl;
  memset(&tl, 0, sizeof tl);
  tl.q = d_q; tl.centers = d_centers; tl.k = d_kv;
  tl.batch = 1; tl.num_heads = p.H; tl.head_dim = p.D;
  tl.num_centers = p.CSZ; tl.cluster_len = p.CLEN; tl.top_clusters = p.TOPC;
  tl.topk_per_cluster = p.TOPK; tl.num_tokens = p.N();
  tl.kv_token_stride = (int64_t)p.H * p.D; tl.kv_head_stride = p.D; tl.sm_scale = scale;
  tl.out_cluster_ids = d_clusters; tl.out_indices = d_ids;
  tl.workspace = ws; tl.workspace_bytes = ws_bytes; tl.stream = stream;
  if (mode == "s3" || mode == "s2") { tl.v = d_v; tl.out = d_out; }   // selection + attention in one call
  ra_center_params ce;
  memset(&ce, 0, sizeof ce);
  ce.q = d_q; ce.centers = d_centers; ce.batch = 1; ce.num_heads = p.H; ce.head_dim = p.D;
  ce.num_centers = p.CSZ; ce.cluster_len = p.CLEN; ce.top_clusters = p.TOPC;
  ce.out_cluster_ids = d_clusters; ce.out_indices = d_ids;
  ce.workspace = ws; ce.workspace_bytes = ws_bytes; ce.stream = stream;
  ra_gather_params ga;
  memset(&ga, 0, sizeof ga);
  ga.q = d_q; ga.k = d_kv; ga.v = d_v; ga.out = d_out;
  ga.batch = 1; ga.num_q_heads = p.H; ga.num_kv_heads = p.H; ga.head_dim = p.D; ga.num_tokens = p.N();
  ga.kv_token_stride = (int64_t)p.H * p.D; ga.kv_head_stride = p.D;
  ga.indices = d_ids; ga.num_indices = n_ids; ga.indices_batch_stride = (int64_t)p.H * n_ids;
  ga.sm_scale = scale; ga.workspace = ws; ga.workspace_bytes = ws_bytes; ga.stream = stream;
  auto step = [&]() -> int {
    if (mode == "center") return ra_center_only_topk(&ce);
    if (mode == "fd") return ra_gathered_attention(&ga);
    const int s = ra_two_level_topk(&tl);
    if (s != RA_OK || mode != "s1") return s;
    return ra_gathered_attention(&ga);
  };

  for (int i = 0; i < 10; ++i) RA(step());
  RA(ra_check_status(ws, stream));
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  CK(cudaEventRecord(e0, stream));
  for (int i = 0; i < iters; ++i) RA(step());
  CK(cudaEventRecord(e1, stream));
  CK(cudaEventSynchronize(e1));
  float ms = 0;
  CK(cudaEventElapsedTime(&ms, e0, e1));
  printf("%s: H=%d CSZ=%d CLEN=%d TOPC=%d TOPK=%d  avg latency %.3f us over %d steps\n",
         mode.c_str(), p.H, p.CSZ, p.CLEN, p.TOPC, p.TOPK, ms * 1000.f / iters, iters);

  int rc = 0;
  if (mode == "s2") {
    // the unfused pipeline on the same inputs: selection only, then attention over its ids
    std::vector<__half> fused(p.q.size()), unfused(p.q.size());
    CK(cudaMemcpy(fused.data(), d_out, fused.size() * 2, cudaMemcpyDeviceToHost));
    __half* d_out2;
    CK(cudaMalloc(&d_out2, p.q.size() * 2));
    ra_two_level_params sel = tl;
    sel.v = nullptr; sel.out = nullptr;
    ra_gather_params ga2 = ga;
    ga2.out = d_out2;
    RA(ra_two_level_topk(&sel));
    RA(ra_gathered_attention(&ga2));
    RA(ra_check_status(ws, stream));
    CK(cudaMemcpy(unfused.data(), d_out2, unfused.size() * 2, cudaMemcpyDeviceToHost));
    cudaFree(d_out2);
    double worst = 0, excess = 0;
    for (size_t i = 0; i < fused.size(); ++i) {
      const double a = __half2float(fused[i]), b = __half2float(unfused[i]);
      worst = std::max(worst, std::fabs(a - b));
      excess = std::max(excess, std::fabs(a - b) - (1e-3 + 1e-2 * std::fabs(b)));
    }
    printf("[S2] max |fused - unfused| = %.3e -> %s\n", worst, excess <= 0 ? "PASS" : "FAIL");
    if (excess > 0) rc = 3;
  }
  if (verify) {
    std::vector<int> gpu(out_elems), cpu;
    CK(cudaMemcpy(gpu.data(), d_ids, out_elems * 4, cudaMemcpyDeviceToHost));
    bool ok = true;
    if (!random_ids) {
      cpu_reference(p, heads, cpu);
      double recall = 0;
      ok = compare(p, heads, cpu, gpu, recall);
      printf("[VERIFY] heads=%d recall=%.4f%% -> %s\n", heads, recall * 100.0, ok ? "PASS" : "FAIL");
    }
    if (p.attend) {
      std::vector<__half> out(p.q.size());
      CK(cudaMemcpy(out.data(), d_out, out.size() * 2, cudaMemcpyDeviceToHost));
      double worst = 0;
      const bool aok = check_attention(p, heads, gpu, n_ids, scale, out, worst);
      printf("[VERIFY] heads=%d attention max |diff| = %.3e -> %s\n", heads, worst,
             aok ? "PASS" : "FAIL");
      ok = ok && aok;
    }
    if (!ok) rc = 3;
  }
  cudaFree(d_q); cudaFree(d_centers); cudaFree(d_kv); cudaFree(d_ids); cudaFree(d_clusters); cudaFree(ws);
  if (d_v) cudaFree(d_v);
  if (d_out) cudaFree(d_out);
  return rc;
}
