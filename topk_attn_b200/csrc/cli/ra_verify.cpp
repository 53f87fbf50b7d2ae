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
//
// Host code only: every device operation goes through topk_attn_b200.h.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
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
  std::vector<__half> q, centers, kv;
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

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) {
    fprintf(stderr, "usage: %s topk|center [--verify [heads]] [--iters N]\n", argv[0]);
    return 1;
  }
  Problem p;
  const std::string mode = argv[1];
  if (mode == "topk") {
    p.CSZ = 32; p.CLEN = 1280; p.TOPC = 5; p.TOPK = 512;       // gemv_topk.cu:21-28
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

  __half *d_q, *d_centers, *d_kv;
  int *d_ids, *d_clusters;
  const size_t out_elems = (size_t)p.H * p.out_per_head();
  CK(cudaMalloc(&d_q, p.q.size() * 2));
  CK(cudaMalloc(&d_centers, p.centers.size() * 2));
  CK(cudaMalloc(&d_kv, p.kv.size() * 2));
  CK(cudaMalloc(&d_ids, out_elems * 4));
  CK(cudaMalloc(&d_clusters, (size_t)p.H * p.TOPC * 4));
  CK(cudaMemcpy(d_q, p.q.data(), p.q.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_centers, p.centers.data(), p.centers.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_kv, p.kv.data(), p.kv.size() * 2, cudaMemcpyHostToDevice));
  const size_t ws_bytes = p.TOPK ? ra_two_level_workspace_bytes(1, p.H, p.CSZ, p.TOPC, p.TOPK)
                                 : ra_center_workspace_bytes(1, p.H, p.CSZ, p.TOPC);
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
  tl.kv_token_stride = (int64_t)p.H * p.D; tl.kv_head_stride = p.D; tl.sm_scale = 1.f;
  tl.out_cluster_ids = d_clusters; tl.out_indices = d_ids;
  tl.workspace = ws; tl.workspace_bytes = ws_bytes; tl.stream = stream;
  ra_center_params ce;
  memset(&ce, 0, sizeof ce);
  ce.q = d_q; ce.centers = d_centers; ce.batch = 1; ce.num_heads = p.H; ce.head_dim = p.D;
  ce.num_centers = p.CSZ; ce.cluster_len = p.CLEN; ce.top_clusters = p.TOPC;
  ce.out_cluster_ids = d_clusters; ce.out_indices = d_ids;
  ce.workspace = ws; ce.workspace_bytes = ws_bytes; ce.stream = stream;
  auto step = [&]() { return p.TOPK ? ra_two_level_topk(&tl) : ra_center_only_topk(&ce); };

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
  printf("%s: H=%d CSZ=%d CLEN=%d TOPC=%d TOPK=%d  avg latency %.3f us over %d launches\n",
         mode.c_str(), p.H, p.CSZ, p.CLEN, p.TOPC, p.TOPK, ms * 1000.f / iters, iters);

  int rc = 0;
  if (verify) {
    std::vector<int> gpu(out_elems), cpu;
    CK(cudaMemcpy(gpu.data(), d_ids, out_elems * 4, cudaMemcpyDeviceToHost));
    cpu_reference(p, heads, cpu);
    double recall = 0;
    const bool ok = compare(p, heads, cpu, gpu, recall);
    printf("[VERIFY] heads=%d recall=%.4f%% -> %s\n", heads, recall * 100.0, ok ? "PASS" : "FAIL");
    rc = ok ? 0 : 3;
  }
  cudaFree(d_q); cudaFree(d_centers); cudaFree(d_kv); cudaFree(d_ids); cudaFree(d_clusters); cudaFree(ws);
  return rc;
}
