// Torch extension `retrieval_attention_cpp`: the reference extension's module name and its 30
// entry points retrieval_attention{,_global,_pipelined,_pipelined_global,_two_kernels,
// _gather_baseline}_{32,128,256,512,1024}(query, key_cache, value_cache, output)
// (retrieval_attn/bind.cpp:726-757), each a thin forward to the C ABI on torch's current stream.
// Differences from the reference, all at the boundary: tensors are validated (the reference reads
// only query.size(0), bind.cpp:252), N comes from key_cache.size(0) instead of a compile-time 8192,
// the call is asynchronous on the current stream (the reference synchronises the device and runs
// ten warm-up launches per call, retrieval_attention.cu:1586-1605), errors raise instead of
// exit(1) (retrieval_attention.cu:17-25), and nothing is printed unless RA_PRINT_TIMING=1.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "topk_attn_b200.h"

namespace {

// Scratch is owned here (torch's caching allocator), one buffer per (device, stream), grown on
// demand; the C ABI itself never allocates.  The entry points are asynchronous on torch's current
// stream, so calls on two streams of one device must not share scratch.  A buffer that is replaced
// by a larger one hands over its status block (the sticky bits a kernel may have set) in stream
// order, and stays alive until the process ends because launches still in flight may use it.
torch::Tensor workspace_for(size_t bytes, const torch::Device& dev, cudaStream_t stream) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, torch::Tensor> cache;
  static std::vector<torch::Tensor> retired;
  std::lock_guard<std::mutex> g(mu);
  const auto key = std::make_pair((int)dev.index(), stream);
  auto it = cache.find(key);
  if (it == cache.end() || (size_t)it->second.numel() < bytes) {
    auto t = torch::zeros({(int64_t)std::max<size_t>(bytes, 1 << 20)},
                          torch::TensorOptions().dtype(torch::kUInt8).device(dev));
    if (it != cache.end()) {
      cudaMemcpyAsync(t.data_ptr(), it->second.data_ptr(), 256, cudaMemcpyDeviceToDevice, stream);
      retired.push_back(it->second);
    }
    cache[key] = t;
    return t;
  }
  return it->second;
}

void check_status(int st, const char* what) {
  TORCH_CHECK(st == RA_OK, what, ": ", ra_strerror(st), " (", ra_last_cuda_error(), ")");
}

void check_half_cuda(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kHalf, name, " must be float16");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

ra_params make_params(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor* v,
                      torch::Tensor* out, int64_t topk, int64_t segments, double sm_scale,
                      int64_t index_base) {
  check_half_cuda(q, "query");
  check_half_cuda(k, "key_cache");
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128, "query must be [B, Hq, 128]");
  TORCH_CHECK((k.dim() == 3 || k.dim() == 4) && k.size(-1) == 128,
              "key_cache must be [N, Hkv, 128] or [B, N, Hkv, 128]");
  if (v) {
    check_half_cuda(*v, "value_cache");
    TORCH_CHECK(v->sizes() == k.sizes(), "value_cache must have the shape of key_cache");
    TORCH_CHECK(v->device() == q.device(), "tensors must be on one device");
  }
  if (out) {
    check_half_cuda(*out, "output");
    TORCH_CHECK(out->sizes() == q.sizes(), "output must have the shape of query");
  }
  TORCH_CHECK(k.device() == q.device(), "tensors must be on one device");
  if (k.dim() == 4) TORCH_CHECK(k.size(0) == q.size(0), "per-sequence cache needs k.size(0) == batch");
  ra_params p;
  memset(&p, 0, sizeof p);
  p.q = q.data_ptr();
  p.k = k.data_ptr();
  p.v = v ? v->data_ptr() : nullptr;
  p.out = out ? out->data_ptr() : nullptr;
  p.batch = (int32_t)q.size(0);
  p.num_q_heads = (int32_t)q.size(1);
  p.num_kv_heads = (int32_t)k.size(-2);
  p.head_dim = 128;
  p.num_tokens = (int32_t)k.size(-3);
  p.kv_batch_stride = k.dim() == 4 ? k.size(1) * k.size(2) * 128 : 0;
  p.kv_token_stride = k.size(-2) * 128;
  p.kv_head_stride = 128;
  p.topk = (int32_t)topk;
  p.num_segments = (int32_t)segments;
  p.sm_scale = (float)sm_scale;
  p.index_base = (int32_t)index_base;
  p.stream = at::cuda::getCurrentCUDAStream(q.device().index()).stream();
  return p;
}

void attach_workspace(ra_params& p, const torch::Device& dev, torch::Tensor& keep) {
  size_t need = ra_workspace_bytes(&p);
  if (need == 0) need = 256;  // the entry point reports what is wrong with the shape
  keep = workspace_for(need, dev, static_cast<cudaStream_t>(p.stream));
  p.workspace = keep.data_ptr();
  p.workspace_bytes = (size_t)keep.numel();
}

// The reference's semantics: 4 chunks, top-K per chunk, exp(s)/sum, no scale.
void legacy(const char* label, int variant, int topk, torch::Tensor query, torch::Tensor key_cache,
            torch::Tensor value_cache, torch::Tensor output) {
  TORCH_CHECK(key_cache.dim() == 3 && key_cache.size(1) == 32 && query.size(1) == 32,
              "the retrieval_attention_* entry points take a shared [N, 32, 128] cache");
  const c10::cuda::CUDAGuard guard(query.device());
  ra_params p = make_params(query, key_cache, &value_cache, &output, topk, 4, 1.0, 0);
  torch::Tensor ws;
  attach_workspace(p, query.device(), ws);
  static const bool timing = getenv("RA_PRINT_TIMING") != nullptr;
  if (!timing) {
    check_status(ra_legacy_retrieval_attention(p.q, p.k, p.v, p.out, p.batch, p.num_tokens, topk,
                                               variant, p.workspace, p.workspace_bytes, p.stream),
                 label);
    return;
  }
  // Optional: reproduce the line the reference prints per call so that scripts which parse it
  // (retrieval_attn/test_ra.py:63-75) keep working.
  cudaStream_t s = static_cast<cudaStream_t>(p.stream);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0, s);
  check_status(ra_legacy_retrieval_attention(p.q, p.k, p.v, p.out, p.batch, p.num_tokens, topk,
                                             variant, p.workspace, p.workspace_bytes, p.stream),
               label);
  cudaEventRecord(e1, s);
  cudaEventSynchronize(e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  printf("%s (TopK=%d, Batch=%d) - Avg time: %.3f ms, Throughput: %.2f iter/s\n", label, topk,
         p.batch, ms, 1000.0f / ms);
  fflush(stdout);
}

// General entry points (not in the reference): global or segmented top-k, explicit scale, GQA,
// per-sequence caches.
std::vector<torch::Tensor> retrieval_attention(torch::Tensor query, torch::Tensor key_cache,
                                               torch::Tensor value_cache, torch::Tensor output,
                                               int64_t topk, int64_t num_segments, double sm_scale,
                                               int64_t index_base, bool return_indices) {
  const c10::cuda::CUDAGuard guard(query.device());
  ra_params p = make_params(query, key_cache, &value_cache, &output, topk, num_segments, sm_scale,
                            index_base);
  std::vector<torch::Tensor> res;
  torch::Tensor idx, sc;
  if (return_indices) {
    idx = torch::empty({query.size(0), query.size(1), num_segments * topk},
                       torch::TensorOptions().dtype(torch::kInt32).device(query.device()));
    sc = torch::empty({query.size(0), query.size(1), num_segments * topk},
                      torch::TensorOptions().dtype(torch::kFloat32).device(query.device()));
    p.out_indices = idx.data_ptr<int32_t>();
    p.out_scores = sc.data_ptr<float>();
    res = {idx, sc};
  }
  torch::Tensor ws;
  attach_workspace(p, query.device(), ws);
  check_status(ra_topk_attention(&p), "retrieval_attention");
  return res;
}

std::vector<torch::Tensor> gemv_topk(torch::Tensor query, torch::Tensor key_cache, int64_t topk,
                                     int64_t num_segments, int64_t index_base) {
  const c10::cuda::CUDAGuard guard(query.device());
  ra_params p = make_params(query, key_cache, nullptr, nullptr, topk, num_segments, 1.0, index_base);
  auto idx = torch::empty({query.size(0), query.size(1), num_segments * topk},
                          torch::TensorOptions().dtype(torch::kInt32).device(query.device()));
  auto sc = torch::empty({query.size(0), query.size(1), num_segments * topk},
                         torch::TensorOptions().dtype(torch::kFloat32).device(query.device()));
  p.out_indices = idx.data_ptr<int32_t>();
  p.out_scores = sc.data_ptr<float>();
  torch::Tensor ws;
  attach_workspace(p, query.device(), ws);
  check_status(ra_gemv_topk(&p), "gemv_topk");
  return {idx, sc};
}

}  // namespace

#define RA_LEGACY(NAME, LABEL, VARIANT, K)                                                        \
  void NAME##_##K(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor o) {          \
    legacy(LABEL, VARIANT, K, q, k, v, o);                                                       \
  }
#define RA_LEGACY_ALL(NAME, LABEL, VARIANT) \
  RA_LEGACY(NAME, LABEL, VARIANT, 32)       \
  RA_LEGACY(NAME, LABEL, VARIANT, 128)      \
  RA_LEGACY(NAME, LABEL, VARIANT, 256)      \
  RA_LEGACY(NAME, LABEL, VARIANT, 512)      \
  RA_LEGACY(NAME, LABEL, VARIANT, 1024)

RA_LEGACY_ALL(retrieval_attention, "Retrieval Attention", 0)
RA_LEGACY_ALL(retrieval_attention_global, "Retrieval Attention Global", 1)
RA_LEGACY_ALL(retrieval_attention_pipelined, "Pipelined Retrieval Attention", 2)
RA_LEGACY_ALL(retrieval_attention_pipelined_global, "Pipelined Retrieval Attention Global", 3)
RA_LEGACY_ALL(retrieval_attention_two_kernels, "Retrieval Attention Two Kernels", 4)
RA_LEGACY_ALL(retrieval_attention_gather_baseline, "Retrieval Attention Gather+Baseline", 5)

#define RA_DEF(NAME, K, DOC) m.def(#NAME "_" #K, &NAME##_##K, DOC " (TopK=" #K ")");
#define RA_DEF_ALL(NAME, DOC) \
  RA_DEF(NAME, 32, DOC) RA_DEF(NAME, 128, DOC) RA_DEF(NAME, 256, DOC) RA_DEF(NAME, 512, DOC) RA_DEF(NAME, 1024, DOC)

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  RA_DEF_ALL(retrieval_attention, "Retrieval Attention")
  RA_DEF_ALL(retrieval_attention_global, "Retrieval Attention Global")
  RA_DEF_ALL(retrieval_attention_pipelined, "Pipelined Retrieval Attention")
  RA_DEF_ALL(retrieval_attention_pipelined_global, "Pipelined Retrieval Attention Global")
  RA_DEF_ALL(retrieval_attention_two_kernels, "Retrieval Attention Two Kernels")
  RA_DEF_ALL(retrieval_attention_gather_baseline, "Retrieval Attention Gather+Baseline")
  m.def("retrieval_attention", &retrieval_attention, "Top-k sparse decode attention (general)",
        py::arg("query"), py::arg("key_cache"), py::arg("value_cache"), py::arg("output"),
        py::arg("topk"), py::arg("num_segments") = 1, py::arg("sm_scale") = 1.0,
        py::arg("index_base") = 0, py::arg("return_indices") = false);
  m.def("gemv_topk", &gemv_topk, "Exact top-k selection (indices, scores)", py::arg("query"),
        py::arg("key_cache"), py::arg("topk"), py::arg("num_segments") = 1,
        py::arg("index_base") = 0);
}
