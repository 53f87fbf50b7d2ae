// Host side of the C ABI: argument validation, launch planning, tensor-map encoding and kernel
// launches.  Nothing here allocates device memory or synchronises (ra_check_status excepted).
#include "topk_attn_b200.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "center_select.cuh"
#include "dense_select.cuh"
#include "exchange.cuh"
#include "flash_decode.cuh"
#include "gather_attend.cuh"
#include "merge_attend.cuh"
#include "scan_select.cuh"
#include "scan_store.cuh"
#include "select_sharded.cuh"

namespace ra {
int scan_max_active_clusters(int hg, int nq, int cluster, size_t smem, int threads);
std::atomic<unsigned long long> g_launch_count{0};
}

extern "C" {
// attention over id lists (defined with the entry points below); with src_score and
// expand_clen == 0 the lists carry their scores and only V is read
static int run_gather(const __half* q, const __half* k, const __half* v, __half* out, float* out_lse,
                      int batch, int hq, int hkv, int n_tokens, long long bs, long long ts,
                      long long hs, const int* src_idx, const float* src_score,
                      long long src_bstride, long long src_hstride, int n_src, int expand_clen,
                      int* out_token_ids, float sm_scale, unsigned* status, bool attend,
                      cudaStream_t stream, int id_shift = 0);
}

namespace {

using namespace ra;

thread_local std::string g_last_error;

int cuda_fail(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  (void)cudaGetLastError();
  return RA_ERR_CUDA;
}
int invalid(const char* why) {
  g_last_error = why;
  return RA_ERR_INVALID_ARGUMENT;
}
int unsupported(const char* why) {
  g_last_error = why;
  return RA_ERR_UNSUPPORTED;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Route and geometry overrides (RA_FORCE_*, RA_NO_*, RA_DEBUG_FLAGS) exist only in a library built
// with -DRA_TUNING (lib/libtopk_attn_b200_tuning.so, used by the A/B tests and the phase profile
// of the bench); the default build reads no environment variable on the call path.
#ifdef RA_TUNING
const char* tuning_env(const char* name) { return getenv(name); }
bool verbose_plan() { return getenv("RA_VERBOSE") != nullptr; }
#else
const char* tuning_env(const char*) { return nullptr; }
bool verbose_plan() {
  static const bool v = getenv("RA_VERBOSE") != nullptr;   // read once, when first asked
  return v;
}
#endif

// Multiprocessors of the current device (queried once per device).
int sm_count() {
  static std::mutex mu;
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return 148;
  }
  std::lock_guard<std::mutex> g(mu);
  if (!cached[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
      (void)cudaGetLastError();
      v = 148;
    }
    cached[dev] = v;
  }
  return cached[dev];
}

// Parameters of the planner's time model: what the whole device and one multiprocessor stream from
// HBM.  They rank launch geometries against each other; absolute accuracy is not needed.
constexpr double kModelHbmBytesPerSec = 6.5e12;
constexpr double kModelSmBytesPerSec = 75e9;

constexpr size_t kSmemBudget = 227 * 1024;
constexpr size_t kStatusBytes = 256;
constexpr int kMaxSplit = 16;  // parts one head's context may be cut into


struct Plan {
  bool ok = false;
  int hg = 0, nq = 0, bshare = 1, nq_valid = 1, qsplit = 1, nq_cta = 1;
  int cluster = 1, nsplit = 1, cap = 0, nstages = 0, per = 0, part_len = 0, grid = 0;
  int groups = 2, rendezvous = 4;
  int det_words = 32;  // bitmap words of the ordered deal in the scan kernel's scratch
  bool parts_in_cluster = false;  // every segment of a (row, head) is one CTA of one cluster
  size_t smem = 0;
  // second stage (only when parts > 1)
  int cluster2 = 1, cap2 = 0, per2 = 0;
  size_t smem2 = 0;
  double cost = 0;
};

struct Shape {
  int batch, hq, hkv, n, topk, segments, per_batch, head_major, fused_ok;
  bool operator<(const Shape& o) const {
    return std::tie(batch, hq, hkv, n, topk, segments, per_batch, head_major, fused_ok) <
           std::tie(o.batch, o.hq, o.hkv, o.n, o.topk, o.segments, o.per_batch, o.head_major,
                    o.fused_ok);
  }
};

int next_pow2(int x) {
  int p = 1;
  while (p < x) p <<= 1;
  return p;
}

bool combo_built(int hg, int nq) {
  static const int ok[][2] = {{1, 1}, {2, 1}, {4, 1}, {8, 1}, {1, 2}, {2, 2}, {4, 2}, {1, 4}, {2, 4}, {1, 8}};
  for (auto& c : ok)
    if (c[0] == hg && c[1] == nq) return true;
  return false;
}

// Most parts the planner may cut one segment into: the largest nsplit that make_plan() accepts for
// any tile height (its own predicate: the tile-rounded part holds k keys and the last part is not
// empty).
int max_parts(int seg_len, int topk) {
  int best = 1;
  for (int T : {16, 32, 64, 128})
    for (int nsplit = 2; nsplit <= kMaxSplit; ++nsplit) {
      const int part_len = ceil_div(ceil_div(seg_len, nsplit), T) * T;
      if (part_len < topk) break;
      if ((long long)part_len * (nsplit - 1) >= seg_len) continue;
      best = std::max(best, nsplit);
    }
  return best;
}

// Queries that share a K row: batch rows on one shared cache times the GQA group, at most 8.
int shared_queries(const Shape& s, int* bshare_out = nullptr) {
  const int group = s.hq / s.hkv;
  int bshare = 1;
  if (!s.per_batch && !(s.fused_ok & 2))
    for (int b = 1; b <= s.batch; ++b)
      if (s.batch % b == 0 && b * group <= 8) bshare = b;
  if (bshare_out) *bshare_out = bshare;
  return bshare * group;
}

// Layout of the workspace: [status block][candidate lists of `parts` parts][stored score keys and
// coarse histograms].  Offsets are multiples of 256 bytes.
size_t cand_bytes(const Shape& s, int parts) {
  return ((size_t)s.batch * s.hq * parts * s.topk * 8 + 255) & ~size_t(255);
}
int store_pitch(int n) { return (n + 127) & ~127; }
size_t store_keys_bytes(const Shape& s) {
  return ((size_t)s.batch * s.hq * store_pitch(s.n) * 4 + 255) & ~size_t(255);
}
size_t store_hist_bytes(const Shape& s, int parts) {
  return (size_t)s.batch * s.hq * parts * kHistBins * 4;
}
// The score-store route is taken for one global selection with several queries per K row (see
// run_store); its scratch replaces the candidate lists.
bool store_shape(const Shape& s) { return s.segments == 1 && !(s.fused_ok & 6) && shared_queries(s) > 1; }

// Second-stage geometry for m_total candidates per row with `topk` winners.
bool plan_merge(int m_total, int topk, Plan& pl) {
  int f_c2 = 0;
  if (const char* f = tuning_env("RA_FORCE_MERGE_CLUSTER")) f_c2 = atoi(f);
  for (int c2 : {1, 2, 4, 8}) {
    if (f_c2 && c2 != f_c2) continue;
    const int cap2 = ceil_div(m_total, c2), per2 = ceil_div(topk, c2);
    const size_t smem2 = merge_attend_smem_bytes(per2, cap2);
    if (smem2 > kSmemBudget) continue;
    // enough CTAs per row to keep the V gather of a CTA short (<= 512 rows) and its list small
    if (!f_c2 && (cap2 > 4096 || per2 > 512) && c2 < 8) continue;
    pl.cluster2 = c2;
    pl.cap2 = cap2;
    pl.per2 = per2;
    pl.smem2 = smem2;
    return true;
  }
  return false;
}

// The single-CTA merge when the row's candidates fit in one CTA's shared memory, else the cluster
// form.
// Whether the single-CTA merge takes these candidates: keys and ids in shared memory when both fit,
// else the keys alone (ids fetched for the winners).  Measured on configuration 4 cut over 8 ranks
// (32 rows x 32768 candidates, cold L2): 41 us against 55 us for a cluster of 8 CTAs per row, so the
// single CTA is taken whenever it fits.  Sets mp.ids_global.
bool merge_fits_one_cta(MergeParams& mp, int rows, size_t& smem) {
  (void)rows;
  if (tuning_env("RA_FORCE_MERGE_CLUSTER")) return false;
  for (int ids_global = 0; ids_global < 2; ++ids_global) {
    smem = merge_attend_cta_smem_bytes(mp.m_total, mp.m.topk, ids_global != 0);
    if (smem <= kSmemBudget) {
      mp.ids_global = ids_global;
      return true;
    }
  }
  return false;
}

cudaError_t dispatch_merge(MergeParams& mp, int rows, const Plan& pl, cudaStream_t stream) {
  size_t one = 0;
  if (merge_fits_one_cta(mp, rows, one)) {
    mp.m.cluster = 1;
    return launch_merge_attend_cta(mp, rows, one, stream);
  }
  return launch_merge_attend(mp, rows, pl.smem2, stream);
}

// Pick the launch geometry with the lowest modelled time.  The model: every CTA streams its
// slab at min(per-SM rate, its fair share of HBM); clusters that do not fit at once run in
// waves; a second kernel costs a fixed latency.
Plan make_plan(const Shape& s) {
  static std::mutex mu;
  static std::map<Shape, Plan> cache;
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(s);
    if (it != cache.end()) return it->second;
  }
  Plan best;
  // RA_FORCE_PLAN="hg,cluster,nsplit" pins the geometry (0 = free); for tuning only
  int f_hg = 0, f_cluster = 0, f_nsplit = 0, f_stages = 0;
  if (const char* f = tuning_env("RA_FORCE_PLAN"))
    sscanf(f, "%d,%d,%d,%d", &f_hg, &f_cluster, &f_nsplit, &f_stages);
  const bool own_parts = (s.fused_ok & 2) != 0;
  int bshare = 1;
  const int nq_valid = shared_queries(s, &bshare);
  const int seg_len = s.n / s.segments;
  const double hbm = kModelHbmBytesPerSec, per_sm = kModelSmBytesPerSec;
  int f_qsplit = 0;
  if (const char* f = tuning_env("RA_FORCE_QSPLIT")) f_qsplit = atoi(f);
  for (int qsplit : {1, 2, 4, 8})
  for (int hg : {8, 4, 2, 1}) {
    if (nq_valid % qsplit || (f_qsplit && qsplit != f_qsplit)) continue;
    const int nq_cta = nq_valid / qsplit;
    const int nq = next_pow2(nq_cta);
    if (qsplit > 1 && hg != 1) continue;
    if (own_parts && hg != 1) continue;
    if (s.hkv % hg || !combo_built(hg, nq)) continue;
    if (s.head_major && hg != 1) continue;
    if (f_hg && hg != f_hg) continue;
    // several queries per K row are scored on the tensor cores, one kv head per CTA
    if (nq > 1 && hg != 1 && !tuning_env("RA_NO_MMA")) continue;
    const int nl = hg * nq, T = kTileRows / hg;
    // bit 8 of fused_ok: the caller attends over all segments of a (row, head) and they are few
    // enough to be the CTAs of one cluster -- each CTA scans and selects its own segment, the
    // attention is merged across the cluster, nothing goes through global memory
    const bool pic = (s.fused_ok & 8) != 0;
    const int groups = (s.batch / bshare) * (s.hkv / hg) * (pic ? 1 : s.segments) * qsplit;
    for (int cluster : {1, 2, 4, 8, 16, 0}) {
      if (pic != (cluster == 0)) continue;
      if (cluster == 0) cluster = s.segments;
      if (f_cluster && cluster != f_cluster && !pic) continue;
      for (int nsplit = 1; nsplit <= kMaxSplit; ++nsplit) {
        if (nsplit > 1 && (s.segments > 1 || (s.fused_ok & 4))) break;
        if (f_nsplit && nsplit != f_nsplit) continue;
        int part_len = ceil_div(ceil_div(seg_len, nsplit), T) * T;
        if (nsplit > 1 && part_len < s.topk) break;           // every part must hold k keys
        if (nsplit > 1 && part_len * (nsplit - 1) >= seg_len) continue;  // empty last part
        if (nsplit == 1) part_len = seg_len;
        const int tiles = ceil_div(part_len, T);
        if (!pic && cluster > 1 && tiles < cluster) continue;
        const int per = pic ? s.topk : ceil_div(s.topk, cluster);
        // scratch of the cluster select in the freed pipeline stages; the bitmap of the ordered
        // deal covers a CTA's token slab in one window when the stages have room for it
        const size_t scratch = merge_scratch_bytes(nl, per, 32);
        const int cta_tiles = pic ? tiles : ceil_div(tiles, cluster);
        const int slab_tokens = cta_tiles * T;
        // stages, consumer groups, check interval and list capacity within the shared-memory
        // budget: the deepest pipeline whose lists still hold k keys plus the keys that may arrive
        // between two overflow checks
        // Long parts take the deepest pipeline that fits.  Short parts (a few tiles) are bound by
        // fixed costs and by how many CTAs run at once: the shallower geometries, which leave room
        // for two CTAs per SM, compete as well, at a penalty on their stream time.
        struct Geo { int nstages, cap, cgroups, rdv; double slow; int det; };
        Geo geos[4];
        int ngeo = 0;
        static const double kSlow[4] = {1.0, 1.05, 1.2, 1.35};
        // one query per K row: scoring is latency-bound, two warp groups and deep rings help;
        // several queries per row (tensor-core scoring): one group and roomier lists win
        static const int kGeo1[4][2] = {{2, 6}, {2, 4}, {1, 3}, {1, 2}};
        static const int kGeoN[4][2] = {{2, 4}, {1, 3}, {1, 2}, {1, 2}};
        const int (*kGeo)[2] = (nq > 1) ? kGeoN : kGeo1;
        for (int gi = 0; gi < 4; ++gi) {
          const int* ge = kGeo[gi];
          const int g2 = ge[0], st = ge[1];
          if (f_stages && st != f_stages) continue;
          if ((size_t)st * kStageBytes < scratch) continue;
          const size_t fixed = scan_smem_bytes(nl, 0, st);
          if (fixed >= kSmemBudget) continue;
          const int fit = (int)((kSmemBudget - fixed) / ((size_t)nl * 8));
          for (int r : {4, 2, 1}) {
            const int margin = r * g2 * T;
            const int c = std::min(fit, 2 * s.topk + margin);
            const int want = (st > 4) ? (3 * s.topk) / 2 + margin : s.topk + margin + 64;
            if (c >= std::min(want, 2 * s.topk + margin)) {
              const int room = (int)(((size_t)st * kStageBytes - merge_scratch_bytes(nl, per, 0)) / 8) & ~31;
              geos[ngeo++] = Geo{st, c, g2, r, kSlow[gi], std::min(det_words_for(slab_tokens), room)};
              break;
            }
          }
          if (ngeo && (tiles > 32 || f_stages)) break;
        }
        for (int gx = 0; gx < ngeo; ++gx) {
        const int nstages = geos[gx].nstages, cap = geos[gx].cap, cgroups = geos[gx].cgroups,
                  rdv = geos[gx].rdv;
        const size_t smem = scan_smem_bytes(nl, cap, nstages);
        const int nclusters = groups * nsplit;
        const int active = scan_max_active_clusters(hg, nq, cluster, smem, 32 * (8 * cgroups + 1));
        if (active <= 0) continue;
        const int waves = ceil_div(nclusters, active);
        const int live = std::min(nclusters, active) * cluster;
        const double bytes_cta = (double)cta_tiles * kStageBytes;
        // clusters that share a K row stream it once from HBM and qsplit - 1 times from L2
        const double rate = std::min(per_sm, hbm * qsplit / live);
        // every cut of a candidate list stalls the CTA's consumers for a few microseconds; the
        // seen-token count grows by (1 + room/k) between two cuts of one list
        const int margin = rdv * cgroups * T;
        const double room = std::max(64, cap - s.topk - margin);
        const double slab = (double)cta_tiles * T;
        const double cuts = slab > cap ? std::log(slab / cap) / std::log1p(room / s.topk) + 1.0 : 0.0;
        const bool two_stage = !pic && (nsplit > 1 || s.segments > 1);
        // clusters of up to 4 CTAs cost little; 8 and more are hard to co-schedule with 227 KiB of
        // shared memory per CTA and measured about twice as slow
        const double cluster_cost = cluster <= 4 ? 0.4e-6 * cluster : 4e-6 * cluster;
        // until a list has filled once every key passes the threshold and is appended: about a
        // microsecond per iteration instead of a fraction of one
        const double warmup = 1e-6 * std::min(cta_tiles, cap / T) / cgroups;
        double cost = waves * (geos[gx].slow * bytes_cta / rate + cuts * nl * 2e-6 + warmup + 6e-6 +
                               cluster_cost) +
                      (two_stage ? 8e-6 : 0.0);
        Plan pl;
        pl.hg = hg; pl.nq = nq; pl.bshare = bshare; pl.nq_valid = nq_valid;
        pl.qsplit = qsplit; pl.nq_cta = nq_cta;
        pl.cluster = cluster; pl.nsplit = nsplit; pl.cap = cap; pl.nstages = nstages;
        pl.groups = cgroups; pl.rendezvous = rdv; pl.det_words = geos[gx].det;
        pl.parts_in_cluster = pic;
        pl.per = per; pl.part_len = part_len; pl.grid = nclusters * cluster; pl.smem = smem;
        pl.cost = cost;
        if (two_stage && !plan_merge(s.segments * nsplit * s.topk,
                                     s.segments > 1 ? s.segments * s.topk : s.topk, pl))
          continue;
        pl.ok = true;
        if (!best.ok || pl.cost < best.cost) best = pl;
        }
      }
    }
  }
  std::lock_guard<std::mutex> g(mu);
  cache[s] = best;
  return best;
}

struct Checked {
  Shape shape;
  int group;
};

int check_shape(const ra_params* p, Checked& c) {
  if (!p) return invalid("params is null");
  if (p->head_dim != kHeadDim) return unsupported("head_dim must be 128");
  if (p->batch < 1 || p->num_q_heads < 1 || p->num_kv_heads < 1 || p->num_tokens < 1)
    return invalid("batch, heads and num_tokens must be positive");
  if (p->num_q_heads % p->num_kv_heads) return invalid("num_kv_heads must divide num_q_heads");
  c.group = p->num_q_heads / p->num_kv_heads;
  if (c.group > 8) return unsupported("more than 8 query heads per kv head");
  if (p->num_segments < 1 || p->num_tokens % p->num_segments)
    return invalid("num_tokens must be a multiple of num_segments");
  if (p->topk < 1 || p->topk > p->num_tokens / p->num_segments)
    return invalid("topk must be in [1, tokens per segment]");
  if (p->topk > 8192) return unsupported("topk above 8192");
  if (p->kv_token_stride < kHeadDim || p->kv_head_stride < kHeadDim || (p->kv_token_stride % 8) ||
      (p->kv_head_stride % 8) || (p->kv_batch_stride % 8) || p->kv_batch_stride < 0)
    return invalid("kv strides must be multiples of 8 elements and at least 128");
  c.shape.batch = p->batch;
  c.shape.hq = p->num_q_heads;
  c.shape.hkv = p->num_kv_heads;
  c.shape.n = p->num_tokens;
  c.shape.topk = p->topk;
  c.shape.segments = p->num_segments;
  c.shape.per_batch = p->kv_batch_stride != 0;
  c.shape.head_major = p->kv_head_stride > p->kv_token_stride;
  c.shape.fused_ok = 1;
  return RA_OK;
}

int check_params(const ra_params* p, bool need_v, bool need_out, Checked& c) {
  int st = check_shape(p, c);
  if (st != RA_OK) return st;
  if (!p->q || !p->k) return invalid("q or k is null");
  if (need_v && !p->v) return invalid("v is null");
  if (need_out && !p->out) return invalid("out is null");
  auto mis = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) != 0; };
  if (mis(p->q) || mis(p->k) || (p->v && mis(p->v)) || (p->out && mis(p->out)))
    return invalid("q, k, v and out must be 16-byte aligned");
  if (!(p->sm_scale > 0.f)) return invalid("sm_scale must be positive");
  if (!p->workspace) {
    g_last_error = "workspace is null";
    return RA_ERR_WORKSPACE;
  }
  if (reinterpret_cast<uintptr_t>(p->workspace) & 255u) return invalid("workspace must be 256-byte aligned");
  return RA_OK;
}

// Device-independent upper bound of the scratch any plan for this shape may use.
size_t workspace_bound(const Shape& s) {
  const int seg_len = s.n / s.segments;
  const int maxsplit = s.segments == 1 ? max_parts(seg_len, s.topk) : 1;
  size_t w = kStatusBytes + cand_bytes(s, s.segments * maxsplit);
  if (store_shape(s)) w = std::max(w, kStatusBytes + store_keys_bytes(s) + store_hist_bytes(s, kMaxSplit));
  return w;
}

int encode_kmap(CUtensorMap* map, const ra_params* p, const Shape& s, int hg, bool swizzled,
                int n_tokens) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) {
    g_last_error = "cuTensorMapEncodeTiled is not available from the driver";
    return RA_ERR_CUDA;
  }
  const cuuint64_t nb = s.per_batch ? (cuuint64_t)p->batch : 1;
  cuuint64_t bstride =
      s.per_batch ? (cuuint64_t)p->kv_batch_stride * 2
                  : (cuuint64_t)16 * (((cuuint64_t)n_tokens * p->kv_token_stride * 2 + 15) / 16);
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  const int T = kTileRows / hg;
  if (s.head_major) {
    dims[0] = kHeadDim; dims[1] = n_tokens; dims[2] = p->num_kv_heads; dims[3] = nb;
    strides[0] = (cuuint64_t)p->kv_token_stride * 2; strides[1] = (cuuint64_t)p->kv_head_stride * 2;
    box[0] = kHeadDim; box[1] = T; box[2] = 1; box[3] = 1;
    if (!s.per_batch) bstride = (cuuint64_t)p->num_kv_heads * p->kv_head_stride * 2;
  } else {
    dims[0] = kHeadDim; dims[1] = p->num_kv_heads; dims[2] = n_tokens; dims[3] = nb;
    strides[0] = (cuuint64_t)p->kv_head_stride * 2; strides[1] = (cuuint64_t)p->kv_token_stride * 2;
    box[0] = kHeadDim; box[1] = hg; box[2] = T; box[3] = 1;
  }
  strides[2] = bstride;
  if (swizzled) box[0] = 64;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(p->k), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[96];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    g_last_error = buf;
    return RA_ERR_CUDA;
  }
  return RA_OK;
}

constexpr float kLog2e = 1.4426950408889634f;

// attend == false: selection only (indices/scores out).
// Two-level retrieval: part i of a (batch row, head) is the cluster ids[row][i] of cluster_len
// tokens instead of the i-th slice of the token axis; p->num_tokens is then parts * cluster_len.
struct PartIds {
  const int* ids;
  int real_tokens;
  // centroid retrieval in one launch: the winners are cluster ids, expanded in rank order
  int expand_clen = 0;
  int* expand_out = nullptr;
  int* expand_ids = nullptr;
  // status block of the caller's workspace when p->workspace is only an inner slice of it
  unsigned* status = nullptr;
  // two-level retrieval with a small centroid table: the scan kernel ranks the centroids itself
  const void* coarse_centers = nullptr;
  int coarse_csz = 0;
  int* coarse_ids_out = nullptr;
};

int run_store(const ra_params* p, const Shape& s, int group, bool attend, unsigned* status,
              const ra_shard_exchange* sx = nullptr, bool scan_only = false);

int run(const ra_params* p, bool attend, const PartIds* ext = nullptr) {
  Checked c;
  int st = check_params(p, attend, attend, c);
  if (st != RA_OK) return st;
  if (!attend && !p->out_indices && !(ext && ext->expand_out)) return invalid("out_indices is required");
  Shape s = c.shape;
  // bit 1: every (row, head) scans its own parts — nothing is shared; bit 2: one part only (the
  // scan kernel itself must produce the final winners)
  s.fused_ok = 1 | ((ext && (ext->ids || ext->coarse_centers)) ? 2 : 0) | ((ext && ext->expand_out) ? 4 : 0);
  // attention over a few per-segment selections of own parts (two-level retrieval): the segments of
  // a (row, head) become the CTAs of one cluster and the whole pipeline is one launch
  if (attend && (s.fused_ok & 2) && s.segments >= 2 && s.segments <= 8 && !tuning_env("RA_NO_SEGMENT_CLUSTER"))
    s.fused_ok |= 8;
  const int real_tokens = (ext && (ext->ids || ext->coarse_centers)) ? ext->real_tokens : s.n;
  const bool verbose = verbose_plan();
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  unsigned* status = (ext && ext->status) ? ext->status : static_cast<unsigned*>(p->workspace);
  // Short segments: score every key into shared memory and select afterwards (no candidate lists),
  // then one pass over the V rows of the lists.
  const int seg_len = s.n / s.segments;
  int dense_bshare = 1;
  if (!s.per_batch)
    for (int b = 1; b <= s.batch; ++b)
      if (s.batch % b == 0 && b * c.group <= 8) dense_bshare = b;
  // (one query per K row and one segment: the fused single launch of the scan kernel is quicker)
  if (!ext && seg_len <= kDenseMaxSeg &&
      (s.segments > 1 || dense_bshare * c.group > 1 || tuning_env("RA_DENSE_SINGLE")) &&
      !tuning_env("RA_NO_DENSE_SELECT")) {
    const int bshare = dense_bshare;
    const int nq_valid = bshare * c.group, nq = next_pow2(nq_valid);
    const size_t lists = (size_t)s.batch * s.hq * s.segments * s.topk;
    if (p->workspace_bytes < kStatusBytes + lists * 8) {
      g_last_error = "workspace smaller than ra_workspace_bytes()";
      return RA_ERR_WORKSPACE;
    }
    float* l_score = reinterpret_cast<float*>(static_cast<char*>(p->workspace) + kStatusBytes);
    int* l_idx = reinterpret_cast<int*>(l_score + lists);
    DenseSelectParams dp;
    memset(&dp, 0, sizeof dp);
    dp.q = static_cast<const __half*>(p->q); dp.k = static_cast<const __half*>(p->k);
    dp.batch_stride = p->kv_batch_stride; dp.token_stride = p->kv_token_stride;
    dp.head_stride = p->kv_head_stride;
    dp.batch = s.batch; dp.hq = s.hq; dp.hkv = s.hkv; dp.group = c.group;
    dp.bshare = bshare; dp.nq_valid = nq_valid;
    dp.seg_len = seg_len; dp.segments = s.segments; dp.topk = s.topk;
    // CTAs per (segment, kv head, batch group): about 512 rows each, but not more CTAs than run
    // at once (two per multiprocessor): a second wave would double the time of a step this short
    const int items = s.segments * s.hkv * (s.batch / bshare);
    int cl = 1;
    while (cl < kDenseMaxCluster && seg_len > 512 * cl && (long long)items * cl * 2 <= 2LL * sm_count()) cl <<= 1;
    dp.cluster = cl; dp.per = (ceil_div(seg_len, cl) + 3) & ~3;
    dp.index_base = p->index_base;
    dp.status = status;
    dp.out_idx = p->out_indices ? p->out_indices : l_idx;
    dp.out_score = p->out_scores ? p->out_scores : l_score;
    if (verbose)
      fprintf(stderr, "[topk_attn_b200] plan: dense select nq=%d(valid %d) cluster=%d seg_len=%d\n", nq,
              nq_valid, cl, seg_len);
    cudaError_t e = launch_dense_select(dp, nq, stream);
    if (e != cudaSuccess) return cuda_fail(e, "dense_select launch");
    if (!attend) return RA_OK;
    const long long per_row = (long long)s.segments * s.topk;
    return run_gather(static_cast<const __half*>(p->q), nullptr, static_cast<const __half*>(p->v),
                      static_cast<__half*>(p->out), p->out_lse, s.batch, s.hq, s.hkv, s.n,
                      p->kv_batch_stride, p->kv_token_stride, p->kv_head_stride, dp.out_idx,
                      dp.out_score, (long long)s.hq * per_row, per_row, (int)per_row, 0, nullptr,
                      p->sm_scale, status, true, stream, p->index_base);
  }
  // Several queries per K row and one global selection: scores are stored and selected afterwards.
  if (!ext && store_shape(s) && !tuning_env("RA_NO_SCORE_STORE")) return run_store(p, s, c.group, attend, status);

  const Plan pl = make_plan(s);
  if (!pl.ok) return unsupported("no launch geometry fits these sizes");
  static thread_local Shape last_shown = {};
  const bool show = verbose && ((last_shown < s) || (s < last_shown));
  if (show) last_shown = s;
  if (show)
    fprintf(stderr,
            "[topk_attn_b200] plan: hg=%d nq=%d(valid %d, qsplit %d) bshare=%d cluster=%d nsplit=%d cap=%d "
            "stages=%d groups=%d rdv=%d per=%d part_len=%d grid=%d smem=%zu | merge: cluster=%d cap=%d smem=%zu | "
            "model %.1f us\n",
            pl.hg, pl.nq, pl.nq_valid, pl.qsplit, pl.bshare, pl.cluster, pl.nsplit, pl.cap, pl.nstages, pl.groups,
            pl.rendezvous, pl.per,
            pl.part_len, pl.grid, pl.smem, pl.cluster2, pl.cap2, pl.smem2, pl.cost * 1e6);
  const int parts = s.segments * pl.nsplit;
  const bool two_stage = parts > 1 && !pl.parts_in_cluster;
  // the candidate lists of this plan must fit in what the caller gave
  if (p->workspace_bytes < kStatusBytes + (two_stage ? cand_bytes(s, parts) : 0)) {
    g_last_error = "workspace smaller than ra_workspace_bytes()";
    return RA_ERR_WORKSPACE;
  }
  float* ws_score = reinterpret_cast<float*>(static_cast<char*>(p->workspace) + kStatusBytes);
  int* ws_idx = reinterpret_cast<int*>(ws_score + (size_t)s.batch * s.hq * parts * s.topk);

  ScanParams sp;
  memset(&sp, 0, sizeof sp);
  // several queries per K row (GQA group, batch rows on one cache): score on the tensor cores
  const bool swizzled = pl.hg == 1 && pl.nq > 1 && !tuning_env("RA_NO_MMA");
  st = encode_kmap(&sp.kmap, p, s, pl.hg, swizzled, real_tokens);
  sp.swizzled = swizzled;
  if (st != RA_OK) return st;
  sp.q = static_cast<const __half*>(p->q);
  sp.status = status;
  sp.batch = s.batch; sp.hq = s.hq; sp.hkv = s.hkv; sp.n_tokens = real_tokens;
  sp.part_ids = ext ? ext->ids : nullptr;
  if (ext && ext->coarse_centers) {
    sp.coarse_centers = static_cast<const __half*>(ext->coarse_centers);
    sp.coarse_csz = ext->coarse_csz;
    sp.coarse_ids_out = ext->coarse_ids_out;
  }
  if (ext && ext->expand_out) {
    sp.m.expand_clen = ext->expand_clen; sp.m.expand_out = ext->expand_out;
    sp.m.expand_ids = ext->expand_ids;
  }
  sp.group = c.group; sp.bshare = pl.bshare; sp.nq_valid = pl.nq_valid;
  sp.qsplit = pl.qsplit; sp.nq_cta = pl.nq_cta;
  sp.kv_per_batch = s.per_batch;
  sp.cap = pl.cap; sp.nstages = pl.nstages; sp.groups = pl.groups; sp.rendezvous = pl.rendezvous; sp.nparts = parts; sp.part_len = pl.part_len;
  sp.head_major = s.head_major;
  sp.wait_limit_ns = kWaitLimitNs;
  if (const char* d = tuning_env("RA_DEBUG_FLAGS")) sp.debug = atoi(d);
  if (const char* d = tuning_env("RA_WAIT_LIMIT_MS")) sp.wait_limit_ns = 1000000ull * (unsigned long long)std::max(1, atoi(d));
  MergeArgs& m = sp.m;
  m.topk = s.topk; m.per = pl.per; m.cluster = pl.cluster; m.det_words = pl.det_words;
  m.per_cta_select = pl.parts_in_cluster ? 1 : 0;
  sp.parts_in_cluster = pl.parts_in_cluster ? 1 : 0;
  m.hq_total = s.hq; m.list_pitch = parts * s.topk; m.list_off = 0;
  m.index_base = two_stage ? 0 : p->index_base;
  m.own_lo = 0; m.own_hi = 0x7fffffff; m.id_shift = 0;
  m.n_tokens = real_tokens; m.status = status;
  m.v = static_cast<const __half*>(p->v);
  m.v_batch_stride = p->kv_batch_stride; m.v_token_stride = p->kv_token_stride;
  m.v_head_stride = p->kv_head_stride;
  m.out = static_cast<__half*>(p->out);
  m.out_lse = p->out_lse; m.out_partial = nullptr;
  m.scale_log2e = p->sm_scale * kLog2e; m.sm_scale = p->sm_scale;
  // Per-chunk selection (segments > 1): every chunk's winners are final, so the scan writes
  // them straight into the caller's lists when given and the second stage only mixes V.
  const bool lists_final = s.segments > 1;
  if (two_stage) {
    m.out_mode = kOutNone;
    m.sel_idx = (lists_final && p->out_indices) ? p->out_indices : ws_idx;
    m.sel_score = (lists_final && p->out_scores) ? p->out_scores : ws_score;
    if (lists_final) m.index_base = p->index_base;
  } else {
    m.out_mode = attend ? kOutFinal : kOutNone;
    m.sel_idx = p->out_indices; m.sel_score = p->out_scores;
  }
  cudaError_t e = launch_scan_select(sp, pl.hg, pl.nq, pl.grid, pl.smem, stream);
  if (e != cudaSuccess) return cuda_fail(e, "scan_select launch");
  if (!two_stage) return RA_OK;

  if (lists_final && !attend) return RA_OK;
  if (lists_final) {
    // every listed key takes part: one pass over the V rows of the lists with the scores the scan
    // wrote, a cluster of CTAs per row
    const long long per_row = (long long)s.segments * s.topk;
    const int st = run_gather(static_cast<const __half*>(p->q), nullptr,
                              static_cast<const __half*>(p->v), static_cast<__half*>(p->out),
                              p->out_lse, s.batch, s.hq, s.hkv, real_tokens, p->kv_batch_stride,
                              p->kv_token_stride, p->kv_head_stride, sp.m.sel_idx, sp.m.sel_score,
                              (long long)s.hq * per_row, per_row, (int)per_row, 0, nullptr,
                              p->sm_scale, status, true, stream, p->index_base);
    if (st != RA_ERR_UNSUPPORTED) return st;   // lists too long for that kernel: the merge below
  }
  MergeParams mp;
  memset(&mp, 0, sizeof mp);
  mp.m = sp.m;
  mp.m.topk = lists_final ? s.segments * s.topk : s.topk;
  mp.m.per = pl.per2; mp.m.cluster = pl.cluster2; mp.m.det_words = det_words_for(pl.cap2);
  mp.m.list_pitch = mp.m.topk; mp.m.list_off = 0;
  mp.m.out_mode = attend ? kOutFinal : kOutNone;
  if (lists_final) {
    // ids in the lists already carry index_base; nothing more to write
    mp.m.index_base = 0;
    mp.m.own_lo = p->index_base; mp.m.id_shift = p->index_base;
    mp.m.sel_idx = nullptr; mp.m.sel_score = nullptr;
  } else {
    mp.m.index_base = p->index_base;
    mp.m.sel_idx = p->out_indices; mp.m.sel_score = p->out_scores;
  }
  mp.cand_score = sp.m.sel_score; mp.cand_idx = sp.m.sel_idx;
  mp.part_len = s.topk; mp.part_stride = s.topk; mp.row_stride = (long long)parts * s.topk;
  mp.m_total = parts * s.topk; mp.cap = pl.cap2; mp.group = c.group; mp.own_part = -1;
  e = dispatch_merge(mp, s.batch * s.hq, pl, stream);
  if (e != cudaSuccess) return cuda_fail(e, "merge_attend launch");
  return RA_OK;
}

// Several queries per K row, one global selection: scan_store_kernel streams K once and stores every
// score, select_stored_kernel picks the exact top-k per (batch row, query head) from the stored
// scores and attends over the winners (or writes them out when attend is false).
int run_store(const ra_params* p, const Shape& s, int group, bool attend, unsigned* status,
              const ra_shard_exchange* sx, bool scan_only) {
  int bshare = 1;
  const int nq_valid = shared_queries(s, &bshare);
  const int rows = s.batch * s.hq;
  const int items = (s.batch / bshare) * s.hkv;   // (batch group, kv head) pairs, each a row of CTAs
  const int sms = sm_count();
  // parts of the token axis per item: the count with the lowest modelled stream time
  int nparts = 1, part_len = store_pitch(s.n);
  double best = 1e30;
  for (int ns = 1; ns <= kMaxSplit; ++ns) {
    const int len = ceil_div(ceil_div(s.n, ns), kTileRows) * kTileRows;
    if (ns > 1 && (long long)len * (ns - 1) >= s.n) continue;
    const int grid = items * ns, live = std::min(grid, sms), waves = ceil_div(grid, sms);
    const double rate = std::min(kModelSmBytesPerSec, kModelHbmBytesPerSec / live);
    const double cost = waves * ((double)ceil_div(len, kTileRows) * kStageBytes / rate + 4e-6);
    if (cost < best) {
      best = cost;
      nparts = ns;
      part_len = len;
    }
  }
  if (const char* f = tuning_env("RA_FORCE_STORE_PARTS")) {
    const int ns = atoi(f);
    const int len = ceil_div(ceil_div(s.n, std::max(ns, 1)), kTileRows) * kTileRows;
    if (ns >= 1 && ns <= kMaxSplit && (ns == 1 || (long long)len * (ns - 1) < s.n)) {
      nparts = ns;
      part_len = len;
    }
  }
  const size_t need = kStatusBytes + store_keys_bytes(s) + store_hist_bytes(s, nparts);
  if (p->workspace_bytes < need) {
    g_last_error = "workspace smaller than ra_workspace_bytes()";
    return RA_ERR_WORKSPACE;
  }
  char* ws = static_cast<char*>(p->workspace);
  uint32_t* keys_ws = reinterpret_cast<uint32_t*>(ws + kStatusBytes);
  uint32_t* hist_ws = reinterpret_cast<uint32_t*>(ws + kStatusBytes + store_keys_bytes(s));
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);

  StoreParams sp;
  memset(&sp, 0, sizeof sp);
  int st = encode_kmap(&sp.kmap, p, s, 1, true, s.n);
  if (st != RA_OK) return st;
  sp.q = static_cast<const __half*>(p->q);
  sp.status = status;
  sp.keys_ws = keys_ws; sp.hist_ws = hist_ws;
  sp.batch = s.batch; sp.hq = s.hq; sp.hkv = s.hkv; sp.n_tokens = s.n; sp.n_pad = store_pitch(s.n);
  sp.group = group; sp.bshare = bshare; sp.nq_valid = nq_valid; sp.kv_per_batch = s.per_batch;
  sp.nstages = nq_valid <= 4 ? 6 : 4;
  sp.groups = 2;
  sp.nparts = nparts; sp.part_len = part_len;

  // selection: a cluster of CTAs per row when there are few rows, each with a candidate list as
  // large as shared memory allows
  int c2 = 1;
  while (c2 < kSelMaxCluster && rows * c2 * 2 <= sms && ceil_div(s.n, c2 * 2) >= 4096) c2 <<= 1;
  int per2 = 0, cap2 = 0, det2 = 32, chunk2 = 0;
  size_t fixed = 0;
  for (;; c2 <<= 1) {
    per2 = ceil_div(s.topk, c2);
    chunk2 = ceil_div(ceil_div(s.n, c2), kTileRows) * kTileRows;
    det2 = det_words_for(chunk2);
    fixed = sx ? select_sharded_fixed_smem_bytes() : select_stored_fixed_smem_bytes(per2, det2);
    // (the sharded kernel also has a few bytes of static shared memory, which count against the limit)
    const size_t budget = kSmemBudget - (sx ? 1024 : 0);
    cap2 = fixed < budget ? (int)std::min<size_t>(16384, (budget - fixed) / 8) : 0;
    if (cap2 >= s.topk + 512 || c2 >= kSelMaxCluster) break;
  }
  if (cap2 < s.topk + 512) return unsupported("topk too large for the stored-score selection");
  // the selection CTAs of all ranks wait for one another row by row: all of them must be resident
  if (sx && rows * c2 > sms) return unsupported("too many (batch row, head) pairs for the histogram exchange");
  // (the ranks' partial rows are staged in the candidate list's shared memory)
  if (sx && cap2 < sx->world * kPartWords) return unsupported("candidate list too small for this many ranks");
  if (verbose_plan()) {
    static thread_local Shape last_shown = {};
    if ((last_shown < s) || (s < last_shown)) {
      last_shown = s;
      fprintf(stderr,
              "[topk_attn_b200] plan: score store nq=%d bshare=%d parts=%d part_len=%d grid=%d stages=%d | "
              "select: cluster=%d cap=%d per=%d | model %.1f us\n",
              nq_valid, bshare, nparts, part_len, items * nparts, sp.nstages, c2, cap2, per2, best * 1e6);
    }
  }
  cudaError_t e = launch_scan_store(sp, items * nparts, scan_store_smem_bytes(nq_valid, sp.nstages), stream);
  if (e != cudaSuccess) return cuda_fail(e, "scan_store launch");
  if (scan_only) return RA_OK;

  SelectStoredParams qp;
  memset(&qp, 0, sizeof qp);
  MergeArgs& m = qp.m;
  m.topk = s.topk; m.per = per2; m.cluster = c2; m.det_words = det2;
  m.out_mode = attend ? kOutFinal : kOutNone;
  m.hq_total = s.hq; m.list_pitch = s.topk; m.list_off = 0; m.index_base = p->index_base;
  m.own_lo = 0; m.own_hi = 0x7fffffff; m.id_shift = 0;
  m.n_tokens = s.n; m.status = status;
  m.sel_idx = p->out_indices; m.sel_score = p->out_scores;
  m.v = static_cast<const __half*>(p->v);
  m.v_batch_stride = p->kv_batch_stride; m.v_token_stride = p->kv_token_stride;
  m.v_head_stride = p->kv_head_stride;
  m.out = static_cast<__half*>(p->out); m.out_lse = p->out_lse; m.out_partial = nullptr;
  m.scale_log2e = p->sm_scale * kLog2e; m.sm_scale = p->sm_scale;
  qp.keys_ws = keys_ws; qp.hist_ws = hist_ws;
  qp.n_tokens = s.n; qp.n_pad = sp.n_pad; qp.nparts = nparts;
  qp.chunk = chunk2;
  qp.cap = cap2; qp.group = group;
  if (sx) {
    SelectShardedParams hp;
    memset(&hp, 0, sizeof hp);
    hp.s = qp;
    hp.x.world = sx->world; hp.x.rank = sx->rank;
    hp.x.epoch = static_cast<const unsigned*>(sx->epoch);
    hp.x.epoch_rw = static_cast<unsigned*>(sx->epoch);
    hp.x.done = static_cast<unsigned*>(sx->done_counter);
    hp.x.limit_ns = sx->wait_timeout_ns;
    for (int r = 0; r < sx->world; ++r) hp.x.buf_peer[r] = static_cast<unsigned long long*>(sx->bufs[r]);
    e = launch_select_sharded(hp, rows, fixed + (size_t)cap2 * 8, stream);
    if (e != cudaSuccess) return cuda_fail(e, "select_sharded launch");
    return RA_OK;
  }
  e = launch_select_stored(qp, rows, fixed + (size_t)cap2 * 8, stream);
  if (e != cudaSuccess) return cuda_fail(e, "select_stored launch");
  return RA_OK;
}

}  // namespace

extern "C" {

const char* ra_strerror(int status) {
  switch (status) {
    case RA_OK: return "ok";
    case RA_ERR_INVALID_ARGUMENT: return "invalid argument";
    case RA_ERR_UNSUPPORTED: return "unsupported configuration";
    case RA_ERR_WORKSPACE: return "workspace missing or too small";
    case RA_ERR_CUDA: return "CUDA call failed";
    case RA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case RA_ERR_NOT_BUILT: return "not built";
    case RA_ERR_DEVICE_CHECK: return "a device-side self-check failed";
    default: return "unknown status";
  }
}

int ra_version(void) { return 100; }

const char* ra_last_cuda_error(void) { return g_last_error.c_str(); }

unsigned long long ra_launch_count(void) { return ra::g_launch_count.load(std::memory_order_relaxed); }

size_t ra_workspace_bytes(const ra_params* p) {
  Checked c;
  if (check_shape(p, c) != RA_OK) return 0;
  return workspace_bound(c.shape);
}

int ra_topk_attention(const ra_params* p) { return run(p, true); }

int ra_gemv_topk(const ra_params* p) { return run(p, false); }

// ---- fused decode step for callers that cannot hand over a workspace ------------------------
// Scratch of this entry point: a fixed array inside the library image.  The name below is only a
// host-side handle; the address kernels may use comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_static_scratch[RA_NOALLOC_SCRATCH_BYTES];

int ra_topk_attention_noalloc(const ra_params* p) {
  if (!p) return invalid("params is null");
  Checked c;
  int st = check_shape(p, c);
  if (st != RA_OK) return st;
  if (workspace_bound(c.shape) > (size_t)RA_NOALLOC_SCRATCH_BYTES) {
    g_last_error = "this shape needs more scratch than the built-in RA_NOALLOC_SCRATCH_BYTES; "
                   "use ra_topk_attention with a workspace";
    return RA_ERR_UNSUPPORTED;
  }
  // set-up, once per device, with that device current
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* scratch_of[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return unsupported("device ordinal above 63");
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> g(mu);
    if (!scratch_of[dev]) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_static_scratch);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
      scratch_of[dev] = ptr;
    }
    scratch = scratch_of[dev];
  }
  // the array keeps the previous call's contents: the status block must start at zero
  e = cudaMemsetAsync(scratch, 0, kStatusBytes, static_cast<cudaStream_t>(p->stream));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(static scratch)");
  ra_params q = *p;
  q.workspace = scratch;
  q.workspace_bytes = RA_NOALLOC_SCRATCH_BYTES;
  return run(&q, true);
}

int ra_check_status(void* workspace, void* stream) {
  if (!workspace) return RA_ERR_WORKSPACE;
  unsigned h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, workspace, sizeof h, cudaMemcpyDeviceToHost,
                                  static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "ra_check_status");
  if (h & ra::kStatusTimeout) return RA_ERR_DEVICE_TIMEOUT;
  if (h & (ra::kStatusBadId | ra::kStatusOverflow)) {
    g_last_error = (h & ra::kStatusBadId) ? "a kernel skipped a key id outside the value cache"
                                          : "a candidate list overflowed";
    return RA_ERR_DEVICE_CHECK;
  }
  return RA_OK;
}

// Launch geometry of the gathered-attention kernel for n_entries ids per row.
static bool plan_gather(int n_entries, int n_src, int rows, int& cluster, int& cap, int& per,
                        size_t& smem) {
  // enough CTAs to fill the machine, not more than 16 rows of K per thread and CTA
  int want = 1;
  while (want < 8 && (rows * want < sm_count() || ceil_div(n_entries, want) > 4096)) want <<= 1;
  for (int c = want; c <= 8; c <<= 1) {
    cap = ceil_div(n_entries, c);
    per = ceil_div(n_entries, c);
    smem = gather_attend_smem_bytes(per, cap, n_src);
    if (smem <= kSmemBudget) {
      cluster = c;
      return true;
    }
  }
  return false;
}

static int run_gather(const __half* q, const __half* k, const __half* v, __half* out, float* out_lse,
                      int batch, int hq, int hkv, int n_tokens, long long bs, long long ts,
                      long long hs, const int* src_idx, const float* src_score,
                      long long src_bstride, long long src_hstride, int n_src, int expand_clen,
                      int* out_token_ids, float sm_scale, unsigned* status, bool attend,
                      cudaStream_t stream, int id_shift) {
  const long long n_entries_ll = (long long)n_src * (expand_clen > 0 ? expand_clen : 1);
  if (n_entries_ll > (1 << 20)) return unsupported("more than 2^20 ids per head");
  const int n_entries = (int)n_entries_ll;
  int cluster = 1, cap = 0, per = 0;
  size_t smem = 0;
  if (!plan_gather(n_entries, n_src, batch * hq, cluster, cap, per, smem))
    return unsupported("id list too long for the gathered-attention kernel");
  GatherParams gp;
  memset(&gp, 0, sizeof gp);
  MergeArgs& m = gp.m;
  m.topk = n_entries; m.per = per; m.cluster = cluster; m.select_all = 1; m.local_deal = 1;
  m.out_mode = attend ? kOutFinal : kOutNone;
  m.hq_total = hq; m.list_pitch = n_entries; m.list_off = 0; m.index_base = 0;
  m.own_lo = 0; m.own_hi = 0x7fffffff; m.id_shift = id_shift; m.n_tokens = n_tokens; m.status = status;
  m.sel_idx = nullptr; m.sel_score = nullptr;
  m.v = v; m.v_batch_stride = bs; m.v_token_stride = ts; m.v_head_stride = hs;
  m.out = out; m.out_lse = out_lse; m.out_partial = nullptr;
  m.scale_log2e = sm_scale * kLog2e; m.sm_scale = sm_scale;
  gp.q = q; gp.k = k; gp.src_idx = src_idx; gp.src_score = src_score;
  gp.src_batch_stride = src_bstride; gp.src_head_stride = src_hstride;
  gp.n_src = n_src; gp.expand_clen = expand_clen; gp.n_entries = n_entries;
  gp.out_token_ids = out_token_ids; gp.cap = cap; gp.group = hq / hkv;
  // attention: one pass over K and V with an online softmax; expansion only: the id writer
  cudaError_t e = attend ? launch_gather_flash(gp, batch * hq, gather_flash_smem_bytes(n_src), stream)
                         : launch_gather_attend(gp, batch * hq, smem, stream);
  if (e != cudaSuccess) return cuda_fail(e, "gather_attend launch");
  return RA_OK;
}

int ra_gathered_attention(const ra_gather_params* p) {
  if (!p) return invalid("params is null");
  if (!p->q || !p->k || !p->v || !p->out || !p->indices) return invalid("a required pointer is null");
  if (p->head_dim != kHeadDim) return unsupported("head_dim must be 128");
  if (p->batch < 1 || p->num_q_heads < 1 || p->num_kv_heads < 1 || p->num_tokens < 1 ||
      p->num_indices < 1)
    return invalid("sizes must be positive");
  if (p->num_q_heads % p->num_kv_heads) return invalid("num_kv_heads must divide num_q_heads");
  if (!(p->sm_scale > 0.f)) return invalid("sm_scale must be positive");
  if (p->kv_token_stride % 8 || p->kv_head_stride % 8 || p->kv_batch_stride % 8)
    return invalid("kv strides must be multiples of 8 elements");
  if (!p->workspace || p->workspace_bytes < kStatusBytes) {
    g_last_error = "workspace missing or too small";
    return RA_ERR_WORKSPACE;
  }
  return run_gather(static_cast<const __half*>(p->q), static_cast<const __half*>(p->k),
                    static_cast<const __half*>(p->v), static_cast<__half*>(p->out), p->out_lse,
                    p->batch, p->num_q_heads, p->num_kv_heads, p->num_tokens, p->kv_batch_stride,
                    p->kv_token_stride, p->kv_head_stride, p->indices, nullptr,
                    p->indices_batch_stride, p->num_indices, p->num_indices, 0, nullptr,
                    p->sm_scale, static_cast<unsigned*>(p->workspace), true,
                    static_cast<cudaStream_t>(p->stream));
}

size_t ra_center_workspace_bytes(int32_t batch, int32_t num_heads, int32_t num_centers,
                                 int32_t top_clusters) {
  if (batch < 1 || num_heads < 1 || num_centers < 1 || top_clusters < 1) return 0;
  Shape s;
  s.batch = batch; s.hq = num_heads; s.hkv = num_heads; s.n = num_centers; s.topk = top_clusters;
  s.segments = 1; s.per_batch = 0; s.head_major = 1; s.fused_ok = 1;
  // selection scratch, then the kept cluster ids and their scores
  return workspace_bound(s) + (size_t)batch * num_heads * top_clusters * 8 + 256;
}

// Centroid tables whose per-head scores fit in shared memory: scores, exact top-C in rank order
// and (optionally) the member ids of the winners in one launch.
static int center_select(const void* q, const void* centers, int batch, int heads, int csz, int topc,
                         int clen, int* ids, float* scores, int* members, cudaStream_t stream) {
  CenterSelectParams cp;
  memset(&cp, 0, sizeof cp);
  cp.q = static_cast<const __half*>(q);
  cp.centers = static_cast<const __half*>(centers);
  cp.heads = heads; cp.csz = csz; cp.topc = topc; cp.clen = clen;
  int cluster = 1;
  while (cluster < kCenterMaxCluster && csz > 256 * cluster) cluster <<= 1;
  if (const char* f = tuning_env("RA_CENTER_CLUSTER")) {
    const int c = atoi(f);
    if (c == 1 || c == 2 || c == 4 || c == 8) cluster = c;
  }
  cp.cluster = cluster;
  cp.per = (ceil_div(csz, cluster) + 3) & ~3;
  cp.out_cluster_ids = ids; cp.out_scores = scores; cp.out_members = members;
  cp.vec_members = members && clen % 4 == 0 && (reinterpret_cast<uintptr_t>(members) & 15u) == 0;
  cudaError_t e = launch_center_select(cp, batch * heads, stream);
  if (e != cudaSuccess) return cuda_fail(e, "center_select launch");
  return RA_OK;
}

int ra_center_only_topk(const ra_center_params* p) {
  if (!p) return invalid("params is null");
  if (!p->q || !p->centers) return invalid("q or centers is null");
  if (p->head_dim != kHeadDim) return unsupported("head_dim must be 128");
  if (p->batch < 1 || p->num_heads < 1 || p->num_centers < 1 || p->cluster_len < 1 ||
      p->top_clusters < 1 || p->top_clusters > p->num_centers)
    return invalid("sizes must be positive and top_clusters <= num_centers");
  const bool attend = p->out != nullptr;
  if (attend && (!p->k || !p->v)) return invalid("k and v are required with out");
  if (!attend && !p->out_indices && !p->out_cluster_ids) return invalid("nothing to compute");
  const size_t need = ra_center_workspace_bytes(p->batch, p->num_heads, p->num_centers, p->top_clusters);
  if (!p->workspace || p->workspace_bytes < need) {
    g_last_error = "workspace smaller than ra_center_workspace_bytes()";
    return RA_ERR_WORKSPACE;
  }
  const long long n_members = (long long)p->top_clusters * p->cluster_len;
  if (attend && (long long)p->num_centers * p->cluster_len > p->num_tokens)
    return invalid("num_centers * cluster_len exceeds num_tokens");
  // 1) exact top-TOPC of the centroid scores (the scan kernel over the head-major table)
  const size_t rows = (size_t)p->batch * p->num_heads;
  char* ws = static_cast<char*>(p->workspace);
  const size_t tail = (need - rows * p->top_clusters * 8 - 256 + 255) & ~size_t(255);
  float* c_score = reinterpret_cast<float*>(ws + tail);
  int* c_ids = reinterpret_cast<int*>(c_score + rows * p->top_clusters);
  ra_params sp;
  memset(&sp, 0, sizeof sp);
  sp.q = p->q; sp.k = p->centers;
  sp.batch = p->batch; sp.num_q_heads = p->num_heads; sp.num_kv_heads = p->num_heads;
  sp.head_dim = kHeadDim; sp.num_tokens = p->num_centers;
  sp.kv_batch_stride = 0; sp.kv_token_stride = kHeadDim;
  sp.kv_head_stride = (int64_t)p->num_centers * kHeadDim;
  sp.topk = p->top_clusters; sp.num_segments = 1; sp.sm_scale = 1.f;
  sp.workspace = p->workspace; sp.workspace_bytes = tail; sp.stream = p->stream;
  if (p->num_centers <= kCenterMaxCsz && !tuning_env("RA_NO_CENTER_SELECT")) {
    if (attend && n_members <= (1 << 20) && !tuning_env("RA_NO_CENTER_ATTEND")) {
      // selection, expansion and attention in one launch; ids only leave the kernel when asked for
      CenterSelectParams cp;
      memset(&cp, 0, sizeof cp);
      cp.q = static_cast<const __half*>(p->q);
      cp.centers = static_cast<const __half*>(p->centers);
      cp.heads = p->num_heads; cp.csz = p->num_centers; cp.topc = p->top_clusters; cp.clen = p->cluster_len;
      // as many CTAs per row as fit on the machine at once (one CTA of this kernel per
      // multiprocessor): a second wave would double the time of a step this short
      int cluster = 1;
      while (cluster < kCenterMaxCluster && (long long)rows * cluster * 2 <= sm_count()) cluster <<= 1;
      cp.cluster = cluster;
      cp.per = (ceil_div(p->num_centers, cluster) + 3) & ~3;
      cp.out_cluster_ids = p->out_cluster_ids; cp.out_scores = nullptr; cp.out_members = p->out_indices;
      cp.k = static_cast<const __half*>(p->k); cp.v = static_cast<const __half*>(p->v);
      cp.out = static_cast<__half*>(p->out);
      cp.batch_stride = p->kv_batch_stride; cp.token_stride = p->kv_token_stride;
      cp.head_stride = p->kv_head_stride; cp.n_tokens = p->num_tokens;
      cp.scale_log2e = (p->sm_scale > 0.f ? p->sm_scale : 1.f) * kLog2e;
      cp.status = static_cast<unsigned*>(p->workspace);
      cudaError_t e = launch_center_attend(cp, (int)rows, static_cast<cudaStream_t>(p->stream));
      if (e != cudaSuccess) return cuda_fail(e, "center_attend launch");
      return RA_OK;
    }
    int* ids = p->out_cluster_ids ? p->out_cluster_ids : c_ids;
    int st = center_select(p->q, p->centers, p->batch, p->num_heads, p->num_centers, p->top_clusters,
                           p->cluster_len, ids, c_score, attend ? nullptr : p->out_indices,
                           static_cast<cudaStream_t>(p->stream));
    if (st != RA_OK || !attend) return st;
    return run_gather(static_cast<const __half*>(p->q), static_cast<const __half*>(p->k),
                      static_cast<const __half*>(p->v), static_cast<__half*>(p->out), nullptr,
                      p->batch, p->num_heads, p->num_heads, p->num_tokens, p->kv_batch_stride,
                      p->kv_token_stride, p->kv_head_stride, ids, /*already in rank order*/ nullptr,
                      (long long)p->num_heads * p->top_clusters, p->top_clusters, p->top_clusters,
                      p->cluster_len, p->out_indices, p->sm_scale > 0.f ? p->sm_scale : 1.f,
                      static_cast<unsigned*>(p->workspace), true,
                      static_cast<cudaStream_t>(p->stream));
  }
  if (!attend && p->out_indices) {
    // selection + expansion in one launch: the scan kernel ranks its winners and writes the
    // member tokens (and the cluster ids) in rank order
    PartIds ext;
    ext.ids = nullptr; ext.real_tokens = 0;
    ext.expand_clen = p->cluster_len; ext.expand_out = p->out_indices;
    ext.expand_ids = p->out_cluster_ids;
    return run(&sp, false, &ext);
  }
  sp.out_indices = p->out_cluster_ids ? p->out_cluster_ids : c_ids;
  sp.out_scores = c_score;
  int st = ra_gemv_topk(&sp);
  if (st != RA_OK) return st;
  if (!attend && !p->out_indices) return RA_OK;
  // 2) expansion in rank order (+ attention over every member token)
  const long long ts = attend ? p->kv_token_stride : kHeadDim;
  return run_gather(static_cast<const __half*>(p->q),
                    static_cast<const __half*>(attend ? p->k : p->centers),
                    static_cast<const __half*>(attend ? p->v : p->centers),
                    static_cast<__half*>(p->out), nullptr, p->batch, p->num_heads, p->num_heads,
                    attend ? p->num_tokens : 0x7fffffff, attend ? p->kv_batch_stride : 0, ts,
                    attend ? p->kv_head_stride : 0, sp.out_indices, c_score,
                    (long long)p->num_heads * p->top_clusters, p->top_clusters, p->top_clusters,
                    p->cluster_len, p->out_indices, p->sm_scale > 0.f ? p->sm_scale : 1.f,
                    static_cast<unsigned*>(p->workspace), attend,
                    static_cast<cudaStream_t>(p->stream));
  (void)n_members;
}

size_t ra_two_level_workspace_bytes(int32_t batch, int32_t num_heads, int32_t num_centers,
                                    int32_t top_clusters, int32_t topk_per_cluster) {
  if (batch < 1 || num_heads < 1 || num_centers < 1 || top_clusters < 1 || topk_per_cluster < 1)
    return 0;
  const size_t rows = (size_t)batch * num_heads;
  // [centroid selection scratch][fine selection scratch][cluster ids + scores, twice]
  const size_t coarse = ra_center_workspace_bytes(batch, num_heads, num_centers, top_clusters);
  // a single cluster may be scanned in up to kMaxSplit parts
  const size_t fine = kStatusBytes + rows * top_clusters * topk_per_cluster * 8 * (top_clusters == 1 ? kMaxSplit : 1) + 256;
  return coarse + fine + rows * top_clusters * 16 + 512;
}

int ra_two_level_topk(const ra_two_level_params* p) {
  if (!p) return invalid("params is null");
  if (!p->q || !p->centers || !p->k) return invalid("q, centers or k is null");
  if (p->head_dim != kHeadDim) return unsupported("head_dim must be 128");
  if (p->batch < 1 || p->num_heads < 1 || p->num_centers < 1 || p->cluster_len < 1 ||
      p->top_clusters < 1 || p->top_clusters > p->num_centers || p->topk_per_cluster < 1 ||
      p->topk_per_cluster > p->cluster_len || p->top_clusters > 1024)
    return invalid("bad two-level sizes");
  if ((long long)p->num_centers * p->cluster_len > p->num_tokens)
    return invalid("num_centers * cluster_len exceeds num_tokens");
  const bool attend = p->out != nullptr;
  if (attend && !p->v) return invalid("v is required with out");
  if (!attend && !p->out_indices) return invalid("nothing to compute");
  const size_t need = ra_two_level_workspace_bytes(p->batch, p->num_heads, p->num_centers,
                                                   p->top_clusters, p->topk_per_cluster);
  if (!p->workspace || p->workspace_bytes < need || (reinterpret_cast<uintptr_t>(p->workspace) & 255u)) {
    g_last_error = "workspace missing, misaligned or smaller than ra_two_level_workspace_bytes()";
    return RA_ERR_WORKSPACE;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  const size_t rows = (size_t)p->batch * p->num_heads;
  char* ws = static_cast<char*>(p->workspace);
  const size_t coarse = (ra_center_workspace_bytes(p->batch, p->num_heads, p->num_centers,
                                                   p->top_clusters) + 255) & ~size_t(255);
  const size_t fine = (kStatusBytes + rows * p->top_clusters * p->topk_per_cluster * 8 * (p->top_clusters == 1 ? kMaxSplit : 1) + 511) & ~size_t(255);
  float* c_score = reinterpret_cast<float*>(ws + coarse + fine);
  int* c_ids = reinterpret_cast<int*>(c_score + rows * p->top_clusters);
  int* c_sorted = c_ids + rows * p->top_clusters;
  // 1) top clusters by centroid score
  ra_params sp;
  memset(&sp, 0, sizeof sp);
  sp.q = p->q; sp.k = p->centers;
  sp.batch = p->batch; sp.num_q_heads = p->num_heads; sp.num_kv_heads = p->num_heads;
  sp.head_dim = kHeadDim; sp.num_tokens = p->num_centers;
  sp.kv_token_stride = kHeadDim; sp.kv_head_stride = (int64_t)p->num_centers * kHeadDim;
  sp.topk = p->top_clusters; sp.num_segments = 1; sp.sm_scale = 1.f;
  sp.out_indices = c_ids; sp.out_scores = c_score;
  sp.workspace = ws; sp.workspace_bytes = coarse; sp.stream = p->stream;
  int* sorted = p->out_cluster_ids ? p->out_cluster_ids : c_sorted;
  // a small table is ranked by the scan kernel's own prologue: no launch for the coarse stage
  const bool coarse_in_scan = p->num_centers <= kMaxCoarse && !tuning_env("RA_NO_COARSE_PROLOGUE");
  if (coarse_in_scan) {
  } else if (p->num_centers <= kCenterMaxCsz && !tuning_env("RA_NO_CENTER_SELECT")) {
    // steps 1 and 2 in one launch
    int st = center_select(p->q, p->centers, p->batch, p->num_heads, p->num_centers, p->top_clusters,
                           p->cluster_len, sorted, nullptr, nullptr, stream);
    if (st != RA_OK) return st;
  } else {
    int st = run(&sp, false);
    if (st != RA_OK) return st;
    // 2) rank order
    cudaError_t e = launch_rank_sort(c_score, c_ids, (int)rows, p->top_clusters, sorted, nullptr, stream);
    if (e != cudaSuccess) return cuda_fail(e, "rank_sort launch");
  }
  // 3) per-cluster top-k over the chosen clusters (+ attention over all kept keys)
  ra_params fp;
  memset(&fp, 0, sizeof fp);
  fp.q = p->q; fp.k = p->k; fp.v = p->v; fp.out = p->out;
  fp.batch = p->batch; fp.num_q_heads = p->num_heads; fp.num_kv_heads = p->num_heads;
  fp.head_dim = kHeadDim;
  fp.num_tokens = p->top_clusters * p->cluster_len;  // the tokens actually scanned per head
  fp.kv_batch_stride = p->kv_batch_stride; fp.kv_token_stride = p->kv_token_stride;
  fp.kv_head_stride = p->kv_head_stride;
  fp.topk = p->topk_per_cluster; fp.num_segments = p->top_clusters;
  fp.sm_scale = p->sm_scale > 0.f ? p->sm_scale : 1.f;
  fp.out_indices = p->out_indices; fp.out_scores = p->out_scores;
  fp.workspace = ws + coarse; fp.workspace_bytes = fine; fp.stream = p->stream;
  PartIds ext;
  ext.ids = coarse_in_scan ? nullptr : sorted;
  ext.real_tokens = p->num_tokens;
  ext.status = static_cast<unsigned*>(p->workspace);   // one status block for every stage
  if (coarse_in_scan) {
    ext.coarse_centers = p->centers;
    ext.coarse_csz = p->num_centers;
    ext.coarse_ids_out = p->out_cluster_ids;
  }
  return run(&fp, attend, &ext);
}

int ra_kv_append(void* k_cache, void* v_cache, const void* new_k, const void* new_v, int32_t caches,
                 int32_t num_kv_heads, int32_t head_dim, int32_t position, int32_t capacity_tokens,
                 int64_t kv_batch_stride, int64_t kv_token_stride, int64_t kv_head_stride,
                 void* centers, int32_t num_centers, int32_t cluster_len, void* stream) {
  if (!k_cache || !v_cache || !new_k || !new_v) return invalid("a required pointer is null");
  if (head_dim != kHeadDim) return unsupported("head_dim must be 128");
  if (caches < 1 || num_kv_heads < 1 || caches > 65535) return invalid("bad cache or head count");
  if (position < 0 || position >= capacity_tokens) return invalid("position outside the cache");
  if (caches > 1 && kv_batch_stride <= 0) return invalid("several caches need kv_batch_stride");
  if (centers && (num_centers < 1 || cluster_len < 1)) return invalid("bad centroid geometry");
  if (centers && caches > 1) return unsupported("centroid maintenance needs one shared cache");
  cudaError_t e = launch_kv_append(static_cast<__half*>(k_cache), static_cast<__half*>(v_cache),
                                   static_cast<const __half*>(new_k), static_cast<const __half*>(new_v),
                                   static_cast<__half*>(centers), caches, num_kv_heads, position,
                                   caches > 1 ? kv_batch_stride : 0, kv_token_stride, kv_head_stride,
                                   num_centers, cluster_len, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "kv_append launch");
  return RA_OK;
}

// Effective split geometry: split_len is a multiple of the 128-token tile.  With asked == 0 the
// library picks about four work items per multiprocessor, never less than two tiles per item.
static void flash_geometry(int batch, int hkv, int n, int asked, int sms, int& splits, int& split_len) {
  int want = asked;
  if (want <= 0) {
    want = std::max(1, ceil_div(4 * sms, batch * hkv));
    want = std::min(want, std::max(1, n / (2 * kFdTile)));
  }
  want = std::max(1, std::min(want, ceil_div(n, kFdTile)));
  split_len = ceil_div(ceil_div(n, want), kFdTile) * kFdTile;
  splits = ceil_div(n, split_len);
}

size_t ra_flash_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                int32_t num_tokens, int32_t num_splits) {
  if (batch < 1 || num_q_heads < 1 || num_kv_heads < 1 || num_tokens < 1) return 0;
  int splits, split_len;
  // device-independent: when the library chooses the splits, room for the count it would pick on a
  // device with 256 multiprocessors (the count never exceeds the `want` it starts from)
  constexpr int kMaxSms = 256;
  flash_geometry(batch, num_kv_heads, num_tokens, num_splits, kMaxSms, splits, split_len);
  if (num_splits <= 0) {
    int want = std::max(1, ceil_div(4 * kMaxSms, batch * num_kv_heads));
    want = std::min(want, std::max(1, num_tokens / (2 * kFdTile)));
    splits = std::max(splits, std::min(want, ceil_div(num_tokens, kFdTile)));
  }
  return kStatusBytes + (size_t)splits * batch * num_q_heads * (kHeadDim + 2) * sizeof(float);
}

int ra_flash_decoding(const ra_dense_params* p) {
  if (!p) return invalid("params is null");
  if (!p->q || !p->k || !p->v || !p->out) return invalid("a required pointer is null");
  if (p->head_dim != kHeadDim) return unsupported("head_dim must be 128");
  if (p->batch < 1 || p->num_q_heads < 1 || p->num_kv_heads < 1 || p->num_tokens < 1)
    return invalid("sizes must be positive");
  if (p->num_q_heads % p->num_kv_heads) return invalid("num_kv_heads must divide num_q_heads");
  const int group = p->num_q_heads / p->num_kv_heads;
  if (group > kFdMaxGroup) return unsupported("more than 8 query heads per kv head");
  if (!(p->sm_scale > 0.f)) return invalid("sm_scale must be positive");
  if (p->kv_token_stride < kHeadDim || p->kv_head_stride < kHeadDim || p->kv_token_stride % 8 ||
      p->kv_head_stride % 8 || p->kv_batch_stride % 8 || p->kv_batch_stride < 0 ||
      p->kv_head_stride > p->kv_token_stride)
    return invalid("kv strides must be token-major multiples of 8 elements");
  auto mis = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) != 0; };
  if (mis(p->q) || mis(p->k) || mis(p->v) || mis(p->out)) return invalid("pointers must be 16-byte aligned");
  const size_t need = ra_flash_workspace_bytes(p->batch, p->num_q_heads, p->num_kv_heads,
                                               p->num_tokens, p->num_splits);
  if (!p->workspace || p->workspace_bytes < need || (reinterpret_cast<uintptr_t>(p->workspace) & 255u)) {
    g_last_error = "workspace missing, misaligned or smaller than ra_flash_workspace_bytes()";
    return RA_ERR_WORKSPACE;
  }
  EncodeTiledFn enc = encode_fn();
  if (!enc) {
    g_last_error = "cuTensorMapEncodeTiled is not available from the driver";
    return RA_ERR_CUDA;
  }
  FlashParams fp;
  memset(&fp, 0, sizeof fp);
  const bool per_batch = p->kv_batch_stride != 0;
  const cuuint64_t nb = per_batch ? (cuuint64_t)p->batch : 1;
  cuuint64_t dims[4] = {kHeadDim, (cuuint64_t)p->num_kv_heads, (cuuint64_t)p->num_tokens, nb};
  cuuint64_t strides[3] = {(cuuint64_t)p->kv_head_stride * 2, (cuuint64_t)p->kv_token_stride * 2,
                           per_batch ? (cuuint64_t)p->kv_batch_stride * 2
                                     : (cuuint64_t)p->num_tokens * p->kv_token_stride * 2};
  cuuint32_t box[4] = {64, 1, kFdTile, 1}, estr[4] = {1, 1, 1, 1};
  for (int which = 0; which < 2; ++which) {
    CUresult r = enc(which ? &fp.vmap : &fp.kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                     const_cast<void*>(which ? p->v : p->k), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      char buf[96];
      snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
      g_last_error = buf;
      return RA_ERR_CUDA;
    }
  }
  int splits, split_len;
  flash_geometry(p->batch, p->num_kv_heads, p->num_tokens, p->num_splits, sm_count(), splits, split_len);
  fp.q = static_cast<const __half*>(p->q);
  fp.partials = reinterpret_cast<float*>(static_cast<char*>(p->workspace) + kStatusBytes);
  fp.status = static_cast<unsigned*>(p->workspace);
  fp.batch = p->batch; fp.hq = p->num_q_heads; fp.hkv = p->num_kv_heads; fp.n_tokens = p->num_tokens;
  fp.group = group; fp.kv_per_batch = per_batch;
  fp.num_splits = splits; fp.split_len = split_len;
  fp.nstages = kFdMaxStages;
  fp.num_items = p->batch * p->num_kv_heads * splits;
  fp.scale_log2e = p->sm_scale * kLog2e;
  const int sms = sm_count();
  const int grid = std::min(fp.num_items, sms);
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  cudaError_t e = launch_flash_decode(fp, grid, flash_decode_smem_bytes(fp.nstages), stream);
  if (e != cudaSuccess) return cuda_fail(e, "flash_decode launch");
  e = launch_lse_combine(fp.partials, splits, p->batch * p->num_q_heads, static_cast<__half*>(p->out),
                         stream);
  if (e != cudaSuccess) return cuda_fail(e, "lse_combine launch");
  return RA_OK;
}

int ra_merge_attend(const ra_merge_params* p) {
  if (!p) return invalid("params is null");
  if (!p->cand_scores || !p->cand_indices) return invalid("candidate buffers are null");
  if (p->head_dim != kHeadDim) return unsupported("head_dim must be 128");
  if (p->batch < 1 || p->num_q_heads < 1 || p->num_kv_heads < 1 || p->num_parts < 1 ||
      p->topk < 1 || p->num_tokens < 0)
    return invalid("sizes must be positive");
  if (p->num_q_heads % p->num_kv_heads) return invalid("num_kv_heads must divide num_q_heads");
  if (p->cand_part_stride < 0) return invalid("cand_part_stride must not be negative");
  const bool attend = p->out || p->out_partial;
  if (attend && !p->v) return invalid("v is null");
  if (!attend && !p->out_indices) return invalid("nothing to compute");
  if (!(p->sm_scale > 0.f)) return invalid("sm_scale must be positive");
  if (!p->workspace || p->workspace_bytes < kStatusBytes) {
    g_last_error = "workspace missing or too small";
    return RA_ERR_WORKSPACE;
  }
  Plan pl;
  const long long m_total = (long long)p->num_parts * p->topk;
  if (m_total > (1 << 20) || !plan_merge((int)m_total, p->topk, pl))
    return unsupported("too many candidates for the merge kernel");
  MergeParams mp;
  memset(&mp, 0, sizeof mp);
  MergeArgs& m = mp.m;
  m.topk = p->topk; m.per = pl.per2; m.cluster = pl.cluster2; m.det_words = det_words_for(pl.cap2);
  m.out_mode = p->out_partial ? kOutPartial : (p->out ? kOutFinal : kOutNone);
  m.hq_total = p->num_q_heads; m.list_pitch = p->topk; m.list_off = 0; m.index_base = 0;
  m.own_lo = p->own_base; m.own_hi = p->own_base + p->num_tokens; m.id_shift = p->own_base;
  m.n_tokens = p->num_tokens; m.status = static_cast<unsigned*>(p->workspace);
  m.sel_idx = p->out_indices; m.sel_score = p->out_scores;
  m.v = static_cast<const __half*>(p->v);
  m.v_batch_stride = p->kv_batch_stride; m.v_token_stride = p->kv_token_stride;
  m.v_head_stride = p->kv_head_stride;
  m.out = static_cast<__half*>(p->out); m.out_lse = nullptr; m.out_partial = p->out_partial;
  m.scale_log2e = p->sm_scale * kLog2e; m.sm_scale = p->sm_scale;
  mp.cand_score = p->cand_scores; mp.cand_idx = p->cand_indices;
  mp.part_len = p->topk;
  mp.part_stride = p->cand_part_stride ? p->cand_part_stride
                                       : (long long)p->batch * p->num_q_heads * p->topk;
  mp.row_stride = p->topk;
  mp.m_total = (int)m_total; mp.cap = pl.cap2; mp.group = p->num_q_heads / p->num_kv_heads;
  mp.own_part = -1;
  if (p->own_part_only) {
    if (p->own_part < 0 || p->own_part >= p->num_parts) return invalid("own_part must name one of the parts");
    mp.own_part = p->own_part;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  const int rows = p->batch * p->num_q_heads;
  const ra_exchange_hooks* xh = p->exchange;
  if (xh) {
    if (!p->out_partial) return invalid("exchange hooks need out_partial");
    if (!xh->epoch) return invalid("exchange hooks need the epoch word");
    if (xh->wait_flags && (xh->num_wait_flags < 1 || xh->num_wait_flags > kMaxPeers || xh->wait_timeout_ns == 0))
      return invalid("bad wait flags in the exchange hooks");
    if (xh->peer_partials && (!xh->peer_flags || !xh->done_counter || xh->num_peers < 1 || xh->num_peers > kMaxPeers))
      return invalid("bad peer slots in the exchange hooks");
  }
  size_t one = 0;
  const bool cta = merge_fits_one_cta(mp, rows, one);
  cudaError_t e;
  if (xh && cta) {
    // wait and push inside the merge kernel
    ExchangeHooks& x = mp.x;
    x.wait_flags = static_cast<const unsigned*>(xh->wait_flags);
    x.wait_n = xh->wait_flags ? xh->num_wait_flags : 0;
    x.epoch = static_cast<const unsigned*>(xh->epoch);
    x.limit_ns = xh->wait_timeout_ns;
    if (xh->peer_partials) {
      x.npeers = xh->num_peers;
      for (int i = 0; i < xh->num_peers; ++i) {
        x.peer_rows[i] = static_cast<float*>(xh->peer_partials[i]);
        x.peer_flag[i] = static_cast<unsigned*>(xh->peer_flags[i]);
      }
      x.done = static_cast<unsigned*>(xh->done_counter);
    }
  } else if (xh && xh->wait_flags) {
    e = launch_exchange_wait(static_cast<const unsigned*>(xh->wait_flags), xh->num_wait_flags,
                             const_cast<unsigned*>(static_cast<const unsigned*>(xh->epoch)), 0,
                             xh->wait_timeout_ns, m.status, stream);
    if (e != cudaSuccess) return cuda_fail(e, "exchange_wait launch");
  }
  e = dispatch_merge(mp, rows, pl, stream);
  if (e != cudaSuccess) return cuda_fail(e, "merge_attend launch");
  if (xh && !cta && xh->peer_partials) {
    const size_t bytes = (size_t)rows * (kHeadDim + 2) * sizeof(float);
    return ra_exchange_push(p->out_partial, bytes, xh->peer_partials, xh->peer_flags, xh->num_peers,
                            xh->epoch, xh->done_counter, p->stream);
  }
  return RA_OK;
}

int ra_lse_combine_wait(const float* partials, int32_t num_parts, int32_t rows, void* out,
                        const void* wait_flags, int32_t num_flags, void* epoch, uint64_t timeout_ns,
                        void* done_counter, void* status_workspace, void* stream) {
  if (!partials || !out || num_parts < 1 || rows < 1) return invalid("bad lse_combine arguments");
  if (!wait_flags || !epoch || !done_counter || !status_workspace || num_flags < 1 ||
      num_flags > kMaxPeers || timeout_ns == 0)
    return invalid("bad exchange arguments");
  ExchangeHooks x;
  memset(&x, 0, sizeof x);
  x.wait_flags = static_cast<const unsigned*>(wait_flags);
  x.wait_n = num_flags;
  x.epoch = static_cast<const unsigned*>(epoch);
  x.limit_ns = timeout_ns;
  x.done = static_cast<unsigned*>(done_counter);
  x.advance = 1;
  x.epoch_rw = static_cast<unsigned*>(epoch);
  cudaError_t e = launch_lse_combine(partials, num_parts, rows, static_cast<__half*>(out),
                                     static_cast<cudaStream_t>(stream), &x,
                                     static_cast<unsigned*>(status_workspace));
  if (e != cudaSuccess) return cuda_fail(e, "lse_combine launch");
  return RA_OK;
}

int ra_lse_combine(const float* partials, int32_t num_parts, int32_t rows, void* out, void* stream) {
  if (!partials || !out || num_parts < 1 || rows < 1) return invalid("bad lse_combine arguments");
  cudaError_t e = launch_lse_combine(partials, num_parts, rows, static_cast<__half*>(out),
                                     static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "lse_combine launch");
  return RA_OK;
}

size_t ra_shard_exchange_bytes(int32_t rows, int32_t world) {
  if (rows < 1 || world < 1) return 0;
  return (size_t)world * rows * (kShardRounds * kHistBins + kPartWords) * sizeof(unsigned long long);
}

int ra_sharded_topk_attention(const ra_params* p, const ra_shard_exchange* x) {
  if (!p || !x) return invalid("params and exchange must be given");
  if (x->world < 1 || x->world > kMaxPeers || x->rank < 0 || x->rank >= x->world)
    return invalid("bad world / rank");
  if (!x->bufs || !x->epoch || !x->done_counter || x->wait_timeout_ns == 0)
    return invalid("receive buffers, epoch word, done counter and a wait bound are required");
  for (int r = 0; r < x->world; ++r)
    if (!x->bufs[r] || (reinterpret_cast<uintptr_t>(x->bufs[r]) & 7u))
      return invalid("a rank's receive buffer is missing or not 8-byte aligned");
  Checked c;
  int st = check_params(p, true, true, c);
  if (st != RA_OK) return st;
  Shape s = c.shape;
  s.fused_ok = 1;
  if (!store_shape(s)) return unsupported("the histogram exchange needs several queries per K row and one segment");
  return run_store(p, s, c.group, true, static_cast<unsigned*>(p->workspace), x);
}

int ra_score_store_probe(const ra_params* p) {
  if (!p) return invalid("params is null");
  Checked c;
  int st = check_params(p, false, false, c);
  if (st != RA_OK) return st;
  Shape s = c.shape;
  s.fused_ok = 1;
  if (!store_shape(s)) return unsupported("not a shape of the stored-score route");
  return run_store(p, s, c.group, false, static_cast<unsigned*>(p->workspace), nullptr, true);
}

int ra_stream_read_probe(const void* src, size_t bytes, void* sink, void* stream) {
  if (!src || !sink || bytes < 16 || (bytes & 15u) || (reinterpret_cast<uintptr_t>(src) & 15u))
    return invalid("src and sink must be given, src 16-byte aligned, bytes a positive multiple of 16");
  cudaError_t e = launch_stream_read(src, bytes, static_cast<unsigned*>(sink), 4 * sm_count(),
                                     static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "stream_read launch");
  return RA_OK;
}

int ra_l2_persist(const void* base, size_t bytes, float hit_ratio, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaStreamAttrValue attr;
  memset(&attr, 0, sizeof attr);
  if (bytes == 0) {
    attr.accessPolicyWindow.num_bytes = 0;
    cudaError_t e = cudaStreamSetAttribute(st, cudaStreamAttributeAccessPolicyWindow, &attr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSetAttribute(access policy window)");
    e = cudaCtxResetPersistingL2Cache();
    if (e != cudaSuccess) return cuda_fail(e, "cudaCtxResetPersistingL2Cache");
    return RA_OK;
  }
  if (!base || !(hit_ratio > 0.f) || hit_ratio > 1.f) return invalid("base must be given and hit_ratio in (0, 1]");
  int dev = 0, max_persist = 0, max_window = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&max_window, cudaDevAttrMaxAccessPolicyWindowSize, dev);
  if (e != cudaSuccess) return cuda_fail(e, "querying the L2 persistence limits");
  if (max_persist <= 0 || max_window <= 0) return unsupported("this device has no persisting L2 lines");
  size_t have = 0;
  e = cudaDeviceGetLimit(&have, cudaLimitPersistingL2CacheSize);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetLimit(persisting L2)");
  const size_t want = std::min<size_t>(bytes, (size_t)max_persist);
  if (have < want) {
    e = cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, want);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSetLimit(persisting L2)");
  }
  attr.accessPolicyWindow.base_ptr = const_cast<void*>(base);
  attr.accessPolicyWindow.num_bytes = std::min<size_t>(bytes, (size_t)max_window);
  attr.accessPolicyWindow.hitRatio = hit_ratio;
  attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
  attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
  e = cudaStreamSetAttribute(st, cudaStreamAttributeAccessPolicyWindow, &attr);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSetAttribute(access policy window)");
  return RA_OK;
}

int ra_exchange_push(const void* src, size_t bytes, void* const* peer_dst, void* const* peer_flags,
                     int32_t num_peers, const void* epoch, void* done_counter, void* stream) {
  if (!src || !peer_dst || !peer_flags || !epoch || !done_counter) return invalid("a required pointer is null");
  if (num_peers < 1 || num_peers > kMaxPeers) return invalid("num_peers must be in [1, 32]");
  if (bytes == 0 || (bytes & 15u) || (reinterpret_cast<uintptr_t>(src) & 15u))
    return invalid("src must be 16-byte aligned and bytes a positive multiple of 16");
  PushParams pp;
  memset(&pp, 0, sizeof pp);
  pp.src = static_cast<const uint4*>(src);
  pp.n16 = bytes / 16;
  pp.npeers = num_peers;
  for (int i = 0; i < num_peers; ++i) {
    if (!peer_dst[i] || !peer_flags[i] || (reinterpret_cast<uintptr_t>(peer_dst[i]) & 15u) ||
        (reinterpret_cast<uintptr_t>(peer_flags[i]) & 3u))
      return invalid("peer pointers must be non-null and aligned (16 bytes for slots, 4 for flags)");
    pp.dst[i] = static_cast<uint4*>(peer_dst[i]);
    pp.flag[i] = static_cast<unsigned*>(peer_flags[i]);
  }
  pp.epoch = static_cast<const unsigned*>(epoch);
  pp.done = static_cast<unsigned*>(done_counter);
  const int grid = (int)std::max<size_t>(1, std::min<size_t>((size_t)2 * sm_count(),
                                                              (pp.n16 + kPushThreads - 1) / kPushThreads));
  cudaError_t e = launch_exchange_push(pp, grid, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "exchange_push launch");
  return RA_OK;
}

int ra_exchange_wait(const void* flags, int32_t num_flags, void* epoch, int32_t advance,
                     uint64_t timeout_ns, void* status_workspace, void* stream) {
  if (!flags || !epoch || !status_workspace) return invalid("a required pointer is null");
  if (num_flags < 1 || num_flags > kMaxPeers) return invalid("num_flags must be in [1, 32]");
  if (timeout_ns == 0) return invalid("timeout_ns must be positive");
  cudaError_t e = launch_exchange_wait(static_cast<const unsigned*>(flags), num_flags,
                                       static_cast<unsigned*>(epoch), advance,
                                       (unsigned long long)timeout_ns,
                                       static_cast<unsigned*>(status_workspace),
                                       static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "exchange_wait launch");
  return RA_OK;
}

static void legacy_params(ra_params* p, const void* q, const void* k, const void* v, void* out,
                          int32_t batch, int32_t num_tokens, int32_t topk, void* ws, size_t wsb,
                          void* stream) {
  memset(p, 0, sizeof *p);
  p->q = q; p->k = k; p->v = v; p->out = out;
  p->batch = batch; p->num_q_heads = 32; p->num_kv_heads = 32; p->head_dim = 128;
  p->num_tokens = num_tokens;
  p->kv_batch_stride = 0; p->kv_token_stride = 32 * 128; p->kv_head_stride = 128;
  p->topk = topk; p->num_segments = 4; p->sm_scale = 1.0f;
  p->workspace = ws; p->workspace_bytes = wsb; p->stream = stream;
}

int ra_legacy_retrieval_attention(const void* q, const void* k, const void* v, void* out,
                                  int32_t batch, int32_t num_tokens, int32_t topk_per_chunk,
                                  int32_t variant, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  if (variant < 0 || variant > 5) return invalid("variant must be 0..5");
  ra_params p;
  legacy_params(&p, q, k, v, out, batch, num_tokens, topk_per_chunk, workspace, workspace_bytes,
                stream);
  return ra_topk_attention(&p);
}

size_t ra_legacy_workspace_bytes(int32_t batch, int32_t num_tokens, int32_t topk_per_chunk) {
  ra_params p;
  legacy_params(&p, reinterpret_cast<void*>(uintptr_t(256)), reinterpret_cast<void*>(uintptr_t(256)),
                reinterpret_cast<void*>(uintptr_t(256)), reinterpret_cast<void*>(uintptr_t(256)), batch,
                num_tokens, topk_per_chunk, nullptr, 0, nullptr);
  return ra_workspace_bytes(&p);
}

}  // extern "C"
