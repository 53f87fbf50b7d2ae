/*
 * topk_attn_b200 — C ABI of the decode-time top-k sparse-attention path for NVIDIA B200
 * (sm_100a).
 *
 * Every entry point is plain C: raw device pointers, sizes and a CUDA stream handle; no
 * torch types, no exceptions, no exit().  Each returns an int status (RA_OK == 0,
 * ra_strerror() gives the text).  Work is enqueued on the caller's stream and the call
 * returns without synchronising; no entry point allocates device memory — scratch comes
 * from a caller-provided workspace sized by ra_workspace_bytes(), zeroed once before its first
 * use (its first 256 bytes are a status block whose bits are sticky).
 *
 * Tensor layouts are the reference project's:
 *   q      fp16 [B, Hq, D]                       retrieval_attn/retrieval_attention.cu:257
 *   k, v   fp16 [N, Hkv, D] token-major, one cache shared by all batch rows (kv_batch_stride
 *          == 0), or one cache per batch row (kv_batch_stride != 0)        ...:258-259,282-284
 *   out    fp16 [B, Hq, D]                                                  ...:260
 *   centers fp16 [H, CSZ, D]                      center_only_topk/gemv_topk.cu:99
 *   indices int32 [.., H, S] global token ids     gemv_topk.cu:373-377, flash_decoding.cu:105
 * D must be 128 (the reference's only head size, retrieval_attention.cu:31).
 */
#ifndef TOPK_ATTN_B200_H_
#define TOPK_ATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RA_OK 0
#define RA_ERR_INVALID_ARGUMENT 1   /* null pointer, bad shape, k > N, misaligned pointer */
#define RA_ERR_UNSUPPORTED 2        /* head_dim != 128, sizes beyond what the kernels hold */
#define RA_ERR_WORKSPACE 3          /* workspace missing or smaller than ra_workspace_bytes() */
#define RA_ERR_CUDA 4               /* a CUDA runtime/driver call failed; see ra_last_cuda_error() */
#define RA_ERR_DEVICE_TIMEOUT 5     /* a bounded wait inside a kernel gave up (ra_check_status) */
#define RA_ERR_NOT_BUILT 6
#define RA_ERR_DEVICE_CHECK 7       /* a kernel found and skipped inconsistent data (ra_check_status) */

/* Operands of one decode step.  Unused optional pointers are NULL. */
typedef struct ra_params {
  const void* q;            /* fp16 [batch, num_q_heads, 128] contiguous */
  const void* k;            /* fp16 key cache */
  const void* v;            /* fp16 value cache, same strides as k */
  void* out;                /* fp16 [batch, num_q_heads, 128]; may be NULL when only
                               candidates/indices are wanted */
  int32_t batch;
  int32_t num_q_heads;
  int32_t num_kv_heads;     /* divides num_q_heads; query head h reads kv head h / group */
  int32_t head_dim;         /* 128 */
  int32_t num_tokens;       /* N, tokens present in the cache (of this shard) */
  int64_t kv_batch_stride;  /* elements between the caches of two batch rows; 0 = shared */
  int64_t kv_token_stride;  /* elements between tokens (num_kv_heads*128 for [N,Hkv,D]) */
  int64_t kv_head_stride;   /* elements between heads (128 for [N,Hkv,D]) */
  int32_t topk;             /* keys kept per segment */
  int32_t num_segments;     /* 1 = global top-k; 4 = the legacy per-chunk selection */
  float sm_scale;           /* softmax(sm_scale * q.k); 1.0 reproduces exp(s)/sum exp(s) */
  int32_t index_base;       /* added to reported token ids (shard offset) */
  int32_t* out_indices;     /* optional int32 [batch, num_q_heads, num_segments*topk] */
  float* out_scores;        /* optional fp32, same shape: raw q.k of each kept key */
  float* out_lse;           /* optional fp32 [batch, num_q_heads, 2]: (max of sm_scale*s,
                               sum of exp) of the kept keys */
  void* workspace;          /* device scratch, 256-byte aligned */
  size_t workspace_bytes;
  void* stream;             /* cudaStream_t */
} ra_params;

const char* ra_strerror(int status);
int ra_version(void);
/* Text of the last failing CUDA call made by this library on the calling thread. */
const char* ra_last_cuda_error(void);
/* Kernels this library has launched since it was loaded, over all threads (a host-side counter
 * bumped beside every launch; no counterpart in the reference).  Benchmarks read it before and
 * after a timed region to state how many launches the region held. */
unsigned long long ra_launch_count(void);

/* Scratch needed by ra_topk_attention / ra_gemv_topk for these operands (the largest any
 * internal plan may use).  Replaces the per-call cudaMalloc of the reference's host runners
 * (retrieval_attn/retrieval_attention.cu:1658-1659,1738-1741). */
size_t ra_workspace_bytes(const ra_params* p);

/* Fused decode step: scan K, keep the exact top-k per (batch row, query head[, segment]),
 * softmax over the kept keys, mix their V rows.  One kernel when a thread-block cluster
 * can cover a head's whole context, scan + merge kernels otherwise.
 * Replaces launch_retrieval_attention*_K and run_retrieval_attention*<K>
 * (retrieval_attn/retrieval_attention.cu:1389-2282) and the fused pipelines
 * topk_attn_fused_kernel (baseline_2.cu:583-1058). */
int ra_topk_attention(const ra_params* p);

/* Same decode step as ra_topk_attention for callers that have no device buffer to lend and
 * must not allocate one: a plugin inside a server that reserved all of HBM for its own pools at
 * start-up, code that runs after an "initialisation is over, no more cudaMalloc" point (a
 * cudaMalloc there may also synchronise the whole device in the middle of a decode step), or a
 * host language binding that can pass pointers it was given but cannot create new ones.
 * It has no counterpart in the reference, whose runners cudaMalloc and cudaFree their scratch on
 * every call.  p->workspace and p->workspace_bytes are ignored; the scratch is a fixed
 * RA_NOALLOC_SCRATCH_BYTES array inside the library image, so every GPU that loads the library
 * gives up that much memory until the process exits.  The call itself performs no cudaMalloc,
 * cudaFree or other allocating call.
 *   - Shapes whose ra_workspace_bytes() exceeds RA_NOALLOC_SCRATCH_BYTES are refused with
 *     RA_ERR_UNSUPPORTED (ra_last_cuda_error() says so); nothing is launched.
 *   - The first call on each device looks up the array's device address (with that device
 *     current).  Make that first call during start-up, before any stream capture begins.
 *   - All calls on one device share the array.  Its status block is cleared at the start of each
 *     call, everything else is overwritten before it is read.  Two calls whose kernels may run at
 *     the same time on one GPU (different streams, no dependency) race on it: order them.
 *   - The device-side self-check word lives in the array too and is not reported back; callers
 *     that want ra_check_status() use the workspace variant. */
#define RA_NOALLOC_SCRATCH_BYTES (4u << 20)
int ra_topk_attention_noalloc(const ra_params* p);

/* Selection only: out_indices (and out_scores) must be given, out/v are ignored.  The role of
 * gemv_topk_kernel (gemv_topk.cu:173-380) with a global top-k over the N keys. */
int ra_gemv_topk(const ra_params* p);

/* After the stream has been synchronised by the caller: RA_OK, or RA_ERR_DEVICE_TIMEOUT if a
 * kernel that used this workspace abandoned a bounded wait, or RA_ERR_DEVICE_CHECK if one
 * skipped data that failed its own bounds checks.  Synchronises the stream itself. */
int ra_check_status(void* workspace, void* stream);

/* The reference extension's entry points (retrieval_attn/bind.cpp:5-243 declare
 * launch_retrieval_attention{,_global,_pipelined,_pipelined_global,_two_kernels,
 * _gather_baseline}_{32,128,256,512,1024}(q, k, v, out, batch)): N = num_tokens keys in a shared
 * [N,32,128] cache cut in 4 chunks, top-K per chunk, raw-exp softmax, no scale.
 * variant (0 fused, 1 global-scratch, 2 pipelined, 3 pipelined-global, 4 two kernels, 5 gather +
 * dense baseline) is accepted so that each of the reference's 30 names has a target, and is
 * validated, but selects nothing: the reference's variants schedule the same arithmetic in
 * different ways, and this library runs its one fastest route for all of them.  There is no A/B
 * between variants here; ra_gemv_topk + ra_gathered_attention is the two-call form. */
int ra_legacy_retrieval_attention(const void* q, const void* k, const void* v, void* out,
                                  int32_t batch, int32_t num_tokens, int32_t topk_per_chunk,
                                  int32_t variant, void* workspace, size_t workspace_bytes,
                                  void* stream);
size_t ra_legacy_workspace_bytes(int32_t batch, int32_t num_tokens, int32_t topk_per_chunk);

/* Attention over given key ids: softmax(sm_scale * q.K[id]) . V[id].  Replaces
 * MHAFlashDecodeKernel (baseline_1.cu:324-610; prototype flash_decoding.cu:100-388), whose
 * kv_indices are [H, S] global token ids shared by the batch (flash_decoding.cu:105); sm_scale is
 * explicit (the reference applies rsqrt(D) inside, baseline_1.cu:369). */
typedef struct ra_gather_params {
  const void* q;            /* fp16 [batch, num_q_heads, 128] */
  const void* k;            /* fp16 caches, strides below */
  const void* v;
  void* out;                /* fp16 [batch, num_q_heads, 128] */
  int32_t batch, num_q_heads, num_kv_heads, head_dim, num_tokens;
  int64_t kv_batch_stride, kv_token_stride, kv_head_stride;
  const int32_t* indices;   /* int32 [batch or 1, num_q_heads, num_indices] */
  int32_t num_indices;
  int64_t indices_batch_stride; /* elements; 0 = one list per head shared by the batch */
  float sm_scale;
  float* out_lse;           /* optional fp32 [batch, num_q_heads, 2] */
  void* workspace;          /* >= 256 bytes (status word) */
  size_t workspace_bytes;
  void* stream;
} ra_gather_params;

int ra_gathered_attention(const ra_gather_params* p);

/* Centroid-only retrieval: score the num_centers centroids of every head, keep the
 * top_clusters best, expand cluster c to its member tokens c*cluster_len .. +cluster_len-1 in
 * descending order of the centroid scores, and (when k, v and out are given) attend over all
 * member tokens.  Replaces gemv_topk_kernel / gemv_topk_cluster_kernel
 * (center_only_topk/gemv_topk.cu:157-280, :283-457) and, with attention, the pipelines of
 * center_only_topk/baselines.cu:546-973. */
typedef struct ra_center_params {
  const void* q;            /* fp16 [batch, num_heads, 128] */
  const void* centers;      /* fp16 [num_heads, num_centers, 128] (center_only_topk/gemv_topk.cu:99) */
  int32_t batch, num_heads, head_dim;
  int32_t num_centers;      /* CSZ */
  int32_t cluster_len;      /* CLEN */
  int32_t top_clusters;     /* TOPC */
  int32_t* out_cluster_ids; /* optional int32 [batch, num_heads, top_clusters]; in descending
                               score order when out_indices is given without out, else unordered */
  int32_t* out_indices;     /* optional int32 [batch, num_heads, top_clusters*cluster_len] */
  const void* k;            /* optional fp16 [num_tokens, num_heads, 128] (or per batch row) */
  const void* v;
  void* out;                /* optional fp16 [batch, num_heads, 128] */
  int32_t num_tokens;
  int64_t kv_batch_stride, kv_token_stride, kv_head_stride;
  float sm_scale;
  void* workspace;          /* ra_center_workspace_bytes() */
  size_t workspace_bytes;
  void* stream;
} ra_center_params;

int ra_center_only_topk(const ra_center_params* p);
size_t ra_center_workspace_bytes(int32_t batch, int32_t num_heads, int32_t num_centers,
                                 int32_t top_clusters);

/* Two-level retrieval: keep the top_clusters best centroids of every head, then inside each
 * kept cluster (cluster_len contiguous tokens) the topk_per_cluster best keys; optionally attend
 * over all kept keys.  out_indices is [batch, num_heads, top_clusters * topk_per_cluster] with
 * one slice per cluster in descending order of the centroid scores, unordered inside a slice —
 * the layout of gemv_topk_kernel (gemv_topk.cu:173-380, baseline_1.cu:103-319); with out it
 * is the pipeline of baseline_1.cu / baseline_2.cu (selection + gathered decode). */
typedef struct ra_two_level_params {
  const void* q;            /* fp16 [batch, num_heads, 128] */
  const void* centers;      /* fp16 [num_heads, num_centers, 128] */
  const void* k;            /* fp16 [num_tokens, num_heads, 128] or one cache per batch row */
  const void* v;            /* needed with out */
  void* out;                /* optional fp16 [batch, num_heads, 128] */
  int32_t batch, num_heads, head_dim;
  int32_t num_centers, cluster_len, top_clusters, topk_per_cluster;
  int32_t num_tokens;       /* >= num_centers * cluster_len */
  int64_t kv_batch_stride, kv_token_stride, kv_head_stride;
  float sm_scale;
  int32_t* out_cluster_ids; /* optional int32 [batch, num_heads, top_clusters], rank order */
  int32_t* out_indices;     /* optional int32, see above */
  float* out_scores;        /* optional fp32, same shape as out_indices */
  void* workspace;          /* ra_two_level_workspace_bytes() */
  size_t workspace_bytes;
  void* stream;
} ra_two_level_params;

int ra_two_level_topk(const ra_two_level_params* p);
size_t ra_two_level_workspace_bytes(int32_t batch, int32_t num_heads, int32_t num_centers,
                                    int32_t top_clusters, int32_t topk_per_cluster);

/* The step of a decode loop that precedes the attention: store the new token's key and value
 * rows (fp16 [caches, num_kv_heads, 128], caches = batch for per-sequence caches, else 1) at token
 * `position` of the caches and, when `centers` (fp16 [num_kv_heads, num_centers, 128]) is given
 * with a shared cache, fold the key into the running mean of centroid position / cluster_len.
 * The reference assumes caches and centroids are given (gemv_topk.cu:218, baseline_1.py:44-68);
 * this keeps them in the layouts its kernels read. */
int ra_kv_append(void* k_cache, void* v_cache, const void* new_k, const void* new_v,
                 int32_t caches, int32_t num_kv_heads, int32_t head_dim, int32_t position,
                 int32_t capacity_tokens, int64_t kv_batch_stride, int64_t kv_token_stride,
                 int64_t kv_head_stride, void* centers, int32_t num_centers, int32_t cluster_len,
                 void* stream);

/* Dense decode attention over the whole cache, split-KV with a log-sum-exp combine
 * ("flash decoding"): the dense baseline of the path and the reference's
 * baseline_attention_kernel (retrieval_attn/retrieval_attention.cu:51-168) /
 * MHAFlashDecodeKernel (flash_decoding.cu:100-388) without the index gather. */
typedef struct ra_dense_params {
  const void* q;            /* fp16 [batch, num_q_heads, 128] */
  const void* k;            /* fp16 caches, token-major */
  const void* v;
  void* out;                /* fp16 [batch, num_q_heads, 128] */
  int32_t batch, num_q_heads, num_kv_heads, head_dim, num_tokens;
  int64_t kv_batch_stride, kv_token_stride, kv_head_stride;
  float sm_scale;
  int32_t num_splits;       /* chunks of the token axis; 0 = chosen by the library */
  void* workspace;          /* ra_flash_workspace_bytes() */
  size_t workspace_bytes;
  void* stream;
} ra_dense_params;

int ra_flash_decoding(const ra_dense_params* p);
size_t ra_flash_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                int32_t num_tokens, int32_t num_splits);

/* ---- sequence-sharded decode (no counterpart in the reference, which is single-device) ----
 * The token axis is cut over ranks.  Per step every rank (1) calls ra_gemv_topk on its shard
 * with index_base = first global token id of the shard, (2) all-gathers the [B,Hq,k] score and
 * id buffers of all ranks, (3) calls ra_merge_attend, which selects the global top-k out of the
 * num_parts*k candidates and mixes only the V rows this rank holds into an un-normalised
 * partial, (4) all-gathers the partials and (5) calls ra_lse_combine.  Every rank merges the same
 * candidates and the merge is deterministic (candidates are ranked by score, then by their
 * position in the candidate array), so every rank selects the same set.  The two all-gathers
 * are either collectives of a library (NCCL) or ra_exchange_push / ra_exchange_wait below. */
/* Optional exchange steps fused into ra_merge_attend (see ra_exchange_push / ra_exchange_wait for
 * the buffers, flags and epoch word): the merge first waits for the candidate flags of all ranks
 * (bounded), and after writing out_partial stores the same rows into this rank's slot on every
 * peer and raises this rank's flag there. */
typedef struct ra_exchange_hooks {
  const void* wait_flags;      /* local flag words to wait for before candidates are read, or NULL */
  int32_t num_wait_flags;
  const void* epoch;           /* device word holding the current epoch */
  uint64_t wait_timeout_ns;
  void* const* peer_partials;  /* host array: out_partial's address in every rank (own entry =
                                  out_partial itself), or NULL */
  void* const* peer_flags;     /* host array: this rank's partial flag word on every rank */
  int32_t num_peers;
  void* done_counter;          /* zero-initialised device word */
} ra_exchange_hooks;

typedef struct ra_merge_params {
  const float* cand_scores;    /* fp32 [num_parts, batch, num_q_heads, topk] */
  const int32_t* cand_indices; /* int32, same shape, global token ids */
  int32_t num_parts;
  int64_t cand_part_stride;    /* elements between two parts in both buffers; 0 = dense
                                  (batch*num_q_heads*topk).  Lets scores and ids travel as the two
                                  halves of one all-gathered buffer. */
  const void* v;               /* this rank's value cache */
  void* out;                   /* optional fp16 [batch, num_q_heads, 128], normalised */
  float* out_partial;          /* optional fp32 [batch, num_q_heads, 130]: 128 un-normalised
                                  sums, their weight, the maximum of sm_scale*score */
  int32_t batch, num_q_heads, num_kv_heads, head_dim;
  int32_t num_tokens;          /* rows of v */
  int64_t kv_batch_stride, kv_token_stride, kv_head_stride;
  int32_t topk;
  float sm_scale;
  int32_t own_base;            /* global id of row 0 of v; ids outside
                                  [own_base, own_base + num_tokens) are not mixed */
  int32_t* out_indices;        /* optional int32 [batch, num_q_heads, topk]: the global winners */
  float* out_scores;           /* optional fp32, same shape */
  void* workspace;             /* >= 256 bytes, 256-byte aligned (status word only) */
  size_t workspace_bytes;
  void* stream;
  const ra_exchange_hooks* exchange;  /* optional, with out_partial only */
  int32_t own_part_only;       /* 1: only the candidates of part `own_part` can be owned by this
                                  rank; cand_indices of every other part is not read, so the ranks
                                  need to exchange the scores only (ties between parts are broken
                                  by position, not by id).  out_indices then lists -1 for winners of
                                  other parts.  0: ownership by id range, all ids are read. */
  int32_t own_part;
} ra_merge_params;

int ra_merge_attend(const ra_merge_params* p);

/* out[r,:] = sum_p w_p o_p / sum_p w_p l_p, w_p = exp(m_p - max_p m_p), over num_parts partials of
 * the layout ra_merge_attend writes ([num_parts, rows, 130]); out is fp16 [rows, 128].  The
 * log-sum-exp merge of baseline_1.cu:549-598 as a stand-alone step. */
int ra_lse_combine(const float* partials, int32_t num_parts, int32_t rows, void* out, void* stream);
/* The same after a bounded wait for the num_flags partial flags of all ranks (ra_exchange_wait's
 * rules); the kernel ends the step by adding one to the epoch word.  done_counter is a
 * zero-initialised device word, status_workspace a workspace whose status block takes the
 * timeout bit. */
int ra_lse_combine_wait(const float* partials, int32_t num_parts, int32_t rows, void* out,
                        const void* wait_flags, int32_t num_flags, void* epoch, uint64_t timeout_ns,
                        void* done_counter, void* status_workspace, void* stream);

/* ---- sequence-sharded decode by exchanged histograms (no counterpart in the reference) ----
 * For shards that take the stored-score route (several queries per K row: a GQA group or one cache
 * shared by the batch, one global selection).  One call per rank and step: the rank scores its
 * shard once and keeps the scores; the ranks then find the exact global k-th score together by a
 * radix select whose histograms travel between them (2048 counters per row, rank and round; 2
 * rounds for distinct scores, 3 at most) instead of k candidates per row and rank; each rank mixes
 * the winners among its own tokens into an un-normalised partial, sends it to every rank, waits
 * for the others' and writes the full output p->out ([batch, num_q_heads, 128] fp16, the same bits
 * on every rank).  Copies of the k-th score are taken in rank order, inside a rank in token
 * order, so the result equals the single-device operator's on the concatenated cache, ties
 * included.
 *
 * bufs[r] (host array of `world` device pointers) is rank r's receive buffer as mapped in this
 * process (peer-mapped memory: CUDA IPC, virtual memory management, symmetric memory), each of
 * ra_shard_exchange_bytes(batch * num_q_heads, world) bytes and zero before the first step; entry
 * `rank` is this rank's own.  All traffic is 8-byte words that carry their step's epoch, polled
 * by the receiver: no flags, no fences, no collective library.  `epoch` is a device word that
 * holds 1 before the first step; the call adds one when it has finished (so a captured call can be
 * replayed).  done_counter is a zero-initialised device word.  Every wait is bounded by
 * wait_timeout_ns (RA_ERR_DEVICE_TIMEOUT through ra_check_status); the timeout bit of the status
 * block is sticky, and while it is set no kernel of the library waits for a peer again, so a rank
 * whose peers are gone finishes its step in one time limit.  Clear the status block to resume.  p->out_indices / out_scores,
 * when given ([batch, num_q_heads, topk], pre-filled by the caller), receive this rank's winners
 * (global ids) from the start of each row.
 * All ranks must call with the same batch, heads, topk and world; the selection kernel needs
 * batch * num_q_heads * its cluster size CTAs resident at once and refuses shapes beyond that. */
typedef struct ra_shard_exchange {
  int32_t world, rank;
  void* const* bufs;
  void* epoch;
  uint64_t wait_timeout_ns;
  void* done_counter;
} ra_shard_exchange;
size_t ra_shard_exchange_bytes(int32_t rows, int32_t world);
int ra_sharded_topk_attention(const ra_params* p, const ra_shard_exchange* x);

/* Measuring aid: the scoring pass of the stored-score route alone (K streamed once, every score
 * and the coarse histograms into the workspace, nothing selected), for timing the dominant kernel
 * of ra_sharded_topk_attention and of ra_topk_attention on such shapes.  RA_ERR_UNSUPPORTED for
 * shapes that take another route. */
int ra_score_store_probe(const ra_params* p);

/* Measuring aid (no counterpart in the reference): one kernel that reads `bytes` (a multiple of 16)
 * from `src` and does nothing else, on `stream`.  Timing it over a buffer much larger than L2 gives
 * the read-only streaming rate of the device, the natural ceiling of a K scan, beside the copy
 * (read + write) figure rooflines are usually quoted against.  `sink` is one writable device word. */
int ra_stream_read_probe(const void* src, size_t bytes, void* sink, void* stream);

/* Keep a cache resident in L2 across consecutive decode steps (no counterpart in the reference,
 * whose pipelined kernels keep K hot only inside one launch, retrieval_attn/
 * retrieval_attention.cu:654-896).  Marks [base, base + bytes) as persisting for every kernel later
 * launched into `stream` (an access-policy window, a stream attribute) and reserves as much of L2
 * for persisting lines as the device allows for that size; hit_ratio in (0, 1] is the fraction of
 * the window that should persist when it is larger than the reservation.  bytes == 0 removes the
 * window and releases the persisting lines.  Both settings belong to the calling process's CUDA
 * context and end with it.  Worth it for caches of up to roughly the L2 size shared by all batch
 * rows (kv_batch_stride == 0): each step then re-reads K from L2 instead of HBM. */
int ra_l2_persist(const void* base, size_t bytes, float hit_ratio, void* stream);

/* ---- exchange step of the sharded decode over peer-mapped memory (no counterpart in the
 * reference; the in-GPU mechanism it generalises is the cluster-wide exchange through
 * distributed shared memory of baseline_1.cu:549-598) ----
 * Every rank owns a receive buffer that all ranks of the node have mapped (CUDA IPC or virtual
 * memory management; the library only sees the resulting pointers).  ra_exchange_push copies
 * `bytes` (a multiple of 16) from `src` into this rank's slot on every peer (peer_dst[i], host
 * array of num_peers device pointers; an entry equal to src is not copied) with plain stores, and
 * when all of it is written stores the current epoch (the 32-bit word at `epoch`, device memory) to
 * this rank's flag on every peer (peer_flags[i]).  `done_counter` is a zero-initialised device word
 * the launch uses and leaves at zero.  ra_exchange_wait makes the stream wait until each of the
 * num_flags local flag words has reached the epoch, at most timeout_ns per flag; a wait that runs
 * out sets the timeout bit of the status block at status_workspace (ra_check_status then reports
 * RA_ERR_DEVICE_TIMEOUT) and the stream carries on.  With advance != 0 the wait ends by adding one
 * to the epoch word, so that a captured sequence of these calls can be replayed unchanged. */
int ra_exchange_push(const void* src, size_t bytes, void* const* peer_dst, void* const* peer_flags,
                     int32_t num_peers, const void* epoch, void* done_counter, void* stream);
int ra_exchange_wait(const void* flags, int32_t num_flags, void* epoch, int32_t advance,
                     uint64_t timeout_ns, void* status_workspace, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TOPK_ATTN_B200_H_ */
