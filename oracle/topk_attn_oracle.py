"""CPU oracle for decode-time top-k sparse attention.  TEST INFRASTRUCTURE ONLY.

This module is a plain torch (CPU, fp32 compute on fp16 inputs) restatement of the
reference project's own torch path for single-token decode attention:

    scores = q . K^T  ->  torch.topk  ->  softmax over the selected keys  ->  . V

It is the checker that the CUDA kernels are compared against.  Nothing in the shipped
package may import it; only the test-suite, the smoke check and the CPU-baseline timing
leg of the benchmark do.  Each function names the reference file:line it follows.

Pinning: ``legacy_retrieval_attention`` and ``coarse_topk``/``fine_topk``/
``compute_attention`` are checked against the reference's own functions (executed from
the reference checkout) by ``tests/golden/make_golden.py``, which stores the resulting
vectors under ``tests/golden/``; ``tests/test_oracle.py`` replays them.

Tensor layouts (the reference's, retrieval_attn/retrieval_attention.cu:257-260,282-284):
    q      [B, Hq, D]  fp16
    k, v   [N, Hkv, D] fp16, one cache shared by every batch row, or
           [Bkv, N, Hkv, D] with Bkv == B for per-sequence caches
    out    [B, Hq, D]
Query head h reads KV head h // (Hq // Hkv).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
from torch import Tensor

__all__ = [
    "legacy_retrieval_attention",
    "full_scores",
    "topk_sparse_attention",
    "gathered_attention",
    "dense_attention",
    "split_kv_attention",
    "lse_combine",
    "center_only_topk",
    "center_only_attention",
    "coarse_topk",
    "fine_topk",
    "two_level_indices",
    "sharded_topk_attention",
    "check_index_sets",
    "check_topk_scores",
    "check_output",
]


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------
def _kv_view(k: Tensor, batch: Optional[int]) -> Tensor:
    """Return the cache as [Bkv, N, Hkv, D] (Bkv == 1 for the shared reference layout)."""
    if k.dim() == 3:
        return k.unsqueeze(0)
    if k.dim() == 4:
        if batch is not None and k.size(0) not in (1, batch):
            raise ValueError("per-sequence cache needs Bkv == B")
        return k
    raise ValueError("cache must be [N,Hkv,D] or [Bkv,N,Hkv,D]")


def full_scores(q: Tensor, k: Tensor) -> Tensor:
    """q.K^T for every key, fp32: [B, Hq, N].

    Same product as retrieval_attn/test_ra.py:117 (``torch.matmul(q_h, k_block^T)``) and
    baseline_1.py:87 (``(selected_k * q).sum(-1)``), computed in fp32 as baseline_1.py:73-74
    does after ``.to(torch.float32)``.
    """
    B, Hq, D = q.shape
    kv = _kv_view(k, B)
    Bkv, N, Hkv, _ = kv.shape
    g = Hq // Hkv
    qf = q.float().view(B, Hkv, g, D)
    out = torch.empty(B, Hq, N, dtype=torch.float32)
    for b in range(B):
        kb = kv[b if Bkv > 1 else 0].float()          # [N, Hkv, D]
        # [Hkv, g, D] x [Hkv, D, N] -> [Hkv, g, N]
        s = torch.matmul(qf[b], kb.permute(1, 2, 0))
        out[b] = s.reshape(Hq, N)
    return out


def _gather_rows(v: Tensor, b: int, Hq: int, idx: Tensor) -> Tensor:
    """Rows v[idx[h, j], h // g, :] as fp32 [Hq, S, D] for batch row b."""
    kv = _kv_view(v, None)
    Bkv, N, Hkv, D = kv.shape
    g = Hq // Hkv
    vb = kv[b if Bkv > 1 else 0]                       # [N, Hkv, D]
    heads = (torch.arange(Hq) // g).view(Hq, 1).expand_as(idx)
    return vb[idx, heads].float()                      # [Hq, S, D]


# --------------------------------------------------------------------------------------
# legacy retrieval_attn semantics (per-chunk top-K, raw exp softmax, no scale)
# --------------------------------------------------------------------------------------
def legacy_retrieval_attention(q: Tensor, k: Tensor, v: Tensor, topk_per_block: int,
                               num_blocks: int = 4) -> Tensor:
    """Restates reference_retrieval_attention, retrieval_attn/test_ra.py:88-160.

    The sequence is cut into ``num_blocks`` equal chunks (test_ra.py:103), each chunk keeps
    its own top-K scores (:121) with indices shifted to global (:124); the chunks'
    selections are concatenated (:131-132), soft-maxed with a raw ``exp`` and no max
    subtraction or 1/sqrt(D) (:136-138), and the selected V rows are mixed (:146-158).
    Computation happens in the dtype of the inputs, exactly as the reference does.
    """
    B, H, D = q.shape
    N = k.size(0)
    q_h = q.unsqueeze(2)                               # [B,H,1,D]
    k_h = k.permute(1, 0, 2).unsqueeze(0)              # [1,H,N,D]
    v_h = v.permute(1, 0, 2).unsqueeze(0)
    per = N // num_blocks
    sc, ix = [], []
    for i in range(num_blocks):
        lo = i * per
        kb = k_h[:, :, lo:lo + per, :]
        s = torch.matmul(q_h, kb.transpose(2, 3)).squeeze(2)       # [B,H,per]
        ts, ti = torch.topk(s, topk_per_block, dim=-1)
        sc.append(ts)
        ix.append(ti + lo)
    gs = torch.cat(sc, dim=2)
    gi = torch.cat(ix, dim=2)
    e = torch.exp(gs)
    p = e / e.sum(dim=-1, keepdim=True)
    idx = gi.unsqueeze(-1).expand(-1, -1, -1, D)
    vsel = torch.gather(v_h.expand(B, -1, -1, -1), 2, idx.long())  # [B,H,S,D]
    return torch.matmul(p.unsqueeze(2), vsel).squeeze(2)


# --------------------------------------------------------------------------------------
# general top-k sparse attention (global or segmented top-k, explicit scale, GQA)
# --------------------------------------------------------------------------------------
def topk_sparse_attention(q: Tensor, k: Tensor, v: Tensor, topk: int, sm_scale: float = 1.0,
                          num_segments: int = 1, index_base: int = 0,
                          scores: Optional[Tensor] = None
                          ) -> Tuple[Tensor, Tensor, Tensor]:
    """q.K^T -> torch.topk -> softmax over the selected keys -> .V, fp32 compute.

    The generalisation of test_ra.py:88-160 that the path's specification states: with
    ``num_segments == 1`` the top-k is global over the N keys; with ``num_segments == S``
    each of the S equal chunks keeps its own ``topk`` (the legacy behaviour, S = 4).
    ``softmax(sm_scale * s)`` equals the reference's raw ``exp(s)/sum`` when
    ``sm_scale == 1`` (test_ra.py:136-138) and baseline_1.py:107-108 when it is 1/sqrt(D).

    Returns (out fp32 [B,Hq,D], indices int64 [B,Hq,S*topk] (+index_base),
    scores fp32 [B,Hq,S*topk]); entries of one segment are in descending score order.
    """
    B, Hq, D = q.shape
    s = full_scores(q, k) if scores is None else scores
    N = s.size(-1)
    if N % num_segments:
        raise ValueError("N must be a multiple of num_segments")
    per = N // num_segments
    if topk > per:
        raise ValueError("topk larger than the segment")
    ts, ti = torch.topk(s.view(B, Hq, num_segments, per), topk, dim=-1)
    ti = ti + (torch.arange(num_segments) * per).view(1, 1, num_segments, 1)
    ts = ts.reshape(B, Hq, -1)
    ti = ti.reshape(B, Hq, -1)
    p = torch.softmax(ts * sm_scale, dim=-1)
    out = torch.empty(B, Hq, D, dtype=torch.float32)
    for b in range(B):
        vsel = _gather_rows(v, b, Hq, ti[b])           # [Hq,S,D]
        out[b] = torch.einsum("hs,hsd->hd", p[b], vsel)
    return out, ti + index_base, ts


def gathered_attention(q: Tensor, k: Tensor, v: Tensor, indices: Tensor,
                       sm_scale: float) -> Tensor:
    """Attention over given key ids.  Restates compute_attention, baseline_1.py:96-110
    (gather K and V rows, ``logits = (k*q).sum(-1) * scale``, softmax, weighted sum), which
    is also the intended math of MHAFlashDecodeKernel, baseline_1.cu:324-610.

    indices: [Hq, S] (shared by the batch) or [B, Hq, S]; returns fp32 [B,Hq,D].
    """
    B, Hq, D = q.shape
    if indices.dim() == 2:
        indices = indices.unsqueeze(0).expand(B, -1, -1)
    indices = indices.long()
    out = torch.empty(B, Hq, D, dtype=torch.float32)
    for b in range(B):
        ksel = _gather_rows(k, b, Hq, indices[b])
        vsel = _gather_rows(v, b, Hq, indices[b])
        logits = torch.einsum("hsd,hd->hs", ksel, q[b].float()) * sm_scale
        p = torch.softmax(logits, dim=-1)
        out[b] = torch.einsum("hs,hsd->hd", p, vsel)
    return out


# --------------------------------------------------------------------------------------
# dense attention and split-KV + log-sum-exp combine
# --------------------------------------------------------------------------------------
def dense_attention(q: Tensor, k: Tensor, v: Tensor, sm_scale: float) -> Tensor:
    """softmax(scale * q.K^T).V over every key, fp32 [B,Hq,D] (the dense role of
    baseline_attention_kernel, retrieval_attn/retrieval_attention.cu:51-168)."""
    B, Hq, D = q.shape
    s = full_scores(q, k) * sm_scale
    p = torch.softmax(s, dim=-1)
    vv = _kv_view(v, B)
    Bkv, N, Hkv, _ = vv.shape
    g = Hq // Hkv
    out = torch.empty(B, Hq, D, dtype=torch.float32)
    for b in range(B):
        vb = vv[b if Bkv > 1 else 0].float()           # [N,Hkv,D]
        pb = p[b].view(Hkv, g, N)
        out[b] = torch.matmul(pb, vb.permute(1, 0, 2)).reshape(Hq, D)
    return out


def lse_combine(o_parts: Tensor, m_parts: Tensor, l_parts: Tensor) -> Tensor:
    """Combine partial attention results.  o_parts [P,...,D] are UNNORMALISED sums
    ``sum_i exp(x_i - m_p) v_i`` with their maxima m_parts [P,...] and weights
    l_parts [P,...] = ``sum_i exp(x_i - m_p)``.  This is the cluster max-then-sum
    reduce of baseline_1.cu:549-598 written as one formula."""
    m = m_parts.max(dim=0).values
    w = torch.exp(m_parts - m)                         # [P,...]
    w = torch.where(torch.isfinite(m_parts), w, torch.zeros_like(w))
    l = (l_parts * w).sum(dim=0)
    o = (o_parts * w.unsqueeze(-1)).sum(dim=0)
    return o / l.unsqueeze(-1)


def split_kv_attention(q: Tensor, k: Tensor, v: Tensor, sm_scale: float,
                       num_splits: int) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """Flash-decoding: cut N into ``num_splits`` chunks, run an independent softmax in
    each (flash_decoding.cu:100-388 / baseline_1.cu:406-517 per cluster CTA) and merge
    with ``lse_combine``.  Returns (out, o_parts, m_parts, l_parts)."""
    B, Hq, D = q.shape
    s = full_scores(q, k) * sm_scale
    N = s.size(-1)
    per = (N + num_splits - 1) // num_splits
    vv = _kv_view(v, B)
    Bkv, _, Hkv, _ = vv.shape
    g = Hq // Hkv
    o_p = torch.zeros(num_splits, B, Hq, D)
    m_p = torch.full((num_splits, B, Hq), -math.inf)
    l_p = torch.zeros(num_splits, B, Hq)
    for i in range(num_splits):
        lo, hi = i * per, min(N, (i + 1) * per)
        if lo >= hi:
            continue
        sc = s[:, :, lo:hi]
        m = sc.max(dim=-1).values
        e = torch.exp(sc - m.unsqueeze(-1))
        m_p[i], l_p[i] = m, e.sum(dim=-1)
        for b in range(B):
            vb = vv[b if Bkv > 1 else 0][lo:hi].float()
            o_p[i, b] = torch.matmul(e[b].view(Hkv, g, hi - lo),
                                     vb.permute(1, 0, 2)).reshape(Hq, D)
    return lse_combine(o_p, m_p, l_p), o_p, m_p, l_p


# --------------------------------------------------------------------------------------
# centroid-only retrieval and two-level retrieval
# --------------------------------------------------------------------------------------
def center_only_topk(q: Tensor, centers: Tensor, topc: int, clen: int
                     ) -> Tuple[Tensor, Tensor, Tensor]:
    """Restates cpu_reference_indices, center_only_topk/gemv_topk.cu:82-119: score each
    of the CSZ centroids of a head in fp64 (:95-103), keep the ``topc`` best (:104-105)
    and expand cluster c to its member tokens ``c*clen + i`` (:108-116).

    q [B,H,D] or [H,D]; centers [H,CSZ,D].  Returns (token ids int64 [B,H,topc*clen],
    cluster ids [B,H,topc] in descending score order, centroid scores fp32 [B,H,CSZ]).
    """
    if q.dim() == 2:
        q = q.unsqueeze(0)
    cs = torch.einsum("hcd,bhd->bhc", centers.double(), q.double()).float()
    top = torch.topk(cs, topc, dim=-1).indices                    # [B,H,topc]
    ids = top.unsqueeze(-1) * clen + torch.arange(clen).view(1, 1, 1, clen)
    return ids.reshape(q.size(0), q.size(1), topc * clen), top, cs


def center_only_attention(q: Tensor, centers: Tensor, k: Tensor, v: Tensor, topc: int,
                          clen: int, sm_scale: float) -> Tuple[Tensor, Tensor]:
    """Centroid selection followed by attention over every member token of the chosen
    clusters (center_only_topk/baselines.cu:1477-1478 feeds the expanded ids to the
    gathered decode).  Returns (out fp32 [B,H,D], token ids [B,H,topc*clen])."""
    if q.dim() == 2:
        q = q.unsqueeze(0)
    ids, _, _ = center_only_topk(q, centers, topc, clen)
    return gathered_attention(q, k, v, ids, sm_scale), ids


def coarse_topk(q: Tensor, centers: Tensor, topc: int) -> Tensor:
    """Restates coarse_topk, baseline_1.py:71-79: fp32 ``einsum('hcd,hd->hc')`` then
    ``torch.topk(..., largest=True, sorted=True)``.  q [H,D], centers [H,CSZ,D]."""
    cs = torch.einsum("hcd,hd->hc", centers.float(), q.float())
    return torch.topk(cs, topc, dim=1, largest=True, sorted=True).indices.long()


def fine_topk(q: Tensor, k: Tensor, top_clusters: Tensor, clen: int,
              topk_per_cluster: int) -> Tensor:
    """Restates fine_topk, baseline_1.py:81-93, for the token-major cache [N,H,D] that
    the CUDA programs use (gemv_topk.cu:110): inside each chosen cluster keep the
    ``topk_per_cluster`` best tokens; ids are global ``c*clen + t``.  Returns
    [H, topc*topk_per_cluster] with one slice per cluster rank."""
    H, D = q.shape
    topc = top_clusters.size(1)
    kf = k.float().view(-1, clen, H, D)                            # [CSZ,clen,H,D]
    out = torch.empty(H, topc, topk_per_cluster, dtype=torch.long)
    for h in range(H):
        sel = kf[top_clusters[h], :, h, :]                         # [topc,clen,D]
        sc = (sel * q[h].float().view(1, 1, D)).sum(-1)
        ti = torch.topk(sc, topk_per_cluster, dim=-1, largest=True, sorted=True).indices
        out[h] = top_clusters[h].view(topc, 1) * clen + ti
    return out.view(H, topc * topk_per_cluster)


def two_level_indices(q: Tensor, centers: Tensor, k: Tensor, topc: int, clen: int,
                      topk_per_cluster: int) -> Tensor:
    """coarse_topk then fine_topk (baseline_1.py:136-140; gemv_topk.cu:75-135)."""
    return fine_topk(q, k, coarse_topk(q, centers, topc), clen, topk_per_cluster)


# --------------------------------------------------------------------------------------
# sequence-sharded variant (what G ranks compute together)
# --------------------------------------------------------------------------------------
def sharded_topk_attention(q: Tensor, k_shards: Sequence[Tensor], v_shards: Sequence[Tensor],
                           topk: int, sm_scale: float) -> Tuple[Tensor, Tensor, Tensor]:
    """The token axis is cut into contiguous shards.  Every shard proposes its local
    top-k (score, global id); the union is reduced to the global top-k; every shard mixes
    the V rows of the winners it owns into an un-normalised partial with its own maximum;
    partials are merged by ``lse_combine``.  The result must equal
    ``topk_sparse_attention`` on the concatenated cache; the reference has no multi-device
    code, so that equality is the definition.  Shards are [n_r, Hkv, D]."""
    B, Hq, D = q.shape
    G = len(k_shards)
    base, cs, ci = 0, [], []
    bases: List[int] = []
    for r in range(G):
        n = k_shards[r].size(0)
        kk = min(topk, n)
        s = full_scores(q, k_shards[r])
        ts, ti = torch.topk(s, kk, dim=-1)
        cs.append(ts)
        ci.append(ti + base)
        bases.append(base)
        base += n
    cand_s = torch.cat(cs, dim=-1)
    cand_i = torch.cat(ci, dim=-1)
    gs, pos = torch.topk(cand_s, topk, dim=-1)
    gi = torch.gather(cand_i, -1, pos)
    o_p = torch.zeros(G, B, Hq, D)
    m_p = torch.full((G, B, Hq), -math.inf)
    l_p = torch.zeros(G, B, Hq)
    for r in range(G):
        lo, hi = bases[r], bases[r] + k_shards[r].size(0)
        mine = (gi >= lo) & (gi < hi)
        x = torch.where(mine, gs * sm_scale, torch.full_like(gs, -math.inf))
        m = x.max(dim=-1).values
        e = torch.where(mine, torch.exp(x - m.unsqueeze(-1)), torch.zeros_like(x))
        e = torch.nan_to_num(e, nan=0.0)
        m_p[r], l_p[r] = m, e.sum(-1)
        loc = torch.where(mine, gi - lo, torch.zeros_like(gi))
        for b in range(B):
            vsel = _gather_rows(v_shards[r], b, Hq, loc[b])
            o_p[r, b] = torch.einsum("hs,hsd->hd", e[b], vsel)
    return lse_combine(o_p, m_p, l_p), gi, gs


def ordered_keys(scores: Tensor) -> Tensor:
    """fp32 scores -> the 32-bit keys (as int64) whose unsigned order is the scores' order: sign
    bit set for non-negative values, all bits flipped for negative ones."""
    u = scores.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return torch.where(u >= 0x80000000, 0xFFFFFFFF - u, u | 0x80000000)


def histogram_select_shard(keys: Tensor, k: int, rank: int, gather_counts) -> Tensor:
    """Which of this shard's tokens belong to the global top-k, found without moving any key or
    candidate: a radix select (11 + 11 + 10 bits) whose per-round histograms are the only thing
    the shards share.  keys int64 [R, n] (ordered_keys of the shard's scores); gather_counts(h) takes
    this shard's counts int64 [R, bins] and returns every shard's [world, R, bins], rank-major.
    A round's bin is split further while it holds more keys than are still wanted from it; at
    the end keys above the k-th key win, and of its copies each shard takes its share in rank
    order, inside a shard in token order -- the policy of a single device that keeps the lowest ids
    (shards hold ascending id ranges).  Returns a bool mask [R, n].  The sharded step's result is
    defined as the single-device operator's on the concatenated cache; this restates how the
    histogram route reaches it."""
    R, n = keys.shape
    lo = torch.zeros(R, dtype=torch.int64)
    rem = torch.full((R,), k, dtype=torch.int64)
    n_in = torch.full((R,), -1, dtype=torch.int64)
    ahead = torch.zeros(R, dtype=torch.int64)      # copies of the bin held by lower ranks
    shift = 32
    for bits in (11, 11, 10):
        active = n_in != rem
        if not bool(active.any()):
            break
        new_shift = shift - bits
        rel = keys - lo.unsqueeze(-1)
        inside = (rel >= 0) & (rel < (1 << shift)) & active.unsqueeze(-1)
        hist = torch.zeros(R, 1 << bits, dtype=torch.int64)
        hist.scatter_add_(1, torch.where(inside, rel >> new_shift, torch.zeros_like(rel)), inside.to(torch.int64))
        per_rank = gather_counts(hist)
        total = per_rank.sum(0)
        from_top = total.flip(-1).cumsum(-1)
        for r in range(R):
            if not bool(active[r]):
                continue
            if int(from_top[r, -1]) < int(rem[r]):      # fewer keys than wanted: everything wins
                n_in[r] = rem[r] = 0
                lo[r] = 0
                continue
            j = int((from_top[r] >= rem[r]).nonzero()[0])
            d = (1 << bits) - 1 - j
            above = int(from_top[r, j] - total[r, d])
            rem[r] -= above
            n_in[r] = total[r, d]
            ahead[r] = per_rank[:rank, r, d].sum()
            lo[r] += d << new_shift
        shift = new_shift
    win = keys > lo.unsqueeze(-1)
    for r in range(R):
        eq = keys[r] == lo[r] if n_in[r] != rem[r] else keys[r] >= lo[r]
        if n_in[r] == rem[r]:
            win[r] |= eq                                 # the whole bin wins
        else:
            quota = int(max(0, min(int(eq.sum()), int(rem[r] - ahead[r]))))
            pos = eq.nonzero().flatten()[:quota]         # token order
            win[r, pos] = True
    return win


# --------------------------------------------------------------------------------------
# the three acceptance checks
# --------------------------------------------------------------------------------------
def check_index_sets(scores: Tensor, got_idx: Tensor, topk: int, band: float = 1e-3,
                     num_segments: int = 1, index_base: int = 0) -> None:
    """Selected index sets must equal the oracle's except for keys whose score lies within
    ``band`` of the k-th score: every key scoring above (kth + band) must be present, no
    key scoring below (kth - band) may be, ids are unique, in range and exactly ``topk``
    per segment.  ``scores`` is the oracle's full [B,Hq,N] matrix."""
    B, Hq, N = scores.shape
    per = N // num_segments
    got = got_idx.long().reshape(B, Hq, num_segments, topk) - index_base
    sc = scores.view(B, Hq, num_segments, per)
    kth = torch.topk(sc, topk, dim=-1).values[..., -1:]            # [B,Hq,S,1]
    seg_lo = (torch.arange(num_segments) * per).view(1, 1, num_segments, 1)
    loc = got - seg_lo
    if not bool(((loc >= 0) & (loc < per)).all()):
        raise AssertionError("selected id outside its segment")
    srt = torch.sort(loc, dim=-1).values
    if topk > 1 and bool((srt[..., 1:] == srt[..., :-1]).any()):
        raise AssertionError("duplicate ids in a selection")
    sel_scores = torch.gather(sc, -1, loc)
    if bool((sel_scores < kth - band).any()):
        bad = (sel_scores < kth - band).sum().item()
        raise AssertionError(f"{bad} selected keys score below kth - band")
    must = sc > kth + band
    chosen = torch.zeros_like(must)
    chosen.scatter_(-1, loc, True)
    missing = (must & ~chosen).sum().item()
    if missing:
        raise AssertionError(f"{missing} keys above kth + band were not selected")


def check_topk_scores(scores: Tensor, got_idx: Tensor, got_scores: Tensor, topk: int,
                      tol: float = 1e-3, num_segments: int = 1, index_base: int = 0) -> None:
    """Top-k scores within ``tol``: each reported score matches the oracle score of the
    reported id, and the sorted score lists agree element-wise."""
    B, Hq, N = scores.shape
    per = N // num_segments
    idx = got_idx.long().reshape(B, Hq, -1) - index_base
    ref_at = torch.gather(scores, -1, idx)
    d = (ref_at - got_scores.float().reshape(B, Hq, -1)).abs().max().item()
    if d > tol:
        raise AssertionError(f"score of a selected key differs by {d}")
    ref_top = torch.topk(scores.view(B, Hq, num_segments, per), topk, dim=-1).values
    got_sorted = torch.sort(got_scores.float().reshape(B, Hq, num_segments, topk), dim=-1,
                            descending=True).values
    d = (ref_top - got_sorted).abs().max().item()
    if d > tol:
        raise AssertionError(f"sorted top-k scores differ by {d}")


def check_output(ref: Tensor, got: Tensor, rtol: float = 1e-2, atol: float = 1e-3) -> None:
    """Outputs within rtol 1e-2 / atol 1e-3 of the oracle."""
    ref = ref.float()
    got = got.float().cpu()
    err = (ref - got).abs()
    lim = atol + rtol * ref.abs()
    if bool((err > lim).any()):
        worst = (err - lim).max().item()
        raise AssertionError(f"output outside tolerance: max |diff| {err.max().item():.3e}, "
                             f"worst excess {worst:.3e}")
