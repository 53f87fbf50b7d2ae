"""Operators on torch CUDA tensors, forwarding to the C ABI on torch's current stream.

torch is used for device memory and streams only; every operator launches the library's own
sm_100a kernels.  Layouts are the reference's: q [B,Hq,128], k/v [N,Hkv,128] (shared cache) or
[B,N,Hkv,128] (one cache per batch row), out [B,Hq,128], all fp16 and contiguous.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch
from torch import Tensor

from . import capi

_workspaces: Dict[Tuple[int, int], Tensor] = {}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_retired = []


def workspace(nbytes: int, device: torch.device) -> Tensor:
    """A cached, zero-initialised scratch buffer of at least ``nbytes`` on ``device`` (one per
    device and stream).  Allocation happens here, outside the C ABI, never per call.  When a
    larger buffer replaces a smaller one it inherits the status block (the sticky bits kernels set)
    in stream order, and the old buffer is kept alive because launches in flight may still use it."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream_ptr())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        new = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        if ws is not None:
            new[:256].copy_(ws[:256])
            _retired.append(ws)
        _workspaces[key] = ws = new
    return ws


def _check_qkv(q: Tensor, k: Tensor, v: Optional[Tensor]) -> Tuple[int, int, int, int, int]:
    if not q.is_cuda:
        raise ValueError("tensors must be CUDA tensors")
    for t in (q, k) + ((v,) if v is not None else ()):
        if t.dtype != torch.float16 or not t.is_contiguous() or t.device != q.device:
            raise ValueError("q, k, v must be contiguous fp16 tensors on one device")
    if q.dim() != 3 or q.size(2) != 128:
        raise ValueError("q must be [B, Hq, 128]")
    if k.dim() not in (3, 4) or k.size(-1) != 128 or (v is not None and v.shape != k.shape):
        raise ValueError("k, v must be [N,Hkv,128] or [B,N,Hkv,128] with equal shapes")
    B, Hq, _ = q.shape
    N, Hkv = k.size(-3), k.size(-2)
    if k.dim() == 4 and k.size(0) != B:
        raise ValueError("per-sequence cache needs k.size(0) == batch")
    return B, Hq, Hkv, N, (N * Hkv * 128 if k.dim() == 4 else 0)


def _params(q, k, v, out, topk, sm_scale, num_segments, index_base, out_indices, out_scores,
            out_lse) -> capi.RaParams:
    B, Hq, Hkv, N, bstride = _check_qkv(q, k, v)
    p = capi.RaParams()
    p.q, p.k = q.data_ptr(), k.data_ptr()
    p.v = v.data_ptr() if v is not None else None
    p.out = out.data_ptr() if out is not None else None
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.num_tokens = B, Hq, Hkv, 128, N
    p.kv_batch_stride, p.kv_token_stride, p.kv_head_stride = bstride, Hkv * 128, 128
    p.topk, p.num_segments, p.sm_scale, p.index_base = topk, num_segments, sm_scale, index_base
    p.out_indices = out_indices.data_ptr() if out_indices is not None else None
    p.out_scores = out_scores.data_ptr() if out_scores is not None else None
    p.out_lse = out_lse.data_ptr() if out_lse is not None else None
    need = capi.lib().ra_workspace_bytes(C.byref(p))
    if need == 0:
        # let the entry point report what is wrong with the shape
        need = 256
    ws = workspace(need, q.device)
    p.workspace, p.workspace_bytes, p.stream = ws.data_ptr(), ws.numel(), _stream_ptr()
    return p


def topk_attention(q: Tensor, k: Tensor, v: Tensor, topk: int, sm_scale: float = 1.0,
                   num_segments: int = 1, index_base: int = 0, out: Optional[Tensor] = None,
                   return_indices: bool = False, return_lse: bool = False):
    """Fused decode step: exact top-k of q.K^T per (batch row, head[, segment]), softmax over the
    kept keys, mix of their V rows.  Returns out [B,Hq,128] fp16, and on request
    (indices int32 [B,Hq,S*topk], scores fp32 [B,Hq,S*topk]) and lse fp32 [B,Hq,2]."""
    B, Hq, _ = q.shape
    if out is None:
        out = torch.empty_like(q)
    idx = sc = lse = None
    if return_indices:
        idx = torch.empty(B, Hq, num_segments * topk, dtype=torch.int32, device=q.device)
        sc = torch.empty(B, Hq, num_segments * topk, dtype=torch.float32, device=q.device)
    if return_lse:
        lse = torch.empty(B, Hq, 2, dtype=torch.float32, device=q.device)
    p = _params(q, k, v, out, topk, sm_scale, num_segments, index_base, idx, sc, lse)
    capi.check(capi.lib().ra_topk_attention(C.byref(p)))
    res = (out,)
    if return_indices:
        res += (idx, sc)
    if return_lse:
        res += (lse,)
    return res[0] if len(res) == 1 else res


def gemv_topk(q: Tensor, k: Tensor, topk: int, num_segments: int = 1, index_base: int = 0,
              out: Optional[Tuple[Tensor, Tensor]] = None) -> Tuple[Tensor, Tensor]:
    """Selection only: (indices int32, scores fp32) [B,Hq,S*topk], unordered inside a segment.
    ``out`` may give the two (contiguous) destination tensors."""
    B, Hq, _ = q.shape
    if out is not None:
        idx, sc = out
        if idx.dtype != torch.int32 or sc.dtype != torch.float32 or not idx.is_contiguous() \
                or not sc.is_contiguous() or idx.shape != (B, Hq, num_segments * topk) \
                or sc.shape != idx.shape:
            raise ValueError("out must be contiguous (int32, fp32) [B,Hq,S*topk]")
    else:
        idx = torch.empty(B, Hq, num_segments * topk, dtype=torch.int32, device=q.device)
        sc = torch.empty(B, Hq, num_segments * topk, dtype=torch.float32, device=q.device)
    p = _params(q, k, None, None, topk, 1.0, num_segments, index_base, idx, sc, None)
    capi.check(capi.lib().ra_gemv_topk(C.byref(p)))
    return idx, sc


def flash_decoding(q: Tensor, k: Tensor, v: Tensor, sm_scale: float, num_splits: int = 0,
                   out: Optional[Tensor] = None) -> Tensor:
    """Dense decode attention over the whole cache (split-KV + log-sum-exp combine)."""
    B, Hq, Hkv, N, bstride = _check_qkv(q, k, v)
    if out is None:
        out = torch.empty_like(q)
    p = capi.RaDenseParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.num_tokens = B, Hq, Hkv, 128, N
    p.kv_batch_stride, p.kv_token_stride, p.kv_head_stride = bstride, Hkv * 128, 128
    p.sm_scale, p.num_splits = sm_scale, num_splits
    need = capi.lib().ra_flash_workspace_bytes(B, Hq, Hkv, N, num_splits)
    ws = workspace(max(need, 256), q.device)
    p.workspace, p.workspace_bytes, p.stream = ws.data_ptr(), ws.numel(), _stream_ptr()
    capi.check(capi.lib().ra_flash_decoding(C.byref(p)))
    return out


def gathered_attention(q: Tensor, k: Tensor, v: Tensor, indices: Tensor, sm_scale: float,
                       out: Optional[Tensor] = None) -> Tensor:
    """softmax(sm_scale * q.K[id]) . V[id] over ``indices`` int32 [Hq,S] (shared by the batch) or
    [B,Hq,S].  Returns fp16 [B,Hq,128]."""
    B, Hq, Hkv, N, bstride = _check_qkv(q, k, v)
    if indices.dtype != torch.int32 or not indices.is_contiguous() or indices.device != q.device:
        raise ValueError("indices must be a contiguous int32 tensor on the device of q")
    if indices.dim() == 2:
        ib, S = 0, indices.size(1)
        ok = indices.size(0) == Hq
    else:
        ib, S = Hq * indices.size(2), indices.size(2)
        ok = indices.shape[:2] == (B, Hq)
    if not ok:
        raise ValueError("indices must be [Hq,S] or [B,Hq,S]")
    if out is None:
        out = torch.empty_like(q)
    p = capi.RaGatherParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.num_tokens = B, Hq, Hkv, 128, N
    p.kv_batch_stride, p.kv_token_stride, p.kv_head_stride = bstride, Hkv * 128, 128
    p.indices, p.num_indices, p.indices_batch_stride = indices.data_ptr(), S, ib
    p.sm_scale = sm_scale
    ws = workspace(256, q.device)
    p.workspace, p.workspace_bytes, p.stream = ws.data_ptr(), ws.numel(), _stream_ptr()
    capi.check(capi.lib().ra_gathered_attention(C.byref(p)))
    return out


def center_only_topk(q: Tensor, centers: Tensor, top_clusters: int, cluster_len: int,
                     k: Optional[Tensor] = None, v: Optional[Tensor] = None, sm_scale: float = 1.0,
                     return_indices: bool = True, out: Optional[Tensor] = None):
    """Centroid-only retrieval.  q [B,H,128], centers [H,CSZ,128].  Returns
    (cluster_ids int32 [B,H,TOPC] unordered, token_ids int32 [B,H,TOPC*CLEN] in descending order
    of the centroid scores[, out fp16 [B,H,128] when k and v are given])."""
    if q.dim() != 3 or centers.dim() != 3 or centers.size(0) != q.size(1) or centers.size(2) != 128:
        raise ValueError("q must be [B,H,128] and centers [H,CSZ,128]")
    for t in (q, centers):
        if t.dtype != torch.float16 or not t.is_contiguous() or not t.is_cuda:
            raise ValueError("q and centers must be contiguous fp16 CUDA tensors")
    B, H, _ = q.shape
    csz = centers.size(1)
    dev = q.device
    p = capi.RaCenterParams()
    p.q, p.centers = q.data_ptr(), centers.data_ptr()
    p.batch, p.num_heads, p.head_dim = B, H, 128
    p.num_centers, p.cluster_len, p.top_clusters = csz, cluster_len, top_clusters
    cids = torch.empty(B, H, top_clusters, dtype=torch.int32, device=dev)
    p.out_cluster_ids = cids.data_ptr()
    tids = None
    out_given = out
    if return_indices:
        tids = torch.empty(B, H, top_clusters * cluster_len, dtype=torch.int32, device=dev)
        p.out_indices = tids.data_ptr()
    out = out_given if k is not None else None
    if k is not None:
        _, _, Hkv, N, bstride = _check_qkv(q, k, v)
        if Hkv != H:
            raise ValueError("centroid retrieval needs one kv head per query head")
        if out is None:
            out = torch.empty_like(q)
        p.k, p.v, p.out, p.num_tokens = k.data_ptr(), v.data_ptr(), out.data_ptr(), N
        p.kv_batch_stride, p.kv_token_stride, p.kv_head_stride = bstride, Hkv * 128, 128
    p.sm_scale = sm_scale
    need = capi.lib().ra_center_workspace_bytes(B, H, csz, top_clusters)
    ws = workspace(max(need, 256), dev)
    p.workspace, p.workspace_bytes, p.stream = ws.data_ptr(), ws.numel(), _stream_ptr()
    capi.check(capi.lib().ra_center_only_topk(C.byref(p)))
    res = (cids, tids)
    return res + (out,) if out is not None else res


def two_level_topk(q: Tensor, centers: Tensor, k: Tensor, top_clusters: int, cluster_len: int,
                   topk_per_cluster: int, v: Optional[Tensor] = None, sm_scale: float = 1.0):
    """Two-level retrieval.  Returns (cluster_ids int32 [B,H,TOPC] in rank order, indices int32
    [B,H,TOPC*K] one slice per cluster rank, scores fp32 of the same shape[, out fp16 [B,H,128]
    when ``v`` is given])."""
    B, H, Hkv, N, bstride = _check_qkv(q, k, v)
    if Hkv != H or centers.dim() != 3 or centers.size(0) != H or centers.size(2) != 128 \
            or centers.dtype != torch.float16 or not centers.is_contiguous():
        raise ValueError("two-level retrieval needs MHA caches and fp16 centers [H,CSZ,128]")
    dev = q.device
    p = capi.RaTwoLevelParams()
    p.q, p.centers, p.k = q.data_ptr(), centers.data_ptr(), k.data_ptr()
    p.batch, p.num_heads, p.head_dim = B, H, 128
    p.num_centers, p.cluster_len = centers.size(1), cluster_len
    p.top_clusters, p.topk_per_cluster, p.num_tokens = top_clusters, topk_per_cluster, N
    p.kv_batch_stride, p.kv_token_stride, p.kv_head_stride = bstride, H * 128, 128
    p.sm_scale = sm_scale
    cids = torch.empty(B, H, top_clusters, dtype=torch.int32, device=dev)
    idx = torch.empty(B, H, top_clusters * topk_per_cluster, dtype=torch.int32, device=dev)
    sc = torch.empty(B, H, top_clusters * topk_per_cluster, dtype=torch.float32, device=dev)
    p.out_cluster_ids, p.out_indices, p.out_scores = cids.data_ptr(), idx.data_ptr(), sc.data_ptr()
    out = None
    if v is not None:
        out = torch.empty_like(q)
        p.v, p.out = v.data_ptr(), out.data_ptr()
    need = capi.lib().ra_two_level_workspace_bytes(B, H, centers.size(1), top_clusters,
                                                  topk_per_cluster)
    ws = workspace(max(need, 256), dev)
    p.workspace, p.workspace_bytes, p.stream = ws.data_ptr(), ws.numel(), _stream_ptr()
    capi.check(capi.lib().ra_two_level_topk(C.byref(p)))
    return (cids, idx, sc) + ((out,) if out is not None else ())


def kv_append(k_cache: Tensor, v_cache: Tensor, new_k: Tensor, new_v: Tensor, position: int,
              centers: Optional[Tensor] = None, cluster_len: int = 0) -> None:
    """In place: caches[.., position, :, :] = new rows ([Hkv,128] for a shared cache, [B,Hkv,128]
    for per-sequence caches) and, with ``centers`` [Hkv,CSZ,128], the running mean of centroid
    position // cluster_len absorbs the key."""
    per_batch = k_cache.dim() == 4
    caches = k_cache.size(0) if per_batch else 1
    N, Hkv = k_cache.size(-3), k_cache.size(-2)
    want = (caches, Hkv, 128) if per_batch else (Hkv, 128)
    for t in (k_cache, v_cache, new_k, new_v):
        if t.dtype != torch.float16 or not t.is_contiguous() or not t.is_cuda:
            raise ValueError("caches and rows must be contiguous fp16 CUDA tensors")
    if tuple(new_k.shape) != want or new_v.shape != new_k.shape or v_cache.shape != k_cache.shape:
        raise ValueError(f"new rows must be {want}")
    cptr, csz = (None, 0)
    if centers is not None:
        if centers.dtype != torch.float16 or not centers.is_contiguous() or centers.size(0) != Hkv:
            raise ValueError("centers must be contiguous fp16 [Hkv,CSZ,128]")
        cptr, csz = centers.data_ptr(), centers.size(1)
    capi.check(capi.lib().ra_kv_append(
        k_cache.data_ptr(), v_cache.data_ptr(), new_k.data_ptr(), new_v.data_ptr(), caches, Hkv, 128,
        position, N, N * Hkv * 128 if per_batch else 0, Hkv * 128, 128, cptr, csz, cluster_len,
        _stream_ptr()))


def merge_attend(cand_scores: Tensor, cand_indices: Tensor, v: Tensor, topk: int, sm_scale: float,
                 own_base: int, partial: bool = True, return_indices: bool = False,
                 out: Optional[Tensor] = None, exchange=None, own_part: Optional[int] = None):
    """Select the global top-k out of ``cand_* [parts,B,Hq,topk]`` (global ids) and mix the V rows
    held in ``v`` (global ids own_base .. own_base+N).  Returns the fp32 partial [B,Hq,130]
    (128 un-normalised sums, weight, maximum) or, with ``partial=False``, the fp16 output."""
    parts, B, Hq, k = cand_scores.shape
    if cand_scores.dtype != torch.float32 or cand_indices.dtype != torch.int32:
        raise ValueError("candidates must be fp32 scores and int32 ids")
    dense = (B * Hq * k, Hq * k, k, 1)
    st = cand_scores.stride()
    if cand_indices.stride() != st or st[1:] != dense[1:] or not v.is_contiguous():
        raise ValueError("candidates must be dense per part with equal strides; v contiguous")
    N, Hkv = v.size(-3), v.size(-2)
    dev = cand_scores.device
    p = capi.RaMergeParams()
    p.cand_scores, p.cand_indices, p.num_parts = cand_scores.data_ptr(), cand_indices.data_ptr(), parts
    p.cand_part_stride = st[0]
    p.v = v.data_ptr()
    if partial:
        if out is None:
            out = torch.empty(B, Hq, 130, dtype=torch.float32, device=dev)
        elif out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (B, Hq, 130):
            raise ValueError("out must be a contiguous fp32 [B,Hq,130] tensor")
        p.out_partial = out.data_ptr()
    else:
        if out is None:
            out = torch.empty(B, Hq, 128, dtype=torch.float16, device=dev)
        p.out = out.data_ptr()
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.num_tokens = B, Hq, Hkv, 128, N
    p.kv_batch_stride = N * Hkv * 128 if v.dim() == 4 else 0
    p.kv_token_stride, p.kv_head_stride = Hkv * 128, 128
    p.topk, p.sm_scale, p.own_base = topk, sm_scale, own_base
    idx = sc = None
    if return_indices:
        idx = torch.empty(B, Hq, topk, dtype=torch.int32, device=dev)
        sc = torch.empty(B, Hq, topk, dtype=torch.float32, device=dev)
        p.out_indices, p.out_scores = idx.data_ptr(), sc.data_ptr()
    ws = workspace(256, dev)
    p.workspace, p.workspace_bytes, p.stream = ws.data_ptr(), ws.numel(), _stream_ptr()
    if own_part is not None:
        # only part `own_part` carries ids (the ranks exchanged scores only)
        p.own_part_only, p.own_part = 1, own_part
    if exchange is not None:
        # exchange: an object with the fields of sharded.PeerExchange -- the merge waits for the
        # candidate flags itself and pushes its partial rows to the peers
        if not partial:
            raise ValueError("the fused exchange works on partial outputs")
        n = len(exchange.dst_p)
        arr = C.c_void_p * n
        h = capi.RaExchangeHooks()
        h.wait_flags, h.num_wait_flags = exchange.flags_c.data_ptr(), exchange.flags_c.numel()
        h.epoch, h.wait_timeout_ns = exchange.epoch.data_ptr(), int(exchange.timeout_s * 1e9)
        keep = (arr(*exchange.dst_p), arr(*exchange.flg_p))
        h.peer_partials = C.cast(keep[0], C.POINTER(C.c_void_p))
        h.peer_flags = C.cast(keep[1], C.POINTER(C.c_void_p))
        h.num_peers, h.done_counter = n, exchange.done[1:2].data_ptr()
        p.exchange = C.pointer(h)
    capi.check(capi.lib().ra_merge_attend(C.byref(p)))
    return (out, idx, sc) if return_indices else out


def stored_scores_probe(q: Tensor, k: Tensor, topk: int) -> None:
    """The scoring pass of the stored-score route alone (a measuring aid)."""
    p = _params(q, k, None, None, topk, 1.0, 1, 0, None, None, None)
    capi.check(capi.lib().ra_score_store_probe(C.byref(p)))


def sharded_topk_attention(q: Tensor, k: Tensor, v: Tensor, topk: int, sm_scale: float, index_base: int,
                           exchange, out: Optional[Tensor] = None, return_indices: bool = False):
    """One rank's call of a sequence-sharded step by exchanged histograms: scores the shard, finds
    the global k-th score together with the other ranks, mixes the winners among the shard's
    tokens, exchanges the partials and writes the full output [B,Hq,128] fp16.  ``exchange`` has the
    fields of sharded.HistExchange.  With ``return_indices`` also gives (ids int32, scores fp32)
    [B,Hq,topk] of this rank's winners, padded with (-1, -inf)."""
    B, Hq, _ = q.shape
    if out is None:
        out = torch.empty_like(q)
    idx = sc = None
    if return_indices:
        idx = torch.full((B, Hq, topk), -1, dtype=torch.int32, device=q.device)
        sc = torch.full((B, Hq, topk), float("-inf"), dtype=torch.float32, device=q.device)
    p = _params(q, k, v, out, topk, sm_scale, 1, index_base, idx, sc, None)
    n = exchange.world
    keep = (C.c_void_p * n)(*exchange.ll_ptrs)
    x = capi.RaShardExchange()
    x.world, x.rank = n, exchange.rank
    x.bufs = C.cast(keep, C.POINTER(C.c_void_p))
    x.epoch, x.wait_timeout_ns = exchange.epoch.data_ptr(), int(exchange.timeout_s * 1e9)
    x.done_counter = exchange.done[2:3].data_ptr()
    capi.check(capi.lib().ra_sharded_topk_attention(C.byref(p), C.byref(x)))
    return (out, idx, sc) if return_indices else out


def lse_combine(partials: Tensor, out: Optional[Tensor] = None, exchange=None) -> Tensor:
    """partials fp32 [parts, B, Hq, 130] -> fp16 [B, Hq, 128].  With ``exchange`` (the fields of
    sharded.PeerExchange) the kernel first waits for every rank's partial flag and ends the step
    by advancing the epoch."""
    parts, B, Hq, w = partials.shape
    if w != 130 or partials.dtype != torch.float32 or not partials.is_contiguous():
        raise ValueError("partials must be contiguous fp32 [parts, B, Hq, 130]")
    if out is None:
        out = torch.empty(B, Hq, 128, dtype=torch.float16, device=partials.device)
    if exchange is not None:
        ws = workspace(256, partials.device)
        capi.check(capi.lib().ra_lse_combine_wait(
            partials.data_ptr(), parts, B * Hq, out.data_ptr(), exchange.flags_p.data_ptr(),
            exchange.flags_p.numel(), exchange.epoch.data_ptr(), int(exchange.timeout_s * 1e9),
            exchange.done[2:3].data_ptr(), ws.data_ptr(), _stream_ptr()))
        return out
    capi.check(capi.lib().ra_lse_combine(partials.data_ptr(), parts, B * Hq, out.data_ptr(),
                                         _stream_ptr()))
    return out


def stream_read_probe(buf: Tensor) -> None:
    """Enqueue one kernel that only reads ``buf`` (a measuring aid: time it over a buffer much larger
    than L2 to get the device's read-only streaming rate)."""
    nbytes = buf.numel() * buf.element_size() // 16 * 16
    sink = workspace(256, buf.device)
    capi.check(capi.lib().ra_stream_read_probe(buf.data_ptr(), nbytes, sink.data_ptr() + 128, _stream_ptr()))


def l2_persist(cache: Optional[Tensor], hit_ratio: float = 1.0) -> None:
    """Mark ``cache`` (a key cache shared by the batch, up to roughly the L2 size) as persisting in
    L2 for the kernels launched into the current stream from now on, so that consecutive decode
    steps re-read it from L2; ``None`` removes the window."""
    if cache is None:
        capi.check(capi.lib().ra_l2_persist(None, 0, 1.0, _stream_ptr()))
        return
    capi.check(capi.lib().ra_l2_persist(cache.data_ptr(), cache.numel() * cache.element_size(),
                                        hit_ratio, _stream_ptr()))


def exchange_push(src: Tensor, peer_dst, peer_flags, epoch: Tensor, done: Tensor) -> None:
    """Store the contiguous tensor ``src`` (a multiple of 16 bytes) into the slots ``peer_dst``
    (device addresses as ints, one per rank; the own slot may be ``src`` itself) and then the epoch
    word into ``peer_flags`` (this rank's flag word on every rank).  Plain stores over peer-mapped
    memory, enqueued on the current stream."""
    n = len(peer_dst)
    if n != len(peer_flags) or not src.is_contiguous():
        raise ValueError("one slot and one flag per rank; src contiguous")
    arr = C.c_void_p * n
    capi.check(capi.lib().ra_exchange_push(src.data_ptr(), src.numel() * src.element_size(),
                                           arr(*peer_dst), arr(*peer_flags), n, epoch.data_ptr(),
                                           done.data_ptr(), _stream_ptr()))


def exchange_wait(flags: Tensor, epoch: Tensor, advance: bool, timeout_s: float = 2.0) -> None:
    """Make the current stream wait until every word of ``flags`` (int32, one per rank) has reached
    the epoch; a wait that outlasts ``timeout_s`` is reported by ``check_status``.  With ``advance``
    the epoch word is incremented afterwards."""
    ws = workspace(256, flags.device)
    capi.check(capi.lib().ra_exchange_wait(flags.data_ptr(), flags.numel(), epoch.data_ptr(),
                                           1 if advance else 0, int(timeout_s * 1e9), ws.data_ptr(),
                                           _stream_ptr()))


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise the current stream and raise if a kernel abandoned a bounded wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    ws = workspace(256, dev)
    capi.check(capi.lib().ra_check_status(ws.data_ptr(), _stream_ptr()))
