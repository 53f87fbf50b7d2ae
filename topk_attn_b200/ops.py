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


def workspace(nbytes: int, device: torch.device) -> Tensor:
    """A cached, zero-initialised scratch buffer of at least ``nbytes`` on ``device`` (one per
    device and stream).  Allocation happens here, outside the C ABI, never per call."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream_ptr())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
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


def gemv_topk(q: Tensor, k: Tensor, topk: int, num_segments: int = 1, index_base: int = 0
              ) -> Tuple[Tensor, Tensor]:
    """Selection only: (indices int32, scores fp32) [B,Hq,S*topk], unordered inside a segment."""
    B, Hq, _ = q.shape
    idx = torch.empty(B, Hq, num_segments * topk, dtype=torch.int32, device=q.device)
    sc = torch.empty(B, Hq, num_segments * topk, dtype=torch.float32, device=q.device)
    p = _params(q, k, None, None, topk, 1.0, num_segments, index_base, idx, sc, None)
    capi.check(capi.lib().ra_gemv_topk(C.byref(p)))
    return idx, sc


def merge_attend(cand_scores: Tensor, cand_indices: Tensor, v: Tensor, topk: int, sm_scale: float,
                 own_base: int, partial: bool = True, return_indices: bool = False):
    """Select the global top-k out of ``cand_* [parts,B,Hq,topk]`` (global ids) and mix the V rows
    held in ``v`` (global ids own_base .. own_base+N).  Returns the fp32 partial [B,Hq,130]
    (128 un-normalised sums, weight, maximum) or, with ``partial=False``, the fp16 output."""
    parts, B, Hq, k = cand_scores.shape
    if cand_scores.dtype != torch.float32 or cand_indices.dtype != torch.int32:
        raise ValueError("candidates must be fp32 scores and int32 ids")
    if not (cand_scores.is_contiguous() and cand_indices.is_contiguous() and v.is_contiguous()):
        raise ValueError("tensors must be contiguous")
    N, Hkv = v.size(-3), v.size(-2)
    dev = cand_scores.device
    p = capi.RaMergeParams()
    p.cand_scores, p.cand_indices, p.num_parts = cand_scores.data_ptr(), cand_indices.data_ptr(), parts
    p.v = v.data_ptr()
    out = None
    if partial:
        out = torch.empty(B, Hq, 130, dtype=torch.float32, device=dev)
        p.out_partial = out.data_ptr()
    else:
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
    capi.check(capi.lib().ra_merge_attend(C.byref(p)))
    return (out, idx, sc) if return_indices else out


def lse_combine(partials: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """partials fp32 [parts, B, Hq, 130] -> fp16 [B, Hq, 128]."""
    parts, B, Hq, w = partials.shape
    if w != 130 or partials.dtype != torch.float32 or not partials.is_contiguous():
        raise ValueError("partials must be contiguous fp32 [parts, B, Hq, 130]")
    if out is None:
        out = torch.empty(B, Hq, 128, dtype=torch.float16, device=partials.device)
    capi.check(capi.lib().ra_lse_combine(partials.data_ptr(), parts, B * Hq, out.data_ptr(),
                                         _stream_ptr()))
    return out


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise the current stream and raise if a kernel abandoned a bounded wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    ws = workspace(256, dev)
    capi.check(capi.lib().ra_check_status(ws.data_ptr(), _stream_ptr()))
