"""Sequence-sharded decode step: one process per GPU, the token axis cut contiguously over ranks.

Per step every rank
  1. scans its shard and proposes its local top-k (score, global id) per (batch row, head);
  2. all-gathers the proposals (k*8 bytes per head and rank — latency-, not bandwidth-bound);
  3. selects the global top-k out of the G*k proposals (every rank computes the same set) and mixes
     the V rows it owns into an un-normalised partial with the common maximum;
  4. all-gathers the partials (130 floats per head and rank);
  5. combines them through their log-sum-exp.  Every rank ends with the full output.

The reference has no multi-device code; the result is defined as equal to the single-device
operator on the concatenated cache.  Collectives go through ``torch.distributed`` (NCCL on GPUs,
gloo in the CPU tests); the compute steps go through the C ABI (``CudaBackend``).  The class only
orchestrates, so the same logic runs in CPU tests with a stand-in backend.
"""
from __future__ import annotations

import json
import os
import time
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor


def _all_gather(out: Tensor, piece: Tensor, group=None) -> None:
    """out [world, *piece.shape] <- every rank's piece (rank-major), one collective."""
    dist.all_gather_into_tensor(out.view(-1, *piece.shape[1:]), piece, group=group)


class CudaBackend:
    """The three compute steps on the local GPU through the C ABI."""

    def select(self, q: Tensor, k: Tensor, topk: int, index_base: int, out=None):
        from . import ops
        return ops.gemv_topk(q, k, topk, index_base=index_base, out=out)

    def merge_partial(self, cand_sc: Tensor, cand_idx: Tensor, v: Tensor, topk: int,
                      sm_scale: float, own_base: int) -> Tensor:
        from . import ops
        return ops.merge_attend(cand_sc, cand_idx, v, topk, sm_scale, own_base, partial=True)

    def combine(self, partials: Tensor) -> Tensor:
        from . import ops
        return ops.lse_combine(partials)


class ShardedTopkAttention:
    def __init__(self, topk: int, sm_scale: float = 1.0, group=None, backend=None):
        self.topk, self.sm_scale, self.group = topk, sm_scale, group
        self.backend = backend if backend is not None else CudaBackend()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._recv = self._send = self._partials = None

    def _buffers(self, B: int, Hq: int, device):
        """Scores and ids of one rank are the two halves of one int32 buffer, so that a single
        all-gather moves both: recv [world, 2, B, Hq, k], send [2, B, Hq, k]."""
        shape = (self.world, 2, B, Hq, self.topk)
        if self._recv is None or self._recv.shape != shape or self._recv.device != device:
            self._recv = torch.empty(shape, dtype=torch.int32, device=device)
            self._send = torch.empty(shape[1:], dtype=torch.int32, device=device)
            self._partials = torch.empty(self.world, B, Hq, 130, dtype=torch.float32, device=device)
        cand_sc = self._recv[:, 0].view(torch.float32)
        cand_idx = self._recv[:, 1]
        return cand_sc, cand_idx, self._partials

    def local_candidates(self, q: Tensor, k: Tensor, index_base: int):
        """Local top-k of this shard, padded with (-inf, -1) when the shard holds fewer than k
        tokens."""
        n = k.size(-3)
        kk = min(self.topk, n)
        if kk == self.topk and self._send is not None and self._send.shape[1:3] == q.shape[:2]:
            # write straight into the send halves
            return self.backend.select(q, k, kk, index_base,
                                       out=(self._send[1], self._send[0].view(torch.float32)))
        idx, sc = self.backend.select(q, k, kk, index_base)
        if kk < self.topk:
            pad = self.topk - kk
            idx = torch.cat([idx, torch.full_like(idx[..., :1], -1).expand(-1, -1, pad)], -1).contiguous()
            sc = torch.cat([sc, torch.full_like(sc[..., :1], float("-inf")).expand(-1, -1, pad)], -1).contiguous()
        return idx, sc

    def step(self, q: Tensor, k: Tensor, v: Tensor, index_base: Optional[int] = None) -> Tensor:
        """q [B,Hq,128] (identical on every rank); k, v this rank's shard.  ``index_base`` is the
        global id of the shard's first token (default rank * shard length)."""
        B, Hq, _ = q.shape
        n = k.size(-3)
        if index_base is None:
            index_base = self.rank * n
        cand_sc, cand_idx, partials = self._buffers(B, Hq, q.device)
        idx, sc = self.local_candidates(q, k, index_base)
        self.exchange_candidates(idx, sc)
        part = self.backend.merge_partial(cand_sc, cand_idx, v, self.topk, self.sm_scale, index_base)
        if self.world > 1:
            _all_gather(partials, part, self.group)
        else:
            partials[0].copy_(part)
        return self.backend.combine(partials)


def _exchange(self, idx: Tensor, sc: Tensor) -> None:
    """All ranks' (score, id) proposals into the receive buffer with one collective."""
    if idx.data_ptr() != self._send[1].data_ptr():
        self._send[1].copy_(idx)
        self._send[0].view(torch.float32).copy_(sc)
    if self.world > 1:
        _all_gather(self._recv, self._send, self.group)
    else:
        self._recv[0].copy_(self._send)


ShardedTopkAttention.exchange_candidates = _exchange


def bench(args, rank: int, local: int, world: int, ClockSampler, measured_peak_gbs) -> None:
    """`bench.py --gpus N` for N > 1: weak scaling, every rank holds a 131072-token shard of each
    of the 4 sequences (32 heads, k = 2048).  Timed on the device, max over ranks."""
    from . import ops, workloads as W
    dev = torch.device("cuda", local)
    strong = args.workload == "cfg4"
    if strong:
        # configuration 4: 1 048 576 tokens in total (32 query / 8 kv heads, k = 4096) cut over the
        # ranks, so the work per rank shrinks as ranks are added
        w = W.sharded_long_context_shard(rank, world, device=dev)
    else:
        w = W.fused_topk_128k_shard(rank, world, device=dev)
    q, k, v = w.q, w.k, w.v
    op = ShardedTopkAttention(w.topk, w.sm_scale)
    n_local = w.n_tokens

    def step():
        return op.step(q, k, v)

    for _ in range(max(args.warmup, 3)):
        step()
    ops.check_status(dev)
    sampler = ClockSampler(local)
    dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sel = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(args.steps)]
    from . import capi
    launches0 = capi.lib().ra_launch_count()
    e0.record()
    for i in range(args.steps):
        # the scan is the dominant kernel: time it separately inside the step
        B, Hq, _ = q.shape
        cand_sc, cand_idx, partials = op._buffers(B, Hq, dev)
        sel[i][0].record()
        idx, sc = op.local_candidates(q, k, rank * n_local)
        sel[i][1].record()
        op.exchange_candidates(idx, sc)
        part = op.backend.merge_partial(cand_sc, cand_idx, v, op.topk, op.sm_scale, rank * n_local)
        _all_gather(partials, part)
        op.backend.combine(partials)
    e1.record()
    launches = capi.lib().ra_launch_count() - launches0      # this rank's, in the timed region
    torch.cuda.synchronize()
    dist.barrier()
    clocks = sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    per_ms = t.item() / args.steps
    scan_ms = sum(a.elapsed_time(b) for a, b in sel) / args.steps
    ops.check_status(dev)

    q_host = q.cpu().pin_memory()
    out_host = torch.empty_like(q_host).pin_memory()
    q_dev = torch.empty_like(q)

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        o = op.step(q_dev, k, v)
        out_host.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    te = torch.tensor([(time.perf_counter() - t0) / args.steps], device=dev)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_s = te.item()

    if rank == 0:
        tokens = world * w.batch * n_local
        peak, kind = measured_peak_gbs()
        alg = w.algorithmic_bytes()
        achieved = alg / (scan_ms * 1e-3) / 1e9
        line = {
            "metric": "tokens_scanned_per_s", "value": tokens / (per_ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": per_ms, "us_per_step": per_ms * 1e3, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f16 inputs, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": "cfg4 token-sharded" if strong else "cfg2 token-sharded", "batch": w.batch, "heads_q": q.size(1),
                       "heads_kv": k.size(-2), "head_dim": 128, "context": world * n_local,
                       "context_per_gpu": n_local, "topk": w.topk, "caches": w.bkv,
                       "l2": "inputs_exceed_l2", "collectives": "nccl all_gather x2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": kind + " (burst copy)",
                         "algorithmic_bytes": alg, "traffic": None,
                         "kernel": "scan_select_kernel (per rank)", "scan_us": scan_ms * 1e3},
            "cpu_baseline": None,
            "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "us_per_step": e2e_s * 1e6,
                    "h2d_bytes_per_step": q_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": launches * world,
            "clocks": clocks,
        }
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
