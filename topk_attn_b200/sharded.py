"""Sequence-sharded decode step: one process per GPU, the token axis cut contiguously over ranks.

Per step every rank
  1. scans its shard and proposes its local top-k (score, global id) per (batch row, head);
  2. all-gathers the proposals (k*8 bytes per head and rank — latency-, not bandwidth-bound);
  3. selects the global top-k out of the G*k proposals (every rank computes the same set) and mixes
     the V rows it owns into an un-normalised partial with the common maximum;
  4. all-gathers the partials (130 floats per head and rank);
  5. combines them through their log-sum-exp.  Every rank ends with the full output.

The reference has no multi-device code; the result is defined as equal to the single-device
operator on the concatenated cache.  The two exchanges (steps 2 and 4) run in one of two ways:

* as collectives of ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests), or
* with the library's own kernels over peer-mapped memory (``PeerExchange``): every rank stores its
  piece straight into its slot of every peer's receive buffer with plain stores and raises a flag
  there; the consumer's stream waits for the flags of all ranks, each wait bounded in time.  The
  whole step is then kernels on one stream and can be replayed as one CUDA graph.

The compute steps go through the C ABI (``CudaBackend``).  The class only orchestrates, so the same
logic runs in CPU tests with a stand-in backend.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import List, Optional

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
                      sm_scale: float, own_base: int, out: Optional[Tensor] = None,
                      exchange=None, own_part: Optional[int] = None) -> Tensor:
        from . import ops
        return ops.merge_attend(cand_sc, cand_idx, v, topk, sm_scale, own_base, partial=True, out=out,
                                exchange=exchange, own_part=own_part)

    def combine(self, partials: Tensor, exchange=None) -> Tensor:
        from . import ops
        return ops.lse_combine(partials, exchange=exchange)

    def sharded_attention(self, q: Tensor, k: Tensor, v: Tensor, topk: int, sm_scale: float,
                          index_base: int, exchange, return_indices: bool = False):
        from . import ops
        return ops.sharded_topk_attention(q, k, v, topk, sm_scale, index_base, exchange,
                                          return_indices=return_indices)


class PeerExchange:
    """Receive buffers of one rank for the two exchanges of a step, laid out identically on every
    rank inside one int32 buffer that all ranks have mapped:

        candidates  [world][2][B][Hq][k]   slot r = rank r's (scores as fp32 bits, ids); only the
                                           score half travels: a rank mixes none but its own
                                           proposals, whose ids it has, and ties between ranks are
                                           broken by position
        partials    [world][B][Hq][130]    slot r = rank r's un-normalised partial (fp32 bits)
        flags       [2][32]                word r of row 0 / 1 = epoch of rank r's last candidate /
                                           partial push

    ``base_ptrs[p]`` is the address of rank p's buffer as seen from this process (how the memory
    got mapped is not this class's business: symmetric memory on real ranks, plain tensors of one
    device for logical ranks in tests).  Slots are written by ``ops.exchange_push`` (plain stores
    over peer memory, then a flag) and read after ``ops.exchange_wait``.  The buffers are reused every
    step without double buffering: a rank pushes the candidates of step s+1 only after its own
    combine of step s, which waited for every rank's partial of step s, and a rank pushes a partial
    only after its merge has finished reading the candidates."""

    ALIGN = 64  # words: regions start on 256-byte boundaries

    @classmethod
    def layout(cls, world: int, B: int, Hq: int, topk: int):
        slot_c, slot_p = 2 * B * Hq * topk, B * Hq * 130
        if slot_c % 4 or slot_p % 4:
            raise ValueError("slots must be multiples of 16 bytes (B*Hq*k and B*Hq even)")
        up = lambda x: (x + cls.ALIGN - 1) // cls.ALIGN * cls.ALIGN
        off_c = 0
        off_p = up(off_c + world * slot_c)
        off_f = up(off_p + world * slot_p)
        return slot_c, slot_p, off_c, off_p, off_f, off_f + 64

    def __init__(self, buf: Tensor, base_ptrs: List[int], rank: int, world: int, B: int, Hq: int,
                 topk: int, timeout_s: float = 2.0):
        slot_c, slot_p, off_c, off_p, off_f, words = PeerExchange.layout(world, B, Hq, topk)
        if buf.dtype != torch.int32 or buf.numel() < words or world > 32:
            raise ValueError("buffer too small or of the wrong type, or more than 32 ranks")
        self.buf, self.rank, self.world, self.timeout_s = buf, rank, world, timeout_s
        self.cand = buf[off_c:off_c + world * slot_c].view(world, 2, B, Hq, topk)
        self.cand_sc = self.cand[:, 0].view(torch.float32)
        self.cand_idx = self.cand[:, 1]
        self.partials = buf[off_p:off_p + world * slot_p].view(torch.float32).view(world, B, Hq, 130)
        self.flags_c = buf[off_f:off_f + world]
        self.flags_p = buf[off_f + 32:off_f + 32 + world]
        self.epoch = torch.ones(1, dtype=torch.int32, device=buf.device)
        self.done = torch.zeros(4, dtype=torch.int32, device=buf.device)   # one word per kernel kind
        self.dst_c = [b + 4 * (off_c + rank * slot_c) for b in base_ptrs]   # the score half comes first
        self.dst_p = [b + 4 * (off_p + rank * slot_p) for b in base_ptrs]
        self.flg_c = [b + 4 * (off_f + rank) for b in base_ptrs]
        self.flg_p = [b + 4 * (off_f + 32 + rank) for b in base_ptrs]

    def push_candidates(self) -> None:
        from . import ops
        ops.exchange_push(self.cand[self.rank, 0], self.dst_c, self.flg_c, self.epoch, self.done[0:1])

    def wait_candidates(self) -> None:
        from . import ops
        ops.exchange_wait(self.flags_c, self.epoch, advance=False, timeout_s=self.timeout_s)

    def push_partial(self) -> None:
        from . import ops
        ops.exchange_push(self.partials[self.rank], self.dst_p, self.flg_p, self.epoch, self.done[1:2])

    def wait_partials(self) -> None:
        """Also ends the step: the epoch advances by one."""
        from . import ops
        ops.exchange_wait(self.flags_p, self.epoch, advance=True, timeout_s=self.timeout_s)


class HistExchange(PeerExchange):
    """PeerExchange plus the receive buffer of the histogram route (``mode="histograms"`` of
    ShardedTopkAttention): after the regions of the base class come, as 8-byte words that carry
    their step's epoch,

        histograms  [3][world][B*Hq][2048]  slot (round, r) = rank r's counts of that round
        partials    [world][B*Hq][132]      slot r = rank r's un-normalised partial row

    The other regions keep their place (a step of the candidate route can run on the same
    buffers)."""

    HIST_ROUNDS, HIST_BINS, PART_WORDS = 3, 2048, 132

    @classmethod
    def layout(cls, world: int, B: int, Hq: int, topk: int):
        base = PeerExchange.layout(world, B, Hq, topk)
        up = lambda x: (x + cls.ALIGN - 1) // cls.ALIGN * cls.ALIGN
        off_ll = up(base[-1])
        ll_words = 2 * world * B * Hq * (cls.HIST_ROUNDS * cls.HIST_BINS + cls.PART_WORDS)
        return base[:-1] + (off_ll, up(off_ll + ll_words))

    def __init__(self, buf: Tensor, base_ptrs: List[int], rank: int, world: int, B: int, Hq: int,
                 topk: int, timeout_s: float = 2.0):
        *_, off_ll, words = self.layout(world, B, Hq, topk)
        if buf.numel() < words:
            raise ValueError("buffer too small for the histogram regions")
        super().__init__(buf, base_ptrs, rank, world, B, Hq, topk, timeout_s)
        self.ll_ptrs = [b + 4 * off_ll for b in base_ptrs]


def make_peer_exchange(B: int, Hq: int, topk: int, device, group=None,
                       histograms: bool = False) -> Optional[PeerExchange]:
    """Receive buffers in symmetric memory (``torch.distributed._symmetric_memory``: one allocation
    per rank, mapped into every rank of the node).  Returns None -- on every rank alike -- when the
    buffers cannot be set up, and the caller stays on the collectives.  Multicast binding of the
    allocation is switched off: only plain peer loads and stores are used."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ex, ok = None, 1
    try:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        kind = HistExchange if histograms else PeerExchange
        words = kind.layout(world, B, Hq, topk)[-1]
        buf = symm.empty(words, dtype=torch.int32, device=device)
        buf.zero_()
        hdl = symm.rendezvous(buf, group if group is not None else dist.group.WORLD)
        ex = kind(buf, [int(p) for p in hdl.buffer_ptrs], rank, world, B, Hq, topk)
        ex._handle = hdl     # keeps the mappings alive
    except Exception as e:   # noqa: BLE001 - any failure means "use the collectives"
        print(f"[topk_attn_b200] rank {rank}: peer exchange unavailable ({type(e).__name__}: {e})",
              file=sys.stderr)
        ok = 0
    flag = torch.tensor([ok], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    torch.cuda.synchronize()
    dist.barrier(group)      # every buffer is zeroed before anyone pushes
    return ex if flag.item() else None


class ShardedTopkAttention:
    def __init__(self, topk: int, sm_scale: float = 1.0, group=None, backend=None,
                 exchange: Optional[PeerExchange] = None, mode: str = "auto"):
        """``mode="histograms"`` (needs a HistExchange and several queries per K row -- a GQA group
        or one cache shared by the batch): the ranks agree on the global k-th score through
        exchanged histograms of their scores and no candidate lists travel; the whole step is one
        call (``ra_sharded_topk_attention``: two kernels, no flags, no collective).
        ``mode="auto"`` (the default) takes that route whenever the exchange is a HistExchange and
        the first step's shapes qualify, else the candidate route."""
        if mode not in ("auto", "candidates", "histograms"):
            raise ValueError("mode must be 'auto', 'candidates' or 'histograms'")
        if mode == "histograms" and not isinstance(exchange, HistExchange):
            raise ValueError("the histogram route needs a HistExchange")
        self.mode = mode
        self.topk, self.sm_scale, self.group = topk, sm_scale, group
        self.backend = backend if backend is not None else CudaBackend()
        self.exchange = exchange
        if exchange is not None:
            self.world, self.rank = exchange.world, exchange.rank
        else:
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._recv = self._send = self._partials = None
        self._graph = None

    def _buffers(self, B: int, Hq: int, device):
        """Scores and ids of one rank are the two halves of one int32 buffer, so that a single
        all-gather moves both: recv [world, 2, B, Hq, k], send [2, B, Hq, k]."""
        if self.exchange is not None:
            ex = self.exchange
            self._recv, self._send, self._partials = ex.cand, ex.cand[self.rank], ex.partials
            return ex.cand_sc, ex.cand_idx, ex.partials
        shape = (self.world, 2, B, Hq, self.topk)
        if self._recv is None or self._recv.shape != shape or self._recv.device != device:
            self._recv = torch.empty(shape, dtype=torch.int32, device=device)
            self._send = torch.empty(shape[1:], dtype=torch.int32, device=device)
            self._partials = torch.empty(self.world, B, Hq, 130, dtype=torch.float32, device=device)
        cand_sc = self._recv[:, 0].view(torch.float32)
        cand_idx = self._recv[:, 1]
        return cand_sc, cand_idx, self._partials

    def resolve_mode(self, q: Tensor, k: Tensor) -> str:
        """Settle ``mode="auto"`` from the shapes of a step: the histogram route needs a
        HistExchange and several queries per K row."""
        if self.mode == "auto":
            B, Hq, _ = q.shape
            shared_queries = (Hq // k.size(-2)) * (B if k.dim() == 3 else 1)
            self.mode = "histograms" if isinstance(self.exchange, HistExchange) and shared_queries > 1 \
                else "candidates"
        return self.mode

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
        self.resolve_mode(q, k)
        if self.mode == "histograms":
            return self.backend.sharded_attention(q, k, v, self.topk, self.sm_scale, index_base, self.exchange)
        idx, sc = self.local_candidates(q, k, index_base)
        self.exchange_candidates(idx, sc)
        self.merge_and_exchange(cand_sc, cand_idx, partials, v, index_base)
        if self.exchange is not None:
            # the combine waits for every rank's partial itself and ends the step
            return self.backend.combine(partials, exchange=self.exchange)
        return self.backend.combine(partials)

    def merge_and_exchange(self, cand_sc: Tensor, cand_idx: Tensor, partials: Tensor, v: Tensor,
                           index_base: int) -> None:
        """Steps 3 and 4: this rank's partial over the global winners it owns, then every rank's
        partial into ``partials``."""
        if self.exchange is not None:
            # the merge waits for the candidate flags, writes this rank's partial and pushes it
            self.backend.merge_partial(cand_sc, cand_idx, v, self.topk, self.sm_scale, index_base,
                                       out=partials[self.rank], exchange=self.exchange,
                                       own_part=self.rank)
            return
        part = self.backend.merge_partial(cand_sc, cand_idx, v, self.topk, self.sm_scale, index_base)
        if self.world > 1:
            _all_gather(partials, part, self.group)
        else:
            partials[0].copy_(part)

    def capture(self, q: Tensor, k: Tensor, v: Tensor, index_base: Optional[int] = None):
        """Capture one step on (q, k, v) into a CUDA graph and return a function that replays it and
        gives the step's output tensor (the same tensor on every replay; new queries are copied
        into ``q`` before a replay).  Only with the peer exchange: then the step is nothing but the
        library's kernels on one stream.  Every rank must call this at the same point, because the
        warm-up step it runs is a real exchange."""
        if self.exchange is None:
            raise RuntimeError("capture() needs the peer exchange")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            self.step(q, k, v, index_base)          # allocates this stream's scratch
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                out = self.step(q, k, v, index_base)
        torch.cuda.current_stream().wait_stream(side)
        self._graph, self._graph_stream = graph, side

        def replay() -> Tensor:
            graph.replay()
            return out
        return replay


def _check_graph_status(self) -> None:
    """Raise if a kernel of the captured step gave up a bounded wait (its status word lives in the
    scratch of the capture stream)."""
    from . import ops
    torch.cuda.synchronize()
    with torch.cuda.stream(self._graph_stream):
        ops.check_status(self.exchange.buf.device)


ShardedTopkAttention.check_graph_status = _check_graph_status


def _exchange(self, idx: Tensor, sc: Tensor) -> None:
    """All ranks' (score, id) proposals into the receive buffer: one collective, or peer stores
    followed by a bounded wait for every rank's flag."""
    if idx.data_ptr() != self._send[1].data_ptr():
        self._send[1].copy_(idx)
        self._send[0].view(torch.float32).copy_(sc)
    if self.exchange is not None:
        self.exchange.push_candidates()      # the merge kernel waits for the flags
    elif self.world > 1:
        _all_gather(self._recv, self._send, self.group)
    else:
        self._recv[0].copy_(self._send)


ShardedTopkAttention.exchange_candidates = _exchange


def local_scores(q: Tensor, k: Tensor) -> Tensor:
    """fp32 q.K^T of this rank's shard by plain torch on the device: [B,Hq,n]."""
    B, Hq, _ = q.shape
    Hkv = k.size(-2)
    grp = Hq // Hkv
    rows = []
    for b in range(B):
        kb = k[b] if k.dim() == 4 else k
        per_head = [q[b, h * grp:(h + 1) * grp].float() @ kb[:, h, :].float().t() for h in range(Hkv)]
        rows.append(torch.cat(per_head, 0))
    return torch.stack(rows)


def verify_winners(q: Tensor, k: Tensor, v: Tensor, out: Tensor, gidx: Tensor, gsc: Tensor,
                   topk: int, sm_scale: float, index_base: int, world: int, band: float = 1e-3) -> dict:
    """Check one step's result on the ranks themselves with plain torch operations on each device
    (no library code): ``out`` is this rank's final output, ``gidx``/``gsc`` the global winners as
    this rank's merge selected them.  Verdicts:

    * ``ranks_agree`` -- every rank holds bit-identical outputs and winner sets;
    * ``selection`` -- against this rank's own fp32 q.K^T: every local key scoring more than
      ``band`` above the k-th winner is among the winners, no owned winner scores more than ``band``
      below it, reported scores match within ``band``, and the owned winners of all ranks add up to
      exactly k distinct ids per (row, head);
    * ``output`` -- ``out`` equals softmax.V recomputed from the winners (every rank mixes the V rows
      it owns in torch, partial sums are all-reduced) within rtol 1e-2 / atol 1e-3.
    """
    B, Hq, _ = q.shape
    n = k.size(-3)
    Hkv = k.size(-2)
    grp = Hq // Hkv
    dev = q.device
    res = {}
    multi = world > 1 and dist.is_initialized()
    if multi:
        outs = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(outs, out.contiguous())
        sets = [torch.empty_like(gidx) for _ in range(world)]
        dist.all_gather(sets, gidx.sort(-1).values.contiguous())
        res["ranks_agree"] = bool(all(torch.equal(o, outs[0]) for o in outs) and
                                  all(torch.equal(x, sets[0]) for x in sets))
    else:
        res["ranks_agree"] = True
    s = local_scores(q, k)
    ids = gidx.long()
    mine = (ids >= index_base) & (ids < index_base + n)
    kth = gsc.min(-1, keepdim=True).values
    slot = torch.where(mine, ids - index_base, torch.full_like(ids, n))
    member = torch.zeros(B, Hq, n + 1, dtype=torch.bool, device=dev).scatter_(-1, slot, True)[..., :n]
    got = torch.cat([s, torch.zeros(B, Hq, 1, device=dev)], -1).gather(-1, slot)
    missed = bool(((s > kth + band) & ~member).any())
    low = bool((mine & (got < kth - band)).any())
    score_err = float(((got - gsc).abs() * mine).max())
    srt = ids.sort(-1).values
    distinct = bool((srt[..., 1:] != srt[..., :-1]).all())
    owned = mine.sum(-1).to(torch.int64)
    if multi:
        dist.all_reduce(owned)
    res["selection"] = bool(not missed and not low and score_err <= band and distinct and
                            bool((owned == topk).all()))
    m = (gsc * sm_scale).max(-1, keepdim=True).values
    w = torch.exp(gsc * sm_scale - m) * mine
    num = torch.zeros(B, Hq, 128, device=dev)
    row = slot.clamp(max=n - 1)
    for b in range(B):
        vb = v[b] if v.dim() == 4 else v
        for h in range(Hq):
            num[b, h] = w[b, h] @ vb[row[b, h], h // grp].float()
    den = w.sum(-1)
    if multi:
        dist.all_reduce(num)
        dist.all_reduce(den)
    ref = num / den.unsqueeze(-1)
    res["output"] = bool(torch.allclose(out.float(), ref, rtol=1e-2, atol=1e-3))
    res["max_abs_err"] = float((out.float() - ref).abs().max())
    res["ok"] = bool(res["ranks_agree"] and res["selection"] and res["output"])
    if multi:
        flag = torch.tensor([1 if res["ok"] else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        res["ok"] = bool(flag.item())
    return res


def verify_sharded_step(op: "ShardedTopkAttention", q: Tensor, k: Tensor, v: Tensor,
                        index_base: int) -> dict:
    """One untimed sharded step and its check (see verify_winners)."""
    from . import ops
    B, Hq, _ = q.shape
    if op.resolve_mode(q, k) == "histograms":
        # every rank reports its own winners; all of them together must be the global top-k
        out, idx, sc = op.backend.sharded_attention(q, k, v, op.topk, op.sm_scale, index_base, op.exchange,
                                                    return_indices=True)
        torch.cuda.synchronize()
        ops.check_status(q.device)
        if op.world > 1 and dist.is_initialized():
            ids = torch.empty(op.world, B, Hq, op.topk, dtype=torch.int32, device=q.device)
            scs = torch.empty(op.world, B, Hq, op.topk, dtype=torch.float32, device=q.device)
            dist.all_gather_into_tensor(ids.view(-1, Hq, op.topk), idx, group=op.group)
            dist.all_gather_into_tensor(scs.view(-1, Hq, op.topk), sc, group=op.group)
            ids = ids.permute(1, 2, 0, 3).reshape(B, Hq, -1)
            scs = scs.permute(1, 2, 0, 3).reshape(B, Hq, -1)
            gsc, pos = scs.topk(op.topk, dim=-1)
            gidx = ids.gather(-1, pos)
        else:
            gidx, gsc = idx, sc
        return verify_winners(q, k, v, out, gidx.contiguous(), gsc.contiguous(), op.topk, op.sm_scale,
                              index_base, op.world)
    out = op.step(q, k, v, index_base)
    cand_sc, cand_idx, _ = op._buffers(B, Hq, q.device)
    if op.exchange is not None and op.world > 1 and dist.is_initialized():
        # the peer exchange moves scores only; the check wants every rank's ids as well
        torch.cuda.synchronize()
        ids = torch.empty(op.world, B, Hq, op.topk, dtype=torch.int32, device=q.device)
        dist.all_gather_into_tensor(ids.view(-1, Hq, op.topk), cand_idx[op.rank].contiguous(), group=op.group)
        cand_idx.copy_(ids)
    _, gidx, gsc = ops.merge_attend(cand_sc, cand_idx, v, op.topk, op.sm_scale, index_base,
                                    partial=True, return_indices=True)
    ops.check_status(q.device)
    return verify_winners(q, k, v, out, gidx, gsc, op.topk, op.sm_scale, index_base, op.world)


def time_sharded(op: "ShardedTopkAttention", q: Tensor, k: Tensor, v: Tensor, index_base: int,
                 steps: int, warmup: int):
    """Device time of ``steps`` sharded steps, max over ranks, and of the local scan alone.  With the
    peer exchange the step is replayed from a CUDA graph.  Returns (ms per step, scan ms per step,
    launches of this rank per step, how the step was issued)."""
    from . import capi, ops
    dev = q.device
    multi = op.world > 1 and dist.is_initialized()
    run, how = (lambda: op.step(q, k, v, index_base)), "eager"
    c0 = capi.lib().ra_launch_count()
    op.step(q, k, v, index_base)
    launches = capi.lib().ra_launch_count() - c0
    if op.exchange is not None:
        run, how = op.capture(q, k, v, index_base), "cuda graph"
    for _ in range(max(warmup, 3)):
        run()
    torch.cuda.synchronize()
    ops.check_status(dev)
    # the local scan alone (the dominant kernel), outside the steps
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    op._buffers(q.size(0), q.size(1), dev)
    if multi:
        dist.barrier()
    a.record()
    for _ in range(steps):
        if op.mode == "histograms":
            ops.stored_scores_probe(q, k, op.topk)     # the scan kernel of this route alone
        else:
            op.local_candidates(q, k, index_base)
    b.record()
    torch.cuda.synchronize()
    scan_ms = a.elapsed_time(b) / steps
    if multi:
        # a step waits for the slowest rank's proposals: report the slowest scan
        sm = torch.tensor([scan_ms], device=dev)
        dist.all_reduce(sm, op=dist.ReduceOp.MAX)
        scan_ms = sm.item()
    run()                       # the exchanged candidates are this step's again
    if multi:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if multi:
        dist.barrier()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ops.check_status(dev)
    if op._graph is not None:
        # the captured kernels report into the scratch of the stream they were captured on
        op.check_graph_status()
    return t.item() / steps, scan_ms, launches, how


HIST_PHASES = ("round 0 (with the wait for the slowest rank's scan)", "collect", "further rounds",
               "winners", "V mixing", "merge + send", "combine (with the wait for the slowest rank's partial)")


def hist_phase_stamps(op: "ShardedTopkAttention", q: Tensor, k: Tensor, v: Tensor, index_base: int,
                      iters: int = 12) -> Optional[dict]:
    """Where a step of the histogram route spends its time on every rank: wall-clock stamps that
    thread 0 of CTA 0 of the selection kernel writes into the status block in the tuning build,
    median over ``iters`` eager steps with L2 flushed and the ranks aligned by a barrier before
    each.  Rank 0 gets {phase: [us on rank 0, rank 1, ...]}; a measuring aid, not a timed result."""
    from . import capi, ops
    dev = q.device
    multi = op.world > 1 and dist.is_initialized()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    with capi.tuning_library():
        for _ in range(iters):
            flush.zero_()
            torch.cuda.synchronize()
            if multi:
                dist.barrier()
            op.step(q, k, v, index_base)
            torch.cuda.synchronize()
            t = ops.workspace(256, dev)[:256].view(torch.int64)[4:12].tolist()
            rows.append([(t[i] - t[i - 1]) / 1e3 for i in range(1, 8)])
    rows = rows[min(3, iters - 1):]
    med = torch.tensor([sorted(r[i] for r in rows)[len(rows) // 2] for i in range(7)], device=dev)
    allm = [torch.empty_like(med) for _ in range(op.world)] if multi else [med]
    if multi:
        dist.all_gather(allm, med)
    if op.rank != 0:
        return None
    return {name: [round(float(m[i]), 2) for m in allm] for i, name in enumerate(HIST_PHASES)}


def bench_long_context(rank: int, world: int, dev, steps: int, warmup: int, peak_gbs: float,
                       collectives: bool = False, histograms: bool = True, phases: bool = False) -> dict:
    """Configuration 4 (1 048 576 tokens, 32 query / 8 kv heads, k = 4096) cut over ``world`` ranks:
    total work is fixed, so the time per step should fall as ranks are added (strong scaling).  On
    one GPU the step is the single fused call; on several it is the sharded step.  Every record
    carries the verdict of a check of its own result (verify_winners)."""
    from . import ops, workloads as W
    w = W.sharded_long_context_shard(rank, world, device=dev)
    q, k, v = w.q, w.k, w.v
    n_local = w.n_tokens
    base = rank * n_local
    if world == 1:
        out, gidx, gsc = ops.topk_attention(q, k, v, w.topk, w.sm_scale, return_indices=True)
        ops.check_status(dev)
        parity = verify_winners(q, k, v, out, gidx, gsc, w.topk, w.sm_scale, 0, 1)
        out = torch.empty_like(q)
        for _ in range(max(warmup, 3)):
            ops.topk_attention(q, k, v, w.topk, w.sm_scale, out=out)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            ops.topk_attention(q, k, v, w.topk, w.sm_scale, out=out)
        e1.record()
        torch.cuda.synchronize()
        ops.check_status(dev)
        per_ms = e0.elapsed_time(e1) / steps
        scan_ms = per_ms
        how, ex = "eager", None
    else:
        ex = None if collectives else make_peer_exchange(q.size(0), q.size(1), w.topk, dev,
                                                         histograms=histograms)
        hist = histograms and isinstance(ex, HistExchange)
        op = ShardedTopkAttention(w.topk, w.sm_scale, exchange=ex,
                                  mode="histograms" if hist else "candidates")
        parity = verify_sharded_step(op, q, k, v, base)
        per_ms, scan_ms, _, how = time_sharded(op, q, k, v, base, steps, warmup)
    n_total = world * n_local
    alg_per_gpu = w.kv_bytes_scanned() + q.size(1) * w.topk * 128 * 2 // world
    stamps = None
    if phases and world > 1 and op.mode == "histograms":
        stamps = hist_phase_stamps(op, q, k, v, base)
    return {"phases_us_per_rank": stamps,
            "workload": "cfg4: B1 Hq32/Hkv8 N1048576 k4096, tokens cut over the ranks",
            "n_gpus": world, "context": n_total, "context_per_gpu": n_local, "scaling": "strong",
            "us_per_step": per_ms * 1e3, "tokens_per_s": n_total / (per_ms * 1e-3),
            "scan_us": scan_ms * 1e3, "exchange_us": (per_ms - scan_ms) * 1e3,
            "exchange": "none" if world == 1 else (
                ("histograms as tagged words over peer stores" if op.mode == "histograms" else "peer stores + flags")
                if ex is not None else "nccl all_gather x2"),
            "issued_as": how,
            "roofline_frac_step": alg_per_gpu / (per_ms * 1e-3) / 1e9 / peak_gbs,
            "algorithmic_bytes_per_gpu": alg_per_gpu, "parity": parity}


def bench(args, rank: int, local: int, world: int, ClockSampler, measured_peak_gbs) -> None:
    """`bench.py --gpus N` for N > 1.  The headline line is weak scaling of configuration 2: every
    rank holds a 131072-token shard of each of the 4 sequences (32 heads, k = 2048), timed on the
    device, max over ranks.  The same process then runs configuration 4 strong-scaled
    (bench_long_context) and adds it as ``cfg4_strong``.  Both results are checked on the ranks
    before they are timed; a failed check fails the run."""
    from . import ops, workloads as W
    dev = torch.device("cuda", local)
    strong = args.workload == "cfg4"
    if strong:
        w = W.sharded_long_context_shard(rank, world, device=dev)
    else:
        w = W.fused_topk_128k_shard(rank, world, device=dev)
    q, k, v = w.q, w.k, w.v
    collectives = bool(getattr(args, "collectives", False))
    hist = strong and not getattr(args, "candidates", False)
    ex = None if collectives else make_peer_exchange(q.size(0), q.size(1), w.topk, dev, histograms=hist)
    hist = hist and isinstance(ex, HistExchange)
    op = ShardedTopkAttention(w.topk, w.sm_scale, exchange=ex, mode="histograms" if hist else "candidates")
    n_local = w.n_tokens
    base = rank * n_local

    parity = verify_sharded_step(op, q, k, v, base)
    sampler = ClockSampler(local)
    sampler.start()
    per_ms, scan_ms, launches, how = time_sharded(op, q, k, v, base, args.steps, args.warmup)
    clocks = sampler.stop()

    q_host = q.cpu().pin_memory()
    out_host = torch.empty_like(q_host).pin_memory()
    q_dev = torch.empty_like(q)

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        o = op.step(q_dev, k, v, base)
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
    tokens = world * w.batch * n_local
    alg = w.algorithmic_bytes()
    heads_q, heads_kv, batch, bkv, topk = q.size(1), k.size(-2), w.batch, w.bkv, w.topk
    peak, kind = measured_peak_gbs()
    exchange_label = (("histograms as tagged words over peer stores" if hist else "peer stores + flags")
                      if ex is not None else "nccl all_gather x2")

    stamps = hist_phase_stamps(op, q, k, v, base) if (getattr(args, "phases", False) and hist) else None
    long_ctx = None
    if not strong and not args.no_cfg4:
        del w, q, k, v, op, q_dev, ex
        torch.cuda.empty_cache()
        long_ctx = bench_long_context(rank, world, dev, min(args.steps, 100), args.warmup, peak,
                                      collectives, histograms=not getattr(args, "candidates", False),
                                      phases=bool(getattr(args, "phases", False)))

    if rank == 0:
        achieved = alg / (scan_ms * 1e-3) / 1e9
        line = {
            "metric": "tokens_scanned_per_s", "value": tokens / (per_ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": per_ms, "us_per_step": per_ms * 1e3, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f16 inputs, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": "cfg4 token-sharded" if strong else "cfg2 token-sharded",
                       "batch": batch, "heads_q": heads_q,
                       "heads_kv": heads_kv, "head_dim": 128, "context": world * n_local,
                       "context_per_gpu": n_local, "topk": topk, "caches": bkv,
                       "l2": "inputs_exceed_l2",
                       "exchange": exchange_label, "issued_as": how},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": kind + " (burst copy)",
                         "algorithmic_bytes": alg, "traffic": None,
                         "kernel": "scan kernel of one rank", "scan_us": scan_ms * 1e3,
                         "exchange_us": (per_ms - scan_ms) * 1e3},
            "cpu_baseline": None,
            "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "us_per_step": e2e_s * 1e6,
                    "h2d_bytes_per_step": q_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": launches * world * args.steps,
            "clocks": clocks,
            "parity": parity,
        }
        if stamps is not None:
            line["phases_us_per_rank"] = stamps
        if long_ctx is not None:
            line["cfg4_strong"] = long_ctx
        print(json.dumps(line), flush=True)
    ok = parity["ok"] and (long_ctx is None or long_ctx["parity"]["ok"])
    dist.barrier()
    dist.destroy_process_group()
    if not ok:
        raise SystemExit("parity check failed on the ranks: " + json.dumps(
            {"cfg2": parity, "cfg4": long_ctx["parity"] if long_ctx else None}))
