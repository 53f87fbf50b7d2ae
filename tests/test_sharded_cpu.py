"""Host logic of the sequence-sharded step on CPU: two gloo ranks, the compute steps replaced by
oracle-based stand-ins (test code only), the exchange/merge/combine orchestration is the
product's."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import topk_attn_oracle as O
from topk_attn_b200.sharded import ShardedTopkAttention


class OracleBackend:
    """CPU stand-in for the three kernels, built from the oracle."""

    def select(self, q, k, topk, index_base, out=None):
        s = O.full_scores(q, k)
        sc, idx = torch.topk(s, topk, dim=-1)
        idx, sc = (idx + index_base).int().contiguous(), sc.contiguous()
        if out is not None:
            out[0].copy_(idx)
            out[1].copy_(sc)
            return out
        return idx, sc

    def merge_partial(self, cand_sc, cand_idx, v, topk, sm_scale, own_base):
        G, B, Hq, k = cand_sc.shape
        assert cand_sc.stride()[1:] == (Hq * k, k, 1) and cand_idx.stride() == cand_sc.stride()
        sc = cand_sc.permute(1, 2, 0, 3).reshape(B, Hq, G * k)
        ix = cand_idx.permute(1, 2, 0, 3).reshape(B, Hq, G * k).long()
        gs, pos = torch.topk(sc, topk, dim=-1)
        gi = torch.gather(ix, -1, pos)
        n = v.size(-3)
        mine = (gi >= own_base) & (gi < own_base + n)
        m = gs.max(-1).values * sm_scale
        e = torch.where(mine, torch.exp(gs * sm_scale - m.unsqueeze(-1)), torch.zeros_like(gs))
        loc = torch.where(mine, gi - own_base, torch.zeros_like(gi))
        out = torch.zeros(B, Hq, 130)
        for b in range(B):
            vs = O._gather_rows(v, b, Hq, loc[b])
            out[b, :, :128] = torch.einsum("hs,hsd->hd", e[b], vs)
        out[..., 128] = e.sum(-1)
        out[..., 129] = m
        return out

    def combine(self, partials):
        o, l, m = partials[..., :128], partials[..., 128], partials[..., 129]
        return O.lse_combine(o, m, l).half()


def _worker(rank, world, port, q, k, v, topk, scale, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = k.size(0) // world
        op = ShardedTopkAttention(topk, scale, backend=OracleBackend())
        out = op.step(q, k[rank * n:(rank + 1) * n].contiguous(), v[rank * n:(rank + 1) * n].contiguous())
        ret[rank] = out.float()
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("topk,n", [(64, 2048), (300, 512)])
def test_two_gloo_ranks_match_single_device(topk, n):
    g = torch.Generator().manual_seed(5)
    q = (torch.randn(2, 8, 128, generator=g) / 11.3).half()
    k = torch.randn(n, 2, 128, generator=g).half()
    v = torch.randn(n, 2, 128, generator=g).half()
    ref, _, _ = O.topk_sparse_attention(q, k, v, topk, 0.7)
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), q, k, v, topk, 0.7, ret), nprocs=world, join=True)
    for r in range(world):
        O.check_output(ref, ret[r])
    assert torch.equal(ret[0], ret[1])        # every rank ends with the same output


def test_short_shard_is_padded():
    """A shard with fewer than k tokens proposes all of them and pads with (-inf, -1)."""
    g = torch.Generator().manual_seed(6)
    q = (torch.randn(1, 2, 128, generator=g) / 11.3).half()
    k = torch.randn(40, 2, 128, generator=g).half()
    op = ShardedTopkAttention(64, 1.0, backend=OracleBackend())
    idx, sc = op.local_candidates(q, k, 1000)
    assert idx.shape == (1, 2, 64) and (idx[..., 40:] == -1).all() and torch.isinf(sc[..., 40:]).all()
    assert idx[..., :40].min().item() >= 1000


# ---- the histogram route: the ranks agree on the k-th score through histograms only ------------

class OracleHistBackend(OracleBackend):
    """Stand-in for ra_sharded_topk_attention: the oracle's restatement of the distributed radix
    select, its histograms gathered over gloo, then partials and the log-sum-exp combine."""

    def sharded_attention(self, q, k, v, topk, sm_scale, index_base, exchange, return_indices=False):
        B, Hq, _ = q.shape
        s = O.full_scores(q, k)                                  # [B,Hq,n] fp32
        n = s.size(-1)

        def gather(h):
            out = torch.empty(exchange.world, *h.shape, dtype=h.dtype)
            dist.all_gather_into_tensor(out.view(-1, h.size(-1)), h.contiguous())
            return out

        win = O.histogram_select_shard(O.ordered_keys(s).view(B * Hq, n), topk, exchange.rank, gather)
        win = win.view(B, Hq, n)
        x = torch.where(win, s * sm_scale, torch.full_like(s, float("-inf")))
        m = x.max(-1).values
        e = torch.nan_to_num(torch.where(win, torch.exp(x - m.unsqueeze(-1)), torch.zeros_like(x)), nan=0.0)
        grp = Hq // v.size(-2)
        part = torch.zeros(B, Hq, 130)
        for h in range(Hq):
            part[:, h, :128] = e[:, h] @ v[:, h // grp].float()
        part[..., 128], part[..., 129] = e.sum(-1), m
        parts = torch.empty(exchange.world, B, Hq, 130)
        dist.all_gather_into_tensor(parts.view(-1, Hq, 130), part)
        out = self.combine(parts)
        if return_indices:
            return out, win
        return out


def _hist_worker(rank, world, port, q, k, v, topk, scale, ret):
    from topk_attn_b200.sharded import HistExchange
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = k.size(0) // world
        B, Hq = q.shape[:2]
        buf = torch.zeros(HistExchange.layout(world, B, Hq, topk)[-1], dtype=torch.int32)
        ex = HistExchange(buf, [buf.data_ptr()] * world, rank, world, B, Hq, topk)
        op = ShardedTopkAttention(topk, scale, backend=OracleHistBackend(), exchange=ex, mode="histograms")
        out = op.step(q, k[rank * n:(rank + 1) * n].contiguous(), v[rank * n:(rank + 1) * n].contiguous())
        ret[rank] = out.float()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("topk,n,ties", [(64, 2048, False), (300, 1024, True)])
def test_two_gloo_ranks_histogram_route_matches_single_device(topk, n, ties):
    g = torch.Generator().manual_seed(9)
    q = (torch.randn(1, 8, 128, generator=g) / 11.3).half()
    k = torch.randn(n, 2, 128, generator=g).half()
    if ties:
        k[::3] = k[0]                                   # a third of the keys are copies of one key
    v = torch.randn(n, 2, 128, generator=g).half()
    # the single-device operator keeps the lowest ids among copies of the k-th score
    ids = (-O.full_scores(q, k)).argsort(dim=-1, stable=True)[..., :topk]
    want = O.gathered_attention(q, k, v, ids, 0.7)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_hist_worker, args=(2, _free_port(), q, k, v, topk, 0.7, ret), nprocs=2, join=True)
    for r in range(2):
        O.check_output(want, ret[r])
    assert torch.equal(ret[0], ret[1])


def test_histogram_select_takes_copies_in_rank_then_token_order():
    """Three shards in lockstep (threads): the winners are exactly the k best with copies of the
    k-th score resolved towards the lowest token ids, whole rows of equal scores included."""
    import threading
    R, n, k, W = 4, 3000, 257, 3
    g = torch.Generator().manual_seed(1)
    s = torch.randn(R, W * n, generator=g)
    s[0, ::7] = 0.5
    s[1] = 1.25
    s[2, 5::2] = s[2, 5]
    keys = O.ordered_keys(s)
    assert torch.equal(keys.argsort(dim=-1, stable=True), s.argsort(dim=-1, stable=True))
    bar, slots, res = threading.Barrier(W), [None] * W, [None] * W

    def run(r):
        def gather(h):
            slots[r] = h
            bar.wait()
            out = torch.stack(slots)
            bar.wait()
            return out
        res[r] = O.histogram_select_shard(keys[:, r * n:(r + 1) * n], k, r, gather)

    ts = [threading.Thread(target=run, args=(r,)) for r in range(W)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    win = torch.cat(res, -1)
    ref = torch.zeros_like(win).scatter_(1, (-s).argsort(dim=-1, stable=True)[:, :k], True)
    assert torch.equal(win, ref)
