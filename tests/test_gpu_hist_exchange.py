"""The histogram route of the sharded step (ra_sharded_topk_attention) on one GPU.

Its selection kernel waits for the other ranks' histograms inside the kernel, so logical ranks
cannot be played by separate launches on one device.  Here a single rank runs the whole route (its
own words satisfy every wait): scoring, the rounds of the radix select over exchanged histograms,
the share-out of copies of the k-th score, the partial and the combine -- against the
single-device operator and the oracle.  The cross-rank sums are checked on real ranks by
``bench.py --gpus N``, which verifies every rank's winners before it times anything.
"""
import pytest
import torch

from oracle import topk_attn_oracle as O

from gpu_util import rand_case

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def one_rank(B, Hq, topk, timeout_s=2.0):
    from topk_attn_b200.sharded import HistExchange
    words = HistExchange.layout(1, B, Hq, topk)[-1]
    buf = torch.zeros(words, dtype=torch.int32, device=DEV)
    return HistExchange(buf, [buf.data_ptr()], 0, 1, B, Hq, topk, timeout_s)


@pytest.mark.parametrize("B,Hq,Hkv,N,topk,per_batch", [
    (1, 8, 2, 20000, 256, False),      # a GQA group of 4
    (2, 4, 4, 16384, 512, False),      # one cache shared by two batch rows
    (1, 32, 8, 65536, 4096, False),    # the long-context configuration, shortened
    (2, 8, 4, 9000, 128, True),        # a cache per batch row, group of 2, ragged length
    (1, 32, 8, 524288, 4096, False),   # a shard of the long-context configuration cut over 2 ranks
])
def test_one_rank_matches_the_single_device_operator(B, Hq, Hkv, N, topk, per_batch):
    from topk_attn_b200 import ops
    from topk_attn_b200.sharded import ShardedTopkAttention, verify_sharded_step
    q, k, v = rand_case(B, Hq, Hkv, N, per_batch, seed=11)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ex = one_rank(B, Hq, topk)
    op = ShardedTopkAttention(topk, 0.5, exchange=ex, mode="histograms")
    ref, ridx, _ = ops.topk_attention(qd, kd, vd, topk, 0.5, return_indices=True)
    for _ in range(2):                                   # the buffers are reused step after step
        out = op.step(qd, kd, vd, 0)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert torch.allclose(out.float(), ref.float(), rtol=1e-2, atol=1e-3)
    out2, idx, _ = ops.sharded_topk_attention(qd, kd, vd, topk, 0.5, 0, ex, return_indices=True)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)                        # the same bits step after step
    assert torch.equal(idx.sort(-1).values, ridx.sort(-1).values)
    res = verify_sharded_step(op, qd, kd, vd, 0)
    assert res["ok"], res
    if N > 100000:
        return                                           # the oracle would take minutes
    want = O.topk_sparse_attention(q, k, v, topk, 0.5)[0]
    assert torch.allclose(out.float().cpu(), want.float(), rtol=1e-2, atol=1e-3)


def test_copies_of_the_kth_score_are_taken_in_token_order():
    """Every key of a head is the same vector: all scores tie, the k winners are tokens 0..k-1
    (round 2 of the select runs, and the copies exceed the candidate list)."""
    from topk_attn_b200 import ops
    from topk_attn_b200.sharded import ShardedTopkAttention
    B, Hq, Hkv, N, topk = 1, 8, 2, 40000, 300
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, Hq, 128, generator=g).half()
    k = torch.randn(1, Hkv, 128, generator=g).half().expand(N, Hkv, 128).contiguous()
    v = torch.randn(N, Hkv, 128, generator=g).half()
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ex = one_rank(B, Hq, topk)
    out, idx, _ = ops.sharded_topk_attention(qd, kd, vd, topk, 1.0, 0, ex, return_indices=True)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    want_ids = torch.arange(topk, dtype=torch.int32, device=DEV).expand(B, Hq, topk)
    assert torch.equal(idx.sort(-1).values, want_ids)
    ref = vd[:topk].float().mean(0)                      # equal weights over tokens 0..k-1
    for h in range(Hq):
        assert torch.allclose(out[0, h].float(), ref[h // (Hq // Hkv)], rtol=1e-2, atol=2e-3)


def test_step_replays_from_a_cuda_graph():
    from topk_attn_b200 import ops
    from topk_attn_b200.sharded import ShardedTopkAttention
    q, k, v = rand_case(1, 8, 2, 30000, False, seed=4)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ex = one_rank(1, 8, 256)
    op = ShardedTopkAttention(256, 1.0, exchange=ex, mode="histograms")
    replay = op.capture(qd, kd, vd, 0)
    ref = ops.topk_attention(qd, kd, vd, 256, 1.0)
    for _ in range(3):
        out = replay()
    op.check_graph_status()
    assert torch.allclose(out.float(), ref.float(), rtol=1e-2, atol=1e-3)


def test_a_histogram_that_never_arrives_ends_in_a_timeout():
    """World of two with nobody playing rank 1: the wait for its histogram runs out, the kernel
    returns, the status word reports it and the context stays usable."""
    import time
    from topk_attn_b200 import capi, ops
    from topk_attn_b200.sharded import HistExchange
    B, Hq, topk = 1, 8, 128
    words = HistExchange.layout(2, B, Hq, topk)[-1]
    bufs = [torch.zeros(words, dtype=torch.int32, device=DEV) for _ in range(2)]
    ex = HistExchange(bufs[0], [b.data_ptr() for b in bufs], 0, 2, B, Hq, topk, timeout_s=0.05)
    q, k, v = rand_case(B, Hq, 2, 8192, False, seed=2)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ops.sharded_topk_attention(qd, kd, vd, topk, 1.0, 0, ex)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0                # one time limit, not one per polled word
    with pytest.raises(capi.RaError) as err:
        ops.check_status(DEV)
    assert err.value.status == capi.RA_ERR_DEVICE_TIMEOUT
    ops.workspace(256, DEV)[:4].zero_()                  # the status bits are sticky
    ops.check_status(DEV)


def test_shapes_outside_the_route_are_refused():
    from topk_attn_b200 import capi, ops
    q, k, v = rand_case(1, 4, 4, 8192, False, seed=1)   # one query per K row
    ex = one_rank(1, 4, 64)
    with pytest.raises(capi.RaError) as err:
        ops.sharded_topk_attention(q.to(DEV), k.to(DEV), v.to(DEV), 64, 1.0, 0, ex)
    assert err.value.status == capi.RA_ERR_UNSUPPORTED


def test_auto_mode_picks_the_route_from_the_shapes():
    from topk_attn_b200 import ops
    from topk_attn_b200.sharded import ShardedTopkAttention
    q, k, v = rand_case(1, 8, 2, 16384, False, seed=6)       # a GQA group of 4: histograms
    op = ShardedTopkAttention(128, 1.0, exchange=one_rank(1, 8, 128))
    out = op.step(q.to(DEV), k.to(DEV), v.to(DEV), 0)
    assert op.mode == "histograms"
    assert torch.allclose(out.float(), ops.topk_attention(q.to(DEV), k.to(DEV), v.to(DEV), 128, 1.0).float(),
                          rtol=1e-2, atol=1e-3)
    q, k, v = rand_case(1, 4, 4, 16384, False, seed=6)       # one query per K row: candidates
    op = ShardedTopkAttention(128, 1.0, exchange=one_rank(1, 4, 128))
    out = op.step(q.to(DEV), k.to(DEV), v.to(DEV), 0)
    torch.cuda.synchronize()
    assert op.mode == "candidates"
    assert torch.allclose(out.float(), ops.topk_attention(q.to(DEV), k.to(DEV), v.to(DEV), 128, 1.0).float(),
                          rtol=1e-2, atol=1e-3)


def _tied_case(N, Hq=8, Hkv=2, every=7, seed=3):
    """All query heads equal, every `every`-th key a copy of one vector along the query: the copies
    score highest and there are far more of them than k, so the k-th score is tied."""
    g = torch.Generator().manual_seed(seed)
    q0 = torch.randn(128, generator=g) / 11.3
    q = q0.expand(1, Hq, 128).contiguous().half()
    k = torch.randn(N, Hkv, 128, generator=g).half()
    k[::every] = (q0 * 40).half()
    v = torch.randn(N, Hkv, 128, generator=g).half()
    return q, k, v


def test_copies_that_fit_the_list_are_shared_out_in_token_order():
    """4286 copies of the best key, 300 wanted: the copies fit in the candidate lists, the CTAs
    share them out in token order through the ordinals of the ordered list."""
    from topk_attn_b200 import ops
    N, topk = 30000, 300
    q, k, v = _tied_case(N)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ex = one_rank(1, 8, topk)
    out, idx, _ = ops.sharded_topk_attention(qd, kd, vd, topk, 1.0, 0, ex, return_indices=True)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    want = torch.arange(0, 7 * topk, 7, dtype=torch.int32, device=DEV).expand(1, 8, topk)
    assert torch.equal(idx.sort(-1).values, want)
    ref = vd[0:7 * topk:7].float().mean(0)               # equal weights over the first 300 copies
    for h in range(8):
        assert torch.allclose(out[0, h].float(), ref[h // 4], rtol=1e-2, atol=2e-3)


def _two_rank_worker(rank, world, port, ret):
    import os
    import torch.distributed as dist
    from topk_attn_b200 import ops
    from topk_attn_b200.sharded import ShardedTopkAttention, make_peer_exchange
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        N, topk = 32768, 2500
        q, k, v = _tied_case(N)
        n = N // world
        qd = q.to(dev)
        ks, vs = k[rank * n:(rank + 1) * n].contiguous().to(dev), v[rank * n:(rank + 1) * n].contiguous().to(dev)
        ex = make_peer_exchange(1, 8, topk, dev, histograms=True)
        assert ex is not None
        op = ShardedTopkAttention(topk, 1.0, exchange=ex)
        out, idx, _ = ops.sharded_topk_attention(qd, ks, vs, topk, 1.0, rank * n, ex, return_indices=True)
        out2 = op.step(qd, ks, vs, rank * n)
        torch.cuda.synchronize()
        ops.check_status(dev)
        ret[rank] = (out.cpu(), out2.cpu(), idx.cpu())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_real_ranks_share_out_copies_of_the_kth_score():
    """4682 copies of the best key lie on both ranks, 2500 are wanted: rank 0 takes all 2341 it has,
    rank 1 the remaining 159 from its lowest ids -- together the lowest k ids, as on one device.
    NVLS is not involved (plain peer stores); every wait is bounded."""
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_two_rank_worker, args=(2, port, ret), nprocs=2, join=True)
    topk = 2500
    assert int((ret[0][2] >= 0).sum(-1)[0, 0]) == 2341 and int((ret[1][2] >= 0).sum(-1)[0, 0]) == 159
    ids = torch.cat([ret[0][2], ret[1][2]], -1)
    got = ids.masked_fill(ids < 0, 2 ** 30).sort(-1).values[..., :topk]
    want = torch.arange(0, 7 * topk, 7, dtype=torch.int32).expand(1, 8, topk)
    assert torch.equal(got, want)
    assert (ids >= 0).sum(-1).eq(topk).all()
    assert torch.equal(ret[0][0], ret[1][0]) and torch.equal(ret[0][0], ret[0][1])
