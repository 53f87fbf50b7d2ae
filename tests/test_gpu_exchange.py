"""The peer-store exchange of the sharded step on one GPU.

Real ranks store into each other's receive buffers over NVLink and wait for each other's flags.
On one device the same kernels run on G logical ranks whose "peer" buffers are plain tensors of that
device, phase by phase (all selects and pushes, then all merges, then all combines), so that no
kernel ever waits for a launch that comes after it.  The wait's time limit is tested with a flag
that nothing sets: the kernel returns, the status word reports the timeout, and the context stays
usable.
"""
import pytest
import torch

from oracle import topk_attn_oracle as O

from gpu_util import rand_case

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def logical_ranks(G, B, Hq, topk, timeout_s=2.0):
    from topk_attn_b200.sharded import PeerExchange, ShardedTopkAttention
    words = PeerExchange.layout(G, B, Hq, topk)[-1]
    bufs = [torch.zeros(words, dtype=torch.int32, device=DEV) for _ in range(G)]
    base = [b.data_ptr() for b in bufs]
    exs = [PeerExchange(bufs[r], base, r, G, B, Hq, topk, timeout_s) for r in range(G)]
    return exs


@pytest.mark.parametrize("G,B,Hq,Hkv,N,topk", [
    (4, 1, 8, 2, 32768, 512),
    (2, 2, 4, 4, 16384, 300),
    (8, 1, 32, 8, 65536, 1024),
])
def test_logical_ranks_exchange_by_peer_stores(G, B, Hq, Hkv, N, topk):
    from topk_attn_b200 import ops
    from topk_attn_b200.sharded import ShardedTopkAttention
    q, k, v = rand_case(B, Hq, Hkv, N, False, seed=G + N)
    n = N // G
    qd = q.to(DEV)
    ks = [k[r * n:(r + 1) * n].contiguous().to(DEV) for r in range(G)]
    vs = [v[r * n:(r + 1) * n].contiguous().to(DEV) for r in range(G)]
    exs = logical_ranks(G, B, Hq, topk)
    shard = [ShardedTopkAttention(topk, 0.9, exchange=exs[r]) for r in range(G)]
    outs = None
    for step in range(2):        # twice: the buffers and flags are reused with the next epoch
        for r in range(G):       # phase 1: every rank proposes and pushes
            shard[r]._buffers(B, Hq, DEV)
            idx, sc = shard[r].local_candidates(qd, ks[r], r * n)
            assert idx.data_ptr() == exs[r].cand_idx[r].data_ptr()     # written in place
            exs[r].push_candidates()
        for r in range(G):       # phase 2: flags are up, merge and push the partial
            exs[r].wait_candidates()
            shard[r].backend.merge_partial(exs[r].cand_sc, exs[r].cand_idx, vs[r], topk, 0.9, r * n,
                                           out=exs[r].partials[r], own_part=r)
            exs[r].push_partial()
        outs = []
        for r in range(G):       # phase 3: combine
            exs[r].wait_partials()
            outs.append(shard[r].backend.combine(exs[r].partials))
        ops.check_status(DEV)
        assert all(int(e.epoch.item()) == step + 2 for e in exs)
    s = O.full_scores(q, k)
    ref, _, _ = O.topk_sparse_attention(q, k, v, topk, 0.9, scores=s)
    for r in range(G):
        O.check_output(ref, outs[r])
        assert torch.equal(outs[r], outs[0])
        # every rank received every rank's scores (ids stay home: a rank mixes only its own proposals)
        assert torch.equal(exs[r].cand[:, 0], exs[0].cand[:, 0])


@pytest.mark.parametrize("G,B,Hq,Hkv,N,topk", [
    (4, 1, 8, 2, 32768, 512),
    (8, 1, 32, 8, 65536, 4096),      # 32768 candidates per row: ids stay in global memory
    (8, 2, 32, 8, 65536, 4096),
    (2, 4, 8, 8, 16384, 1024),
])
def test_logical_ranks_with_the_exchange_fused_into_merge_and_combine(G, B, Hq, Hkv, N, topk):
    """The product's step: the merge kernel waits for the candidate flags itself and stores its
    partial rows into every peer's slot, the combine kernel waits for the partial flags and ends the
    step by advancing the epoch."""
    from topk_attn_b200 import ops
    from topk_attn_b200.sharded import ShardedTopkAttention
    q, k, v = rand_case(B, Hq, Hkv, N, False, seed=G + N + 1)
    n = N // G
    qd = q.to(DEV)
    ks = [k[r * n:(r + 1) * n].contiguous().to(DEV) for r in range(G)]
    vs = [v[r * n:(r + 1) * n].contiguous().to(DEV) for r in range(G)]
    exs = logical_ranks(G, B, Hq, topk)
    shard = [ShardedTopkAttention(topk, 0.9, exchange=exs[r]) for r in range(G)]
    for step in range(2):
        bufs = [shard[r]._buffers(B, Hq, DEV) for r in range(G)]
        for r in range(G):
            idx, sc = shard[r].local_candidates(qd, ks[r], r * n)
            shard[r].exchange_candidates(idx, sc)
        for r in range(G):
            shard[r].merge_and_exchange(bufs[r][0], bufs[r][1], bufs[r][2], vs[r], r * n)
        outs = [shard[r].backend.combine(bufs[r][2], exchange=exs[r]) for r in range(G)]
        ops.check_status(DEV)
        assert all(int(e.epoch.item()) == step + 2 for e in exs)
    s = O.full_scores(q, k)
    ref, _, _ = O.topk_sparse_attention(q, k, v, topk, 0.9, scores=s)
    for r in range(G):
        O.check_output(ref, outs[r])
        assert torch.equal(outs[r], outs[0])
        assert torch.equal(exs[r].partials, exs[0].partials)   # every rank received every partial


def test_one_rank_step_replays_from_a_cuda_graph():
    from topk_attn_b200 import ops
    from topk_attn_b200.sharded import ShardedTopkAttention
    q, k, v = rand_case(1, 8, 2, 20000, False, seed=3)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ex = logical_ranks(1, 1, 8, 256)[0]
    op = ShardedTopkAttention(256, 1.0, exchange=ex)
    replay = op.capture(qd, kd, vd, 0)
    ref = ops.topk_attention(qd, kd, vd, 256, 1.0)
    for _ in range(3):
        out = replay()
    op.check_graph_status()
    assert torch.allclose(out.float(), ref.float(), rtol=1e-2, atol=1e-3)
    q2 = (q * 0.5).to(DEV)
    qd.copy_(q2)                                            # a new query in the captured buffer
    out = replay()
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), ops.topk_attention(q2, kd, vd, 256, 1.0).float(),
                          rtol=1e-2, atol=1e-3)


def test_wait_runs_out_and_reports_a_timeout():
    """A flag that no rank ever sets: the bounded wait gives up after its (short) limit, the kernel
    returns, ra_check_status says RA_ERR_DEVICE_TIMEOUT, and after the status word is cleared the
    next call works."""
    import time
    from topk_attn_b200 import capi, ops
    ex = logical_ranks(2, 1, 8, 64, timeout_s=0.005)[0]     # rank 1 never pushes
    ops.check_status(DEV)
    ex.push_candidates()
    t0 = time.perf_counter()
    ex.wait_candidates()
    with pytest.raises(capi.RaError) as e:
        ops.check_status(DEV)
    assert e.value.status == capi.RA_ERR_DEVICE_TIMEOUT
    assert time.perf_counter() - t0 < 1.0
    ops.workspace(256, DEV)[:4].zero_()                      # the status bits are sticky
    q, k, v = rand_case(1, 8, 8, 4096, False, seed=1)
    out = ops.topk_attention(q.to(DEV), k.to(DEV), v.to(DEV), 64)
    ops.check_status(DEV)
    assert torch.isfinite(out.float()).all()


def test_pipeline_wait_runs_out_and_reports_a_timeout(monkeypatch):
    """The bounded wait on a TMA pipeline barrier of the scan kernel: in the tuning build the
    producer can be told to leave its last tile out (no access out of place, the consumers simply
    never see that tile arrive).  With a limit of a few milliseconds the kernel returns, the status
    word reports the timeout, and after it is cleared the next call is fine."""
    import time
    from topk_attn_b200 import capi, ops
    q, k, v = rand_case(1, 8, 8, 8192, False, seed=2)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    monkeypatch.setenv("RA_DEBUG_FLAGS", "32")
    monkeypatch.setenv("RA_WAIT_LIMIT_MS", "5")
    with capi.tuning_library():
        ops.check_status(DEV)
        t0 = time.perf_counter()
        ops.topk_attention(qd, kd, vd, 64)
        with pytest.raises(capi.RaError) as e:
            ops.check_status(DEV)
        assert e.value.status == capi.RA_ERR_DEVICE_TIMEOUT
        assert time.perf_counter() - t0 < 2.0
        ops.workspace(256, DEV)[:4].zero_()
        monkeypatch.delenv("RA_DEBUG_FLAGS")
        out = ops.topk_attention(qd, kd, vd, 64)
        ops.check_status(DEV)
    ref = ops.topk_attention(qd, kd, vd, 64)
    ops.check_status(DEV)
    assert torch.equal(out, ref)


def test_cluster_merge_with_separate_wait_and_push(monkeypatch):
    """When the candidates of a row do not fit one CTA the merge runs as a cluster of CTAs and the
    exchange steps run as kernels of their own around it; forced here through the tuning build."""
    from topk_attn_b200 import capi, ops
    from topk_attn_b200.sharded import ShardedTopkAttention
    G, B, Hq, Hkv, N, topk = 4, 1, 8, 2, 32768, 512
    q, k, v = rand_case(B, Hq, Hkv, N, False, seed=77)
    n = N // G
    qd = q.to(DEV)
    ks = [k[r * n:(r + 1) * n].contiguous().to(DEV) for r in range(G)]
    vs = [v[r * n:(r + 1) * n].contiguous().to(DEV) for r in range(G)]
    monkeypatch.setenv("RA_FORCE_MERGE_CLUSTER", "8")
    with capi.tuning_library():
        exs = logical_ranks(G, B, Hq, topk)
        shard = [ShardedTopkAttention(topk, 0.9, exchange=exs[r]) for r in range(G)]
        bufs = [shard[r]._buffers(B, Hq, DEV) for r in range(G)]
        for r in range(G):
            idx, sc = shard[r].local_candidates(qd, ks[r], r * n)
            shard[r].exchange_candidates(idx, sc)
        for r in range(G):
            shard[r].merge_and_exchange(bufs[r][0], bufs[r][1], bufs[r][2], vs[r], r * n)
        outs = [shard[r].backend.combine(bufs[r][2], exchange=exs[r]) for r in range(G)]
        ops.check_status(DEV)
    s = O.full_scores(q, k)
    ref, _, _ = O.topk_sparse_attention(q, k, v, topk, 0.9, scores=s)
    for r in range(G):
        O.check_output(ref, outs[r])
        assert torch.equal(outs[r], outs[0])
