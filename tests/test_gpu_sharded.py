"""Sequence-sharded path on one GPU: G logical shards are run one after another through the same
C-ABI calls the ranks make (select, merge with an ownership window, log-sum-exp combine); the
result must equal the single-device operator and the oracle on the concatenated cache."""
import pytest
import torch

from oracle import topk_attn_oracle as O

from gpu_util import rand_case

pytestmark = pytest.mark.gpu


def run_shards(q, k, v, topk, scale, G):
    from topk_attn_b200 import ops
    dev = torch.device("cuda:0")
    n = k.size(-3) // G
    qd = q.to(dev)
    ks = [k[..., r * n:(r + 1) * n, :, :].contiguous().to(dev) for r in range(G)]
    vs = [v[..., r * n:(r + 1) * n, :, :].contiguous().to(dev) for r in range(G)]
    cand = [ops.gemv_topk(qd, ks[r], topk, index_base=r * n) for r in range(G)]
    cand_idx = torch.stack([c[0] for c in cand]).contiguous()
    cand_sc = torch.stack([c[1] for c in cand]).contiguous()
    parts = torch.stack([ops.merge_attend(cand_sc, cand_idx, vs[r], topk, scale, r * n)
                         for r in range(G)]).contiguous()
    out = ops.lse_combine(parts)
    _, gidx, gsc = ops.merge_attend(cand_sc, cand_idx, vs[0], topk, scale, 0, return_indices=True)
    ops.check_status(dev)
    return out, gidx, gsc


@pytest.mark.parametrize("G", [1, 2, 8])
@pytest.mark.parametrize("B,Hq,Hkv,N,topk,per_batch", [
    (1, 32, 8, 32768, 512, False),
    (2, 8, 8, 16384, 1024, True),
])
def test_logical_shards_match_oracle(G, B, Hq, Hkv, N, topk, per_batch):
    q, k, v = rand_case(B, Hq, Hkv, N, per_batch, seed=G + N)
    out, gidx, gsc = run_shards(q, k, v, topk, 0.9, G)
    s = O.full_scores(q, k)
    ref, _, _ = O.topk_sparse_attention(q, k, v, topk, 0.9, scores=s)
    O.check_index_sets(s, gidx.cpu(), topk)
    O.check_topk_scores(s, gidx.cpu(), gsc.cpu(), topk)
    O.check_output(ref, out)


def test_lse_combine_matches_oracle():
    from topk_attn_b200 import ops
    g = torch.Generator().manual_seed(3)
    parts = torch.randn(5, 3, 4, 130, generator=g)
    parts[..., 128] = parts[..., 128].abs() + 0.1
    parts[1, ..., 128] = 0.0            # a rank that owns no winner
    parts[1, ..., :128] = 0.0
    ref = O.lse_combine(parts[..., :128], parts[..., 129], parts[..., 128])
    out = ops.lse_combine(parts.cuda().contiguous())
    assert torch.allclose(out.float().cpu(), ref, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("G", [2, 8])
def test_ties_straddling_shards_give_one_global_set(G, monkeypatch):
    """Small-integer scores with hundreds of exact ties at the k-th score, spread over all shards.
    Every rank merges the same candidates, so every rank must pick the same winners: the first k keys
    in the order (score descending, id ascending) -- the unsharded operator's choice.  Both forms of
    the merge kernel (one CTA per row, a cluster per row) must agree on the set and on its order, and
    the owned winners of all ranks add up to exactly k distinct ids."""
    from topk_attn_b200 import capi, ops
    dev = torch.device("cuda:0")
    N, H, topk = 16384, 4, 1000
    g = torch.Generator().manual_seed(31)
    q = torch.zeros(1, H, 128)
    q[:, :, 0] = 1.0
    k = torch.zeros(N, H, 128)
    k[:, :, 0] = torch.randint(0, 20, (N, H), generator=g).float()
    v = torch.randn(N, H, 128, generator=g)
    q, k, v = q.half(), k.half(), v.half()
    n = N // G
    qd = q.to(dev)
    ks = [k[r * n:(r + 1) * n].contiguous().to(dev) for r in range(G)]
    vs = [v[r * n:(r + 1) * n].contiguous().to(dev) for r in range(G)]
    cand = [ops.gemv_topk(qd, ks[r], topk, index_base=r * n) for r in range(G)]
    cand_idx = torch.stack([c[0] for c in cand]).contiguous()
    cand_sc = torch.stack([c[1] for c in cand]).contiguous()
    _, gidx, gsc = ops.merge_attend(cand_sc, cand_idx, vs[0], topk, 0.05, 0, return_indices=True)
    monkeypatch.setenv("RA_FORCE_MERGE_CLUSTER", "8")
    with capi.tuning_library():
        _, cidx, csc = ops.merge_attend(cand_sc, cand_idx, vs[0], topk, 0.05, 0, return_indices=True)
    ops.check_status(dev)
    assert torch.equal(gidx, cidx) and torch.equal(gsc, csc)
    s = O.full_scores(q, k)
    expect = torch.sort(s, dim=-1, descending=True, stable=True).indices[..., :topk]
    assert torch.equal(gidx.cpu().long().sort(-1).values, expect.sort(-1).values)
    owned = sum(int(((gidx >= r * n) & (gidx < (r + 1) * n)).sum()) for r in range(G))
    assert owned == H * topk
    # the sharded output equals the unsharded operator's on the same keys
    parts = torch.stack([ops.merge_attend(cand_sc, cand_idx, vs[r], topk, 0.05, r * n)
                         for r in range(G)]).contiguous()
    out = ops.lse_combine(parts)
    ref = ops.topk_attention(qd, k.to(dev), v.to(dev), topk, 0.05)
    ops.check_status(dev)
    assert torch.allclose(out.float(), ref.float(), rtol=1e-2, atol=1e-3)
