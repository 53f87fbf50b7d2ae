"""The benchmark configurations at their full sizes.

The CPU oracle needs tens of seconds per call at these sizes, so the checks here are properties
that hold at any size and are evaluated with plain torch operations on the device, a scorer that
shares no code with the library:

* threshold property of an exact top-k: with s = q.K^T in fp32, every key scoring more than
  1e-3 above the k-th largest value is selected, no selected key scores more than 1e-3 below it,
  the ids are distinct and in range (the acceptance rule of the reference's own verifier,
  gemv_topk.cu:138-170, with the tolerance band of the parity tests);
* the returned scores equal s at the returned ids within 1e-3;
* the output equals softmax(scale * s[ids]) . V[ids] recomputed from the returned ids
  (rtol 1e-2 / atol 1e-3), and the (max, sum) pair matches;
* splitting the token axis into logical shards and merging gives the same selection and output
  (the sequence-sharded path at its full length);
* dense decoding equals torch's softmax over the whole cache.
"""
import pytest
import torch

from topk_attn_b200 import workloads as W

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
BAND = 1e-3


def device_scores(q, k):
    """fp32 q.K^T [B,Hq,N] by torch on the device; k [N,Hkv,D] or [B,N,Hkv,D]."""
    B, Hq, D = q.shape
    Hkv = k.size(-2)
    grp = Hq // Hkv
    rows = []
    for b in range(B):
        kb = k[b] if k.dim() == 4 else k
        per_head = []
        for h in range(Hkv):                                     # bounded fp32 staging
            kh = kb[:, h, :].float()                             # [N,D]
            qh = q[b, h * grp:(h + 1) * grp].float()             # [grp,D]
            per_head.append(qh @ kh.t())
        rows.append(torch.cat(per_head, 0))
    return torch.stack(rows)


def check_selection(s, idx, sc, topk, index_base=0):
    B, Hq, N = s.shape
    ids = idx.long() - index_base
    assert ids.min() >= 0 and ids.max() < N
    srt = ids.sort(-1).values
    assert (srt[..., 1:] != srt[..., :-1]).all(), "duplicate ids"
    kth = s.topk(topk, -1).values[..., -1:]
    got = s.gather(-1, ids)
    assert (got >= kth - BAND).all(), "a selected key lies below the band"
    member = torch.zeros_like(s, dtype=torch.bool).scatter_(-1, ids, True)
    assert not ((s > kth + BAND) & ~member).any(), "a key above the band was missed"
    assert (got - sc).abs().max() <= BAND
    return got


def check_attention(got, idx, v, out, lse, scale, index_base=0):
    B, Hq, k = got.shape
    Hkv = v.size(-2)
    grp = Hq // Hkv
    ids = idx.long() - index_base
    m = (got * scale).max(-1, keepdim=True).values
    w = torch.exp(got * scale - m)
    ref = torch.empty(B, Hq, 128, device=got.device)
    for b in range(B):
        vb = v[b] if v.dim() == 4 else v
        for h in range(Hq):
            rows = vb[ids[b, h], h // grp].float()               # [k,D]
            ref[b, h] = (w[b, h].unsqueeze(0) @ rows).squeeze(0) / w[b, h].sum()
    assert torch.allclose(out.float(), ref, rtol=1e-2, atol=1e-3)
    if lse is not None:
        assert torch.allclose(lse[..., 0], m.squeeze(-1), atol=1e-3, rtol=1e-4)
        assert torch.allclose(lse[..., 1], w.sum(-1), atol=1e-3, rtol=2e-3)


@pytest.mark.parametrize("shared_cache", [False, True])
def test_headline_configuration(shared_cache):
    """B=4, 32 heads, N=131072, k=2048 with 2 % planted keys: one cache per row (the headline) and
    one shared cache (four queries scored per K row)."""
    from topk_attn_b200 import ops
    w = W.fused_topk_128k(device=DEV, shared_cache=shared_cache)
    out, idx, sc, lse = ops.topk_attention(w.q, w.k, w.v, w.topk, w.sm_scale,
                                           return_indices=True, return_lse=True)
    ops.check_status(torch.device(DEV))
    s = device_scores(w.q, w.k)
    got = check_selection(s, idx, sc, w.topk)
    check_attention(got, idx, w.v, out, lse, w.sm_scale)
    # the kept keys are the upper tail of the score distribution
    assert (got.min(-1).values > s.mean(-1) + 1.5 * s.std(-1)).all()


def test_dense_configuration():
    """B=8, 32 query / 8 KV heads, N=32768, 64 splits, against torch's dense softmax."""
    from topk_attn_b200 import ops
    w = W.dense_flash_decoding(device=DEV)
    out = ops.flash_decoding(w.q, w.k, w.v, 1.0, w.num_splits)
    ops.check_status(torch.device(DEV))
    s = device_scores(w.q, w.k)
    p = torch.softmax(s, -1)
    ref = torch.empty(8, 32, 128, device=DEV)
    for b in range(8):
        for h in range(8):
            ref[b, 4 * h:4 * h + 4] = p[b, 4 * h:4 * h + 4] @ w.v[b, :, h, :].float()
    assert torch.allclose(out.float(), ref, rtol=1e-2, atol=1e-3)


def test_sharded_configuration_on_logical_shards():
    """N=1 048 576, 8 KV heads, k=4096: the whole cache in one call, and cut into 8 token shards
    that go through select -> merge (ownership window) -> log-sum-exp combine."""
    from topk_attn_b200 import ops
    G = 8
    shards = [W.sharded_long_context_shard(r, G, device=DEV) for r in range(G)]
    q, topk = shards[0].q, shards[0].topk
    k = torch.cat([s.k for s in shards])
    v = torch.cat([s.v for s in shards])
    out, idx, sc, lse = ops.topk_attention(q, k, v, topk, 1.0, return_indices=True, return_lse=True)
    s = device_scores(q, k)
    got = check_selection(s, idx, sc, topk)
    check_attention(got, idx, v, out, lse, 1.0)

    n = k.size(0) // G
    cand = [ops.gemv_topk(q, shards[r].k, topk, index_base=r * n) for r in range(G)]
    cand_idx = torch.stack([c[0] for c in cand]).contiguous()
    cand_sc = torch.stack([c[1] for c in cand]).contiguous()
    parts = torch.stack([ops.merge_attend(cand_sc, cand_idx, shards[r].v, topk, 1.0, r * n)
                         for r in range(G)]).contiguous()
    out_sh = ops.lse_combine(parts)
    _, gidx, gsc = ops.merge_attend(cand_sc, cand_idx, shards[0].v, topk, 1.0, 0,
                                    return_indices=True)
    ops.check_status(torch.device(DEV))
    check_selection(s, gidx, gsc, topk)
    assert torch.allclose(out_sh.float(), out.float(), rtol=1e-2, atol=1e-3)


def test_centroid_configuration():
    """32 heads, 2048 clusters of 64: best 64 clusters by centroid score (threshold property on the
    centroid scores), member expansion, attention over the 4096 members."""
    from topk_attn_b200 import ops
    w = W.centroid_retrieval(device=DEV)
    res = ops.center_only_topk(w.q, w.centers, w.topc, w.clen, k=w.k, v=w.v, sm_scale=1.0)
    ops.check_status(torch.device(DEV))
    cids, ids, out = res[0], res[1], res[2]
    cs = torch.einsum("bhd,hcd->bhc", w.q.float(), w.centers.float())
    kth = cs.topk(w.topc, -1).values[..., -1:]
    gotc = cs.gather(-1, cids.long())
    assert (gotc >= kth - BAND).all()
    member = torch.zeros_like(cs, dtype=torch.bool).scatter_(-1, cids.long(), True)
    assert not ((cs > kth + BAND) & ~member).any()
    expect = (cids.long().unsqueeze(-1) * w.clen + torch.arange(w.clen, device=DEV)).flatten(-2)
    assert torch.equal(ids.long().sort(-1).values, expect.sort(-1).values)
    s = device_scores(w.q, w.k)
    got = s.gather(-1, ids.long())
    check_attention(got, ids, w.v, out, None, 1.0)
