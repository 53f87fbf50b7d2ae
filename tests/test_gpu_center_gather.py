"""GPU parity of centroid-only retrieval and gathered attention through the C ABI."""
import math

import numpy as np
import pytest
import torch

from oracle import topk_attn_oracle as O
from topk_attn_b200 import workloads as W

from gpu_util import rand_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def check_cluster_sets(cs, cids, topc, band=1e-3):
    """cluster ids against the oracle's centroid scores [B,H,CSZ] by the band rule"""
    O.check_index_sets(cs, cids, topc, band=band)


@pytest.mark.parametrize("csz,clen,topc,heads,batch", [
    (2048, 64, 64, 32, 1),      # configuration 3
    (1024, 128, 64, 32, 1),     # center_only_topk/gemv_topk.cu:31-37
    (256, 8, 16, 4, 3),
    (100, 5, 100, 2, 1),        # keep every cluster
])
def test_center_only_selection_and_attention(csz, clen, topc, heads, batch):
    from topk_attn_b200 import ops
    w = W.centroid_retrieval(csz=csz, clen=clen, topc=topc, heads=heads)
    if batch > 1:
        g = torch.Generator().manual_seed(9)
        w.q = (torch.randn(batch, heads, 128, generator=g) / math.sqrt(128)).half()
    scale = 1.0 / math.sqrt(128)
    cids, tids, out = ops.center_only_topk(w.q.to(DEV), w.centers.to(DEV), topc, clen,
                                           w.k.to(DEV), w.v.to(DEV), scale)
    ops.check_status(torch.device(DEV))
    ids_ref, top_ref, cs = O.center_only_topk(w.q, w.centers, topc, clen)
    check_cluster_sets(cs, cids.cpu(), topc)
    # token ids: clusters appear in descending score order, members ascending inside a cluster
    t = tids.cpu().long().view(batch, heads, topc, clen)
    assert torch.equal(t - t[..., :1], torch.arange(clen).expand_as(t))
    got_clusters = t[..., 0] // clen
    assert torch.equal(got_clusters.sort(-1).values, cids.cpu().long().sort(-1).values)
    sc_of = torch.gather(cs, -1, got_clusters)
    assert bool((sc_of[..., :-1] >= sc_of[..., 1:] - 1e-6).all()) or topc == 1
    # same per-head sets as the reference's CPU check (order ignored) when no near tie exists
    ref_out = O.gathered_attention(w.q, w.k, w.v, tids.cpu().long(), scale)
    O.check_output(ref_out, out)
    kth = torch.topk(cs, topc, dim=-1).values
    if topc < csz and float((kth[..., -1] - torch.topk(cs, topc + 1, dim=-1).values[..., -1]).min()) > 2e-3:
        assert torch.equal(tids.cpu().long().sort(-1).values, ids_ref.sort(-1).values)
        out_ref2, _ = O.center_only_attention(w.q, w.centers, w.k, w.v, topc, clen, scale)
        O.check_output(out_ref2, out)


def test_center_only_selection_without_attention():
    from topk_attn_b200 import ops
    w = W.centroid_retrieval(csz=512, clen=16, topc=32, heads=8)
    cids, tids = ops.center_only_topk(w.q.to(DEV), w.centers.to(DEV), 32, 16)
    ops.check_status(torch.device(DEV))
    ids_ref, top_ref, cs = O.center_only_topk(w.q, w.centers, 32, 16)
    check_cluster_sets(cs, cids.cpu(), 32)
    assert torch.equal(tids.cpu().long().sort(-1).values, ids_ref.sort(-1).values)


def expected_rank_order(cs, topc):
    """ids by descending score, ties by ascending id: the order both centroid paths promise"""
    csz = cs.size(-1)
    order = torch.argsort(cs.double() * 1.0, dim=-1, descending=True, stable=True)
    return order[..., :topc]


@pytest.mark.parametrize("csz,clen,topc,heads,batch", [
    (37, 3, 5, 3, 2),          # odd everything, members not a multiple of four
    (1000, 6, 1000, 2, 1),     # keep all, slices that do not divide
    (4096, 4, 300, 2, 2),      # eight CTAs per row
    (8192, 2, 1024, 1, 1),     # largest table the shared-memory kernel takes
    (9000, 2, 16, 2, 1),       # beyond it: the streaming kernel takes over
])
def test_center_selection_rank_order_exact_on_exact_scores(csz, clen, topc, heads, batch):
    """Centroids and queries with small integer entries: every score is exact in fp16 x fp32, so
    the expected order is unambiguous, and ties are plentiful."""
    from topk_attn_b200 import ops
    g = torch.Generator().manual_seed(csz + topc)
    q = torch.randint(-2, 3, (batch, heads, 128), generator=g).half()
    centers = torch.randint(-2, 3, (heads, csz, 128), generator=g).half()
    cids, tids = ops.center_only_topk(q.to(DEV), centers.to(DEV), topc, clen)
    ops.check_status(torch.device(DEV))
    cs = torch.einsum("bhd,hcd->bhc", q.float(), centers.float())
    want = expected_rank_order(cs, topc)
    t = tids.cpu().long().view(batch, heads, topc, clen)
    assert torch.equal(t - t[..., :1], torch.arange(clen).expand_as(t))
    got_scores = torch.gather(cs, -1, t[..., 0] // clen)
    want_scores = torch.gather(cs, -1, want)
    assert torch.equal(got_scores, want_scores)               # same scores rank by rank
    assert torch.equal(cids.cpu().long().sort(-1).values, (t[..., 0] // clen).sort(-1).values)
    if csz <= 8192:
        assert torch.equal(t[..., 0] // clen, want)           # ties broken by the lower id
        assert torch.equal(cids.cpu().long(), want)


def test_center_selection_all_scores_equal():
    from topk_attn_b200 import ops
    q = torch.zeros(1, 4, 128).half()
    centers = torch.randn(4, 700, 128).half()
    cids, tids = ops.center_only_topk(q.to(DEV), centers.to(DEV), 9, 4)
    ops.check_status(torch.device(DEV))
    assert torch.equal(cids.cpu().long(), torch.arange(9).expand(1, 4, 9))
    assert torch.equal(tids.cpu().long(), torch.arange(36).expand(1, 4, 36))


def test_center_selection_paths_agree(monkeypatch):
    """The shared-memory kernel and the streaming kernel give the same clusters."""
    from topk_attn_b200 import ops
    w = W.centroid_retrieval(csz=1024, clen=128, topc=64, heads=32)
    q, c = w.q.to(DEV), w.centers.to(DEV)
    a_c, a_t = ops.center_only_topk(q, c, 64, 128)
    monkeypatch.setenv("RA_NO_CENTER_SELECT", "1")
    b_c, b_t = ops.center_only_topk(q, c, 64, 128)
    ops.check_status(torch.device(DEV))
    assert torch.equal(a_c.sort(-1).values, b_c.sort(-1).values)
    assert torch.equal(a_t, b_t)


@pytest.mark.parametrize("B,Hq,Hkv,N,S,per_batch,shared_idx", [
    (1, 32, 32, 40960, 2560, False, True),     # flash_decoding.cu:32-37 shape
    (2, 8, 2, 5000, 777, True, False),
    (3, 4, 4, 300, 1, False, False),
    (1, 32, 32, 131072, 12800, False, True),   # center_only_topk/baselines.cu:47-55
])
def test_gathered_attention(B, Hq, Hkv, N, S, per_batch, shared_idx):
    from topk_attn_b200 import ops
    q, k, v = rand_case(B, Hq, Hkv, N, per_batch, seed=S)
    g = torch.Generator().manual_seed(S)
    shape = (Hq, S) if shared_idx else (B, Hq, S)
    idx = torch.stack([torch.randperm(N, generator=g)[:S] for _ in range(math.prod(shape[:-1]))])
    idx = idx.view(*shape).int()
    scale = 1.0 / math.sqrt(128)
    out = ops.gathered_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx.to(DEV), scale)
    ops.check_status(torch.device(DEV))
    O.check_output(O.gathered_attention(q, k, v, idx.long(), scale), out)


def test_two_level_golden_output(golden_dir):
    """Attention over the reference's own two-level selection (baseline_1.py) reproduces the
    output it printed."""
    import os
    from topk_attn_b200 import ops
    g = np.load(os.path.join(golden_dir, "two_level_baseline_1.npz"))
    hn, hd, csz, clen, topc, tpk = [int(x) for x in g["dims"]]
    w = W.two_level_case(hn=hn, hd=hd, csz=csz, clen=clen, topc=topc, topk_per_cluster=tpk)
    idx = torch.from_numpy(g["kv_indices"]).int()
    out = ops.gathered_attention(w.q.to(DEV), w.k.to(DEV), w.v.to(DEV), idx.to(DEV), w.sm_scale)
    ops.check_status(torch.device(DEV))
    ref = torch.from_numpy(g["output"]).unsqueeze(0)
    assert torch.allclose(out.float().cpu(), ref, rtol=1e-2, atol=2e-3)


def test_out_of_range_id_is_reported_not_read():
    from topk_attn_b200 import capi, ops
    q, k, v = rand_case(1, 2, 2, 256, False, seed=1)
    idx = torch.tensor([[1, 2, 3, 100000], [4, 5, 6, 7]], dtype=torch.int32)
    ops.gathered_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx.to(DEV), 1.0)
    with pytest.raises(capi.RaError) as e:
        ops.check_status(torch.device(DEV))
    assert e.value.status == capi.RA_ERR_DEVICE_CHECK
    # the status word is sticky until cleared by the owner of the workspace
    ops.workspace(256, torch.device(DEV))[:256].zero_()
    ops.check_status(torch.device(DEV))
