"""CPU tests: the oracle against the golden vectors produced by the reference's own torch
functions (tests/golden/make_golden.py), and the oracle's internal consistency."""
import hashlib
import math
import os

import numpy as np
import pytest
import torch

from oracle import topk_attn_oracle as O
from topk_attn_b200 import workloads as W


def sha(t):
    return hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()


@pytest.fixture(scope="module")
def legacy():
    return W.legacy_test_case()


def test_legacy_inputs_match_golden_digests(legacy, golden_dir):
    g = np.load(os.path.join(golden_dir, "legacy_retrieval_attention.npz"))
    assert sha(legacy.q) == str(g["sha_q"])
    assert sha(legacy.k) == str(g["sha_k"])
    assert sha(legacy.v) == str(g["sha_v"])


@pytest.mark.parametrize("topk", [32, 128, 256, 512, 1024])
def test_legacy_oracle_matches_reference_output(legacy, golden_dir, topk):
    g = np.load(os.path.join(golden_dir, "legacy_retrieval_attention.npz"))
    ref = torch.from_numpy(g[f"out_{topk}"])
    got = O.legacy_retrieval_attention(legacy.q.float(), legacy.k.float(), legacy.v.float(), topk)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-7)
    # the general formulation with 4 segments and scale 1 is the same function
    out, idx, sc = O.topk_sparse_attention(legacy.q, legacy.k, legacy.v, topk, 1.0, num_segments=4)
    # a different fp32 summation order may flip a tie at the K-th score of a (batch, head)
    # row; such rows stay inside the acceptance tolerance, all others agree tightly
    O.check_output(ref, out)
    rows_off = ((out - ref).abs().amax(-1) > 1e-5).sum().item()
    assert rows_off <= 2
    assert idx.shape == (4, 32, 4 * topk)


def test_two_level_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "two_level_baseline_1.npz"))
    hn, hd, csz, clen, topc, tpk = [int(x) for x in g["dims"]]
    w = W.two_level_case(hn=hn, hd=hd, csz=csz, clen=clen, topc=topc, topk_per_cluster=tpk)
    assert sha(w.q[0]) == str(g["sha_q"])
    assert sha(w.centers) == str(g["sha_centers"])
    assert sha(w.extra["k_head_major"]) == str(g["sha_k"])
    top = O.coarse_topk(w.q[0], w.centers, topc)
    assert np.array_equal(top.numpy(), g["top_clusters"])
    idx = O.fine_topk(w.q[0], w.k, top, clen, tpk)
    ref_idx = torch.from_numpy(g["kv_indices"]).long()
    # same per-(head, cluster-rank) sets, order ignored (verify_gpu_vs_cpu, gemv_topk.cu:138-170)
    a = idx.view(hn, topc, tpk).sort(-1).values
    b = ref_idx.view(hn, topc, tpk).sort(-1).values
    assert torch.equal(a, b)
    out = O.gathered_attention(w.q, w.k, w.v, ref_idx, 1.0 / math.sqrt(hd))[0]
    ref = torch.from_numpy(g["output"])
    assert torch.allclose(out, ref, rtol=2e-3, atol=2e-3)   # the reference rounds to fp16


def test_center_only_matches_coarse_topk():
    w = W.centroid_retrieval(csz=256, clen=8, topc=16, heads=4)
    ids, top, cs = O.center_only_topk(w.q, w.centers, 16, 8)
    assert torch.equal(top[0].sort(-1).values, O.coarse_topk(w.q[0], w.centers, 16).sort(-1).values)
    assert ids.shape == (1, 4, 128)
    assert torch.equal(ids[0, 0, :8], top[0, 0, 0] * 8 + torch.arange(8))


def small(seed=0, B=2, Hq=8, Hkv=8, N=1024, per_batch=False):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, Hq, 128, generator=g) / math.sqrt(128)).half()
    shape = (B, N, Hkv, 128) if per_batch else (N, Hkv, 128)
    k = torch.randn(shape, generator=g).half()
    v = torch.randn(shape, generator=g).half()
    return q, k, v


@pytest.mark.parametrize("per_batch", [False, True])
@pytest.mark.parametrize("hkv", [8, 2])
def test_topk_equals_dense_when_k_is_n(per_batch, hkv):
    q, k, v = small(Hkv=hkv, per_batch=per_batch, N=256)
    out, idx, sc = O.topk_sparse_attention(q, k, v, 256, 0.7)
    assert torch.allclose(out, O.dense_attention(q, k, v, 0.7), rtol=1e-4, atol=1e-5)
    assert torch.allclose(out, O.gathered_attention(q, k, v, idx, 0.7), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("splits", [1, 3, 64])
def test_split_kv_equals_dense(splits):
    q, k, v = small(Hkv=2, per_batch=True, N=1000)
    out, *_ = O.split_kv_attention(q, k, v, 0.5, splits)
    assert torch.allclose(out, O.dense_attention(q, k, v, 0.5), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("shards", [1, 2, 8])
def test_sharded_equals_single(shards):
    q, k, v = small(B=1, Hq=8, Hkv=2, N=2048)
    ref, ridx, rsc = O.topk_sparse_attention(q, k, v, 128, 1.0)
    out, gi, gs = O.sharded_topk_attention(q, list(k.chunk(shards)), list(v.chunk(shards)), 128, 1.0)
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-5)
    assert torch.equal(gi.sort(-1).values, ridx.sort(-1).values)


def test_checkers_accept_oracle_and_reject_errors():
    q, k, v = small(N=512)
    s = O.full_scores(q, k)
    out, idx, sc = O.topk_sparse_attention(q, k, v, 64, 1.0)
    O.check_index_sets(s, idx, 64)
    O.check_topk_scores(s, idx, sc, 64)
    O.check_output(out, out.half())
    bad = idx.clone()
    worst = s.argmin(-1)
    bad[..., 0] = worst
    with pytest.raises(AssertionError):
        O.check_index_sets(s, bad, 64)
    dup = idx.clone()
    dup[..., 1] = dup[..., 0]
    with pytest.raises(AssertionError):
        O.check_index_sets(s, dup, 64)
    with pytest.raises(AssertionError):
        O.check_output(out, out + 0.1)
    with pytest.raises(AssertionError):
        O.check_topk_scores(s, idx, sc + 0.01, 64)


def test_band_rule_tolerates_near_ties():
    q, k, v = small(B=1, Hq=1, Hkv=1, N=256)
    s = O.full_scores(q, k)
    out, idx, sc = O.topk_sparse_attention(q, k, v, 16, 1.0)
    # make the 17th key a near tie of the 16th, then swap them in the selection
    order = s[0, 0].argsort(descending=True)
    s2 = s.clone()
    s2[0, 0, order[16]] = s2[0, 0, order[15]] - 5e-4
    swapped = idx.clone()
    swapped[0, 0][swapped[0, 0] == order[15]] = order[16]
    O.check_index_sets(s2, swapped, 16)
