"""The torch extension keeps the reference module's name and entry points
(retrieval_attn/bind.cpp:726-757) and passes the reference's own test: every variant and every K
against the torch oracle with max |diff| < 1e-2 (retrieval_attn/test_ra.py:162-352)."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import topk_attn_oracle as O
from topk_attn_b200 import workloads as W

pytestmark = pytest.mark.gpu

VARIANTS = ["retrieval_attention", "retrieval_attention_global", "retrieval_attention_pipelined",
            "retrieval_attention_pipelined_global", "retrieval_attention_two_kernels",
            "retrieval_attention_gather_baseline"]


@pytest.fixture(scope="module")
def ra_ops():
    import topk_attn_b200
    return topk_attn_b200.load_extension()


def test_module_has_the_reference_entry_points(ra_ops):
    for v in VARIANTS:
        for k in (32, 128, 256, 512, 1024):
            assert callable(getattr(ra_ops, f"{v}_{k}"))


@pytest.mark.parametrize("topk", [32, 128, 256, 512, 1024])
def test_reference_test_loop(ra_ops, golden_dir, topk):
    w = W.legacy_test_case()
    g = np.load(os.path.join(golden_dir, "legacy_retrieval_attention.npz"))
    ref = torch.from_numpy(g[f"out_{topk}"])
    dev = torch.device("cuda:0")
    q, k, v = w.q.to(dev), w.k.to(dev), w.v.to(dev)
    for name in VARIANTS:
        out = torch.zeros(4, 32, 128, device=dev, dtype=torch.float16)
        getattr(ra_ops, f"{name}_{topk}")(q, k, v, out)
        torch.cuda.synchronize()
        diff = (out.float().cpu() - ref).abs().max().item()
        assert diff < 1e-2, (name, topk, diff)
        O.check_output(ref, out)


def test_general_entry_points(ra_ops):
    from gpu_util import rand_case
    q, k, v = rand_case(2, 8, 2, 10000, True, seed=3)
    dev = torch.device("cuda:0")
    out = torch.empty(2, 8, 128, device=dev, dtype=torch.float16)
    idx, sc = ra_ops.retrieval_attention(q.to(dev), k.to(dev), v.to(dev), out, 256, 1, 0.5, 0, True)
    s = O.full_scores(q, k)
    ref, _, _ = O.topk_sparse_attention(q, k, v, 256, 0.5, scores=s)
    O.check_index_sets(s, idx.cpu(), 256)
    O.check_topk_scores(s, idx.cpu(), sc.cpu(), 256)
    O.check_output(ref, out)
    idx2, sc2 = ra_ops.gemv_topk(q.to(dev), k.to(dev), 256)
    O.check_index_sets(s, idx2.cpu(), 256)


def test_bad_tensors_raise(ra_ops):
    dev = torch.device("cuda:0")
    q = torch.zeros(4, 32, 128, device=dev, dtype=torch.float16)
    k = torch.zeros(8192, 32, 128, device=dev, dtype=torch.float16)
    out = torch.zeros_like(q)
    with pytest.raises(RuntimeError):
        ra_ops.retrieval_attention_128(q.float(), k, k, out)          # wrong dtype
    with pytest.raises(RuntimeError):
        ra_ops.retrieval_attention_128(q.cpu(), k, k, out)            # wrong device
    with pytest.raises(RuntimeError):
        ra_ops.retrieval_attention_128(q, k[:, :16], k[:, :16], out)  # not contiguous / heads
