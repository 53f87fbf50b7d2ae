"""The route for several queries per K row with one global selection: scan_store_kernel stores every
score and a coarse histogram, select_stored_kernel picks the exact top-k from them.  Parity against
the oracle on the three acceptance checks, plus the inputs that stress the selection: scores
crowded into one coarse bin (the bin must be refined by passes over the stored scores) and exact
ties on a scale no candidate list can hold (copies are taken in ascending token order)."""
import math

import pytest
import torch

from oracle import topk_attn_oracle as O

from gpu_util import check_topk_attention, rand_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("B,Hq,Hkv,N,k,per_batch", [
    (1, 32, 8, 65536, 1024, False),    # GQA 4: four queries per row, cluster of CTAs per row in the select
    (4, 32, 32, 16384, 512, False),    # four batch rows on one cache
    (2, 8, 2, 9000, 700, True),        # GQA with a cache per row, ragged N
    (1, 8, 1, 5000, 100, False),       # eight queries per row (shallower pipeline)
    (3, 6, 3, 4500, 4500, False),      # k == N, three rows on one cache, two heads per kv head
    (1, 8, 2, 70000, 4096, False),
    (8, 4, 4, 20001, 33, False),       # eight batch rows on one cache
])
def test_parity(B, Hq, Hkv, N, k, per_batch):
    q, k_, v = rand_case(B, Hq, Hkv, N, per_batch, seed=N + k)
    check_topk_attention(q, k_, v, k, sm_scale=0.8)


def test_plan_line_names_the_route(monkeypatch, capfd):
    from topk_attn_b200 import capi
    monkeypatch.setenv("RA_VERBOSE", "1")
    q, k, v = rand_case(1, 8, 2, 50048, False, seed=21)
    with capi.tuning_library():
        check_topk_attention(q, k, v, 4096, sm_scale=0.7)
    assert "score store" in capfd.readouterr().err


def test_selection_only_and_index_base():
    from topk_attn_b200 import ops
    q, k, v = rand_case(2, 8, 4, 30000, False, seed=5)
    idx, sc = ops.gemv_topk(q.to(DEV), k.to(DEV), 900, index_base=1 << 20)
    ops.check_status(torch.device(DEV))
    s = O.full_scores(q, k)
    O.check_index_sets(s, idx.cpu(), 900, index_base=1 << 20)
    O.check_topk_scores(s, idx.cpu(), sc.cpu(), 900, index_base=1 << 20)


def test_scores_crowded_into_one_coarse_bin():
    """All scores lie in [1.00, 1.06): one bin of the 11-bit histogram holds every key, far more
    than a candidate list, so the bin is refined from the stored scores before the exact select."""
    N, H = 60000, 2
    g = torch.Generator().manual_seed(4)
    q = torch.zeros(2, H, 128)
    q[:, :, 0] = 1.0
    q[1, :, 1] = 0.5
    k = torch.zeros(N, H, 128)
    k[:, :, 0] = 1.0 + 0.03 * torch.rand(N, H, generator=g)
    k[:, :, 1] = 0.06 * torch.rand(N, H, generator=g)
    v = torch.randn(N, H, 128, generator=g)
    # fp16 keys leave only a few dozen distinct scores per head, so the k-th score has thousands
    # of copies and any of them may be kept: band rule for the ids, attention over the reported ids
    from topk_attn_b200 import ops
    q, k, v = q.half(), k.half(), v.half()
    out, idx, sc = ops.topk_attention(q.to(DEV), k.to(DEV), v.to(DEV), 300, return_indices=True)
    ops.check_status(torch.device(DEV))
    s = O.full_scores(q, k)
    O.check_index_sets(s, idx.cpu(), 300)
    O.check_topk_scores(s, idx.cpu(), sc.cpu(), 300)
    O.check_output(O.gathered_attention(q, k, v, idx.cpu().long(), 1.0), out)


def test_ties_beyond_any_list_take_the_lowest_tokens():
    """Every key is identical: the k-th score has N copies.  The selection takes copies in
    ascending token order, so the winners are exactly tokens 0 .. k-1, on every call."""
    from topk_attn_b200 import ops
    N, H, k = 50000, 2, 777
    q = (torch.ones(2, H, 128) * 0.1).half()
    kk = torch.ones(N, H, 128).half()
    v = torch.randn(N, H, 128, generator=torch.Generator().manual_seed(1)).half()
    for _ in range(2):
        out, idx, sc = ops.topk_attention(q.to(DEV), kk.to(DEV), v.to(DEV), k, return_indices=True)
        ops.check_status(torch.device(DEV))
        assert torch.equal(idx.sort(-1).values.cpu(),
                           torch.arange(k, dtype=torch.int32).expand(2, H, k))
        O.check_output(O.gathered_attention(q, kk, v, idx.cpu().long(), 1.0), out)


def test_ties_at_the_cut_inside_one_cta_range():
    """Small-integer scores: thousands of exact ties at the k-th score, few enough to sit in the
    candidate lists.  Index sets obey the band rule and the output is the attention over exactly
    the reported keys."""
    from topk_attn_b200 import ops
    N, H, k = 30000, 4, 2000
    g = torch.Generator().manual_seed(9)
    q = torch.zeros(2, H, 128)
    q[:, :, 0] = 1.0
    kk = torch.zeros(N, H, 128)
    kk[:, :, 0] = torch.randint(0, 40, (N, H), generator=g).float()
    v = torch.randn(N, H, 128, generator=g)
    q, kk, v = q.half(), kk.half(), v.half()
    out, idx, sc = ops.topk_attention(q.to(DEV), kk.to(DEV), v.to(DEV), k, sm_scale=0.05,
                                      return_indices=True)
    ops.check_status(torch.device(DEV))
    s = O.full_scores(q, kk)
    O.check_index_sets(s, idx.cpu(), k)
    O.check_topk_scores(s, idx.cpu(), sc.cpu(), k)
    O.check_output(O.gathered_attention(q, kk, v, idx.cpu().long(), 0.05), out)
