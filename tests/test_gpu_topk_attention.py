"""GPU parity of the fused scan + top-k + softmax.V path, called through the C ABI."""
import math

import numpy as np
import pytest
import torch

from oracle import topk_attn_oracle as O
from topk_attn_b200 import workloads as W

from gpu_util import check_topk_attention, rand_case

pytestmark = pytest.mark.gpu


def test_config0_reference_cpu_case():
    w = W.reference_cpu_case()
    check_topk_attention(w.q, w.k, w.v, w.topk, w.sm_scale)


@pytest.mark.parametrize("B,Hq,Hkv,N,k,per_batch", [
    (1, 8, 8, 1024, 64, False),
    (2, 8, 8, 5000, 300, True),        # ragged N: not a multiple of any tile
    (2, 8, 2, 4096, 128, False),       # GQA 4 and a shared cache: 8 queries per K row
    (1, 32, 8, 65536, 1024, False),    # GQA, context split over several clusters
    (4, 32, 32, 16384, 512, False),    # shared cache MHA, batch scored together
    (3, 4, 4, 777, 777, True),         # k == N, odd batch
    (1, 1, 1, 1, 1, False),            # single key
    (1, 2, 1, 130, 1, False),          # k == 1
    (2, 16, 16, 40000, 2048, True),
    (1, 8, 1, 3000, 100, False),       # 8 query heads on one kv head
    (5, 6, 3, 2049, 33, False),        # batch that does not share evenly
    (1, 8, 2, 40000, 2048, False),     # GQA with lists too large for shared memory (global lists)
    (1, 8, 2, 70000, 4096, False),     # the same at k = 4096
    (2, 4, 4, 30000, 3000, False),     # two batch rows on one cache, k not a power of two
])
def test_random_shapes(B, Hq, Hkv, N, k, per_batch):
    q, k_, v = rand_case(B, Hq, Hkv, N, per_batch, seed=N + k)
    check_topk_attention(q, k_, v, k, sm_scale=1.0)


@pytest.mark.parametrize("B,Hq,Hkv,N,k,S,per_batch", [
    (1, 8, 8, 1024, 64, 1, False),
    (2, 8, 2, 4096, 128, 1, False),       # GQA 4
    (3, 4, 4, 777, 777, 1, True),         # k == N
    (1, 2, 1, 130, 1, 1, False),
    (5, 6, 3, 2049, 33, 1, False),        # three batch rows... one cache, two heads per kv head
    (4, 32, 32, 8192, 128, 4, False),     # the reference extension's shape: 4 chunks of 2048
    (2, 8, 8, 4096, 1024, 2, True),
])
def test_short_segments_on_both_paths(B, Hq, Hkv, N, k, S, per_batch, monkeypatch):
    """Segments of at most 4096 keys go through the score-everything kernel; the streaming kernel
    stays reachable in the tuning build of the library (RA_NO_DENSE_SELECT) and must agree with the
    oracle on the same inputs."""
    from topk_attn_b200 import capi
    q, k_, v = rand_case(B, Hq, Hkv, N, per_batch, seed=N + k + S)
    check_topk_attention(q, k_, v, k, sm_scale=0.7, num_segments=S)
    monkeypatch.setenv("RA_NO_DENSE_SELECT", "1")
    with capi.tuning_library():
        check_topk_attention(q, k_, v, k, sm_scale=0.7, num_segments=S)


@pytest.mark.parametrize("scale", [0.25, 1.0 / math.sqrt(128), 2.0])
def test_softmax_scale(scale):
    q, k, v = rand_case(2, 8, 8, 4096, True, seed=5)
    check_topk_attention(q, k, v, 256, sm_scale=scale)


def test_index_base_is_added():
    q, k, v = rand_case(1, 8, 8, 2048, False, seed=7)
    check_topk_attention(q, k, v, 64, index_base=1 << 20)


@pytest.mark.parametrize("topk", [32, 128, 1024])
def test_segmented_selection(topk):
    q, k, v = rand_case(2, 32, 32, 8192, False, seed=topk)
    q = (q.float() * 3).half()
    check_topk_attention(q, k, v, topk, num_segments=4)


def test_ties_everywhere():
    """All keys identical: any k distinct keys are a valid selection.  The output must be the
    attention over exactly the keys that were reported."""
    from topk_attn_b200 import ops
    q = torch.ones(1, 4, 128).half() * 0.1
    k = torch.ones(512, 4, 128).half()
    v = torch.randn(512, 4, 128, generator=torch.Generator().manual_seed(1)).half()
    dev = torch.device("cuda:0")
    out, idx, sc = ops.topk_attention(q.to(dev), k.to(dev), v.to(dev), 100, return_indices=True)
    ops.check_status(dev)
    s = O.full_scores(q, k)
    O.check_index_sets(s, idx.cpu(), 100)
    O.check_topk_scores(s, idx.cpu(), sc.cpu(), 100)
    O.check_output(O.gathered_attention(q, k, v, idx.cpu().long(), 1.0), out)


def test_ascending_scores_worst_case_for_the_filter():
    """Scores rise with the token index, so every key beats the running threshold and the
    candidate lists are cut back as often as they can be."""
    N = 20000
    q = torch.zeros(1, 2, 128)
    q[:, :, 0] = 1.0
    k = torch.zeros(N, 2, 128)
    k[:, 0, 0] = torch.linspace(-4, 4, N)
    k[:, 1, 0] = torch.linspace(4, -4, N)          # descending on the other head
    k[:, :, 1:] = torch.randn(N, 2, 127, generator=torch.Generator().manual_seed(2))
    v = torch.randn(N, 2, 128, generator=torch.Generator().manual_seed(3))
    # fp16 rounds neighbouring scores to the same value, so the boundary of the selection is a
    # run of exact ties: check the selection by the band rule and the output against attention
    # over the keys that were reported
    from topk_attn_b200 import ops
    dev = torch.device("cuda:0")
    q, k, v = q.half(), k.half(), v.half()
    out, idx, sc = ops.topk_attention(q.to(dev), k.to(dev), v.to(dev), 512, return_indices=True)
    ops.check_status(dev)
    s = O.full_scores(q, k)
    O.check_index_sets(s, idx.cpu(), 512)
    O.check_topk_scores(s, idx.cpu(), sc.cpu(), 512)
    O.check_output(O.gathered_attention(q, k, v, idx.cpu().long(), 1.0), out)
    top = idx.cpu()[0, 0].sort().values
    assert top.min().item() >= N - 600


def test_infinite_and_nan_keys():
    """+inf scores are kept first, -inf never; NaN sorts above everything as in torch.topk."""
    from topk_attn_b200 import ops
    q, k, v = rand_case(1, 2, 2, 1024, False, seed=11)
    k[5, 0, :] = float("inf") * torch.sign(q[0, 0].float()).half()     # score +inf on head 0
    k[9, 0, :] = -float("inf") * torch.sign(q[0, 0].float()).half()    # score -inf on head 0
    dev = torch.device("cuda:0")
    idx, sc = ops.gemv_topk(q.to(dev), k.to(dev), 16)
    ops.check_status(dev)
    i0 = set(idx[0, 0].cpu().tolist())
    assert 5 in i0 and 9 not in i0
    s = O.full_scores(q, k)
    ref = set(torch.topk(torch.nan_to_num(s[0, 1], nan=float("inf")), 16).indices.tolist())
    assert set(idx[0, 1].cpu().tolist()) == ref


def test_selection_only_matches_fused_lists():
    from topk_attn_b200 import ops
    q, k, v = rand_case(2, 8, 8, 30000, True, seed=13)
    dev = torch.device("cuda:0")
    idx, sc = ops.gemv_topk(q.to(dev), k.to(dev), 700)
    ops.check_status(dev)
    s = O.full_scores(q, k)
    O.check_index_sets(s, idx.cpu(), 700)
    O.check_topk_scores(s, idx.cpu(), sc.cpu(), 700)


@pytest.mark.parametrize("B,Hq,Hkv,N,topk,S,per_batch", [
    (2, 8, 8, 20000, 512, 1, True),       # streaming kernel, one launch
    (1, 8, 8, 65536, 512, 1, False),      # context cut into parts + second stage
    (1, 32, 8, 40000, 1024, 1, False),    # stored scores
    (4, 32, 32, 8192, 128, 4, False),     # short segments
    (2, 8, 8, 32768, 300, 4, True),       # segmented selection on the streaming kernel
])
def test_repeat_gives_the_same_bits(B, Hq, Hkv, N, topk, S, per_batch):
    """Winners are dealt in a fixed order (ascending token id inside a CTA, CTAs in rank order) and
    ties go to the lower id, so a repeated call returns the same lists in the same order and the
    same output bits."""
    from topk_attn_b200 import ops
    q, k, v = rand_case(B, Hq, Hkv, N, per_batch, seed=17)
    dev = torch.device("cuda:0")
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    a = ops.topk_attention(qd, kd, vd, topk, num_segments=S, return_indices=True)
    b = ops.topk_attention(qd, kd, vd, topk, num_segments=S, return_indices=True)
    ops.check_status(dev)
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    assert torch.equal(a[0], b[0])


def test_ties_go_to_the_lowest_ids():
    """Small-integer scores: hundreds of exact ties at the k-th score.  The selection is the first k
    keys in the order (score descending, id ascending), exactly."""
    from topk_attn_b200 import ops
    N, H, k = 30000, 4, 2000
    g = torch.Generator().manual_seed(9)
    q = torch.zeros(1, H, 128)
    q[:, :, 0] = 1.0
    kk = torch.zeros(N, H, 128)
    kk[:, :, 0] = torch.randint(0, 25, (N, H), generator=g).float()
    v = torch.randn(N, H, 128, generator=g)
    q, kk, v = q.half(), kk.half(), v.half()
    dev = torch.device("cuda:0")
    out, idx, sc = ops.topk_attention(q.to(dev), kk.to(dev), v.to(dev), k, sm_scale=0.05,
                                      return_indices=True)
    ops.check_status(dev)
    s = O.full_scores(q, kk)                                   # exact small integers
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[..., :k]
    assert torch.equal(idx.cpu().long().sort(-1).values, order.sort(-1).values)
    O.check_output(O.gathered_attention(q, kk, v, idx.cpu().long(), 0.05), out)


def test_golden_legacy_outputs(golden_dir):
    """The reference extension's own test shape (B=4, N=8192, 4 chunks) against the vectors its
    torch oracle produced, through the legacy C entry point."""
    import ctypes as C
    import os
    from topk_attn_b200 import capi, ops
    w = W.legacy_test_case()
    g = np.load(os.path.join(golden_dir, "legacy_retrieval_attention.npz"))
    dev = torch.device("cuda:0")
    q, k, v = w.q.to(dev), w.k.to(dev), w.v.to(dev)
    lib = capi.lib()
    for variant, topk in [(0, 32), (1, 128), (2, 256), (3, 512), (4, 1024), (5, 128)]:
        out = torch.zeros_like(q)
        need = lib.ra_legacy_workspace_bytes(4, 8192, topk)
        ws = ops.workspace(need, dev)
        st = lib.ra_legacy_retrieval_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                               out.data_ptr(), 4, 8192, topk, variant,
                                               ws.data_ptr(), ws.numel(),
                                               torch.cuda.current_stream().cuda_stream)
        capi.check(st)
        ops.check_status(dev)
        ref = torch.from_numpy(g[f"out_{topk}"])
        O.check_output(ref, out)
        assert (out.float().cpu() - ref).abs().max().item() < 1e-2      # the reference's own bar


def test_bad_arguments_are_rejected():
    import ctypes as C
    from topk_attn_b200 import capi, ops
    q, k, v = rand_case(1, 8, 8, 1024, False)
    dev = torch.device("cuda:0")
    with pytest.raises(capi.RaError) as e:
        ops.topk_attention(q.to(dev), k.to(dev), v.to(dev), 2000)       # k > N
    assert e.value.status == capi.RA_ERR_INVALID_ARGUMENT
    with pytest.raises(capi.RaError):
        ops.topk_attention(q.to(dev), k.to(dev), v.to(dev), 64, num_segments=3)   # 1024 % 3
    with pytest.raises(capi.RaError):
        ops.topk_attention(q.to(dev), k.to(dev), v.to(dev), 64, sm_scale=0.0)
    p = capi.RaParams()
    assert capi.lib().ra_topk_attention(C.byref(p)) != capi.RA_OK
    assert capi.lib().ra_topk_attention(None) == capi.RA_ERR_INVALID_ARGUMENT


def test_candidate_lists_with_several_queries_per_row(monkeypatch, capfd):
    """The streaming kernel with tensor-core scoring and per-query candidate lists (the route of
    segmented selections on long inputs) stays reachable for a global selection in the tuning
    build; the plan line proves that this path ran."""
    from topk_attn_b200 import capi
    monkeypatch.setenv("RA_NO_SCORE_STORE", "1")
    monkeypatch.setenv("RA_VERBOSE", "1")
    q, k, v = rand_case(1, 8, 2, 50048, False, seed=21)
    with capi.tuning_library():
        check_topk_attention(q, k, v, 1024, sm_scale=0.7)
    err = capfd.readouterr().err
    assert "nq=4" in err and "score store" not in err, err[-400:]


@pytest.mark.parametrize("B,Hq,Hkv,N,k", [
    (1, 8, 8, 20000, 2048),      # context length that is no multiple of the split granularity
    (1, 4, 4, 36000, 4096),
    (1, 16, 2, 2000, 32),        # eight queries per row
    (1, 8, 2, 20000, 500),       # stored scores and histograms
])
def test_exact_size_workspace_is_never_overrun(B, Hq, Hkv, N, k):
    """A caller that allocates exactly ra_workspace_bytes() must be safe: a guard pattern behind
    the workspace stays untouched and the result still matches the oracle."""
    import ctypes as C
    from topk_attn_b200 import capi
    lib = capi.lib()
    dev = torch.device("cuda:0")
    q, k_, v = rand_case(B, Hq, Hkv, N, False, seed=N)
    qd, kd, vd = q.to(dev), k_.to(dev), v.to(dev)
    out = torch.empty_like(qd)
    idx = torch.empty(B, Hq, k, dtype=torch.int32, device=dev)
    sc = torch.empty(B, Hq, k, dtype=torch.float32, device=dev)
    p = capi.RaParams()
    p.q, p.k, p.v, p.out = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr()
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.num_tokens = B, Hq, Hkv, 128, N
    p.kv_batch_stride, p.kv_token_stride, p.kv_head_stride = 0, Hkv * 128, 128
    p.topk, p.num_segments, p.sm_scale = k, 1, 1.0
    p.out_indices, p.out_scores = idx.data_ptr(), sc.data_ptr()
    p.stream = torch.cuda.current_stream().cuda_stream
    need = lib.ra_workspace_bytes(C.byref(p))
    guard = 1 << 20
    buf = torch.zeros(need + guard + 256, dtype=torch.uint8, device=dev)
    off = (-buf.data_ptr()) % 256
    buf[off + need:].fill_(0xAB)
    p.workspace, p.workspace_bytes = buf.data_ptr() + off, need
    capi.check(lib.ra_topk_attention(C.byref(p)))
    capi.check(lib.ra_check_status(p.workspace, p.stream))
    assert bool((buf[off + need:] == 0xAB).all()), "a kernel wrote past ra_workspace_bytes()"
    s = O.full_scores(q, k_)
    ref, _, _ = O.topk_sparse_attention(q, k_, v, k, 1.0, scores=s)
    O.check_index_sets(s, idx.cpu(), k)
    O.check_output(ref, out)
    # a workspace that only holds the status block is refused when the plan needs lists
    p.workspace_bytes = 256
    st = lib.ra_topk_attention(C.byref(p))
    assert st in (capi.RA_OK, capi.RA_ERR_WORKSPACE)
