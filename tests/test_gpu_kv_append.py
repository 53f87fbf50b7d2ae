"""The decode-loop step before the attention: append a token to the caches, keep centroids as the
running mean of their members, then attend over the grown cache."""
import math

import pytest
import torch

from oracle import topk_attn_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_append_then_attend_shared_cache_with_centroids():
    from topk_attn_b200 import ops
    g = torch.Generator().manual_seed(8)
    H, cap, clen = 8, 512, 16
    k = torch.zeros(cap, H, 128, dtype=torch.float16, device=DEV)
    v = torch.zeros_like(k)
    centers = torch.zeros(H, cap // clen, 128, dtype=torch.float16, device=DEV)
    rows_k = torch.randn(300, H, 128, generator=g).half()
    rows_v = torch.randn(300, H, 128, generator=g).half()
    for pos in range(300):
        ops.kv_append(k, v, rows_k[pos].to(DEV), rows_v[pos].to(DEV), pos, centers, clen)
    assert torch.equal(k[:300].cpu(), rows_k) and torch.equal(v[:300].cpu(), rows_v)
    assert not k[300:].any()
    full = 300 // clen
    ref_c = rows_k[:full * clen].float().view(full, clen, H, 128).mean(1).permute(1, 0, 2)
    assert torch.allclose(centers[:, :full].float().cpu(), ref_c, atol=4e-3, rtol=1e-2)
    tail = rows_k[full * clen:300].float().mean(0)
    assert torch.allclose(centers[:, full].float().cpu(), tail, atol=4e-3, rtol=1e-2)
    q = (torch.randn(2, H, 128, generator=g) / math.sqrt(128)).half()
    kk, vv = k[:300].contiguous(), v[:300].contiguous()
    out = ops.topk_attention(q.to(DEV), kk, vv, 64)
    ops.check_status(torch.device(DEV))
    ref, _, _ = O.topk_sparse_attention(q, rows_k, rows_v, 64, 1.0)
    O.check_output(ref, out)


def test_append_per_sequence_caches_and_bounds():
    from topk_attn_b200 import capi, ops
    g = torch.Generator().manual_seed(9)
    B, H, cap = 3, 4, 64
    k = torch.zeros(B, cap, H, 128, dtype=torch.float16, device=DEV)
    v = torch.zeros_like(k)
    nk = torch.randn(B, H, 128, generator=g).half().to(DEV)
    nv = torch.randn(B, H, 128, generator=g).half().to(DEV)
    ops.kv_append(k, v, nk, nv, 5)
    assert torch.equal(k[:, 5], nk) and torch.equal(v[:, 5], nv)
    assert not k[:, :5].any() and not k[:, 6:].any()
    with pytest.raises(capi.RaError):
        ops.kv_append(k, v, nk, nv, cap)


def test_l2_persistence_window_can_be_set_and_removed():
    """ra_l2_persist marks a shared cache as persisting in L2 for the current stream (consecutive
    decode steps of one sequence); results do not change, and the window can be removed again."""
    from topk_attn_b200 import ops
    from gpu_util import rand_case
    q, k, v = rand_case(1, 8, 8, 4096, False, seed=4)
    dev = torch.device("cuda:0")
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    ref = ops.topk_attention(qd, kd, vd, 128)
    ops.l2_persist(kd)
    for _ in range(3):
        out = ops.topk_attention(qd, kd, vd, 128)
    ops.l2_persist(None)
    ops.check_status(dev)
    assert torch.equal(out, ref)


def test_stream_read_probe_runs():
    """The read-only stream used by the bench to measure the device's streaming rate."""
    from topk_attn_b200 import ops
    dev = torch.device("cuda:0")
    buf = torch.ones(1 << 22, dtype=torch.int32, device=dev)
    ops.stream_read_probe(buf)
    torch.cuda.synchronize()
    ops.check_status(dev)
