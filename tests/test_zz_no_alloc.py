"""The entry point for callers that cannot allocate or lend device memory
(ra_topk_attention_noalloc) must give what ra_topk_attention gives.

It is called straight through the C ABI with a NULL workspace, twice in a row on different
queries: the built-in scratch keeps the first call's contents, so the second call shows that
stale contents do no harm.  The shapes cover every route that writes to the scratch: a context
scanned by several clusters (candidate lists), short segments (winner lists of the
score-everything kernel), several queries per K row (stored scores and histograms), and a shape
whose scratch need sits just under the built-in array's size.  This file sorts last on purpose: a
run that stops at the first failure has then already run every other test.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

NOALLOC_BYTES = 4 << 20


def _params(capi, q, k, v, out, topk, scale, segments=1):
    p = capi.RaParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim = q.size(0), q.size(1), k.size(-2), 128
    p.num_tokens = k.size(-3)
    p.kv_batch_stride = k.size(1) * k.size(2) * 128 if k.dim() == 4 else 0
    p.kv_token_stride, p.kv_head_stride = k.size(-2) * 128, 128
    p.topk, p.num_segments, p.sm_scale, p.index_base = topk, segments, scale, 0
    p.stream = torch.cuda.current_stream().cuda_stream
    return p


@pytest.mark.parametrize("B,Hq,Hkv,N,topk,segments,per_batch,near_limit", [
    (1, 8, 8, 65536, 512, 1, False, False),     # one query per row, context cut into parts
    (4, 32, 32, 8192, 128, 4, False, False),    # the extension's shape: 4 short segments
    (1, 8, 2, 16384, 256, 1, False, False),     # four queries per row: stored scores
    (2, 16, 16, 16384, 1000, 1, True, True),    # 256 + 32*16*1000*8 bytes: just under 4 MiB
])
def test_noalloc_matches_workspace_variant_twice(B, Hq, Hkv, N, topk, segments, per_batch, near_limit):
    from topk_attn_b200 import capi, ops
    lib = capi.lib()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(123 + N + topk)
    shape = (B, N, Hkv, 128) if per_batch else (N, Hkv, 128)
    k = torch.randn(shape, generator=g).half().to(dev)
    v = torch.randn(shape, generator=g).half().to(dev)
    scale = 0.5
    for call in range(2):
        q = (torch.randn(B, Hq, 128, generator=g) / math.sqrt(128)).half().to(dev)
        ref = torch.empty_like(q)
        p = _params(capi, q, k, v, ref, topk, scale, segments)
        need = lib.ra_workspace_bytes(C.byref(p))
        assert 0 < need <= NOALLOC_BYTES
        if near_limit:
            assert need > NOALLOC_BYTES - (128 << 10)
        ws = ops.workspace(need, dev)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        capi.check(lib.ra_topk_attention(C.byref(p)))
        ops.check_status(dev)

        got = torch.full_like(q, float("nan"))
        p2 = _params(capi, q, k, v, got, topk, scale, segments)      # workspace stays NULL
        capi.check(lib.ra_topk_attention_noalloc(C.byref(p2)))
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # same tolerance as the parity tests: rtol 1e-2 / atol 1e-3
        err = (got.float() - ref.float()).abs()
        assert bool((err <= 1e-3 + 1e-2 * ref.float().abs()).all()), (call, err.max().item())


def test_noalloc_refuses_shapes_beyond_its_scratch():
    from topk_attn_b200 import capi
    lib = capi.lib()
    dev = torch.device("cuda:0")
    q = torch.zeros(4, 32, 128, dtype=torch.float16, device=dev)
    k = torch.zeros(131072, 32, 128, dtype=torch.float16, device=dev)
    out = torch.empty_like(q)
    p = _params(capi, q, k, k, out, 2048, 1.0)
    assert lib.ra_workspace_bytes(C.byref(p)) > NOALLOC_BYTES
    assert lib.ra_topk_attention_noalloc(C.byref(p)) == capi.RA_ERR_UNSUPPORTED
    assert b"scratch" in lib.ra_last_cuda_error()
