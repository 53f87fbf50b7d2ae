"""The entry point for callers that cannot allocate or lend device memory
(ra_topk_attention_noalloc) must give what ra_topk_attention gives.

It is called straight through the C ABI with a NULL workspace, twice in a row on different
queries: the built-in scratch keeps the first call's candidates, so the second call shows that
stale contents do no harm.  The shape is one whose context is scanned by several clusters, i.e. one
that really writes candidate lists to the scratch.  This file sorts last on purpose: a run that
stops at the first failure has then already run every other test.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(capi, q, k, v, out, topk, scale):
    p = capi.RaParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim = q.size(0), q.size(1), k.size(1), 128
    p.num_tokens = k.size(0)
    p.kv_batch_stride, p.kv_token_stride, p.kv_head_stride = 0, k.size(1) * 128, 128
    p.topk, p.num_segments, p.sm_scale, p.index_base = topk, 1, scale, 0
    p.stream = torch.cuda.current_stream().cuda_stream
    return p


def test_noalloc_matches_workspace_variant_twice():
    from topk_attn_b200 import capi, ops
    lib = capi.lib()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(123)
    B, Hq, Hkv, N, topk, scale = 1, 32, 8, 65536, 512, 0.5
    k = torch.randn(N, Hkv, 128, generator=g).half().to(dev)
    v = torch.randn(N, Hkv, 128, generator=g).half().to(dev)
    for call in range(2):
        q = (torch.randn(B, Hq, 128, generator=g) / math.sqrt(128)).half().to(dev)
        ref = torch.empty_like(q)
        p = _params(capi, q, k, v, ref, topk, scale)
        need = lib.ra_workspace_bytes(C.byref(p))
        assert 0 < need <= (4 << 20)
        ws = ops.workspace(need, dev)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        capi.check(lib.ra_topk_attention(C.byref(p)))
        ops.check_status(dev)

        got = torch.full_like(q, float("nan"))
        p2 = _params(capi, q, k, v, got, topk, scale)      # workspace stays NULL
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
    assert lib.ra_workspace_bytes(C.byref(p)) > (4 << 20)
    assert lib.ra_topk_attention_noalloc(C.byref(p)) == capi.RA_ERR_UNSUPPORTED
    assert b"scratch" in lib.ra_last_cuda_error()
