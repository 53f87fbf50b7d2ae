"""Helpers for the GPU parity tests: run an operator through the C ABI and apply the three
acceptance checks against the CPU oracle."""
import math

import torch

from oracle import topk_attn_oracle as O
from topk_attn_b200 import workloads as W


def rand_case(B, Hq, Hkv, N, per_batch, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, Hq, 128, generator=g) * scale / math.sqrt(128)).half()
    shape = (B, N, Hkv, 128) if per_batch else (N, Hkv, 128)
    k = torch.randn(shape, generator=g).half()
    v = torch.randn(shape, generator=g).half()
    return q, k, v


def check_topk_attention(q, k, v, topk, sm_scale=1.0, num_segments=1, index_base=0):
    """q,k,v CPU fp16.  Runs the fused operator on cuda:0 and checks index sets (band rule),
    top-k scores (1e-3) and outputs (rtol 1e-2 / atol 1e-3) against the oracle."""
    from topk_attn_b200 import ops
    dev = torch.device("cuda:0")
    out, idx, sc, lse = ops.topk_attention(q.to(dev), k.to(dev), v.to(dev), topk, sm_scale,
                                           num_segments, index_base, return_indices=True,
                                           return_lse=True)
    ops.check_status(dev)
    s = O.full_scores(q, k)
    ref, ridx, rsc = O.topk_sparse_attention(q, k, v, topk, sm_scale, num_segments, scores=s)
    O.check_index_sets(s, idx.cpu(), topk, num_segments=num_segments, index_base=index_base)
    O.check_topk_scores(s, idx.cpu(), sc.cpu(), topk, num_segments=num_segments,
                        index_base=index_base)
    O.check_output(ref, out)
    # log-sum-exp pair: (max of scaled kept scores, sum of exp)
    m_ref = rsc.max(-1).values * sm_scale
    l_ref = torch.exp(rsc * sm_scale - m_ref.unsqueeze(-1)).sum(-1)
    assert torch.allclose(lse[..., 0].cpu(), m_ref, atol=1e-3, rtol=1e-4)
    assert torch.allclose(lse[..., 1].cpu(), l_ref, atol=1e-3, rtol=2e-3)
    return out, idx, sc
