"""GPU parity of the dense split-KV decode kernel against the oracle's dense attention."""
import math

import pytest
import torch

from oracle import topk_attn_oracle as O

from gpu_util import rand_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("B,Hq,Hkv,N,per_batch,splits", [
    (2, 32, 8, 4096, True, 8),        # configuration 1 geometry, small
    (8, 32, 8, 32768, True, 64),      # configuration 1 in full
    (2, 32, 8, 32768, False, 64),     # the reference's shared cache
    (1, 8, 8, 1000, False, 0),        # MHA, ragged N, automatic splits
    (3, 16, 2, 777, True, 5),         # group of 8, splits that do not divide N
    (1, 4, 4, 1, False, 1),           # one key
    (1, 32, 32, 8192, False, 3),      # the reference extension's shape
])
def test_flash_decoding_matches_dense_oracle(B, Hq, Hkv, N, per_batch, splits):
    from topk_attn_b200 import ops
    q, k, v = rand_case(B, Hq, Hkv, N, per_batch, seed=N + splits, scale=3.0)
    scale = 0.8
    out = ops.flash_decoding(q.to(DEV), k.to(DEV), v.to(DEV), scale, splits)
    ops.check_status(torch.device(DEV))
    O.check_output(O.dense_attention(q, k, v, scale), out)


def test_flash_decoding_equals_topk_with_k_equal_n():
    from topk_attn_b200 import ops
    q, k, v = rand_case(2, 8, 2, 2048, True, seed=4, scale=3.0)
    a = ops.flash_decoding(q.to(DEV), k.to(DEV), v.to(DEV), 0.5)
    b = ops.topk_attention(q.to(DEV), k.to(DEV), v.to(DEV), 2048, 0.5)
    ops.check_status(torch.device(DEV))
    O.check_output(a.float().cpu(), b)
