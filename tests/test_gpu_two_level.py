"""Two-level retrieval (coarse top clusters, fine top-k inside each) through the C ABI, against
the vectors of the reference's own torch pipeline (baseline_1.py) and against the oracle."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import topk_attn_oracle as O
from topk_attn_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_reference_pipeline_vectors(golden_dir):
    """Same per-(head, cluster rank) index sets as baseline_1.py's fine_topk (order inside a
    slice ignored, as verify_gpu_vs_cpu does, gemv_topk.cu:138-170) and the output it printed."""
    from topk_attn_b200 import ops
    g = np.load(os.path.join(golden_dir, "two_level_baseline_1.npz"))
    hn, hd, csz, clen, topc, tpk = [int(x) for x in g["dims"]]
    w = W.two_level_case(hn=hn, hd=hd, csz=csz, clen=clen, topc=topc, topk_per_cluster=tpk)
    cids, idx, sc, out = ops.two_level_topk(w.q.to(DEV), w.centers.to(DEV), w.k.to(DEV), topc, clen,
                                            tpk, v=w.v.to(DEV), sm_scale=w.sm_scale)
    ops.check_status(torch.device(DEV))
    assert np.array_equal(cids.cpu().numpy()[0], g["top_clusters"])
    got = idx.cpu().long().view(hn, topc, tpk).sort(-1).values
    ref = torch.from_numpy(g["kv_indices"]).long().view(hn, topc, tpk).sort(-1).values
    assert torch.equal(got, ref)
    assert torch.allclose(out.float().cpu()[0], torch.from_numpy(g["output"]), rtol=1e-2, atol=2e-3)


@pytest.mark.parametrize("B,H,csz,clen,topc,tpk,per_batch", [
    (1, 32, 32, 1280, 5, 512, False),     # gemv_topk.cu:21-28
    (2, 4, 16, 200, 3, 200, True),        # keep whole clusters, ragged cluster length
    (3, 8, 64, 96, 8, 7, False),          # clusters shorter than a tile
    (1, 2, 4, 4096, 1, 1024, False),      # a single cluster
])
def test_against_oracle(B, H, csz, clen, topc, tpk, per_batch):
    from topk_attn_b200 import ops
    g = torch.Generator().manual_seed(csz + clen)
    n = csz * clen
    q = (torch.randn(B, H, 128, generator=g) / math.sqrt(128)).half()
    centers = torch.randn(H, csz, 128, generator=g).half()
    shape = (B, n, H, 128) if per_batch else (n, H, 128)
    k = (torch.randn(shape, generator=g) * 0.3).half()
    base = centers.permute(1, 0, 2).unsqueeze(1).expand(csz, clen, H, 128).reshape(n, H, 128)
    k = (k.float() + base.float()).half()
    v = torch.randn(shape, generator=g).half()
    scale = 0.3
    cids, idx, sc, out = ops.two_level_topk(q.to(DEV), centers.to(DEV), k.to(DEV), topc, clen, tpk,
                                            v=v.to(DEV), sm_scale=scale)
    ops.check_status(torch.device(DEV))
    _, _, cs = O.center_only_topk(q, centers, topc, clen)
    O.check_index_sets(cs, cids.cpu(), topc)
    chosen = cids.cpu().long()
    sc_of = torch.gather(cs, -1, chosen)
    assert bool((sc_of[..., :-1] >= sc_of[..., 1:]).all()) or topc == 1     # rank order
    # fine level: band rule inside every chosen cluster
    s = O.full_scores(q, k).view(B, H, csz, clen)
    sel = torch.gather(s, 2, chosen.unsqueeze(-1).expand(-1, -1, -1, clen)).reshape(B, H, topc * clen)
    local = idx.cpu().long().view(B, H, topc, tpk) - chosen.unsqueeze(-1) * clen
    assert bool(((local >= 0) & (local < clen)).all())
    local = local + (torch.arange(topc) * clen).view(1, 1, topc, 1)
    O.check_index_sets(sel, local.reshape(B, H, -1), tpk, num_segments=topc)
    O.check_topk_scores(sel, local.reshape(B, H, -1), sc.cpu(), tpk, num_segments=topc)
    O.check_output(O.gathered_attention(q, k, v, idx.cpu().long(), scale), out)
