"""Seeded synthetic inputs for the decode-attention path.

The reference measures on synthetic tensors only (every program regenerates its inputs
from a fixed seed: retrieval_attn/test_ra.py:164-170, gemv_topk.cu:411-447,
baseline_1.py:44-68).  These generators produce the same shapes, layouts and value
distributions for the five benchmark configurations and for the reference's own test
shapes.  Everything is a function of (configuration, seed, device); the CPU and CUDA
generators of torch are different streams, so parity tests generate once and move the
tensors, they never generate twice.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch
from torch import Tensor


@dataclass
class Workload:
    """One decode step's operands.  k/v are [N,Hkv,D] (shared cache) or [Bkv,N,Hkv,D]."""
    name: str
    q: Tensor
    k: Tensor
    v: Tensor
    topk: int = 0
    sm_scale: float = 1.0
    num_segments: int = 1
    centers: Optional[Tensor] = None        # [H, CSZ, D]
    clen: int = 0
    topc: int = 0
    num_splits: int = 0
    extra: Dict[str, object] = field(default_factory=dict)

    @property
    def batch(self) -> int:
        return self.q.size(0)

    @property
    def n_tokens(self) -> int:
        return self.k.size(-3)

    @property
    def bkv(self) -> int:
        return self.k.size(0) if self.k.dim() == 4 else 1

    def kv_bytes_scanned(self) -> int:
        """fp16 bytes of K streamed by one step (every distinct cache once)."""
        return self.bkv * self.n_tokens * self.k.size(-2) * self.k.size(-1) * 2

    def algorithmic_bytes(self) -> int:
        """Bytes one step must move: the K scan plus the selected V rows
        (Bkv*N*Hkv*D*2 + B*Hq*k*D*2); dense attention reads K and V in full."""
        B, Hq, D = self.q.shape
        if self.num_splits:
            return 2 * self.kv_bytes_scanned()
        if self.centers is not None:
            return self.centers.numel() * 2 + 2 * B * Hq * self.topc * self.clen * D * 2
        return self.kv_bytes_scanned() + B * Hq * self.topk * self.num_segments * D * 2


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _randn16(shape, gen, device) -> Tensor:
    """N(0,1) fp16, generated in slabs so the fp32 staging buffer stays small."""
    out = torch.empty(shape, dtype=torch.float16, device=device)
    flat = out.view(-1)
    step = 1 << 26
    for lo in range(0, flat.numel(), step):
        hi = min(flat.numel(), lo + step)
        flat[lo:hi] = torch.randn(hi - lo, generator=gen, device=device, dtype=torch.float32).half()
    return out


def _plant(k: Tensor, qdir: Tensor, frac: float, gen, amp: float = 3.0,
           positions: Optional[Tensor] = None) -> Tensor:
    """K[pos, h] += amp * qdir[h] on a random ``frac`` of positions per head (fp32 add,
    then cast).  k [N,H,D], qdir [H,D] unit vectors.  Returns the planted positions
    [cnt,H]."""
    N, H, D = k.shape
    cnt = int(round(frac * N))
    if positions is None:
        r = torch.rand(N, H, generator=gen, device=k.device)
        positions = r.topk(cnt, dim=0).indices                     # [cnt,H]
    heads = torch.arange(H, device=k.device).view(1, H).expand(cnt, H)
    rows = k[positions, heads].float() + amp * qdir.float().view(1, H, D)
    k[positions, heads] = rows.half()
    return positions


def reference_cpu_case(seed: int = 0, device="cpu") -> Workload:
    """Configuration 0: B=1, 32 heads (MHA), D=128, N=4096, N(0,1) fp16, q scaled by
    1/sqrt(128), global top-256."""
    g = _gen(device, seed)
    q = (torch.randn(1, 32, 128, generator=g, device=device) / math.sqrt(128)).half()
    k = _randn16((4096, 32, 128), g, device)
    v = _randn16((4096, 32, 128), g, device)
    return Workload("cfg0_ref_cpu", q, k, v, topk=256)


def dense_flash_decoding(seed: int = 1, device="cpu", batch: int = 8, n: int = 32768,
                         hq: int = 32, hkv: int = 8, shared_cache: bool = False,
                         num_splits: int = 64) -> Workload:
    """Configuration 1: dense split-KV decode, B=8, 32 query / 8 KV heads, N=32768, 64
    splits.  ``shared_cache`` gives the reference's single [N,Hkv,D] cache."""
    g = _gen(device, seed)
    q = (torch.randn(batch, hq, 128, generator=g, device=device) / math.sqrt(128)).half()
    shape = (n, hkv, 128) if shared_cache else (batch, n, hkv, 128)
    k = _randn16(shape, g, device)
    v = _randn16(shape, g, device)
    return Workload("cfg1_dense", q, k, v, num_splits=num_splits)


def fused_topk_128k(seed: int = 2, device="cpu", batch: int = 4, n: int = 131072,
                    heads: int = 32, topk: int = 2048, shared_cache: bool = False,
                    frac: float = 0.02) -> Workload:
    """Configuration 2 (the headline): B=4, 32 heads MHA, N=131072, k=2048; K,V ~ N(0,1)
    except a random 2 % of positions per (batch row, head) where K += 3 q/|q|.  Each batch
    row has its own cache because planting depends on that row's query; ``shared_cache``
    plants from row 0 into one cache."""
    g = _gen(device, seed)
    q = (torch.randn(batch, heads, 128, generator=g, device=device) / math.sqrt(128)).half()
    qdir = q.float() / q.float().norm(dim=-1, keepdim=True)
    if shared_cache:
        k = _randn16((n, heads, 128), g, device)
        v = _randn16((n, heads, 128), g, device)
        _plant(k, qdir[0], frac, g)
    else:
        k = _randn16((batch, n, heads, 128), g, device)
        v = _randn16((batch, n, heads, 128), g, device)
        for b in range(batch):
            _plant(k[b], qdir[b], frac, g)
    return Workload("cfg2_fused_topk", q, k, v, topk=topk)


def fused_topk_128k_shard(rank: int, world: int, seed: int = 2, device="cpu", batch: int = 4,
                          n_local: int = 131072, heads: int = 32, topk: int = 2048,
                          frac: float = 0.02) -> Workload:
    """One rank's token shard of the headline geometry stretched over ``world`` ranks (weak
    scaling: the context is world * n_local).  The query depends on ``seed`` only, so it is
    identical on every rank; the shard's cache is drawn from ``seed * 2**16 + rank``."""
    g0 = _gen(device, seed)
    q = (torch.randn(batch, heads, 128, generator=g0, device=device) / math.sqrt(128)).half()
    qdir = q.float() / q.float().norm(dim=-1, keepdim=True)
    g = _gen(device, seed * (1 << 16) + rank)
    k = _randn16((batch, n_local, heads, 128), g, device)
    v = _randn16((batch, n_local, heads, 128), g, device)
    for b in range(batch):
        _plant(k[b], qdir[b], frac, g)
    w = Workload("cfg2_token_shard", q, k, v, topk=topk)
    w.extra.update(index_base=rank * n_local, n_shards=world)
    return w


def centroid_retrieval(seed: int = 3, device="cpu", heads: int = 32, csz: int = 2048,
                       clen: int = 64, topc: int = 64, noise: float = 0.3) -> Workload:
    """Configuration 3: B=1, centroids [H,CSZ,D] ~ N(0,1); member keys
    K[c*clen+t, h] = centroid[h,c] + 0.3 N(0,1); V ~ N(0,1); keep the best 64 of 2048
    clusters and attend over their 4096 member tokens."""
    g = _gen(device, seed)
    n = csz * clen
    q = (torch.randn(1, heads, 128, generator=g, device=device) / math.sqrt(128)).half()
    centers = _randn16((heads, csz, 128), g, device)
    k = _randn16((n, heads, 128), g, device)
    k.mul_(noise)
    base = centers.permute(1, 0, 2).unsqueeze(1).expand(csz, clen, heads, 128).reshape(n, heads, 128)
    k.copy_((k.float() + base.float()).half())
    v = _randn16((n, heads, 128), g, device)
    return Workload("cfg3_centroid", q, k, v, centers=centers, clen=clen, topc=topc)


def sharded_long_context_shard(shard: int, n_shards: int, seed: int = 4, device="cpu",
                               n_total: int = 1 << 20, hq: int = 32, hkv: int = 8,
                               topk: int = 4096, frac: float = 0.01) -> Workload:
    """Configuration 4, one token shard: B=1, 32 query / 8 KV heads, N=1 048 576 cut
    contiguously over ``n_shards`` ranks, 1 % planted keys, k=4096.  The query comes from
    ``seed`` alone (identical on every rank); shard r draws its cache from the seed
    ``seed * 2**16 + r`` so ranks generate independently.  Every query head plants into its
    KV head on its own residue class of positions (position % g == head % g), which keeps
    the planted sets of one GQA group disjoint."""
    g0 = _gen(device, seed)
    q = (torch.randn(1, hq, 128, generator=g0, device=device) / math.sqrt(128)).half()
    qdir = q[0].float() / q[0].float().norm(dim=-1, keepdim=True)
    n = n_total // n_shards
    g = _gen(device, seed * (1 << 16) + shard)
    k = _randn16((n, hkv, 128), g, device)
    v = _randn16((n, hkv, 128), g, device)
    grp = hq // hkv
    cnt = int(round(frac * n))
    slots = n // grp
    r = torch.rand(slots, hq, generator=g, device=device)
    pos = r.topk(cnt, dim=0).indices * grp                         # [cnt,hq]
    pos = pos + (torch.arange(hq, device=device) % grp).view(1, hq)
    kvh = (torch.arange(hq, device=device) // grp).view(1, hq).expand(cnt, hq)
    rows = k[pos, kvh].float() + 3.0 * qdir.view(1, hq, 128)
    k[pos, kvh] = rows.half()
    w = Workload("cfg4_sharded", q, k, v, topk=topk)
    w.extra.update(index_base=shard * n, n_total=n_total, n_shards=n_shards)
    return w


def legacy_test_case(batch: int = 4, n: int = 8192, device="cpu") -> Workload:
    """The reference extension's own test inputs (retrieval_attn/test_ra.py:164-170):
    ``torch.manual_seed(0)``, ``randn * 0.1`` in fp16, H=32, D=128, N=8192, 4 chunks."""
    torch.manual_seed(0)
    q = torch.randn(batch, 32, 128, dtype=torch.float16) * 0.1
    k = torch.randn(n, 32, 128, dtype=torch.float16) * 0.1
    v = torch.randn(n, 32, 128, dtype=torch.float16) * 0.1
    return Workload("legacy_ra", q.to(device), k.to(device), v.to(device), num_segments=4)


def two_level_case(device="cpu", hn: int = 32, hd: int = 128, csz: int = 20, clen: int = 2048,
                   topc: int = 5, topk_per_cluster: int = 512) -> Workload:
    """The two-level retrieval inputs of baseline_1.py:44-68 (generator seed 12345,
    centroids U(-0.5,0.5), members = centroid + N(0,0.05), V = K, q U(-0.5,0.5)), returned
    in the token-major [N,H,D] layout the CUDA programs use (gemv_topk.cu:110)."""
    rng = torch.Generator(device="cpu")
    rng.manual_seed(12345)
    centers = torch.empty(hn, csz, hd, dtype=torch.float16).uniform_(-0.5, 0.5, generator=rng)
    noise = torch.empty(hn, csz, clen, hd, dtype=torch.float16)
    noise.normal_(mean=0.0, std=0.05, generator=rng)
    k_hm = centers.unsqueeze(2) + noise
    q = torch.empty(hn, hd, dtype=torch.float16).uniform_(-0.5, 0.5, generator=rng)
    k = k_hm.permute(1, 2, 0, 3).reshape(csz * clen, hn, hd).contiguous()
    w = Workload("two_level", q.unsqueeze(0).to(device), k.to(device), k.clone().to(device),
                 topk=topk_per_cluster, sm_scale=1.0 / math.sqrt(hd),
                 centers=centers.to(device), clen=clen, topc=topc)
    w.extra["k_head_major"] = k_hm
    return w
