#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ by EXECUTING the reference's own torch
functions from a checkout of the reference project (read-only, never copied).

    python tests/golden/make_golden.py --reference /path/to/topk_attn

Two sources are run:

* ``reference_retrieval_attention`` (retrieval_attn/test_ra.py:88-160).  That file
  compiles and loads a CUDA extension at import time (:80-85), so the function is pulled
  out of the parsed source with ``ast`` and executed with the module constants it reads
  (:10-14); nothing else of the file runs.  Inputs follow run_test (:164-170):
  ``torch.manual_seed(0)``, ``randn * 0.1`` in fp16, B = 4 — generated on the CPU.  The
  function is evaluated on the fp32 up-cast of those fp16 values (so the stored vectors do
  not depend on a CPU half-precision matmul) for K in {32, 128, 256, 512, 1024}.
* ``generate_data``, ``coarse_topk``, ``fine_topk``, ``compute_attention`` imported from
  baseline_1.py (:44-110) and run as they are (CPU, fp16 base dtype).

Outputs (numpy ``.npz``): the results plus SHA-256 digests of the inputs, so that the
replaying test can prove it regenerated identical inputs without the reference present.
"""
from __future__ import annotations

import argparse
import ast
import hashlib
import importlib.util
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()


def legacy_inputs(batch: int = 4, n: int = 8192, heads: int = 32, dim: int = 128):
    """The tensors of run_test (retrieval_attn/test_ra.py:164-170), on the CPU."""
    torch.manual_seed(0)
    q = torch.randn(batch, heads, dim, dtype=torch.float16) * 0.1
    k = torch.randn(n, heads, dim, dtype=torch.float16) * 0.1
    v = torch.randn(n, heads, dim, dtype=torch.float16) * 0.1
    return q, k, v


def load_reference_oracle(ref_root: str):
    path = os.path.join(ref_root, "retrieval_attn", "test_ra.py")
    tree = ast.parse(open(path).read(), filename=path)
    consts, fn = [], None
    for node in tree.body:
        if isinstance(node, ast.Assign) and all(isinstance(t, ast.Name) for t in node.targets) \
                and isinstance(node.value, ast.Constant):
            consts.append(node)
        if isinstance(node, ast.FunctionDef) and node.name == "reference_retrieval_attention":
            fn = node
    assert fn is not None, "reference_retrieval_attention not found"
    mod = ast.Module(body=consts + [fn], type_ignores=[])
    env = {"torch": torch}
    exec(compile(mod, path, "exec"), env)
    return env["reference_retrieval_attention"]


def make_legacy(ref_root: str) -> None:
    ref_fn = load_reference_oracle(ref_root)
    q, k, v = legacy_inputs()
    out = {"sha_q": digest(q), "sha_k": digest(k), "sha_v": digest(v)}
    for topk in (32, 128, 256, 512, 1024):
        o = ref_fn(q.float(), k.float(), v.float(), topk)
        out[f"out_{topk}"] = o.numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "legacy_retrieval_attention.npz"), **out)
    print("legacy_retrieval_attention.npz written")


def make_two_level(ref_root: str) -> None:
    path = os.path.join(ref_root, "baseline_1.py")
    spec = importlib.util.spec_from_file_location("ref_baseline_1", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    torch.manual_seed(2025)                              # baseline_1.py:128
    q, k, v, centers = mod.generate_data(torch.device("cpu"), dtype=torch.float16)
    top = mod.coarse_topk(q, centers)
    idx = mod.fine_topk(q, k, top)
    o = mod.compute_attention(q, k, v, idx)
    np.savez_compressed(
        os.path.join(HERE, "two_level_baseline_1.npz"),
        sha_q=digest(q), sha_k=digest(k), sha_centers=digest(centers),
        top_clusters=top.numpy().astype(np.int32), kv_indices=idx.numpy().astype(np.int32),
        output=o.float().numpy(),
        dims=np.array([mod.HN, mod.HD, mod.CSZ, mod.CLEN, mod.TOPC, mod.TOPK_PER_CLUSTER]))
    print("two_level_baseline_1.npz written")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    a = ap.parse_args()
    torch.set_num_threads(os.cpu_count() or 1)
    make_legacy(a.reference)
    make_two_level(a.reference)
