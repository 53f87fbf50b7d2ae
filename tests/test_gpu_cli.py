"""The stand-alone C++ driver: data generated like the reference's benchmark programs, selection
on the GPU through the C ABI, verified against a double-precision CPU reference with the
reference's own check (exact id sets per (head, cluster rank) slice, order ignored); the modes
that attend (random ids, selection then attention as two calls or as one) also compare the
output with a double-precision softmax.V over the ids used."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "topk_attn_b200", "bin", "ra_verify")


@pytest.mark.parametrize("mode,heads", [("topk", "4"), ("center", "32"), ("fd", "8"), ("s1", "4"),
                                        ("s2", "4"), ("s3", "4")])
def test_cli_verify(mode, heads):
    assert os.path.exists(BIN), "build with python -m topk_attn_b200.build"
    r = subprocess.run([BIN, mode, "--verify", heads, "--iters", "20"], capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASS" in r.stdout and "FAIL" not in r.stdout
    if mode != "fd":
        assert "recall=100.0000%" in r.stdout
    if mode in ("fd", "s1", "s2", "s3"):
        assert "attention max |diff|" in r.stdout
    if mode == "s2":      # the fused and the two-call pipeline agree (`make s2`'s printout)
        assert "[S2] max |fused - unfused|" in r.stdout
