"""topk_attn_b200 — decode-time top-k sparse attention for NVIDIA B200 (sm_100a).

The package is a thin host layer over hand-written CUDA kernels reached through the C ABI of
``include/topk_attn_b200.h``.  ``ops`` holds the torch-tensor operators, ``capi`` the ctypes
binding, ``workloads`` the seeded synthetic inputs, ``build`` the nvcc build.  There is no CPU
or PyTorch fallback: importing an operator without the built library raises.
"""
import importlib.util
import os

__all__ = ["load_extension"]


def load_extension():
    """Import the in-tree torch extension ``retrieval_attention_cpp`` (the reference's module
    name, retrieval_attn/setup_ra.py:8).  Raises ImportError if it has not been built."""
    import torch  # noqa: F401  (libtorch must be loaded first)
    from . import build
    path = build.extension_path()
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: run `python -m topk_attn_b200.build`")
    spec = importlib.util.spec_from_file_location("retrieval_attention_cpp", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
