"""ctypes binding of the C ABI declared in include/topk_attn_b200.h.

The library is the product: if it has not been built (``python -m topk_attn_b200.build``) the
import of any operator fails loudly; there is no Python or CPU fallback.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libtopk_attn_b200.so")
TUNING_LIB_PATH = os.path.join(_PKG, "lib", "libtopk_attn_b200_tuning.so")

RA_OK = 0
RA_ERR_INVALID_ARGUMENT = 1
RA_ERR_UNSUPPORTED = 2
RA_ERR_WORKSPACE = 3
RA_ERR_CUDA = 4
RA_ERR_DEVICE_TIMEOUT = 5
RA_ERR_DEVICE_CHECK = 7


class RaParams(C.Structure):
    """Mirror of ``struct ra_params``."""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("num_tokens", C.c_int32),
        ("kv_batch_stride", C.c_int64), ("kv_token_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("topk", C.c_int32), ("num_segments", C.c_int32), ("sm_scale", C.c_float),
        ("index_base", C.c_int32),
        ("out_indices", C.c_void_p), ("out_scores", C.c_void_p), ("out_lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class RaExchangeHooks(C.Structure):
    """Mirror of ``struct ra_exchange_hooks``."""
    _fields_ = [
        ("wait_flags", C.c_void_p), ("num_wait_flags", C.c_int32), ("epoch", C.c_void_p),
        ("wait_timeout_ns", C.c_uint64),
        ("peer_partials", C.POINTER(C.c_void_p)), ("peer_flags", C.POINTER(C.c_void_p)),
        ("num_peers", C.c_int32), ("done_counter", C.c_void_p),
    ]


class RaShardExchange(C.Structure):
    """Mirror of ``struct ra_shard_exchange``."""
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("bufs", C.POINTER(C.c_void_p)),
        ("epoch", C.c_void_p), ("wait_timeout_ns", C.c_uint64), ("done_counter", C.c_void_p),
    ]


class RaMergeParams(C.Structure):
    """Mirror of ``struct ra_merge_params``."""
    _fields_ = [
        ("cand_scores", C.c_void_p), ("cand_indices", C.c_void_p), ("num_parts", C.c_int32),
        ("cand_part_stride", C.c_int64), ("v", C.c_void_p), ("out", C.c_void_p), ("out_partial", C.c_void_p),
        ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("num_tokens", C.c_int32),
        ("kv_batch_stride", C.c_int64), ("kv_token_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("topk", C.c_int32), ("sm_scale", C.c_float), ("own_base", C.c_int32),
        ("out_indices", C.c_void_p), ("out_scores", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
        ("exchange", C.POINTER(RaExchangeHooks)),
        ("own_part_only", C.c_int32), ("own_part", C.c_int32),
    ]


class RaGatherParams(C.Structure):
    """Mirror of ``struct ra_gather_params``."""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("num_tokens", C.c_int32),
        ("kv_batch_stride", C.c_int64), ("kv_token_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("indices", C.c_void_p), ("num_indices", C.c_int32), ("indices_batch_stride", C.c_int64),
        ("sm_scale", C.c_float), ("out_lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class RaCenterParams(C.Structure):
    """Mirror of ``struct ra_center_params``."""
    _fields_ = [
        ("q", C.c_void_p), ("centers", C.c_void_p),
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32),
        ("num_centers", C.c_int32), ("cluster_len", C.c_int32), ("top_clusters", C.c_int32),
        ("out_cluster_ids", C.c_void_p), ("out_indices", C.c_void_p),
        ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("num_tokens", C.c_int32),
        ("kv_batch_stride", C.c_int64), ("kv_token_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("sm_scale", C.c_float),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class RaDenseParams(C.Structure):
    """Mirror of ``struct ra_dense_params``."""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("num_tokens", C.c_int32),
        ("kv_batch_stride", C.c_int64), ("kv_token_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("sm_scale", C.c_float), ("num_splits", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class RaTwoLevelParams(C.Structure):
    """Mirror of ``struct ra_two_level_params``."""
    _fields_ = [
        ("q", C.c_void_p), ("centers", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("out", C.c_void_p),
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32),
        ("num_centers", C.c_int32), ("cluster_len", C.c_int32), ("top_clusters", C.c_int32),
        ("topk_per_cluster", C.c_int32), ("num_tokens", C.c_int32),
        ("kv_batch_stride", C.c_int64), ("kv_token_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("sm_scale", C.c_float),
        ("out_cluster_ids", C.c_void_p), ("out_indices", C.c_void_p), ("out_scores", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class RaError(RuntimeError):
    def __init__(self, status: int, text: str, detail: str = ""):
        super().__init__(f"topk_attn_b200: {text} (status {status})" + (f": {detail}" if detail else ""))
        self.status = status


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m topk_attn_b200.build` "
                "(nvcc, sm_100a). There is no fallback implementation.")
        _lib = C.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


_tuning_lib = None


@contextlib.contextmanager
def tuning_library():
    """Inside the block every operator runs on the tuning build of the library, the one that
    honours the route and phase overrides (RA_FORCE_*, RA_NO_*, RA_DEBUG_FLAGS, RA_VERBOSE per
    call).  For A/B tests and phase timing; the default library ignores those variables."""
    global _lib, _tuning_lib
    if _tuning_lib is None:
        if not os.path.exists(TUNING_LIB_PATH):
            raise ImportError(f"{TUNING_LIB_PATH} is missing: run `python -m topk_attn_b200.build`")
        _tuning_lib = C.CDLL(TUNING_LIB_PATH)
        _declare(_tuning_lib)
    prev, _lib = _lib, _tuning_lib
    try:
        yield _tuning_lib
    finally:
        _lib = prev


def _declare(l: C.CDLL) -> None:
    P = C.POINTER(RaParams)
    vp, i32, sz, f32 = C.c_void_p, C.c_int32, C.c_size_t, C.c_float
    sigs = {
        "ra_strerror": (C.c_char_p, [C.c_int]),
        "ra_version": (C.c_int, []),
        "ra_last_cuda_error": (C.c_char_p, []),
        "ra_launch_count": (C.c_ulonglong, []),
        "ra_workspace_bytes": (sz, [P]),
        "ra_topk_attention": (C.c_int, [P]),
        "ra_gemv_topk": (C.c_int, [P]),
        "ra_topk_attention_noalloc": (C.c_int, [P]),
        "ra_check_status": (C.c_int, [vp, vp]),
        "ra_legacy_retrieval_attention": (C.c_int, [vp, vp, vp, vp, i32, i32, i32, i32, vp, sz, vp]),
        "ra_legacy_workspace_bytes": (sz, [i32, i32, i32]),
        "ra_merge_attend": (C.c_int, [C.POINTER(RaMergeParams)]),
        "ra_gathered_attention": (C.c_int, [C.POINTER(RaGatherParams)]),
        "ra_flash_decoding": (C.c_int, [C.POINTER(RaDenseParams)]),
        "ra_two_level_topk": (C.c_int, [C.POINTER(RaTwoLevelParams)]),
        "ra_kv_append": (C.c_int, [vp, vp, vp, vp, i32, i32, i32, i32, i32, C.c_int64, C.c_int64,
                                   C.c_int64, vp, i32, i32, vp]),
        "ra_two_level_workspace_bytes": (sz, [i32, i32, i32, i32, i32]),
        "ra_flash_workspace_bytes": (sz, [i32, i32, i32, i32, i32]),
        "ra_center_only_topk": (C.c_int, [C.POINTER(RaCenterParams)]),
        "ra_center_workspace_bytes": (sz, [i32, i32, i32, i32]),
        "ra_lse_combine": (C.c_int, [vp, i32, i32, vp, vp]),
        "ra_stream_read_probe": (C.c_int, [vp, sz, vp, vp]),
        "ra_l2_persist": (C.c_int, [vp, sz, f32, vp]),
        "ra_score_store_probe": (C.c_int, [C.POINTER(RaParams)]),
        "ra_shard_exchange_bytes": (C.c_size_t, [i32, i32]),
        "ra_sharded_topk_attention": (C.c_int, [C.POINTER(RaParams), C.POINTER(RaShardExchange)]),
        "ra_lse_combine_wait": (C.c_int, [vp, i32, i32, vp, vp, i32, vp, C.c_uint64, vp, vp, vp]),
        "ra_exchange_push": (C.c_int, [vp, sz, C.POINTER(vp), C.POINTER(vp), i32, vp, vp, vp]),
        "ra_exchange_wait": (C.c_int, [vp, i32, vp, i32, C.c_uint64, vp, vp]),
    }
    for name, (res, args) in sigs.items():
        if not hasattr(l, name):
            continue
        fn = getattr(l, name)
        fn.restype = res
        fn.argtypes = args


def check(status: int) -> None:
    if status != RA_OK:
        l = lib()
        raise RaError(status, l.ra_strerror(status).decode(), l.ra_last_cuda_error().decode())
