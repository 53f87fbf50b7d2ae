"""CPU checks of the boundary: the C-ABI library loads without a GPU, exports every function the
header declares, the ctypes mirrors match the header's structs field by field, and argument
validation that needs no device works."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "topk_attn_b200.h")


def header_text():
    return open(HEADER).read()


def declared_functions():
    txt = re.sub(r"/\*.*?\*/", "", header_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ra_[a-z_0-9]+)\s*\(", txt)))


def test_library_exports_every_declared_symbol():
    from topk_attn_b200 import capi
    lib = capi.lib()
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"


def struct_fields(name):
    txt = re.sub(r"/\*.*?\*/", "", header_text(), flags=re.S)
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), txt, flags=re.S).group(1)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        names = [x.strip().lstrip("*").strip() for x in decl.split(",")]
        first = names[0].split()[-1].lstrip("*")
        fields.append(first)
        fields.extend(names[1:])
    return fields


@pytest.mark.parametrize("cname,pyname", [
    ("ra_params", "RaParams"), ("ra_merge_params", "RaMergeParams"),
    ("ra_exchange_hooks", "RaExchangeHooks"), ("ra_shard_exchange", "RaShardExchange"),
    ("ra_gather_params", "RaGatherParams"), ("ra_center_params", "RaCenterParams"),
    ("ra_dense_params", "RaDenseParams"), ("ra_two_level_params", "RaTwoLevelParams"),
])
def test_ctypes_mirrors_match_header(cname, pyname):
    from topk_attn_b200 import capi
    py = [f[0] for f in getattr(capi, pyname)._fields_]
    assert py == struct_fields(cname)


def test_strerror_and_version():
    from topk_attn_b200 import capi
    lib = capi.lib()
    assert lib.ra_version() >= 100
    assert lib.ra_strerror(0) == b"ok"
    for code in range(1, 8):
        assert lib.ra_strerror(code) not in (b"ok", b"unknown status")


def test_shape_validation_without_a_device():
    from topk_attn_b200 import capi
    lib = capi.lib()
    p = capi.RaParams()
    assert lib.ra_workspace_bytes(C.byref(p)) == 0           # empty shape
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.num_tokens = 4, 32, 32, 128, 131072
    p.kv_token_stride, p.kv_head_stride, p.topk, p.num_segments, p.sm_scale = 4096, 128, 2048, 1, 1.0
    need = lib.ra_workspace_bytes(C.byref(p))
    assert need >= 256 + 4 * 32 * 2048 * 8
    p.head_dim = 64
    assert lib.ra_workspace_bytes(C.byref(p)) == 0
    assert lib.ra_topk_attention(C.byref(p)) == capi.RA_ERR_UNSUPPORTED
    p.head_dim, p.topk = 128, 0
    assert lib.ra_topk_attention(C.byref(p)) == capi.RA_ERR_INVALID_ARGUMENT
    assert lib.ra_legacy_workspace_bytes(4, 8192, 128) > 0
    assert lib.ra_flash_workspace_bytes(8, 32, 8, 32768, 64) == 256 + 64 * 8 * 32 * 130 * 4
    assert lib.ra_center_workspace_bytes(1, 32, 2048, 64) > 0


def test_missing_library_fails_loudly(monkeypatch):
    from topk_attn_b200 import capi
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", "/nonexistent/libtopk_attn_b200.so")
    with pytest.raises(ImportError):
        capi.lib()


def test_extension_module_is_built_with_the_reference_names():
    import topk_attn_b200
    mod = topk_attn_b200.load_extension()
    names = [f"retrieval_attention{v}_{k}" for v in
             ("", "_global", "_pipelined", "_pipelined_global", "_two_kernels", "_gather_baseline")
             for k in (32, 128, 256, 512, 1024)]
    assert all(hasattr(mod, n) for n in names)


def _planner_max_parts(seg_len, topk):
    """The planner's own acceptance rule for cutting a context into parts, restated: tile heights
    16..128, at most 16 parts, the tile-rounded part holds k keys and the last part is not empty."""
    best = 1
    for tile in (16, 32, 64, 128):
        for nsplit in range(2, 17):
            part = -(-(-(-seg_len // nsplit)) // tile) * tile
            if part < topk:
                break
            if part * (nsplit - 1) >= seg_len:
                continue
            best = max(best, nsplit)
    return best


def test_workspace_bound_covers_every_plan_the_planner_accepts():
    """ra_workspace_bytes() must hold the candidate lists of the largest part count any plan may
    pick, also for context lengths that are no multiple of the split granularity."""
    from topk_attn_b200 import capi
    lib = capi.lib()
    p = capi.RaParams()
    p.head_dim, p.kv_head_stride, p.num_segments, p.sm_scale = 128, 128, 1, 1.0
    cases = 0
    for B, Hq, Hkv in ((1, 32, 32), (1, 32, 8), (2, 8, 8), (4, 16, 2)):
        p.batch, p.num_q_heads, p.num_kv_heads, p.kv_token_stride = B, Hq, Hkv, Hkv * 128
        for n in (2000, 4097, 20000, 36000, 65536, 100003, 131072):
            for k in (1, 32, 500, 2048, 4096):
                if k > n:
                    continue
                p.num_tokens, p.topk = n, k
                need = lib.ra_workspace_bytes(C.byref(p))
                lists = B * Hq * _planner_max_parts(n, k) * k * 8
                assert need >= 256 + lists, (B, Hq, Hkv, n, k, need, lists)
                cases += 1
    assert cases > 100


def test_tuning_library_is_built_and_default_ignores_overrides():
    from topk_attn_b200 import capi
    assert os.path.exists(capi.TUNING_LIB_PATH)
    default = capi.lib()
    with capi.tuning_library() as t:
        assert capi.lib() is t and t is not default
        assert t.ra_version() == default.ra_version()
    assert capi.lib() is default


def test_setup_ra_build_ext_leaves_an_importable_module():
    """The reference's flow: `python setup_ra.py build_ext --inplace`, then
    `import retrieval_attention_cpp` from that directory (retrieval_attn/setup_ra.py:4-24,
    test_ra.py:80-85)."""
    import subprocess
    import sys
    pkg = os.path.join(ROOT, "topk_attn_b200")
    subprocess.check_call([sys.executable, "setup_ra.py", "build_ext", "--inplace"], cwd=pkg,
                          stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    code = ("import torch, retrieval_attention_cpp as m; "
            "assert hasattr(m, 'retrieval_attention_128') and hasattr(m, 'retrieval_attention_pipelined_global_1024')")
    subprocess.check_call([sys.executable, "-c", code], cwd=pkg)


def test_histogram_exchange_layout_and_argument_checks():
    """The receive buffer of the histogram route: its region inside the Python layout is exactly
    what the library asks for, 8-byte aligned, after the regions of the candidate route; bad
    arguments are refused before anything touches a device."""
    import torch
    from topk_attn_b200 import capi
    from topk_attn_b200.sharded import HistExchange, PeerExchange
    lib = capi.lib()
    for world, B, Hq, topk in [(1, 1, 8, 256), (2, 1, 32, 4096), (8, 4, 32, 2048)]:
        base = PeerExchange.layout(world, B, Hq, topk)
        lay = HistExchange.layout(world, B, Hq, topk)
        off_ll, words = lay[-2], lay[-1]
        assert lay[:len(base) - 1] == base[:-1] and off_ll >= base[-1] and off_ll % 2 == 0
        assert (words - off_ll) * 4 >= lib.ra_shard_exchange_bytes(B * Hq, world) > 0
        buf = torch.zeros(words, dtype=torch.int32)
        ex = HistExchange(buf, [buf.data_ptr()] * world, 0, world, B, Hq, topk)
        assert all(p % 8 == 0 for p in ex.ll_ptrs)
    assert lib.ra_shard_exchange_bytes(0, 2) == 0
    p, x = capi.RaParams(), capi.RaShardExchange()
    assert lib.ra_sharded_topk_attention(None, None) == capi.RA_ERR_INVALID_ARGUMENT
    x.world, x.rank = 2, 2
    assert lib.ra_sharded_topk_attention(C.byref(p), C.byref(x)) == capi.RA_ERR_INVALID_ARGUMENT
    x.rank = 1                                               # no buffers, no epoch word
    assert lib.ra_sharded_topk_attention(C.byref(p), C.byref(x)) == capi.RA_ERR_INVALID_ARGUMENT
