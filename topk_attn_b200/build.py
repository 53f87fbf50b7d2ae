"""Build the native parts in-tree with nvcc for sm_100a.

    python -m topk_attn_b200.build            # C-ABI library (+ torch extension)

* ``lib/libtopk_attn_b200.so`` — the CUDA kernels behind the C ABI of
  ``include/topk_attn_b200.h`` (no torch dependency).
* ``retrieval_attention_cpp*.so`` — the torch extension with the reference's module name and
  its 30 entry points (retrieval_attn/setup_ra.py:8, bind.cpp:726-757), a thin pybind layer
  that forwards to the C ABI on torch's current stream.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libtopk_attn_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
TUNING_LIB = os.path.join(LIBDIR, "libtopk_attn_b200_tuning.so")
CU_SOURCES = ["api.cu", "scan_select.cu", "scan_store.cu", "select_stored.cu", "select_sharded.cu", "merge_attend.cu",
              "gather_attend.cu", "flash_decode.cu", "center_select.cu", "dense_select.cu", "exchange.cu"]
# sources that read the route / phase overrides when compiled with -DRA_TUNING
TUNING_SOURCES = ["api.cu", "scan_select.cu", "select_stored.cu", "select_sharded.cu", "dense_select.cu", "center_select.cu", "merge_attend.cu"]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _all_deps():
    deps = [os.path.join(ROOT, "include", "topk_attn_b200.h")]
    for f in os.listdir(CSRC):
        if f.endswith((".cu", ".cuh", ".cpp", ".h")):
            deps.append(os.path.join(CSRC, f))
    return deps


def _compile(sources, objdir, extra, deps, force, verbose):
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    for src in sources:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _newer(obj, deps):
            cmd = [NVCC, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", *extra,
                   "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c",
                   os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((src, subprocess.Popen(cmd)))
    for src, pr in procs:
        if pr.wait() != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    return objs, bool(procs)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """The C-ABI library, and beside it the tuning build: the same kernels with the route and
    phase overrides (RA_FORCE_*, RA_NO_*, RA_DEBUG_FLAGS) compiled in, for A/B tests and the
    bench's phase profile.  The default library reads no such variable."""
    os.makedirs(LIBDIR, exist_ok=True)
    deps = _all_deps()
    objs, fresh = _compile(CU_SOURCES, os.path.join(PKG, "build"), [], deps, force, verbose)
    if force or fresh or _newer(LIB, objs):
        subprocess.check_call([NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-cudart", "static"])
    tobjs, tfresh = _compile(TUNING_SOURCES, os.path.join(PKG, "build", "tuning"), ["-DRA_TUNING"],
                             deps, force, False)
    tall = tobjs + [o for o, src in zip(objs, CU_SOURCES) if src not in TUNING_SOURCES]
    if force or fresh or tfresh or _newer(TUNING_LIB, tall):
        subprocess.check_call([NVCC, *ARCH, "-shared", "-o", TUNING_LIB, *tall, "-cudart", "static"])
    return LIB


def extension_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(PKG, "retrieval_attention_cpp" + suffix)


def build_extension(force: bool = False) -> str:
    """Compile bind.cpp against torch's headers and link it to the C-ABI library."""
    import torch
    from torch.utils import cpp_extension as ce

    out = extension_path()
    src = os.path.join(CSRC, "bind.cpp")
    if not force and not _newer(out, [src, LIB, os.path.join(ROOT, "include", "topk_attn_b200.h")]):
        return out
    inc = ce.include_paths()
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", src, "-o", out,
           "-DTORCH_EXTENSION_NAME=retrieval_attention_cpp", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I", os.path.join(ROOT, "include"), "-I", sysconfig.get_paths()["include"],
           "-I", "/usr/local/cuda/include"]
    for i in inc:
        cmd += ["-I", i]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd += ["-L", tlib, "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda",
            "-L", LIBDIR, "-ltopk_attn_b200",
            f"-Wl,-rpath,{tlib}", "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{LIBDIR}"]
    subprocess.check_call(cmd)
    return out


def build_cli(force: bool = False) -> str:
    """The stand-alone C++ driver (host code only, links the C-ABI library)."""
    bindir = os.path.join(PKG, "bin")
    os.makedirs(bindir, exist_ok=True)
    src = os.path.join(CSRC, "cli", "ra_verify.cpp")
    out = os.path.join(bindir, "ra_verify")
    if force or _newer(out, [src, LIB]):
        subprocess.check_call([NVCC, "-O2", "-std=c++17", "-x", "cu", *ARCH, "-I",
                               os.path.join(ROOT, "include"), src, "-o", out, "-L", LIBDIR,
                               "-ltopk_attn_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib"])
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_library(force, verbose)
    build_cli(force)
    if os.path.exists(os.path.join(CSRC, "bind.cpp")):
        build_extension(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
