"""Build entry point with the reference's name (retrieval_attn/setup_ra.py): compiles the kernels
for sm_100a and the torch extension ``retrieval_attention_cpp``.

    python setup_ra.py build_ext --inplace     # leaves retrieval_attention_cpp*.so beside this file
    python setup_ra.py install                 # or into site-packages, like the reference's flow
    python setup_ra.py [--force]               # no command: build in-tree and print the paths

after which ``import torch, retrieval_attention_cpp`` works from that directory (or anywhere after
``install``), exactly as with the reference (setup_ra.py:4-24, test_ra.py:80-85).  The reference
hands two sources to torch's CUDAExtension with ``-arch=sm_120a``; here nvcc builds the C-ABI
library first (``-gencode arch=compute_100a,code=sm_100a -O3 -lineinfo``) and ``bind.cpp`` is linked
against it, so ``build_ext`` delegates to ``topk_attn_b200.build`` and copies the result to where
setuptools wants it.  The extension finds ``libtopk_attn_b200.so`` through its run path
(``$ORIGIN/lib`` and the absolute path of this package's ``lib/``).
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from topk_attn_b200 import build  # noqa: E402


def _setup():
    from setuptools import Extension, setup
    from setuptools.command.build_ext import build_ext

    class BuildExt(build_ext):
        def build_extension(self, ext):
            build.build_all()
            dst = self.get_ext_fullpath(ext.name)
            os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
            src = build.extension_path()
            if os.path.abspath(src) != os.path.abspath(dst):
                shutil.copyfile(src, dst)

    os.chdir(HERE)
    setup(name="retrieval_attention", version="1.0",
          ext_modules=[Extension("retrieval_attention_cpp", sources=[])],
          cmdclass={"build_ext": BuildExt}, script_args=[a for a in sys.argv[1:] if a != "--force"])


if __name__ == "__main__":
    commands = [a for a in sys.argv[1:] if not a.startswith("-")]
    if commands:
        _setup()
    else:
        build.build_all(force="--force" in sys.argv)
        print(build.LIB)
        print(build.extension_path())
