"""Build entry point with the reference's name (retrieval_attn/setup_ra.py): compiles the kernels
for sm_100a and the torch extension ``retrieval_attention_cpp`` in-tree.

    python topk_attn_b200/setup_ra.py [build_ext] [--force]

The reference hands two sources to torch's CUDAExtension with ``-arch=sm_120a``
(setup_ra.py:4-24); here nvcc builds the C-ABI library first
(``-gencode arch=compute_100a,code=sm_100a -O3 -lineinfo``) and ``bind.cpp`` is linked against it.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from topk_attn_b200 import build  # noqa: E402

if __name__ == "__main__":
    build.build_all(force="--force" in sys.argv)
    print(build.LIB)
    print(build.extension_path())
