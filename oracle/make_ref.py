"""Stage the UNMODIFIED reference packages under ``oracle/_ref/`` so they travel to the GPU machine.

    python oracle/make_ref.py /path/to/alexdremov-kernels

TEST / CONTEXT INFRASTRUCTURE, not product code.  The reference is pure Python + Triton: there is
nothing to compile, "building" it means placing its three importable packages
(``src/streaming_attention``, ``src/self_attention``, ``src/softmax``) where a separate process can
import them.  ``oracle/_ref/`` is git-ignored (the files are the reference's, not this repository's)
but is carried to the benchmark machine with the rest of the tree.

Who uses it: ``bench.py --impl context`` times the reference's own Triton kernel
(``streaming_attention(..., autotune=False)``, src/streaming_attention/kernel.py:1599-1652) on the same
GPU and inputs as this library, in a child process of its own because both packages register operators
of the same names.  Nothing under ``kernels_b200/`` ever imports from here.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
PACKAGES = ("streaming_attention", "self_attention", "softmax")


def stage(reference_root: str) -> str:
    src_root = os.path.join(reference_root, "src")
    missing = [p for p in PACKAGES if not os.path.isfile(os.path.join(src_root, p, "kernel.py"))]
    if missing:
        raise SystemExit(f"{reference_root}: not the reference project (no src/{missing[0]}/kernel.py)")
    dst_root = os.path.join(DEST, "src")
    os.makedirs(dst_root, exist_ok=True)
    for p in PACKAGES:
        dst = os.path.join(dst_root, p)
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(os.path.join(src_root, p), dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as fh:
        fh.write("Unmodified copies of src/{streaming_attention,self_attention,softmax} of alexdremov/kernels,\n"
                 "staged by oracle/make_ref.py for timing the reference's Triton kernels as context.\n")
    return dst_root


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(stage(sys.argv[1]))
