"""Build the C-ABI library ``lib/libkernels_b200.so`` in-tree with nvcc for sm_100a.

    python -m kernels_b200.build [--force] [--verbose]

Every ``csrc/*.cu`` is compiled to an object file (in parallel) and linked into one shared
library with a static CUDA runtime.  The library does not link ``libcuda``: the one driver
entry point it needs (tensor-map encoding for TMA) is looked up at run time, so the library
also loads on a machine without a GPU driver.  Objects are rebuilt only when a source or
header changed.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG_DIR, "csrc")
INC_DIR = os.path.join(os.path.dirname(PKG_DIR), "include")
OUT_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB_PATH = os.path.join(OUT_DIR, "libkernels_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]

# translation units whose presence switches on a kernel family in capi.cu
FEATURE_DEFINES = {"sa_fwd_sm100.cu": "-DKB_HAVE_SM100", "sa_bwd_sm100.cu": "-DKB_HAVE_SM100_BWD",
                   "sa_bwd_fused_sm100.cu": "-DKB_HAVE_SM100_BWD_FUSED"}


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the kernels_b200 library cannot be built")
    return cand


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(SRC_DIR) if f.endswith(".cu"))


def _digest(paths: list[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    srcs = _sources()
    headers = sorted(
        [os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR) if f.endswith((".h", ".cuh"))]
        + [os.path.join(INC_DIR, f) for f in os.listdir(INC_DIR) if f.endswith(".h")]
    )
    defines = [FEATURE_DEFINES[s] for s in srcs if s in FEATURE_DEFINES]
    extra = os.environ.get("KB_NVCC_EXTRA", "").split()  # e.g. -DKB_TRACE for the clock-trace build
    flags = NVCC_FLAGS + defines + extra + ["-I", INC_DIR]

    def compile_one(src: str) -> tuple[str, bool, str]:
        src_path = os.path.join(SRC_DIR, src)
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        stamp = obj + ".sha"
        dig = _digest([src_path] + headers, " ".join(flags))
        if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
            return obj, False, ""
        cmd = [nvcc, *flags, "-c", src_path, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        with open(stamp, "w") as fh:
            fh.write(dig)
        return obj, True, res.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(compile_one, srcs))
    objs = [r[0] for r in results]
    rebuilt = any(r[1] for r in results)
    if verbose:
        for (_, did, log), src in zip(results, srcs):
            if did:
                print(f"--- {src}\n{log}")
    if rebuilt or force or not os.path.exists(LIB_PATH):
        cmd = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-cudart", "static", "-Xlinker", "--no-undefined", "-ldl", "-lpthread", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))


if __name__ == "__main__":
    main()
