"""Build ``lmdeploy_b200/_lib/libtm_b200.so`` (sm_100a only) with nvcc, in tree.

    python -m lmdeploy_b200.build [--force] [--verbose]

The library is the product: every Python entry point in this package calls into it through
ctypes and raises if it is missing.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_lib")
LIB = os.path.join(OUT_DIR, "libtm_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _nccl_flags():
    """NCCL is optional at build time: without it the tensor-parallel entry points return
    TM_ERR_NOT_BUILT."""
    for inc, lib in (("/usr/include", "/usr/lib/x86_64-linux-gnu"), ("/usr/local/cuda/include", "/usr/local/cuda/lib64")):
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return ["-DTM_B200_WITH_NCCL=1", "-I", inc], ["-L", lib, "-lnccl"]
    return [], []


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cc")))


def _digest(paths, extra) -> str:
    h = hashlib.sha256(" ".join(extra).encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode() + b"\0" + f.read())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    srcs = sources()
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hdrs += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include")) if f.endswith(".h")]
    nccl_c, nccl_l = _nccl_flags()
    flags = NVCC_FLAGS + nccl_c + (["-Xptxas", "-v"] if ptxas_info else [])
    stamp = os.path.join(OUT_DIR, "build.sha256")
    dig = _digest(srcs + hdrs, flags + nccl_l)
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read().strip() == dig:
        return LIB
    nvcc = _nvcc()

    def compile_one(src):
        obj = os.path.join(OUT_DIR, os.path.basename(src) + ".o")
        cmd = [nvcc, "-x", "cu"] + flags + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or ptxas_info or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcublas"] + nccl_l
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("link failed")
    with open(stamp, "w") as f:
        f.write(dig)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.ptxas_info))
