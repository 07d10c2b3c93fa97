"""Builds the sm_100a kernel library in-tree with nvcc.

`python -m sglang_jax_b200.csrc.build` (or `build()` from Python) compiles every `.cu`
file in this directory into `sglang_jax_b200/ops/libsglb200.so`.  nvcc cross-compiles
without a GPU, so the library can be produced on a build box and shipped as is.
"""

from __future__ import annotations

import glob
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(os.path.dirname(HERE), "ops")
# `SGLB_BOUNDS_CHECK=1` selects the checked build: kernels compiled with -DSGLB_BOUNDS_CHECK verify the indices they
# write through against the extents given to `sglb_debug_set_kv_pages`, report a violation through the status word
# and skip the access.  It is a library of its own so the regular one stays as it is.
CHECKED = os.environ.get("SGLB_BOUNDS_CHECK", "0") == "1"
LIB_PATH = os.path.join(OUT_DIR, "libsglb200_checked.so" if CHECKED else "libsglb200.so")
STAMP = LIB_PATH + ".stamp"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-shared"] + (["-DSGLB_BOUNDS_CHECK"] if CHECKED else [])


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def _digest() -> str:
    h = hashlib.sha256()
    for f in sources() + sorted(glob.glob(os.path.join(HERE, "*.cuh"))) + sorted(glob.glob(os.path.join(HERE, "*.h"))):
        h.update(f.encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == _digest()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and is_current():
        return LIB_PATH
    objs = []
    tmp = os.path.join(HERE, "build_checked" if CHECKED else "build")
    os.makedirs(tmp, exist_ok=True)
    procs = []
    for src in sources():
        obj = os.path.join(tmp, os.path.basename(src)[:-3] + ".o")
        cmd = [_nvcc(), *[f for f in NVCC_FLAGS if f != "-shared"], "-c", src, "-o", obj, "-I", HERE]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{out}")
    link = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    with open(STAMP, "w") as f:
        f.write(_digest())
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
