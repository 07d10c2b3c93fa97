"""Builds the native scheduler structures (`sched_native.cpp`, pybind11) in-tree with g++:
`python -m sglang_jax_b200.csrc.sched.build` -> `sglang_jax_b200/mem_cache/_sched_native*.so`."""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "sched_native.cpp")
OUT_DIR = os.path.join(os.path.dirname(os.path.dirname(HERE)), "mem_cache")
LIB_PATH = os.path.join(OUT_DIR, "_sched_native" + sysconfig.get_config_var("EXT_SUFFIX"))
STAMP = LIB_PATH + ".stamp"


def _digest() -> str:
    with open(SRC, "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB_PATH) and os.path.exists(STAMP) and open(STAMP).read().strip() == _digest():
        return LIB_PATH
    import pybind11
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-shared", "-fPIC", "-I", pybind11.get_include(),
           "-I", sysconfig.get_paths()["include"], SRC, "-o", LIB_PATH]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {SRC}:\n{r.stdout}")
    with open(STAMP, "w") as f:
        f.write(_digest())
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
