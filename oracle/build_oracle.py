"""Build recipe for the CPU checkers.  TEST INFRASTRUCTURE ONLY.

* ``oracle/c/libsocket_oracle.so`` — the plain-C restatement (`oracle/c/socket_oracle.c`).
* ``oracle/_ref/libref_scorer.so`` — the reference's own scorer kernel source compiled as
  C++ through `oracle/ref_shim.cpp`.  Built only where the reference tree is present
  (``SOCKET_REFERENCE_ROOT``, else a ``reference`` directory beside the repository); the sources are compiled where they
  lie and never copied.  The output directory is git-ignored.

Run ``python oracle/build_oracle.py``.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: named by SOCKET_REFERENCE_ROOT, else a `reference` directory beside this repository
REF_ROOT = os.environ.get("SOCKET_REFERENCE_ROOT") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))
REF_KERNEL = os.path.join(REF_ROOT, "GPT-FAST", "kernels", "soft_hash_collision.cu")
C_SRC = os.path.join(HERE, "c", "socket_oracle.c")
C_LIB = os.path.join(HERE, "c", "libsocket_oracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libref_scorer.so")


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_c(force: bool = False) -> str:
    if force or not _newer(C_LIB, C_SRC):
        cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-std=c11",
               "-o", C_LIB, C_SRC, "-lm"]
        subprocess.check_call(cmd)
    return C_LIB


def build_ref(force: bool = False):
    """Returns the library path, or None when the reference tree is not on this machine
    and no prebuilt library travelled with the repository."""
    if not os.path.exists(REF_KERNEL):
        return REF_LIB if os.path.exists(REF_LIB) else None
    shim = os.path.join(HERE, "ref_shim.cpp")
    if force or not _newer(REF_LIB, shim, REF_KERNEL):
        os.makedirs(os.path.dirname(REF_LIB), exist_ok=True)
        cmd = ["g++", "-O2", "-std=c++17", "-fopenmp", "-fPIC", "-shared", "-x", "c++",
               f'-DSOCKET_REF_KERNEL_SRC="{REF_KERNEL}"', "-o", REF_LIB, shim]
        subprocess.check_call(cmd)
    return REF_LIB


if __name__ == "__main__":
    print(build_c(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
