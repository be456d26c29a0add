"""Build the checker libraries.  TEST INFRASTRUCTURE ONLY.

* ``oracle/libhogwild_oracle.so`` -- the plain-C restatement (``hogwild_oracle.c``), gcc.
* ``oracle/_ref/librope_ref.so``  -- the REFERENCE's own ``rope_cpu`` (``src/q_rope.h``) behind a C
  symbol, compiled from the reference checkout where it lies; only when that checkout is present
  (the build container).  ``oracle/_ref/`` is git-ignored and travels with the tree to the GPU box.

The reference's CUDA sources are not built here: their launcher accepts only head size 128 with
16 query heads per kv head, which none of the benchmark shapes has, and its static workspaces and
default-stream launches make it unsuitable as a general checker.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
C_ORACLE = os.path.join(HERE, "libhogwild_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_ROPE = os.path.join(REF_DIR, "librope_ref.so")


def _stale(out, srcs):
    return not os.path.exists(out) or any(os.path.getmtime(s) > os.path.getmtime(out) for s in srcs)


def build_c_oracle() -> str:
    src = os.path.join(HERE, "hogwild_oracle.c")
    if _stale(C_ORACLE, [src]):
        subprocess.run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-o", C_ORACLE, src, "-lm"],
                       check=True)
    return C_ORACLE


def build_ref(reference: str = "/root/reference"):
    hdr = os.path.join(reference, "src", "q_rope.h")
    if not os.path.exists(hdr):
        return REF_ROPE if os.path.exists(REF_ROPE) else None
    os.makedirs(REF_DIR, exist_ok=True)
    src = os.path.join(HERE, "ref_rope_shim.cpp")
    if _stale(REF_ROPE, [src, hdr]):
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off",
                        f"-I{os.path.join(reference, 'src')}", "-o", REF_ROPE, src], check=True)
    return REF_ROPE


if __name__ == "__main__":
    print(build_c_oracle(), build_ref())
