"""Build the checker libraries.  TEST INFRASTRUCTURE ONLY.

* ``oracle/libhogwild_oracle.so`` -- the plain-C restatement (``hogwild_oracle.c``), gcc.
* ``oracle/_ref/librope_ref.so``  -- the REFERENCE's own ``rope_cpu`` (``src/q_rope.h``) behind a C
  symbol, compiled from the reference checkout where it lies.
* ``oracle/_ref/hogwild/attention.py`` -- the REFERENCE's own Python module (``python/hogwild/attention.py``),
  staged unmodified so that the benchmark's CPU legs can time ``hogwild_sdpa_pt`` itself on machines
  that have no checkout (``load_reference_python`` imports it).

Both ``_ref`` artefacts are made only where a checkout of the reference is present (``HOGWILD_REFERENCE``
or the ``reference`` argument); ``oracle/_ref/`` is kept out of version control and is never read by the
package itself.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
C_ORACLE = os.path.join(HERE, "libhogwild_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_ROPE = os.path.join(REF_DIR, "librope_ref.so")
REF_PY = os.path.join(REF_DIR, "hogwild", "attention.py")


def _stale(out, srcs):
    return not os.path.exists(out) or any(os.path.getmtime(s) > os.path.getmtime(out) for s in srcs)


def build_c_oracle() -> str:
    src = os.path.join(HERE, "hogwild_oracle.c")
    if _stale(C_ORACLE, [src]):
        subprocess.run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-o", C_ORACLE, src, "-lm"],
                       check=True)
    return C_ORACLE


def default_reference() -> str:
    return os.environ.get("HOGWILD_REFERENCE", os.path.join(os.sep, "root", "reference"))


def build_ref(reference: str = None):
    reference = reference or default_reference()
    hdr = os.path.join(reference, "src", "q_rope.h")
    if not os.path.exists(hdr):
        return REF_ROPE if os.path.exists(REF_ROPE) else None
    os.makedirs(REF_DIR, exist_ok=True)
    src = os.path.join(HERE, "ref_rope_shim.cpp")
    if _stale(REF_ROPE, [src, hdr]):
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off",
                        f"-I{os.path.join(reference, 'src')}", "-o", REF_ROPE, src], check=True)
    py = os.path.join(reference, "python", "hogwild", "attention.py")
    if os.path.exists(py) and _stale(REF_PY, [py]):
        os.makedirs(os.path.dirname(REF_PY), exist_ok=True)
        shutil.copyfile(py, REF_PY)
    return REF_ROPE


def load_reference_python():
    """The reference's ``hogwild.attention`` module from ``oracle/_ref`` (``None`` if it was never staged).

    It imports as shipped except for one thing: it looks up an installed ``hogwild`` distribution and only
    catches ``OSError``; a wrapper around ``importlib.metadata.distribution`` turns "not installed" into that
    ``OSError`` so that the module takes its own eager (pure PyTorch) branch."""
    if not os.path.exists(REF_PY):
        return None
    import importlib.metadata as md
    import importlib.util
    import warnings
    real = md.distribution

    def shim(name):
        if name == "hogwild":
            raise OSError("hogwild wheel is not installed here")
        return real(name)

    md.distribution = shim
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            spec = importlib.util.spec_from_file_location("hogwild_reference_attention", REF_PY)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
    finally:
        md.distribution = real
    return mod


if __name__ == "__main__":
    print(build_c_oracle(), build_ref())
