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
REF_CUDA = os.path.join(REF_DIR, "hogatt_ref.so")


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


def build_ref_cuda(reference: str = None, verbose: bool = False):
    """The REFERENCE's own CUDA extension (``src/binding.cu`` + ``src/tpl/kernel_v21.cu``), compiled for sm_100a from
    the checkout where it lies into ``oracle/_ref/hogatt_ref.so`` with one nvcc command (the reference's CMake build is
    not run).  Its launcher only accepts head size 128 with 16 query heads per kv head (``kernel_v21.cuh:982-986``), so
    it serves as a timed competitor and as the checker of the paged operators at such a shape, in a process of its
    own (it registers the same ``libhogatt`` operator names as this package).  Returns the path, or ``None`` when
    there is neither a checkout nor an earlier build."""
    reference = reference or default_reference()
    srcs = [os.path.join(reference, "src", "binding.cu"), os.path.join(reference, "src", "tpl", "kernel_v21.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return REF_CUDA if os.path.exists(REF_CUDA) else None
    deps = srcs + [os.path.join(reference, "src", "kernels", "kernel_v21.cuh")]
    if not _stale(REF_CUDA, deps):
        return REF_CUDA
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(REF_DIR, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = [os.path.join(reference, "src")] + ce.include_paths() + [sysconfig.get_paths()["include"]]
    libs = ce.library_paths() + [os.path.join(cuda_home, "lib64")]
    cmd = [os.path.join(cuda_home, "bin", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
           "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared", "-w",
           "-DHOGDILD_ENABLE_FLOAT=1", "-DHOGDILD_ENABLE_HALF=1", "-DHOGDILD_ENABLE_BFLOAT=1",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{i}" for i in inc] + srcs + ["-o", REF_CUDA] + [f"-L{d}" for d in libs]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"]
    cmd += [f"-Xlinker=-rpath,{d}" for d in libs]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        if verbose:
            print(res.stdout[-3000:], res.stderr[-3000:])
        return None
    return REF_CUDA


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
    print(build_c_oracle(), build_ref(), build_ref_cuda(verbose=True))
