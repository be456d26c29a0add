"""In-tree builds: the CUDA library (C ABI) and the torch binding.

Everything is compiled for sm_100a only.  Outputs land next to this file so that they travel with
the source tree:

* ``libhogatt_b200.so``   nvcc, no torch dependency: kernels + C ABI (``include/hogatt.h``)
* ``hogatt.abi3.so``      g++, links torch + the library above: registers ``torch.ops.libhogatt``

A build is skipped when its output is newer than all of its sources.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from typing import List

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
CABI_SO = os.path.join(PKG, "libhogatt_b200.so")
TORCH_SO = os.path.join(PKG, "hogatt.abi3.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]


def _stale(out: str, sources: List[str]) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: List[str], what: str, verbose: bool) -> None:
    if verbose:
        print("[build]", " ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {what} failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr, flush=True)


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return cand


def cabi_sources() -> List[str]:
    names = ["hogatt_api.cu", "hogatt_device.cuh", "hogatt_fma.cuh", "hogatt_mma.cuh", "hogatt_merge.cuh",
             "hogatt_plan.h"]
    extra = [n for n in sorted(os.listdir(CSRC)) if n.endswith((".cuh", ".h", ".cu")) and n not in names]
    return [os.path.join(CSRC, n) for n in names + extra] + [os.path.join(ROOT, "include", "hogatt.h")]


def build_cabi(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    srcs = cabi_sources()
    if force or _stale(CABI_SO, srcs):
        units = [s for s in srcs if s.endswith(".cu")]
        cmd = [nvcc_path()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-shared", "-o", CABI_SO] + units
        _run(cmd, "libhogatt_b200.so", verbose or ptxas_info)
    return CABI_SO


def build_torch_binding(force: bool = False, verbose: bool = False) -> str:
    build_cabi(force=False, verbose=verbose)
    src = os.path.join(CSRC, "hogatt_torch.cpp")
    if force or _stale(TORCH_SO, [src, CABI_SO, os.path.join(ROOT, "include", "hogatt.h")]):
        import torch
        from torch.utils import cpp_extension as ce
        cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        inc = ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]
        lib_dirs = ce.library_paths() + [os.path.join(cuda_home, "lib64")]
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wno-deprecated-declarations",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-DPy_LIMITED_API=0x03090000"]
        cmd += [f"-I{i}" for i in inc] + [src, "-o", TORCH_SO]
        cmd += [f"-L{d}" for d in lib_dirs] + [f"-L{PKG}", "-l:libhogatt_b200.so", "-lc10", "-lc10_cuda", "-ltorch_cpu",
                                                "-ltorch", "-lcudart"]
        cmd += ["-Wl,-rpath,$ORIGIN"] + [f"-Wl,-rpath,{d}" for d in lib_dirs]
        _run(cmd, "hogatt.abi3.so", verbose)
    return TORCH_SO


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cabi(force, verbose)
    build_torch_binding(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built", CABI_SO, TORCH_SO)
