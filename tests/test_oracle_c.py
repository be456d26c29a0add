"""The plain-C oracle and the compiled reference RoPE against the reference outputs (tests/golden)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from inference_lib_b200 import workloads as wl
from oracle import build_oracle

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


@pytest.fixture(scope="module")
def clib():
    lib = C.CDLL(build_oracle.build_c_oracle())
    lib.hogwild_rope_ref.restype = None
    lib.hogwild_sdpa_ref.restype = None
    return lib


def _f32(t):
    return np.ascontiguousarray(t.to(torch.float32).numpy())


def c_fused(clib, p):
    q, cos, sin = _f32(p.queries), _f32(p.cos), _f32(p.sin)
    F, W, Hq, S, E, Ev, Hkv, R = p.F, p.W, p.Hq, p.S, p.E, p.Ev, p.Hkv, p.cos.shape[-1]
    rq = np.empty((F, W, Hq, S, E), dtype=np.float32)
    fp = lambda a: a.ctypes.data_as(C.c_void_p)
    clib.hogwild_rope_ref(fp(rq), fp(q), fp(cos), fp(sin), F, W, Hq, S, E, R, DT[p.dtype])
    ks = [_f32(k[0]) for k in p.keys]
    vs = [_f32(v[0]) for v in p.values]
    kp = (C.c_void_p * F)(*[a.ctypes.data for a in ks])
    vp = (C.c_void_p * F)(*[a.ctypes.data for a in vs])
    lens = np.array([k.shape[1] for k in ks], dtype=np.int32)
    loc = np.ascontiguousarray(p.locations.numpy())
    out = np.empty((W, Hq, S, Ev), dtype=np.float32)
    clib.hogwild_sdpa_ref(fp(out), fp(rq), fp(loc), kp, vp, fp(lens), C.c_float(p.scale), F, W, Hq, Hkv, S, E, Ev)
    return out, rq


@pytest.mark.parametrize("name", ["cfg1"] + sorted(n for n in wl.EDGE_CASES if not n.startswith("split_many")))
def test_c_oracle_matches_reference(clib, golden, name):
    p = wl.baseline_problem(name) if name.startswith("cfg") else wl.edge_problem(name)
    out, rq = c_fused(clib, p)
    ref = golden[f"{name}/out"]
    assert np.array_equal(np.isnan(out), np.isnan(ref))
    assert np.nanmax(np.abs(out - ref), initial=0.0) <= 3e-5
    if f"{name}/rq" in golden.files:
        assert np.array_equal(rq, golden[f"{name}/rq"]), "rotation (and storage rounding) must be bit-exact"


def test_reference_rope_cpu_compiled_from_the_checkout(golden):
    """`rope_cpu` of the reference itself (oracle/_ref) == its PyTorch rotation, on fp32 inputs."""
    path = build_oracle.build_ref()
    if path is None or not os.path.exists(path):
        pytest.skip("oracle/_ref was not built (no reference checkout on this machine)")
    lib = C.CDLL(path)
    for name in ("cfg1", "ragged_f32"):
        p = wl.baseline_problem(name) if name.startswith("cfg") else wl.edge_problem(name)
        q, cos, sin = _f32(p.queries), _f32(p.cos), _f32(p.sin)
        rq = np.empty((p.F, p.W, p.Hq, p.S, p.E), dtype=np.float32)
        fp = lambda a: a.ctypes.data_as(C.c_void_p)
        lib.ref_rope_cpu_f32(fp(rq), fp(q), fp(cos), fp(sin), p.F, p.W, p.Hq, p.S, p.E, p.cos.shape[-1])
        assert np.array_equal(rq, golden[f"{name}/rq"])
