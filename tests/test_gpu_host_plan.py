"""GPU parity of the host-planned launch: the tiles come from lengths the HOST knows (``hogatt_problem.host_lengths``),
nothing is read from device memory before the first K/V copy, and tiles of "stable" fragments may be fetched
before the kernel waits for the stream's preceding kernel (programmatic dependent launch).

Visibility is still decided on the device from ``locations`` and ``fragment_lengths``, so a bound that is larger
than the true length must only cost traffic, never change a result -- whatever the rows past the true length hold.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from inference_lib_b200 import _cabi
from inference_lib_b200 import workloads as wl
from oracle import hogwild_oracle as oracle
from tests.gpu_util import check_against, run_cabi

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))

MMA_SHAPES = [_cabi.KERNEL_MMA, _cabi.KERNEL_MMA_CLUSTER]


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "target", "cfg4"])
@pytest.mark.parametrize("kernel", MMA_SHAPES)
def test_exact_host_lengths_give_the_device_plan_bit_for_bit(golden, name, kernel):
    """With host lengths equal to what the device would derive, the decomposition is the same: identical bits."""
    p = wl.baseline_problem(name)
    dev_plan = run_cabi(p, kernel=kernel, want_rq=True)
    host_plan = run_cabi(p, kernel=kernel, want_rq=True, host_lengths="rows", stable_fragments=1)
    assert dev_plan.rc == 0 and host_plan.rc == 0 and host_plan.status == 0
    assert torch.equal(dev_plan.out, host_plan.out)
    assert torch.equal(dev_plan.rq, host_plan.rq)
    check_against(host_plan.out, golden[f"{name}/out"], p.dtype, what=f"{name} host plan")


@pytest.mark.parametrize("name", sorted(n for n, c in wl.EDGE_CASES.items()
                                        if c["dtype"] != torch.float32 and c.get("Ev", c["E"]) == c["E"]))
def test_edge_cases_under_a_host_plan(golden, name):
    """Hidden fragments, partially visible fragments, blind rows, causal chunks, empty fragments: the host only
    knows the tensors' row counts, the device masks."""
    p = wl.edge_problem(name)
    rows = p.W * (p.Hq // p.Hkv) * p.S
    units = -(-rows // (16 if rows <= 16 else 32 if rows <= 32 else 64)) * p.Hkv
    for kernel in MMA_SHAPES:
        if kernel == _cabi.KERNEL_MMA_CLUSTER and 2 * units > torch.cuda.get_device_properties(0).multi_processor_count:
            continue
        for stable in (0, p.F):
            r = run_cabi(p, kernel=kernel, want_rq=True, host_lengths="rows", stable_fragments=stable)
            assert r.rc == 0 and r.status == 0, (name, kernel, r.rc, r.status)
            check_against(r.out, golden[f"{name}/out"], p.dtype, what=f"{name} kernel {kernel} host plan")
            if f"{name}/rq" in golden.files:
                assert np.array_equal(r.rq.float().cpu().numpy(), golden[f"{name}/rq"])


@pytest.mark.parametrize("max_ctas", [1, 3, 7, 31])
@pytest.mark.parametrize("name", ["ragged_bf16", "causal_chunk_bf16", "hidden_and_partial_bf16", "row_blocks_bf16"])
def test_host_plan_on_any_grid(golden, name, max_ctas):
    p = wl.edge_problem(name)
    r = run_cabi(p, kernel=_cabi.KERNEL_MMA, max_ctas=max_ctas, host_lengths="rows")
    assert r.rc == 0 and r.status == 0
    check_against(r.out, golden[f"{name}/out"], p.dtype, what=f"{name} ctas {max_ctas} host plan")


@pytest.mark.parametrize("kernel", MMA_SHAPES)
def test_rows_past_the_true_length_never_reach_a_result(kernel):
    """Slabs with spare capacity: the device lengths are shorter than the tensors, the host passes a loose bound,
    and the spare rows hold NaN (keys) and Inf (values).  They are fetched and masked."""
    p = wl.edge_problem("ragged_bf16")                            # lengths 37, 1, 9, 130
    true_len = [20, 1, 4, 77]
    bound = [37, 1, 9, 130]                                       # what the host believes: the tensors' row counts
    short = torch.tensor(true_len, dtype=torch.int32)
    q = wl.Problem(**{**p.__dict__, "fragment_lengths": short})
    ref, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, [k[:, :, :n] for k, n in zip(p.keys, true_len)],
                          [v[:, :, :n] for v, n in zip(p.values, true_len)], p.scale)
    keys, values = [], []
    for k, v, n in zip(p.keys, p.values, true_len):
        k, v = k.clone(), v.clone()
        k[:, :, n:] = float("nan")
        v[:, :, n:] = float("inf")
        keys.append(k.to("cuda:0"))
        values.append(v.to("cuda:0"))
    for hl in (bound, [25, 1, 8, 100], true_len):
        r = run_cabi(q, kernel=kernel, host_lengths=hl, keys=keys, values=values)
        assert r.rc == 0 and r.status == 0
        check_against(r.out, ref.numpy(), p.dtype, what=f"host bound {hl}")


def test_host_lengths_are_clamped_to_the_tensors():
    p = wl.edge_problem("gqa5_bf16")
    ref, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale)
    r = run_cabi(p, kernel=_cabi.KERNEL_MMA, host_lengths=[10 ** 9, -5, 18, 19, 20])
    assert r.rc == 0 and r.status == 0
    # fragment 1 is planned as empty (bound -5 -> 0): its keys are not attended at all, which the oracle shows too
    keys = [k if f != 1 else k[:, :, :0] for f, k in enumerate(p.keys)]
    vals = [v if f != 1 else v[:, :, :0] for f, v in enumerate(p.values)]
    ref2, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, keys, vals, p.scale)
    check_against(r.out, ref2.numpy(), p.dtype)
    assert (ref - ref2).abs().max() > 1e-3        # (the dropped fragment mattered)


def test_the_fma_kernel_ignores_the_host_plan(golden):
    p = wl.edge_problem("ragged_f32")
    r = run_cabi(p, host_lengths="rows", stable_fragments=2)
    assert r.rc == 0 and r.status == 0
    check_against(r.out, golden["ragged_f32/out"], p.dtype)


PDL_SCRIPT = r"""
import sys, numpy as np, torch
sys.path.insert(0, {root!r})
from inference_lib_b200 import _cabi, workloads as wl
dev = torch.device("cuda:0")
golden = np.load({root!r} + "/tests/golden/reference_outputs.npz")
stream = torch.cuda.Stream(dev)
status = torch.zeros(1, dtype=torch.int32, device=dev)
calls = []
for name, stable in (("cfg2", 1), ("ragged_bf16", 4), ("target", 1), ("gqa5_bf16", 0), ("cfg3", 5), ("target", 5),
                     ("hidden_and_partial_bf16", 4), ("cfg2", 3)):
    p = wl.baseline_problem(name) if name in wl.BASELINE_CONFIGS else wl.edge_problem(name)
    d = p.to(dev)
    out = torch.full((p.W, p.Hq, p.S, p.Ev), float("nan"), dtype=p.dtype, device=dev)
    rq = torch.zeros((p.F, p.W, p.Hq, p.S, p.E), dtype=p.dtype, device=dev)
    for kernel in (_cabi.KERNEL_MMA, _cabi.KERNEL_MMA_CLUSTER):
        bp = _cabi.bind(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values, scale=p.scale,
                        fragment_lengths=d.fragment_lengths, cos=d.cos, sin=d.sin, rq=rq, status=status, kernel=kernel,
                        host_lengths="rows", stable_fragments=stable)
        ws = _cabi.attach_workspace(bp, dev)
        ws.fill_(0xFF)
        calls.append((name, p, out, rq, bp))
torch.cuda.synchronize()

def check(tag):
    torch.cuda.synchronize()
    assert int(status.item()) == 0, (tag, int(status.item()))
    for name, p, out, rq, bp in calls:
        got, ref = out.float().cpu().numpy(), golden[name + "/out"]
        blind = np.isnan(ref)
        diff = np.abs(got - np.where(blind, 0, ref))[~blind]
        assert np.isfinite(got).all() and diff.max() <= 2e-2 and diff.mean() <= 2e-3, (tag, name, float(diff.max()))
        if name + "/rq" in golden.files:
            assert np.array_equal(rq.float().cpu().numpy(), golden[name + "/rq"]), (tag, name)

# every call runs on its own output, back to back on one stream: each kernel may start while its predecessor runs
with torch.cuda.stream(stream):
    for rep in range(3):
        for c in calls:
            assert _cabi.launch(c[4], stream.cuda_stream) == 0
    check("eager")
    for c in calls:
        c[2].fill_(float("nan"))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for c in calls:
            assert _cabi.launch(c[4], torch.cuda.current_stream().cuda_stream) == 0
    for rep in range(5):
        g.replay()
    check("graph")
print("PDL_OK")
"""


@pytest.mark.parametrize("pdl", ["1", "0"])
def test_back_to_back_calls_with_and_without_programmatic_dependent_launch(pdl):
    """HOGATT_PDL is read once per process, hence the child.  With it (the default) consecutive calls overlap: a
    kernel is scheduled while its predecessor still runs and fetches tiles of its stable fragments before waiting
    for it.  Eager and replayed from a CUDA graph, both launch shapes, results against the reference's."""
    env = dict(os.environ, HOGATT_PDL=pdl)
    res = subprocess.run([sys.executable, "-c", PDL_SCRIPT.format(root=ROOT)], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "PDL_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
