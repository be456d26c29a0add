"""The entry point that takes no workspace (``hogatt_fused_launch_static``).

It serves hosts that may not allocate device memory where they call the library (host callbacks of
another runtime, processes whose device memory belongs to another allocator, loops that must not
synchronise the device): the split-K
scratch is a fixed array inside the library.  Its results must equal those of the regular entry
point, call after call, although every call reuses the same array with the previous call's contents
still in it.  This file sorts last on purpose, so that a run which stops at the first failure has
already been through every other test.
"""
import pytest
import torch

from inference_lib_b200 import _cabi
from inference_lib_b200 import workloads as wl
from tests.gpu_util import check_against, run_cabi

pytestmark = pytest.mark.gpu


def _static_call(p: wl.Problem):
    dev = torch.device("cuda:0")
    d = p.to(dev)
    out = torch.full((p.W, p.Hq, p.S, p.Ev), float("nan"), dtype=p.dtype, device=dev)
    rq = torch.zeros((p.F, p.W, p.Hq, p.S, p.E), dtype=p.dtype, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    bp = _cabi.bind(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values, scale=p.scale,
                    fragment_lengths=d.fragment_lengths, cos=d.cos, sin=d.sin, rq=rq, status=status)   # no workspace
    rc = _cabi.launch_static(bp, torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize(dev)
    return rc, out, rq, int(status.item())


def test_static_scratch_entry_point_matches_the_regular_one_on_consecutive_calls(golden):
    # three calls in a row; the second needs far less scratch than the first, so it runs on top of
    # the first call's leftovers; the third is fp32 through the FMA kernel
    for name in ("split_many_bf16", "ragged_bf16", "split_many_f32", "hidden_and_partial_bf16"):
        p = wl.edge_problem(name)
        rc, out, rq, status = _static_call(p)
        assert rc == 0 and status == 0, (name, rc, _cabi.status_string(rc))
        ref = run_cabi(p, want_rq=True)
        assert ref.rc == 0
        # same kernels, same decomposition: not merely within tolerance but identical
        assert torch.equal(out, ref.out), name
        assert torch.equal(rq, ref.rq), name
        check_against(out, golden[f"{name}/out"], p.dtype, what=name)


def test_static_scratch_entry_point_refuses_problems_beyond_its_fixed_size():
    # 2048 query rows per kv head -> 64 units of 64 rows with 4 partial slots each: about 8.5 MB of scratch
    p = wl.make_problem("too_big_for_static", W=64, Hq=16, Hkv=2, E=128, S=4, lengths=[8] + [4] * 64, theta=1e4,
                        dtype=torch.bfloat16, seed=3)
    dev = torch.device("cuda:0")
    d = p.to(dev)
    out = torch.zeros((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device=dev)
    bp = _cabi.bind(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values, scale=p.scale,
                    fragment_lengths=d.fragment_lengths, cos=d.cos, sin=d.sin)
    assert _cabi.workspace_bytes(bp) > _cabi.STATIC_SCRATCH_BYTES
    rc = _cabi.launch_static(bp, torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize(dev)
    assert rc == -11 and "HOGATT_STATIC_SCRATCH_BYTES" in _cabi.status_string(rc)
    assert (out == 0).all(), "a refused call must not launch anything"
    # the regular entry point takes the same problem with a caller workspace
    assert run_cabi(p).rc == 0
