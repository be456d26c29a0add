"""GPU parity of the tcgen05 kernel (``HOGATT_KERNEL_DENSE``): calls with at least 128 query rows per kv head.

Every row of every output is compared, against the reference's own outputs where they are stored
(``tests/golden/``) and against the oracle otherwise; tolerance as everywhere: 16-bit output against the fp32
reference max-abs <= 2e-2 and mean-abs <= 2e-3.
"""
import os

import numpy as np
import pytest
import torch

from inference_lib_b200 import _cabi
from inference_lib_b200 import workloads as wl
from oracle import hogwild_oracle as oracle
from tests.gpu_util import check_against, run_cabi

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
CFG5_SLICE = (slice(None), slice(None, None, 8), slice(None, None, 4), slice(None))
DENSE_CASES = ["dense_chunk_bf16", "dense_small_gs_bf16", "dense_big_gs_f16", "dense_partial_block_bf16"]


@pytest.mark.parametrize("name", DENSE_CASES)
@pytest.mark.parametrize("host_plan", [False, True])
def test_dense_edge_cases_match_reference(golden, name, host_plan):
    p = wl.edge_problem(name)
    r = run_cabi(p, kernel=_cabi.KERNEL_DENSE, want_rq=True, host_lengths="rows" if host_plan else None)
    assert r.rc == 0 and r.status == 0, (r.rc, r.status)
    check_against(r.out, golden[f"{name}/out"], p.dtype, what=name)
    assert torch.equal(r.rq.cpu(), oracle.rotate_queries(p.queries, p.cos, p.sin)), "rotated queries must be bit-exact"


@pytest.mark.parametrize("name", DENSE_CASES)
def test_auto_takes_the_dense_kernel_and_agrees_with_the_other_kernels(golden, name):
    p = wl.edge_problem(name)
    d = p.to("cuda:0")
    out = torch.empty((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device="cuda:0")
    bp = _cabi.bind(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values, scale=p.scale,
                    cos=d.cos, sin=d.sin)
    assert _cabi.launch_shape(bp)["kernel"] == _cabi.KERNEL_DENSE
    auto = run_cabi(p)
    mma = run_cabi(p, kernel=_cabi.KERNEL_MMA)
    assert auto.rc == 0 and mma.rc == 0
    check_against(auto.out, golden[f"{name}/out"], p.dtype, what=name)
    assert (auto.out.float() - mma.out.float()).abs().max() <= 2e-2


@pytest.mark.parametrize("max_ctas", [1, 2, 5, 37])
def test_dense_result_does_not_depend_on_the_grid(golden, max_ctas):
    for name in ("dense_chunk_bf16", "dense_partial_block_bf16"):
        p = wl.edge_problem(name)
        r = run_cabi(p, kernel=_cabi.KERNEL_DENSE, max_ctas=max_ctas, host_lengths="rows")
        assert r.rc == 0 and r.status == 0
        check_against(r.out, golden[f"{name}/out"], p.dtype, what=f"{name} ctas {max_ctas}")


def test_dense_prerotated_entry_point_equals_fused():
    p = wl.edge_problem("dense_chunk_bf16")
    rq = oracle.rotate_queries(p.queries, p.cos, p.sin)
    a = run_cabi(p, kernel=_cabi.KERNEL_DENSE, fused=True)
    b = run_cabi(p, kernel=_cabi.KERNEL_DENSE, fused=False, pre_rotated=rq)
    assert a.rc == 0 and b.rc == 0
    assert torch.equal(a.out, b.out)


def test_dense_rows_past_the_true_length_never_reach_a_result():
    """Slabs with spare rows holding NaN / Inf, device lengths shorter than the tensors, a loose host bound."""
    p = wl.edge_problem("dense_chunk_bf16")                       # lengths 300, 40, 150
    true_len = [200, 33, 129]
    short = torch.tensor(true_len, dtype=torch.int32)
    # locations as they would be for the true lengths
    orders = [[0, 2, 1], [0, 1, 2]]
    loc = wl.hogwild_locations(true_len, orders, p.S)
    cos, sin = wl.rope_tables(loc, p.E, p.theta)
    q = wl.Problem(**{**p.__dict__, "fragment_lengths": short, "locations": loc, "cos": cos.contiguous(), "sin": sin.contiguous()})
    ref, _ = oracle.fused(q.queries, q.cos, q.sin, q.locations, [k[:, :, :n] for k, n in zip(p.keys, true_len)],
                          [v[:, :, :n] for v, n in zip(p.values, true_len)], p.scale)
    keys, values = [], []
    for k, v, n in zip(p.keys, p.values, true_len):
        k, v = k.clone(), v.clone()
        k[:, :, n:] = float("nan")
        v[:, :, n:] = float("inf")
        keys.append(k.to("cuda:0"))
        values.append(v.to("cuda:0"))
    for hl in (None, "rows", true_len):
        r = run_cabi(q, kernel=_cabi.KERNEL_DENSE, host_lengths=hl, keys=keys, values=values)
        assert r.rc == 0 and r.status == 0
        check_against(r.out, ref.numpy(), p.dtype, what=f"host bound {hl}")


@pytest.mark.parametrize("group", range(4))
def test_causal_chunk_config_every_group_every_row(golden, group):
    """BASELINE configuration 5 (8 workers x 16-token chunks, GQA 8, 24,576 keys): each of the four groups, every
    output row against the oracle; the rows the reference's own outputs are stored for against those as well
    (group 0: all of them)."""
    p = wl.baseline_problem("cfg5", seed=group)
    r = run_cabi(p, want_rq=False, host_lengths="rows")
    assert r.rc == 0 and r.status == 0
    check_against(r.out[CFG5_SLICE], golden[f"cfg5_g{group}/out"], p.dtype, what=f"cfg5 group {group} (stored rows)")
    if group == 0:
        full = np.load(os.path.join(ROOT, "tests", "golden", "cfg5_g0_full.npz"))["out"]
        check_against(r.out, full, p.dtype, what="cfg5 group 0, every row, reference output")
    else:
        torch.set_num_threads(os.cpu_count() or 1)
        ref, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale)
        check_against(r.out, ref.numpy(), p.dtype, what=f"cfg5 group {group}, every row")


def test_dense_is_refused_where_it_cannot_run():
    # 12 rows per kv head; G*S = 5 divides nothing; 40 rows of fp32 -- none of them can take the tcgen05 kernel
    for name in ("ragged_bf16", "gqa5_bf16", "causal_chunk_f32"):
        p = wl.edge_problem(name)
        d = p.to("cuda:0")
        out = torch.zeros((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device="cuda:0")
        ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda:0")
        bp = _cabi.bind(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values, scale=p.scale,
                        cos=d.cos, sin=d.sin, workspace=ws, kernel=_cabi.KERNEL_DENSE)
        assert _cabi.workspace_bytes(bp) == 0
        assert _cabi.launch(bp, torch.cuda.current_stream().cuda_stream) == -9
        torch.cuda.synchronize()
        assert (out == 0).all()
