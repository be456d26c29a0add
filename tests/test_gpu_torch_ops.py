"""GPU parity through the torch operator surface (the drop-in boundary)."""
import numpy as np
import pytest
import torch

from inference_lib_b200 import workloads as wl
from oracle import hogwild_oracle as oracle
from tests.gpu_util import check_against

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def A():
    import inference_lib_b200.attention as mod
    return mod


@pytest.mark.parametrize("name", ["cfg1", "cfg2", "ragged_bf16", "ragged_f16", "causal_chunk_bf16", "blind_worker_bf16"])
def test_hogwild_fused_operator(A, golden, name):
    p = wl.baseline_problem(name) if name.startswith("cfg") else wl.edge_problem(name)
    d = p.to("cuda:0")
    rq = torch.empty((p.F, p.W, p.Hq, p.S, p.E), dtype=p.dtype, device="cuda:0")
    out = torch.empty((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device="cuda:0")
    res = A.hogwild_fused(d.queries, d.locations, d.keys, d.values, p.scale, d.fragment_lengths, d.cos, d.sin,
                          rotated_queries=rq, out=out)
    torch.cuda.synchronize()
    assert res is out
    check_against(out, golden[f"{name}/out"], p.dtype, what=name)
    ref_rq = oracle.rotate_queries(p.queries, p.cos, p.sin)
    assert torch.equal(rq.cpu(), ref_rq)


@pytest.mark.parametrize("name", ["cfg1", "gqa5_bf16", "d64_bf16"])
def test_hogwild_sdpa_and_rope_operators(A, golden, name):
    p = wl.baseline_problem(name) if name.startswith("cfg") else wl.edge_problem(name)
    d = p.to("cuda:0")
    rq = A.hogwild_rope(d.queries, d.cos, d.sin)
    assert torch.equal(rq.cpu(), oracle.rotate_queries(p.queries, p.cos, p.sin))
    out = A.hogwild_sdpa(rq, d.locations, d.keys, d.values, p.scale)       # lengths derived from the tensors
    torch.cuda.synchronize()
    check_against(out, golden[f"{name}/out"], p.dtype, what=name)


def test_operators_run_on_a_side_stream(A, golden):
    p = wl.edge_problem("ragged_bf16")
    d = p.to("cuda:0")
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        rq = torch.empty((p.F, p.W, p.Hq, p.S, p.E), dtype=p.dtype, device="cuda:0")
        out = torch.empty((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device="cuda:0")
        for _ in range(3):
            A.hogwild_fused(d.queries, d.locations, d.keys, d.values, p.scale, d.fragment_lengths, d.cos, d.sin,
                            rotated_queries=rq, out=out)
    s.synchronize()
    check_against(out, golden["ragged_bf16/out"], p.dtype)


def test_operator_rejects_what_the_reference_silently_ignores(A):
    """Unsupported head size / dtype: the reference prints and returns success; here it raises."""
    q = torch.zeros(1, 2, 1, 24, device="cuda:0", dtype=torch.bfloat16)
    k = [torch.zeros(1, 1, 8, 24, device="cuda:0", dtype=torch.bfloat16)]
    loc = torch.zeros(1, 1, 1, dtype=torch.int32, device="cuda:0")
    with pytest.raises(RuntimeError):
        A.hogwild_sdpa(q.unsqueeze(0), loc, k, k, 1.0)
    with pytest.raises(RuntimeError):
        A.hogwild_sdpa(q.unsqueeze(0).double(), loc, [x.double() for x in k], [x.double() for x in k], 1.0)
