"""GPU parity: the CUDA path (through the C ABI) against the reference's outputs and the oracle."""
import numpy as np
import pytest
import torch

from inference_lib_b200 import _cabi
from inference_lib_b200 import workloads as wl
from oracle import hogwild_oracle as oracle
from tests.gpu_util import check_against, run_cabi

pytestmark = pytest.mark.gpu

CFG5_SLICE = (slice(None), slice(None, None, 8), slice(None, None, 4), slice(None))


def _kernels_for(p, cluster=True):
    ks = []
    if p.dtype != torch.float32 and p.E == p.Ev and p.E in (64, 128):
        ks.append(_cabi.KERNEL_MMA)
        rows = p.W * (p.Hq // p.Hkv) * p.S
        rows_per_block = 16 if rows <= 16 else (32 if rows <= 32 else 64)
        units = -(-rows // rows_per_block) * p.Hkv
        if cluster and 2 * units <= torch.cuda.get_device_properties(0).multi_processor_count:
            ks.append(_cabi.KERNEL_MMA_CLUSTER)      # same kernel, launched in clusters that merge by themselves
    if p.Ev in (32, 64, 128, 256):
        ks.append(_cabi.KERNEL_FMA)
    return ks


@pytest.mark.parametrize("name", ["cfg1", "cfg2", "cfg3", "target", "cfg4"])
def test_baseline_shapes_match_reference(golden, name):
    p = wl.baseline_problem(name)
    r = run_cabi(p)
    assert r.rc == 0 and r.status == 0
    check_against(r.out, golden[f"{name}/out"], p.dtype, what=name)


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "target", "cfg4"])
@pytest.mark.parametrize("kernel", [_cabi.KERNEL_MMA, _cabi.KERNEL_MMA_CLUSTER])
def test_both_launch_shapes_of_the_tensor_core_kernel(golden, name, kernel):
    p = wl.baseline_problem(name)
    r = run_cabi(p, kernel=kernel, want_rq=True)
    assert r.rc == 0 and r.status == 0
    check_against(r.out, golden[f"{name}/out"], p.dtype, what=f"{name} kernel {kernel}")
    if f"{name}/rq" in golden.files:
        assert np.array_equal(r.rq.float().cpu().numpy(), golden[f"{name}/rq"])


def test_cluster_shape_is_refused_when_units_exceed_half_the_sms():
    p = wl.baseline_problem("cfg5", seed=0)          # 128 units
    r = run_cabi(p, kernel=_cabi.KERNEL_MMA_CLUSTER)
    assert r.rc == -9


def test_one_workspace_serves_many_launches_and_shapes(golden):
    """The workspace carries nothing from one launch to the next: any contents, any sequence of shapes."""
    names = ["cfg2", "target", "ragged_bf16", "cfg3", "cfg2", "gqa5_bf16", "target"]
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream(dev).cuda_stream
    ws = torch.full((64 << 20,), 0xFF, dtype=torch.uint8, device=dev)       # NaN in every fp32 word
    ptr = ws.data_ptr() + (-ws.data_ptr()) % 256
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for name in names:
        p = wl.baseline_problem(name) if name in wl.BASELINE_CONFIGS else wl.edge_problem(name)
        d = p.to(dev)
        out = torch.full((p.W, p.Hq, p.S, p.Ev), float("nan"), dtype=p.dtype, device=dev)
        bp = _cabi.bind(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values, scale=p.scale,
                        fragment_lengths=d.fragment_lengths, cos=d.cos, sin=d.sin, status=status)
        need = _cabi.workspace_bytes(bp)
        assert 0 < need <= 32 << 20
        bp.struct.workspace, bp.struct.workspace_bytes = ptr, need
        assert _cabi.launch(bp, stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0, name
        check_against(out, golden[f"{name}/out"], p.dtype, what=name)


def test_launch_shape_matches_what_runs():
    p = wl.baseline_problem("target")
    d = p.to("cuda:0")
    out = torch.empty((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device="cuda:0")
    mk = lambda k: _cabi.bind(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values,
                              scale=p.scale, cos=d.cos, sin=d.sin, kernel=k)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    shape = _cabi.launch_shape(mk(_cabi.KERNEL_MMA))
    assert shape == dict(kernel=_cabi.KERNEL_MMA, ctas=sms, cluster=0, kernels_per_call=2)
    shape = _cabi.launch_shape(mk(_cabi.KERNEL_MMA_CLUSTER))
    assert shape["kernel"] == _cabi.KERNEL_MMA_CLUSTER and shape["kernels_per_call"] == 1
    assert 2 <= shape["cluster"] <= 16 and shape["ctas"] == 8 * shape["cluster"] <= sms
    # left to itself the library takes the persistent grid for this shape ...
    assert _cabi.launch_shape(mk(_cabi.KERNEL_AUTO))["kernels_per_call"] == 2
    # ... and for one rank's share of it when the kv heads are spread over 4 GPUs (clusters only on request)
    part = p.shard(0, 4).to("cuda:0")
    out4 = torch.empty((part.W, part.Hq, part.S, part.Ev), dtype=p.dtype, device="cuda:0")
    mk4 = lambda k: _cabi.bind(out=out4, queries=part.queries, locations=part.locations, keys=part.keys, values=part.values,
                               scale=part.scale, cos=part.cos, sin=part.sin, kernel=k)
    assert _cabi.launch_shape(mk4(_cabi.KERNEL_AUTO)) == dict(kernel=_cabi.KERNEL_MMA, ctas=sms, cluster=0, kernels_per_call=2)
    shape = _cabi.launch_shape(mk4(_cabi.KERNEL_MMA_CLUSTER))
    assert shape["kernel"] == _cabi.KERNEL_MMA_CLUSTER and shape["cluster"] == 16 and shape["ctas"] == 32


def test_causal_chunk_config_matches_reference(golden):
    p = wl.baseline_problem("cfg5", seed=2)
    r = run_cabi(p)
    assert r.rc == 0 and r.status == 0
    check_against(r.out[CFG5_SLICE], golden["cfg5_g2/out"], p.dtype, what="cfg5 group 2")


@pytest.mark.parametrize("name", sorted(wl.EDGE_CASES))
def test_edge_cases_match_reference_on_every_eligible_kernel(golden, name):
    p = wl.edge_problem(name)
    kernels = _kernels_for(p)
    assert kernels
    for k in kernels:
        r = run_cabi(p, kernel=k, want_rq=True)
        assert r.rc == 0 and r.status == 0, (name, k, r.rc, r.status)
        check_against(r.out, golden[f"{name}/out"], p.dtype, what=f"{name} kernel {k}")
        if f"{name}/rq" in golden.files:
            assert np.array_equal(r.rq.float().cpu().numpy(), golden[f"{name}/rq"]), "rotated queries must be bit-exact"


@pytest.mark.parametrize("name", ["ragged_bf16", "causal_chunk_bf16", "ragged_f32", "hidden_and_partial_bf16",
                                  "split_many_bf16", "many_rows_bf16", "row_blocks_bf16"])
@pytest.mark.parametrize("max_ctas", [1, 2, 3, 7, 31])
def test_result_does_not_depend_on_the_grid(golden, name, max_ctas):
    """Any number of CTAs cuts the tile list differently; the merged result must stay within tolerance."""
    p = wl.edge_problem(name)
    for k in _kernels_for(p, cluster=False):
        r = run_cabi(p, kernel=k, max_ctas=max_ctas)
        assert r.rc == 0 and r.status == 0
        check_against(r.out, golden[f"{name}/out"], p.dtype, what=f"{name} ctas {max_ctas} kernel {k}")


@pytest.mark.parametrize("name", ["ragged_bf16", "cfg1", "causal_chunk_bf16", "gqa5_bf16"])
def test_prerotated_entry_point_equals_fused(golden, name):
    p = wl.baseline_problem(name) if name.startswith("cfg") else wl.edge_problem(name)
    rq = oracle.rotate_queries(p.queries, p.cos, p.sin)
    a = run_cabi(p, fused=True)
    b = run_cabi(p, fused=False, pre_rotated=rq)
    assert a.rc == 0 and b.rc == 0
    assert torch.equal(a.out, b.out), "same rounded queries, same kernel: results must be identical"
    check_against(b.out, golden[f"{name}/out"], p.dtype, what=name)


def test_mma_and_fma_kernels_agree():
    p = wl.edge_problem("split_many_bf16")
    a = run_cabi(p, kernel=_cabi.KERNEL_MMA)
    b = run_cabi(p, kernel=_cabi.KERNEL_FMA)
    assert a.rc == 0 and b.rc == 0
    assert (a.out.float() - b.out.float()).abs().max() <= 1e-2


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes_against_oracle(seed):
    rng = np.random.default_rng(seed)
    dtype = [torch.bfloat16, torch.float16, torch.float32][seed % 3]
    E = int(rng.choice([64, 128]))
    W, S = int(rng.integers(1, 5)), int(rng.integers(1, 4))
    Hkv, G = int(rng.integers(1, 4)), int(rng.choice([1, 2, 4, 7]))
    lengths = [int(rng.integers(1, 400))] + [int(rng.integers(S, 70)) for _ in range(W)]
    p = wl.make_problem(f"rand{seed}", W=W, Hq=Hkv * G, Hkv=Hkv, E=E, S=S, lengths=lengths, theta=1e4, dtype=dtype,
                        seed=100 + seed)
    ref, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale)
    for k in _kernels_for(p):
        r = run_cabi(p, kernel=k)
        assert r.rc == 0 and r.status == 0
        check_against(r.out, ref.numpy(), p.dtype, what=f"seed {seed} kernel {k}")


@pytest.mark.parametrize("kernel", [_cabi.KERNEL_AUTO, _cabi.KERNEL_MMA, _cabi.KERNEL_MMA_CLUSTER])
def test_one_kv_head_spread_over_the_whole_gpu(kernel):
    """What one rank sees when 8 kv heads are sharded over 8 GPUs: a single (kv head, row block) unit, cut into
    one partial per SM on the persistent grid (the merge kernel's batched and strided passes both run) or into
    one cluster of 16 CTAs."""
    p = wl.make_problem("one_head", W=4, Hq=4, Hkv=1, E=128, S=1, lengths=[30000, 2048, 2048, 2048, 2049], theta=5e5,
                        dtype=torch.bfloat16, seed=77)
    ref, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale)
    r = run_cabi(p, kernel=kernel, want_rq=True)
    assert r.rc == 0 and r.status == 0
    check_against(r.out, ref.numpy(), p.dtype, what=f"one kv head, kernel {kernel}")


def test_device_lengths_shorter_than_the_tensors():
    """fragment_lengths (device) may be shorter than the tensors' row extent: only that prefix is visible."""
    p = wl.edge_problem("ragged_bf16")
    short = torch.tensor([20, 1, 4, 77], dtype=torch.int32)
    q = wl.Problem(**{**p.__dict__, "fragment_lengths": short})
    keys = [k[:, :, :int(n)] for k, n in zip(p.keys, short)]
    vals = [v[:, :, :int(n)] for v, n in zip(p.values, short)]
    ref, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, keys, vals, p.scale)
    r = run_cabi(q)
    assert r.rc == 0 and r.status == 0
    check_against(r.out, ref.numpy(), p.dtype)


def test_rope_entry_point_is_bit_exact(golden):
    import ctypes as C
    lib = _cabi.load()
    for name in ("cfg1", "ragged_f16", "ragged_bf16", "partial_rotary_bf16", "causal_chunk_bf16"):
        p = wl.baseline_problem(name) if name.startswith("cfg") else wl.edge_problem(name)
        d = p.to("cuda:0")
        rq = torch.empty((p.F, p.W, p.Hq, p.S, p.E), dtype=p.dtype, device="cuda:0")
        rc = lib.hogatt_rope_launch(rq.data_ptr(), d.queries.data_ptr(), d.cos.data_ptr(), d.sin.data_ptr(), p.F, p.W,
                                    p.Hq, p.S, p.E, p.cos.shape[-1], _cabi.dtype_code(p.dtype),
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert rc == 0
        assert np.array_equal(rq.float().cpu().numpy(), golden[f"{name}/rq"])


def test_bad_arguments_are_refused_without_launching():
    p = wl.edge_problem("ragged_bf16")
    d = p.to("cuda:0")
    out = torch.zeros((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device="cuda:0")
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda:0")
    mk = lambda **kw: _cabi.bind(**{**dict(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values,
                                           scale=p.scale, cos=d.cos, sin=d.sin, workspace=ws), **kw})
    bp = mk(); bp.struct.workspace_bytes = 16
    assert _cabi.launch(bp) == -7
    bp = mk(); bp.struct.Hkv = 3
    assert _cabi.launch(bp) == -2
    bp = mk(); bp.struct.F = 1000
    assert _cabi.launch(bp) == -5
    bp = mk(); bp.struct.dtype = 9
    assert _cabi.launch(bp) == -4
    bp = mk(kernel=_cabi.KERNEL_MMA); bp.struct.dtype = _cabi.F32
    assert _cabi.launch(bp) == -9
    bp = mk(); bp.struct.queries = d.queries.data_ptr() + 2
    assert _cabi.launch(bp) == -6
    bp = mk(); bp.struct.out = None
    assert _cabi.launch(bp) == -1
    torch.cuda.synchronize()
    assert (out == 0).all(), "a refused call must not touch the output"


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("name", ["target", "cfg3"])
@pytest.mark.parametrize("host_plan", [True, False])
def test_every_ranks_share_of_a_sharded_call_matches_the_reference_heads(golden, name, world, host_plan):
    """One GPU computes, rank by rank, what each rank of a kv-head-sharded call would: 32, 64 and 128-148 partials per
    row, i.e. every instantiation of the merge step (one warp per row with 32 slots; one CTA per row with four warps
    x 16, four x 24 and eight x 24).  The heads of each share against the same heads of the reference's output."""
    p = wl.baseline_problem(name)
    ref = golden[f"{name}/out"]
    hq = p.Hq // world
    for rank in (0, world - 1):
        part = p.shard(rank, world)
        r = run_cabi(part, host_lengths="rows" if host_plan else None, stable_fragments=1 if host_plan else 0)
        assert r.rc == 0 and r.status == 0
        check_against(r.out, ref[:, rank * hq:(rank + 1) * hq], p.dtype, what=f"{name} rank {rank} of {world}")
