"""The CPU oracle against the outputs of the reference itself (tests/golden)."""
import numpy as np
import pytest
import torch

from inference_lib_b200 import workloads as wl
from oracle import hogwild_oracle as oracle

CFG5_SLICE = (slice(None), slice(None, None, 8), slice(None, None, 4), slice(None))
FAST_BASELINE = ["cfg1", "cfg2", "cfg3", "target"]


def _same(a: torch.Tensor, b: np.ndarray, atol):
    a = a.to(torch.float32).numpy()
    assert a.shape == b.shape
    nan_a, nan_b = np.isnan(a), np.isnan(b)
    assert (nan_a == nan_b).all(), "rows without any visible key must be NaN in both"
    diff = np.abs(np.where(nan_a, 0, a) - np.where(nan_b, 0, b))
    assert diff.max() <= atol, diff.max()


@pytest.mark.parametrize("name", FAST_BASELINE)
def test_oracle_matches_reference_on_baseline_shapes(golden, name):
    p = wl.baseline_problem(name)
    out, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale)
    # same fp32 math, only the GEMM blocking may differ
    _same(out, golden[f"{name}/out"], atol=2e-5)


def test_oracle_matches_reference_on_one_causal_chunk_group(golden):
    p = wl.baseline_problem("cfg5", seed=2)
    out, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale)
    _same(out[CFG5_SLICE], golden["cfg5_g2/out"], atol=2e-5)


@pytest.mark.parametrize("name", sorted(wl.EDGE_CASES))
def test_oracle_matches_reference_on_edge_cases(golden, name):
    p = wl.edge_problem(name)
    out, rq = oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale)
    _same(out, golden[f"{name}/out"], atol=2e-5)
    if f"{name}/rq" in golden.files:
        assert np.array_equal(rq.to(torch.float32).numpy(), golden[f"{name}/rq"]), "rotation must be bit-exact"


def test_blind_rows_are_the_nan_rows(golden):
    for name in ("blind_worker_bf16", "blind_worker_f32", "hidden_and_partial_bf16"):
        p = wl.edge_problem(name)
        blind = oracle.blind_rows(p.locations, p.fragment_lengths)          # [W,S]
        nan_rows = np.isnan(golden[f"{name}/out"]).all(axis=(1, 3))         # [W,S]
        assert np.array_equal(blind.numpy(), nan_rows)


def test_scalar_rope_matches_tensor_rope(golden):
    """rope_cpu-style scalar loops == apply_rotary_pos_emb-style tensor code == the reference."""
    for name in ("cfg1", "ragged_f32"):
        p = wl.baseline_problem(name) if name == "cfg1" else wl.edge_problem(name)
        rows = oracle.rope_rows(p.queries.numpy(), p.cos.numpy(), p.sin.numpy())
        assert np.array_equal(rows, golden[f"{name}/rq"])
    p = wl.edge_problem("partial_rotary_bf16")
    rows = oracle.rope_rows(p.queries.float().numpy(), p.cos.numpy(), p.sin.numpy())
    rows = torch.from_numpy(rows).to(torch.bfloat16).float().numpy()
    assert np.array_equal(rows, golden["partial_rotary_bf16/rq"])


def test_intermediates_are_consistent():
    p = wl.edge_problem("causal_chunk_f32")
    rq = oracle.rotate_queries(p.queries, p.cos, p.sin)
    out, qk, att = oracle.sdpa(rq, p.locations, p.keys, p.values, p.scale, return_intermediate=True)
    assert qk.shape[-1] == sum(p.meta["lengths"])
    assert torch.allclose(att.sum(-1), torch.ones_like(att.sum(-1)), atol=1e-5)
    assert torch.isinf(qk).any()            # causal masking inside the worker's own fragment


def test_paged_oracle_equals_fragment_oracle_on_gathered_blocks():
    torch.manual_seed(0)
    W, Hq, Hkv, E, S, bs, F = 2, 4, 2, 64, 1, 16, 2
    lens = torch.tensor([37, 20], dtype=torch.int32)
    nblk = 8
    kc, vc = torch.randn(nblk, Hkv, bs, E), torch.randn(nblk, Hkv, bs, E)
    table = torch.tensor([[3, 1, 6, 0], [2, 7, 5, 4]], dtype=torch.int32)
    rq = torch.randn(F, W, Hq, S, E)
    loc = torch.tensor([[[36], [30]], [[19], [5]]], dtype=torch.int32)
    out = oracle.paged_sdpa(rq, loc, lens, kc, vc, table, 0.125)
    for w in range(W):
        ks = [oracle.gather_pages(kc, table[w], int(lens[f])) for f in range(F)]
        vs = [oracle.gather_pages(vc, table[w], int(lens[f])) for f in range(F)]
        ref = oracle.sdpa(rq[:, w:w + 1], loc[:, w:w + 1], ks, vs, 0.125)
        assert torch.equal(out[w:w + 1], ref)
    # token l of worker w lives in block table[w, l // bs], row l % bs
    assert torch.equal(oracle.gather_pages(kc, table[1], 20)[0, :, 17], kc[7, :, 1])


def test_varlen_oracle_equals_fixed_layout_oracle_when_lengths_are_equal():
    torch.manual_seed(1)
    W, S, Hq, Hkv, E, bs, F = 2, 3, 4, 2, 64, 8, 2
    kc, vc = torch.randn(12, Hkv, bs, E), torch.randn(12, Hkv, bs, E)
    table = torch.tensor([[3, 1, 6, 0, 9], [2, 7, 5, 4, 8]], dtype=torch.int32)
    lens = torch.tensor([33, 20], dtype=torch.int32)
    rq = torch.randn(F, W, Hq, S, E)
    loc = torch.randint(0, 40, (F, W, S), dtype=torch.int32)
    fixed = oracle.paged_sdpa(rq, loc, lens, kc, vc, table, 0.125)                       # [W,Hq,S,Ev]
    packed_q = rq.permute(0, 1, 3, 2, 4).reshape(F, W * S, Hq, E)
    packed = oracle.varlen_paged_sdpa(packed_q, loc.reshape(F, W * S), lens[:, None].expand(F, W).contiguous(), kc, vc,
                                      table, torch.tensor([0, S, 2 * S], dtype=torch.int32), 0.125)
    assert torch.allclose(packed.reshape(W, S, Hq, E).permute(0, 2, 1, 3), fixed, atol=1e-6)


def test_copy_to_blocks_oracle_addresses():
    kc, vc = torch.zeros(6, 2, 4, 8), torch.zeros(6, 2, 4, 8)
    table = torch.tensor([[5, 2, 0], [1, 3, 4]], dtype=torch.int32)
    ks, vs = torch.ones(2, 2, 3, 8), 2 * torch.ones(2, 2, 3, 8)
    oracle.copy_to_blocks(ks, vs, kc, vc, table, torch.tensor([3, 0], dtype=torch.int32))
    assert kc[5, :, 3].eq(1).all() and kc[2, :, 0].eq(1).all() and kc[2, :, 1].eq(1).all() and kc[2, :, 2].eq(0).all()
    assert vc[1, :, :3].eq(2).all() and vc[1, :, 3].eq(0).all()
