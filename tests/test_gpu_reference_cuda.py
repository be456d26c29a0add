"""The reference's own CUDA kernels, recompiled for sm_100a (``oracle/_ref/hogatt_ref.so``), as a checker.

Their launchers take one head layout only -- head size 128, 16 query heads per kv head
(``src/kernels/kernel_v21.cuh:982-986,1025,1074``) -- so at that layout this package's operators are compared with
them directly: the fragment op, and the three paged operators, for which the reference has no other implementation
(this is what pins ``hogwild_paged_sdpa`` / ``hogwild_varlen_paged_sdpa`` / ``copy_to_blocks``).  The reference runs
in a child process (``oracle/ref_cuda_runner.py``): it registers the same operator names, keeps static device buffers
and uses the default stream.  Skipped where the library was never built (no reference checkout at build time).
"""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from inference_lib_b200 import workloads as wl
from oracle import hogwild_oracle as oracle
from tests.gpu_util import check_against, run_cabi

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "hogatt_ref.so")
DEV = "cuda:0"


def _reference(jobs):
    if not os.path.exists(REF_LIB):
        pytest.skip("the reference's CUDA extension was not built (no reference checkout at build time)")
    with tempfile.TemporaryDirectory() as tmp:
        src, dst = os.path.join(tmp, "jobs.pt"), os.path.join(tmp, "results.pt")
        torch.save(jobs, src)
        res = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "ref_cuda_runner.py"), "check", src, dst],
                             capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
        return torch.load(dst)


@pytest.fixture(scope="module")
def A():
    import inference_lib_b200.attention as mod
    return mod


@pytest.mark.parametrize("name", ["gqa16_bf16", "gqa16"])
def test_fragment_op_against_the_reference_kernel(golden, name):
    p = wl.edge_problem(name) if name in wl.EDGE_CASES else wl.baseline_problem(name)
    ref = _reference({"fragment": dict(queries=p.queries, keys=p.keys, values=p.values, locations=p.locations, cos=p.cos,
                                       sin=p.sin, fragment_lengths=p.fragment_lengths, scale=p.scale)})["fragment"]
    ours = run_cabi(p, want_rq=True)
    assert ours.rc == 0 and ours.status == 0
    # The reference's two rotations do not agree with each other to the last bit: its PyTorch path rounds both products
    # before adding them (what this package reproduces bit for bit, see the goldens), its rope kernel lets the compiler
    # fuse a multiply-add.  Against the kernel, then: at most one unit in the last place, on few elements.
    mine, theirs = ours.rq.float().cpu(), ref["rq"].float()
    differ = mine != theirs
    assert differ.float().mean() < 0.02
    assert ((mine - theirs).abs() <= theirs.abs() * 2.0 ** -7 + 1e-30).all()
    truth, _ = oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale)
    check_against(ours.out, truth.numpy(), p.dtype, what=f"{name}: this package")
    check_against(ref["out"], truth.numpy(), p.dtype, what=f"{name}: reference kernel")
    assert (ours.out.float().cpu() - ref["out"].float()).abs().max() <= 2e-2


def _caches(rng, W, Hkv, bs, E, Ev, max_len, dtype):
    max_blocks = (max_len + bs - 1) // bs + 1
    nblk = W * max_blocks + 3
    g = torch.Generator().manual_seed(int(rng.integers(1 << 30)))
    kc = torch.randn(nblk, Hkv, bs, E, generator=g).to(dtype)
    vc = torch.randn(nblk, Hkv, bs, Ev, generator=g).to(dtype)
    perm = torch.from_numpy(rng.permutation(nblk)[: W * max_blocks].astype(np.int32)).reshape(W, max_blocks)
    return kc, vc, perm.contiguous(), g


@pytest.mark.parametrize("dtype,W,S,Hkv,bs,F", [(torch.bfloat16, 2, 2, 1, 8, 2), (torch.float16, 3, 1, 2, 16, 3),
                                                (torch.bfloat16, 4, 3, 2, 32, 1)])
def test_paged_sdpa_against_the_reference_kernel(A, dtype, W, S, Hkv, bs, F):
    rng = np.random.default_rng(W * 100 + S * 10 + F)
    E, Hq = 128, 16 * Hkv
    lens = torch.tensor([int(rng.integers(1, 300)) for _ in range(F)], dtype=torch.int32)
    kc, vc, table, g = _caches(rng, W, Hkv, bs, E, E, int(lens.max()), dtype)
    rq = torch.randn(F, W, Hq, S, E, generator=g).to(dtype)
    loc = torch.from_numpy(rng.integers(-1, int(lens.max()) + 20, size=(F, W, S)).astype(np.int32))
    loc[0] = torch.clamp(loc[0], min=0)                           # every row sees at least one key
    scale = E ** -0.5
    ref = _reference({"paged": dict(queries=rq, locations=loc, fragment_lengths=lens, key_cache=kc, value_cache=vc,
                                    block_table=table, scale=scale)})["paged"]["out"]
    out = A.hogwild_paged_sdpa(rq.to(DEV), loc.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), scale, lens.to(DEV))
    torch.cuda.synchronize()
    truth = oracle.paged_sdpa(rq, loc, lens, kc, vc, table, scale)
    check_against(ref, truth.numpy(), dtype, what="reference paged kernel against the gathered-fragment oracle")
    check_against(out, truth.numpy(), dtype, what="paged operator of this package")
    assert (out.float().cpu() - ref.float()).abs().max() <= 2e-2


@pytest.mark.parametrize("dtype,bs,seqs", [(torch.bfloat16, 16, [3, 2, 4]), (torch.float16, 8, [1, 5])])
def test_varlen_paged_sdpa_against_the_reference_kernel(A, dtype, bs, seqs):
    rng = np.random.default_rng(len(seqs) * 7 + bs)
    W, Hkv, F, E = len(seqs), 2, 2, 128
    Hq = 16 * Hkv
    cu = torch.tensor([0] + list(np.cumsum(seqs)), dtype=torch.int32)
    total_q = int(cu[-1])
    lens = torch.from_numpy(rng.integers(1, 200, size=(F, W)).astype(np.int32))
    kc, vc, table, g = _caches(rng, W, Hkv, bs, E, E, int(lens.max()), dtype)
    rq = torch.randn(F, total_q, Hq, E, generator=g).to(dtype)
    loc = torch.from_numpy(rng.integers(-1, 220, size=(F, total_q)).astype(np.int32))
    loc[0] = torch.clamp(loc[0], min=0)
    scale = E ** -0.5
    ref = _reference({"varlen": dict(queries=rq, locations=loc, fragment_lengths=lens, key_cache=kc, value_cache=vc,
                                     block_table=table, cu_seqlens_q=cu, scale=scale)})["varlen"]["out"]
    out = A.hogwild_varlen_paged_sdpa(rq.to(DEV), loc.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), scale, lens.to(DEV),
                                      cu.to(DEV))
    torch.cuda.synchronize()
    truth = oracle.varlen_paged_sdpa(rq, loc, lens, kc, vc, table, cu, scale)
    check_against(ref, truth.numpy(), dtype, what="reference packed-query kernel against the gathered-fragment oracle")
    check_against(out, truth.numpy(), dtype, what="packed-query operator of this package")
    assert (out.float().cpu() - ref.float()).abs().max() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_copy_to_blocks_against_the_reference_kernel(A, dtype):
    rng = np.random.default_rng(5)
    B, Hkv, S_new, E, bs = 3, 2, 5, 128, 16
    kc, vc, table, g = _caches(rng, B, Hkv, bs, E, E, 100, dtype)
    ks = torch.randn(B, Hkv, S_new, E, generator=g).to(dtype)
    vs = torch.randn(B, Hkv, S_new, E, generator=g).to(dtype)
    seq = torch.tensor([0, 14, 61], dtype=torch.int32)            # crosses block boundaries
    ref = _reference({"copy": dict(key_states=ks, value_states=vs, key_cache=kc, value_cache=vc, block_table=table,
                                   seq_lengths=seq)})["copy"]
    dk, dv = kc.to(DEV), vc.to(DEV)
    A.copy_to_blocks(ks.to(DEV), vs.to(DEV), dk, dv, table.to(DEV), seq.to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(dk.cpu(), ref["key_cache"]) and torch.equal(dv.cpu(), ref["value_cache"])
    ok, ov = oracle.copy_to_blocks(ks, vs, kc.clone(), vc.clone(), table, seq)
    assert torch.equal(ref["key_cache"], ok) and torch.equal(ref["value_cache"], ov), "the by-construction oracle equals the reference"
