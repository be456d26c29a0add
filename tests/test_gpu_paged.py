"""GPU parity of the paged operators against their oracle by construction (gather the blocks into
contiguous fragments, then the fragment oracle).  The reference has no CPU path for these operators,
so their parity is pinned only through the fragment oracle's own pin."""
import numpy as np
import pytest
import torch

from oracle import hogwild_oracle as oracle
from tests.gpu_util import check_against

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def A():
    import inference_lib_b200.attention as mod
    return mod


def _caches(rng, W, Hkv, bs, E, Ev, max_len, dtype):
    max_blocks = (max_len + bs - 1) // bs + 1
    nblk = W * max_blocks + 3
    g = torch.Generator().manual_seed(int(rng.integers(1 << 30)))
    kc = torch.randn(nblk, Hkv, bs, E, generator=g).to(dtype)
    vc = torch.randn(nblk, Hkv, bs, Ev, generator=g).to(dtype)
    perm = torch.from_numpy(rng.permutation(nblk)[: W * max_blocks].astype(np.int32)).reshape(W, max_blocks)
    return kc, vc, perm.contiguous(), g


CASES = [
    # dtype, W, S, Hkv, G, E, Ev, bs, F
    (torch.bfloat16, 2, 1, 2, 4, 128, 128, 16, 1),
    (torch.bfloat16, 3, 3, 2, 5, 128, 128, 32, 2),
    (torch.float16, 2, 2, 1, 16, 128, 128, 8, 2),
    (torch.float32, 2, 1, 2, 2, 64, 64, 16, 1),
    (torch.bfloat16, 2, 2, 1, 32, 128, 64, 16, 1),      # more than 16 heads per kv head, Ev != E
    (torch.float32, 4, 5, 2, 1, 64, 32, 4, 3),
]


@pytest.mark.parametrize("case", CASES, ids=[str(i) for i in range(len(CASES))])
def test_paged_sdpa_matches_the_gathered_fragment_oracle(A, case):
    dtype, W, S, Hkv, G, E, Ev, bs, F = case
    rng = np.random.default_rng(hash(case[1:]) % (1 << 31))
    Hq = Hkv * G
    lens = torch.tensor([int(rng.integers(1, 150)) for _ in range(F)], dtype=torch.int32)
    kc, vc, table, g = _caches(rng, W, Hkv, bs, E, Ev, int(lens.max()), dtype)
    rq = torch.randn(F, W, Hq, S, E, generator=g).to(dtype)
    loc = torch.from_numpy(rng.integers(-1, int(lens.max()) + 20, size=(F, W, S)).astype(np.int32))
    loc[0, :, :] = torch.clamp(loc[0], min=0)                       # every row sees at least one key
    ref = oracle.paged_sdpa(rq, loc, lens, kc, vc, table, E ** -0.5)
    out = A.hogwild_paged_sdpa(rq.to(DEV), loc.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), E ** -0.5, lens.to(DEV))
    torch.cuda.synchronize()
    check_against(out, ref.numpy(), dtype, what=str(case))


@pytest.mark.parametrize("dtype,G,E,bs,seqs", [(torch.bfloat16, 4, 128, 16, [3, 0, 7, 1]), (torch.float32, 2, 64, 8, [5, 2]),
                                                (torch.float16, 8, 128, 32, [1, 1, 1]), (torch.bfloat16, 20, 128, 16, [2, 3])])
def test_varlen_paged_sdpa_matches_the_gathered_fragment_oracle(A, dtype, G, E, bs, seqs):
    rng = np.random.default_rng(len(seqs) * 1000 + G)
    W, Hkv, F, Ev = len(seqs), 2, 2, E
    Hq = Hkv * G
    cu = torch.tensor([0] + list(np.cumsum(seqs)), dtype=torch.int32)
    total_q = int(cu[-1])
    lens = torch.from_numpy(rng.integers(1, 120, size=(F, W)).astype(np.int32))
    kc, vc, table, g = _caches(rng, W, Hkv, bs, E, Ev, int(lens.max()), dtype)
    rq = torch.randn(F, total_q, Hq, E, generator=g).to(dtype)
    loc = torch.from_numpy(rng.integers(-1, 140, size=(F, total_q)).astype(np.int32))
    loc[0] = torch.clamp(loc[0], min=0)
    ref = oracle.varlen_paged_sdpa(rq, loc, lens, kc, vc, table, cu, E ** -0.5)
    out = A.hogwild_varlen_paged_sdpa(rq.to(DEV), loc.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), E ** -0.5,
                                      lens.to(DEV), cu.to(DEV))
    torch.cuda.synchronize()
    check_against(out, ref.numpy(), dtype, what=f"varlen {seqs}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_copy_to_blocks_is_bit_exact(A, dtype):
    rng = np.random.default_rng(5)
    B, Hkv, S_new, E, Ev, bs = 3, 2, 5, 128, 64, 16
    kc, vc, table, g = _caches(rng, B, Hkv, bs, E, Ev, 100, dtype)
    ks = torch.randn(B, Hkv, S_new, E, generator=g).to(dtype)
    vs = torch.randn(B, Hkv, S_new, Ev, generator=g).to(dtype)
    seq = torch.tensor([0, 14, 61], dtype=torch.int32)              # crosses block boundaries
    ref_k, ref_v = oracle.copy_to_blocks(ks, vs, kc.clone(), vc.clone(), table, seq)
    dk, dv = kc.to(DEV), vc.to(DEV)
    A.copy_to_blocks(ks.to(DEV), vs.to(DEV), dk, dv, table.to(DEV), seq.to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(dk.cpu(), ref_k) and torch.equal(dv.cpu(), ref_v)


def test_append_then_attend_round_trip(A):
    """copy_to_blocks followed by paged attention sees the appended keys (write path + read path)."""
    rng = np.random.default_rng(11)
    dtype, W, Hkv, G, E, bs = torch.bfloat16, 2, 2, 4, 128, 16
    kc, vc, table, g = _caches(rng, W, Hkv, bs, E, E, 80, dtype)
    seq = torch.tensor([30, 47], dtype=torch.int32)
    ks = torch.randn(W, Hkv, 1, E, generator=g).to(dtype)
    vs = torch.randn(W, Hkv, 1, E, generator=g).to(dtype)
    rq = torch.randn(1, W, Hkv * G, 1, E, generator=g).to(dtype)
    dk, dv = kc.to(DEV), vc.to(DEV)
    A.copy_to_blocks(ks.to(DEV), vs.to(DEV), dk, dv, table.to(DEV), seq.to(DEV))
    lens = torch.tensor([48], dtype=torch.int32)                    # worker 0 sees 31 keys through its location
    loc = torch.tensor([[[30], [47]]], dtype=torch.int32)
    out = A.hogwild_paged_sdpa(rq.to(DEV), loc.to(DEV), dk, dv, table.to(DEV), E ** -0.5, lens.to(DEV))
    torch.cuda.synchronize()
    ck, cv = oracle.copy_to_blocks(ks, vs, kc.clone(), vc.clone(), table, seq)
    ref = oracle.paged_sdpa(rq, loc, lens, ck, cv, table, E ** -0.5)
    check_against(out, ref.numpy(), dtype)


# ---- the tensor-core paged kernel by name, against the CUDA-core one and the oracle ---------------------------------
MMA_CASES = [
    # dtype, W, S, Hkv, G, E, bs, F, max_len
    (torch.bfloat16, 3, 1, 2, 16, 128, 16, 2, 1500),      # decode, 16 heads per kv head: one m-tile of heads
    (torch.bfloat16, 2, 3, 2, 4, 128, 24, 3, 700),        # block size that is no multiple of the copy group; 3 tokens x 4 heads
    (torch.float16, 2, 2, 1, 40, 64, 8, 2, 333),          # head size 64, 40 heads per kv head (three head blocks)
    (torch.bfloat16, 5, 1, 1, 8, 128, 256, 1, 2100),      # large blocks
]


def _run_paged(kernel, rq, loc, lens, kc, vc, table, scale, cu=None):
    from inference_lib_b200 import _cabi
    d = lambda t: t.to(DEV).contiguous()
    if cu is None:
        out = torch.full((rq.shape[1], rq.shape[2], rq.shape[3], vc.shape[3]), float("nan"), dtype=rq.dtype, device=DEV)
    else:
        out = torch.full((rq.shape[1], rq.shape[2], vc.shape[3]), float("nan"), dtype=rq.dtype, device=DEV)
    keep = [d(rq), d(loc), d(lens), d(kc), d(vc), d(table)] + ([d(cu)] if cu is not None else [])
    rc, ws = _cabi.paged_sdpa(out=out, queries=keep[0], locations=keep[1], fragment_lengths=keep[2], key_cache=keep[3],
                              value_cache=keep[4], block_table=keep[5], scale=scale,
                              cu_seqlens_q=keep[6] if cu is not None else None, kernel=kernel,
                              stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, out


@pytest.mark.parametrize("case", MMA_CASES, ids=[str(i) for i in range(len(MMA_CASES))])
def test_tensor_core_paged_kernel_matches_oracle_and_cuda_core_kernel(case):
    from inference_lib_b200 import _cabi
    dtype, W, S, Hkv, G, E, bs, F, max_len = case
    rng = np.random.default_rng(sum(case[1:]))
    Hq = Hkv * G
    lens = torch.tensor([max_len] + [int(rng.integers(1, max_len)) for _ in range(F - 1)], dtype=torch.int32)
    kc, vc, table, g = _caches(rng, W, Hkv, bs, E, E, max_len, dtype)
    rq = torch.randn(F, W, Hq, S, E, generator=g).to(dtype)
    loc = torch.from_numpy(rng.integers(-1, max_len + 20, size=(F, W, S)).astype(np.int32))
    loc[0, :, :] = torch.clamp(loc[0], min=0)
    # whatever lies in a block past a sequence's visible rows must never reach a result
    last = (max_len - 1) // bs
    if (max_len % bs) != 0:
        for w in range(W):
            kc[table[w, last], :, max_len % bs:] = float("nan")
            vc[table[w, last], :, max_len % bs:] = float("inf")
    ref = oracle.paged_sdpa(rq, loc, lens, kc.nan_to_num(0.0, 0.0, 0.0), vc.nan_to_num(0.0, 0.0, 0.0), table, E ** -0.5)
    rc_m, out_m = _run_paged(_cabi.KERNEL_MMA, rq, loc, lens, kc, vc, table, E ** -0.5)
    rc_f, out_f = _run_paged(_cabi.KERNEL_FMA, rq, loc, lens, kc, vc, table, E ** -0.5)
    rc_a, out_a = _run_paged(_cabi.KERNEL_AUTO, rq, loc, lens, kc, vc, table, E ** -0.5)
    assert (rc_m, rc_f, rc_a) == (0, 0, 0)
    check_against(out_m, ref.numpy(), dtype, what=f"tensor-core paged kernel {case}")
    check_against(out_f, ref.numpy(), dtype, what=f"CUDA-core paged kernel {case}")
    assert torch.equal(out_a, out_m), "AUTO takes the tensor-core kernel for 16-bit types with equal head sizes of 64 / 128"


def test_tensor_core_paged_kernel_packed_layout():
    from inference_lib_b200 import _cabi
    dtype, G, E, bs, seqs = torch.bfloat16, 8, 128, 16, [3, 0, 5, 1, 2]
    rng = np.random.default_rng(77)
    W, Hkv, F = len(seqs), 2, 2
    Hq = Hkv * G
    cu = torch.tensor([0] + list(np.cumsum(seqs)), dtype=torch.int32)
    total_q = int(cu[-1])
    lens = torch.from_numpy(rng.integers(1, 900, size=(F, W)).astype(np.int32))
    kc, vc, table, g = _caches(rng, W, Hkv, bs, E, E, int(lens.max()), dtype)
    rq = torch.randn(F, total_q, Hq, E, generator=g).to(dtype)
    loc = torch.from_numpy(rng.integers(-1, 950, size=(F, total_q)).astype(np.int32))
    loc[0] = torch.clamp(loc[0], min=0)
    ref = oracle.varlen_paged_sdpa(rq, loc, lens, kc, vc, table, cu, E ** -0.5)
    for kernel in (_cabi.KERNEL_MMA, _cabi.KERNEL_FMA):
        rc, out = _run_paged(kernel, rq, loc, lens, kc, vc, table, E ** -0.5, cu=cu)
        assert rc == 0
        check_against(out, ref.numpy(), dtype, what=f"packed layout, kernel {kernel}")


def test_tensor_core_paged_kernel_is_refused_where_it_cannot_run():
    from inference_lib_b200 import _cabi
    rng = np.random.default_rng(5)
    for dtype, E, Ev in ((torch.float32, 64, 64), (torch.bfloat16, 128, 64), (torch.float16, 32, 32)):
        kc, vc, table, g = _caches(rng, 2, 2, 16, E, Ev, 40, dtype)
        rq = torch.randn(1, 2, 4, 1, E, generator=g).to(dtype)
        loc = torch.full((1, 2, 1), 30, dtype=torch.int32)
        lens = torch.tensor([35], dtype=torch.int32)
        rc, out = _run_paged(_cabi.KERNEL_MMA, rq, loc, lens, kc, vc, table, 0.1)
        assert rc == -9
        assert torch.isnan(out).all()                    # nothing ran
        rc, out = _run_paged(_cabi.KERNEL_AUTO, rq, loc, lens, kc, vc, table, 0.1)
        assert rc == 0 and torch.isfinite(out).all()
