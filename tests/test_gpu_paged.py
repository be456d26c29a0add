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
