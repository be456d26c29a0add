"""GPU parity of the steps either side of the attention op (step metadata, key rotation + append, merge)
against golden vectors produced by the reference's own Python, through the C ABI and the host class."""
import json
import os

import numpy as np
import pytest
import torch

from inference_lib_b200 import _cabi
from oracle import hogwild_cache_oracle as oc
from oracle import hogwild_oracle as oracle

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
DEV = "cuda:0"


@pytest.fixture(scope="module")
def steps():
    return np.load(os.path.join(HERE, "golden", "cache_steps.npz"))


@pytest.fixture(scope="module")
def scenarios():
    with open(os.path.join(HERE, "golden", "cache_steps.json")) as fh:
        return json.load(fh)["scenarios"]


def _dev(a, dtype):
    return torch.from_numpy(np.asarray(a)).to(device=DEV, dtype=dtype)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _plan(order, frags, inv_freq, S, round_to):
    W, F = order.shape
    R = 2 * len(inv_freq)
    loc = torch.full((F, W, S), -7, dtype=torch.int32, device=DEV)
    cos = torch.full((F, W, S, R), float("nan"), dtype=torch.float32, device=DEV)
    sin = torch.full_like(cos, float("nan"))
    rc = _cabi.step_plan(order=_dev(order, torch.int32), fragment_lengths=_dev(frags, torch.int32),
                         inv_freq=_dev(inv_freq, torch.float32), S=S, locations=loc, cosines=cos, sines=sin,
                         round_tables_to=round_to, stream=_stream())
    torch.cuda.synchronize()
    assert rc == 0
    return loc.cpu().numpy(), cos.cpu().numpy(), sin.cpu().numpy()


def test_step_metadata_matches_the_reference(steps, scenarios):
    """locations exactly; tables: cos/sin of the GPU's libm and of the CPU's may differ in the last fp32 bit, which
    moves a rounding to 16 bits now and then -- at most one 16-bit ulp, on few entries."""
    for name, cfg in scenarios.items():
        dtype = getattr(torch, cfg["dtype"])
        for step in range(cfg["steps"]):
            pre = f"{name}/step{step}"
            loc, cos, sin = _plan(steps[f"{name}/order"], steps[f"{pre}/frags"], steps[f"{name}/inv_freq"], cfg["S"],
                                  _cabi.dtype_code(dtype))
            assert np.array_equal(loc, steps[f"{pre}/loc"]), pre
            for got, want in ((cos, steps[f"{pre}/cos"]), (sin, steps[f"{pre}/sin"])):
                diff = np.abs(got - want)
                ulp = {torch.float32: 2.5e-7, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}[dtype]
                assert diff.max() <= ulp, (pre, diff.max())
                assert (diff > 0).mean() <= 0.02 or dtype == torch.float32, (pre, (diff > 0).mean())
            # unrounded tables against the fp32 restatement
            _, cos32, sin32 = _plan(steps[f"{name}/order"], steps[f"{pre}/frags"], steps[f"{name}/inv_freq"], cfg["S"], _cabi.F32)
            rc32, rs32 = oc.rotary_tables(steps[f"{pre}/loc"], steps[f"{name}/inv_freq"])
            assert np.abs(cos32 - rc32.numpy()).max() <= 2.5e-7 and np.abs(sin32 - rs32.numpy()).max() <= 2.5e-7
            assert np.array_equal(cos32[..., : cos32.shape[-1] // 2], cos32[..., cos32.shape[-1] // 2:])


def test_fragment_missing_from_a_workers_order_is_invisible():
    order = np.array([[0, 2, 1], [0, 2, -1]], dtype=np.int32)      # worker 1 does not have fragment 1
    loc, _, _ = _plan(order, np.array([10, 4, 6], dtype=np.int32), np.array([1.0, 0.5], dtype=np.float32), 2, _cabi.F32)
    assert np.array_equal(loc[:, 0], [[18, 19], [2, 3], [8, 9]])
    assert np.array_equal(loc[:, 1], [[14, 15], [-1, -1], [4, 5]])


def _slabs(steps, name, layer, F, Hkv, E, dtype, extra):
    ks, vs, lens = [], [], []
    for f in range(F):
        k0 = _dev(steps[f"{name}/init/k{f}_l{layer}"], dtype)
        v0 = _dev(steps[f"{name}/init/v{f}_l{layer}"], dtype)
        L = k0.shape[1]
        k = torch.full((Hkv, L + extra, E), 77.0, dtype=dtype, device=DEV)
        v = torch.full((Hkv, L + extra, E), 77.0, dtype=dtype, device=DEV)
        k[:, :L], v[:, :L] = k0, v0
        ks.append(k); vs.append(v); lens.append(L)
    return ks, vs, torch.tensor(lens, dtype=torch.int32, device=DEV)


def test_key_rotation_and_append_match_the_reference_bit_for_bit(steps, scenarios):
    for name, cfg in scenarios.items():
        dtype = getattr(torch, cfg["dtype"])
        W, Hkv, E, S, F = cfg["W"], cfg["Hkv"], cfg["E"], cfg["S"], cfg["W"] + 1
        write_to = [int(x) for x in steps[f"{name}/write_to"]]
        for layer in range(cfg["layers"]):
            ks, vs, lens = _slabs(steps, name, layer, F, Hkv, E, dtype, extra=cfg["steps"] * S + 3)
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            for step in range(cfg["steps"]):
                pre = f"{name}/step{step}/l{layer}"
                # keys arrive as the transposed view of a [W,S,Hkv,E] projection output, as in the model
                k_new = _dev(steps[f"{pre}/k_new"], dtype).transpose(1, 2).contiguous().transpose(1, 2)
                v_new = _dev(steps[f"{pre}/v_new"], dtype).transpose(1, 2).contiguous().transpose(1, 2)
                assert k_new.stride(1) == E or Hkv == 1 or S == 1
                cos, sin = _dev(steps[f"{pre}/key_cos"], dtype), _dev(steps[f"{pre}/key_sin"], dtype)
                key = f"{name}/step{step}/new_rows"
                new_rows = _dev(steps[key], torch.int32) if key in steps.files else None
                out_lens = torch.zeros_like(lens)
                rc = _cabi.append(keys=k_new, values=v_new, cosines=cos, sines=sin, write_to=write_to, key_fragments=ks,
                                  value_fragments=vs, lengths_in=lens, lengths_out=out_lens, new_rows=new_rows,
                                  status=status, stream=_stream())
                torch.cuda.synchronize()
                assert rc == 0 and int(status.item()) == 0
                lens = out_lens
                if layer == 0:
                    assert np.array_equal(lens.cpu().numpy(), steps[f"{name}/step{step}/frags"]), pre
                for f in range(F):
                    want_k, want_v = steps[f"{pre}/k{f}"], steps[f"{pre}/v{f}"]
                    L = want_k.shape[1]
                    assert int(lens[f]) == L
                    assert np.array_equal(ks[f][:, :L].float().cpu().numpy(), want_k), (pre, f)
                    assert np.array_equal(vs[f][:, :L].float().cpu().numpy(), want_v), (pre, f)
                    assert (ks[f][:, L:] == 77).all() and (vs[f][:, L:] == 77).all(), "rows past the end must stay untouched"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("E,R", [(128, 128), (64, 32), (40, 24)])
def test_append_with_fp32_tables_matches_the_restatement(dtype, E, R):
    """fp32 tables: products in fp32, one rounding -- the arithmetic of the query path; vectorised and scalar paths."""
    g = torch.Generator().manual_seed(E * 1000 + R)
    W, Hkv, S, cap = 3, 2, 5, 40
    k_new = torch.randn(W, Hkv, S, E, generator=g).to(dtype)
    v_new = torch.randn(W, Hkv, S, E, generator=g).to(dtype)
    pos = torch.randint(0, 5000, (W, S), generator=g)
    inv = 1.0 / (1e4 ** (torch.arange(0, R, 2, dtype=torch.float32) / R))
    cos, sin = oc.rotary_tables(pos.numpy(), inv.numpy())
    want = oc.rotate_keys(k_new, cos, sin)
    ks = [torch.zeros((Hkv, cap, E), dtype=dtype, device=DEV) for _ in range(W)]
    vs = [torch.zeros((Hkv, cap, E), dtype=dtype, device=DEV) for _ in range(W)]
    lens = torch.tensor([0, 7, 35], dtype=torch.int32, device=DEV)
    out_lens = torch.zeros_like(lens)
    rc = _cabi.append(keys=k_new.to(DEV), values=v_new.to(DEV), cosines=cos.to(DEV), sines=sin.to(DEV), write_to=[0, 1, 2],
                      key_fragments=ks, value_fragments=vs, lengths_in=lens, lengths_out=out_lens, stream=_stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert out_lens.tolist() == [5, 12, 40]
    for w, start in enumerate([0, 7, 35]):
        assert torch.equal(ks[w][:, start:start + S].cpu(), want[w]), (w, dtype)
        assert torch.equal(vs[w][:, start:start + S].cpu(), v_new[w])


def test_append_that_does_not_fit_is_dropped_and_reported():
    dtype, W, Hkv, S, E, cap = torch.bfloat16, 1, 2, 4, 64, 6
    slab_k = torch.full((Hkv * cap * E + 256,), 9.0, dtype=dtype, device=DEV)      # canary after the slab
    slab_v = torch.full_like(slab_k, 9.0)
    ks, vs = [slab_k[:Hkv * cap * E].view(Hkv, cap, E)], [slab_v[:Hkv * cap * E].view(Hkv, cap, E)]
    lens = torch.tensor([4], dtype=torch.int32, device=DEV)
    out_lens = torch.zeros_like(lens)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.ones((W, Hkv, S, E), dtype=dtype, device=DEV)
    cos = torch.ones((W, S, E), dtype=torch.float32, device=DEV)
    sin = torch.zeros_like(cos)
    rc = _cabi.append(keys=x, values=x, cosines=cos, sines=sin, write_to=[0], key_fragments=ks, value_fragments=vs,
                      lengths_in=lens, lengths_out=out_lens, status=status, stream=_stream())
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 256 and out_lens.tolist() == [6]
    assert (ks[0][:, 4:6] == 1).all() and (ks[0][:, :4] == 9).all()
    assert (slab_k[Hkv * cap * E:] == 9).all() and (slab_v[Hkv * cap * E:] == 9).all()


def test_append_refuses_bad_arguments():
    x = torch.ones((1, 1, 1, 64), dtype=torch.bfloat16, device=DEV)
    t = torch.ones((1, 1, 64), dtype=torch.float32, device=DEV)
    slab = [torch.zeros((1, 4, 64), dtype=torch.bfloat16, device=DEV)]
    lens = torch.zeros(1, dtype=torch.int32, device=DEV)
    other = torch.zeros(1, dtype=torch.int32, device=DEV)
    mk = dict(keys=x, values=x, cosines=t, sines=t, write_to=[0], key_fragments=slab, value_fragments=slab)
    assert _cabi.append(**mk, lengths_in=lens, lengths_out=lens) == -2          # lengths must be two buffers
    assert _cabi.append(**{**mk, "write_to": [3]}, lengths_in=lens, lengths_out=other) == -2
    assert _cabi.append(**{**mk, "cosines": t.half(), "sines": t.half()}, lengths_in=lens, lengths_out=other) == -4
    torch.cuda.synchronize()
    assert (slab[0] == 0).all()


def test_fragment_cache_replays_the_reference_steps_and_feeds_the_attention_op(steps, scenarios):
    """The host class end to end: prefill, a few decode steps over all layers (append + metadata + attention),
    then merge_caches; the attention result is checked against the restated reference on the golden fragments."""
    from inference_lib_b200 import attention as ours
    from inference_lib_b200.cache import FragmentCache
    for name, cfg in scenarios.items():
        dtype = getattr(torch, cfg["dtype"])
        if cfg["E"] not in (32, 64, 128):
            continue
        W, Hkv, E, S, F, L = cfg["W"], cfg["Hkv"], cfg["E"], cfg["S"], cfg["W"] + 1, cfg["layers"]
        G = 2
        caps = [steps[f"{name}/init/k{f}_l0"].shape[1] + cfg["steps"] * S + 64 for f in range(F)]
        cache = FragmentCache(layers=L, capacities=caps, Hkv=Hkv, E=E, dtype=dtype, device=DEV, order=steps[f"{name}/order"].tolist(),
                              write_to=steps[f"{name}/write_to"].tolist(), inv_freq=torch.from_numpy(steps[f"{name}/inv_freq"]))
        for f in range(F):
            cache.load_fragment(f, [_dev(steps[f"{name}/init/k{f}_l{l}"], dtype) for l in range(L)],
                                [_dev(steps[f"{name}/init/v{f}_l{l}"], dtype) for l in range(L)])
        g = torch.Generator().manual_seed(5)
        for step in range(cfg["steps"]):
            key = f"{name}/step{step}/new_rows"
            new_rows = _dev(steps[key], torch.int32) if key in steps.files else None
            for layer in range(L):
                pre = f"{name}/step{step}/l{layer}"
                cs = cache.update(_dev(steps[f"{pre}/k_new"], dtype), _dev(steps[f"{pre}/v_new"], dtype), layer,
                                  _dev(steps[f"{pre}/key_cos"], dtype), _dev(steps[f"{pre}/key_sin"], dtype), new_rows)
                q = torch.randn(W, Hkv * G, S, E, generator=g).to(dtype)
                out = torch.empty((W, Hkv * G, S, E), dtype=dtype, device=DEV)
                rq = torch.empty((F, W, Hkv * G, S, E), dtype=dtype, device=DEV)
                ours.hogwild_fused(q.to(DEV), cs.loc, cs.keys, cs.values, E ** -0.5, cs.frags, cs.cos, cs.sin,
                                   rotated_queries=rq, out=out)
                torch.cuda.synchronize()
                assert int(cache.status.item()) == 0
                gk = [torch.from_numpy(steps[f"{pre}/k{f}"]).to(dtype)[None] for f in range(F)]
                gv = [torch.from_numpy(steps[f"{pre}/v{f}"]).to(dtype)[None] for f in range(F)]
                ref, _ = oracle.fused(q, torch.from_numpy(steps[f"{name}/step{step}/cos"]), torch.from_numpy(steps[f"{name}/step{step}/sin"]),
                                      torch.from_numpy(steps[f"{name}/step{step}/loc"]), gk, gv, E ** -0.5)
                refn = ref.numpy()
                got = out.float().cpu().numpy()
                seen = ~np.isnan(refn)
                tol = 1e-4 if dtype == torch.float32 else 2e-2
                assert np.abs(got[seen] - refn[seen]).max() <= tol, (pre, np.abs(got[seen] - refn[seen]).max())
        # merge_caches: worker 1's fragment behind worker 0's
        tf, sf = int(steps[f"{name}/write_to"][0]), int(steps[f"{name}/write_to"][1])
        cache.merge(tf, sf)
        torch.cuda.synchronize()
        assert int(cache.status.item()) == 0
        for layer in range(L):
            want_k, want_v = steps[f"{name}/merge/k_l{layer}"], steps[f"{name}/merge/v_l{layer}"]
            n = want_k.shape[1]
            assert int(cache.frags(layer)[tf]) == n
            got_k = cache.keys[layer][tf][:, :n].float().cpu().numpy()
            assert np.array_equal(cache.values[layer][tf][:, :n].float().cpu().numpy(), want_v)
            diff = np.abs(got_k - want_k)
            # the single table row comes from the GPU's cos/sin: a last-bit difference can move a 16-bit rounding
            assert diff.max() <= (1e-5 if dtype == torch.float32 else 0.07) and (diff > 0).mean() <= 0.05, (name, layer, diff.max())
