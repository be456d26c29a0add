"""The CPU restatement of the cache steps against golden vectors produced by the reference's own Python."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import hogwild_cache_oracle as oc

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def steps():
    return np.load(os.path.join(HERE, "golden", "cache_steps.npz"))


@pytest.fixture(scope="module")
def scenarios():
    with open(os.path.join(HERE, "golden", "cache_steps.json")) as fh:
        return json.load(fh)["scenarios"]


def _t(a, dtype):
    return torch.from_numpy(np.asarray(a)).to(dtype)


def test_locations_and_tables_match_the_reference(steps, scenarios):
    for name, cfg in scenarios.items():
        dtype = getattr(torch, cfg["dtype"])
        for step in range(cfg["steps"]):
            pre = f"{name}/step{step}"
            loc = oc.step_locations(steps[f"{name}/order"], steps[f"{pre}/frags"], cfg["S"])
            assert np.array_equal(loc, steps[f"{pre}/loc"]), pre
            cos, sin = oc.rotary_tables(loc, steps[f"{name}/inv_freq"], 1.0, dtype)
            assert np.array_equal(cos.numpy(), steps[f"{pre}/cos"]) and np.array_equal(sin.numpy(), steps[f"{pre}/sin"]), pre


def test_own_positions_match_the_reference(steps, scenarios):
    for name, cfg in scenarios.items():
        own = list(cfg["own"])
        for step in range(cfg["steps"]):
            n = steps[f"{name}/step{step}/new_rows"] if f"{name}/step{step}/new_rows" in steps.files else [cfg["S"]] * cfg["W"]
            got = np.stack([oc.own_positions(own[w], int(n[w]), cfg["S"]) for w in range(cfg["W"])])
            assert np.array_equal(got, steps[f"{name}/step{step}/position_ids"]), (name, step)
            own = [own[w] + int(n[w]) for w in range(cfg["W"])]


def test_key_rotation_and_append_match_the_reference(steps, scenarios):
    for name, cfg in scenarios.items():
        dtype = getattr(torch, cfg["dtype"])
        F = cfg["W"] + 1
        write_to = steps[f"{name}/write_to"]
        for layer in range(cfg["layers"]):
            frag_k = [_t(steps[f"{name}/init/k{f}_l{layer}"], dtype) for f in range(F)]
            frag_v = [_t(steps[f"{name}/init/v{f}_l{layer}"], dtype) for f in range(F)]
            for step in range(cfg["steps"]):
                pre = f"{name}/step{step}/l{layer}"
                k_new, v_new = _t(steps[f"{pre}/k_new"], dtype), _t(steps[f"{pre}/v_new"], dtype)
                cos, sin = _t(steps[f"{pre}/key_cos"], dtype), _t(steps[f"{pre}/key_sin"], dtype)
                k_rot = oc.rotate_keys(k_new, cos, sin)
                assert torch.equal(k_rot.float(), _t(steps[f"{pre}/k_rot"], torch.float32)), pre
                key = f"{name}/step{step}/new_rows"
                for w in range(cfg["W"]):
                    f = int(write_to[w])
                    n = int(steps[key][w]) if key in steps.files else None
                    frag_k[f], frag_v[f] = oc.append(frag_k[f], frag_v[f], k_rot[w], v_new[w], n)
                for f in range(F):
                    assert torch.equal(frag_k[f].float(), _t(steps[f"{pre}/k{f}"], torch.float32)), (pre, f)
                    assert torch.equal(frag_v[f].float(), _t(steps[f"{pre}/v{f}"], torch.float32)), (pre, f)


def test_merge_matches_the_reference(steps, scenarios):
    for name, cfg in scenarios.items():
        dtype = getattr(torch, cfg["dtype"])
        last = cfg["steps"] - 1
        write_to = steps[f"{name}/write_to"]
        tf, sf = int(write_to[0]), int(write_to[1])
        L = cfg["layers"]
        tk = [_t(steps[f"{name}/step{last}/l{l}/k{tf}"], dtype) for l in range(L)]
        tv = [_t(steps[f"{name}/step{last}/l{l}/v{tf}"], dtype) for l in range(L)]
        sk = [_t(steps[f"{name}/step{last}/l{l}/k{sf}"], dtype) for l in range(L)]
        sv = [_t(steps[f"{name}/step{last}/l{l}/v{sf}"], dtype) for l in range(L)]
        assert tk[0].shape[-2] == int(steps[f"{name}/merge/target_len"][0])
        mk, mv = oc.merge(tk, tv, sk, sv, steps[f"{name}/inv_freq"])
        for l in range(L):
            assert torch.equal(mk[l].float(), _t(steps[f"{name}/merge/k_l{l}"], torch.float32)), (name, l)
            assert torch.equal(mv[l].float(), _t(steps[f"{name}/merge/v_l{l}"], torch.float32)), (name, l)
