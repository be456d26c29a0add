"""Golden vectors for the steps either side of the attention op, from the REFERENCE's own Python.

Run in the build container only (needs the reference checkout):

    python tests/golden/make_cache_golden.py [--reference /path/to/reference]

It drives ``HogwildCache.update`` / ``get_input_kwargs``, ``apply_rotary_pos_emb`` and ``merge_caches``
(``python/hogwild/attention.py:112-257, :77-90``) exactly as ``AttentionModule.forward`` does (``:309-318``)
and records what they produce: per-step ``locations``, ``cos``, ``sin``, fragment lengths, the rotated keys
and the grown fragments.  Two stand-ins are needed because the reference was written against an older
``transformers`` cache API and a real checkpoint:

* ``ListCache``: the per-fragment cache object the reference expects (``key_cache`` / ``value_cache`` lists
  per layer, ``get_seq_length``, ``update`` that concatenates along the token axis);
* ``TinyModel``: only ``model.rotary_emb(x, position_ids)``, the standard rotary embedding: fp32
  ``position * inv_freq``, both halves equal, cos/sin returned in ``x``'s dtype.

No reference file is edited or copied.  Output: ``tests/golden/cache_steps.npz`` (+ ``.json`` index).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from tests.golden.make_golden import load_reference  # noqa: E402


class ListCache:
    def __init__(self, layers: int):
        self.key_cache = [None] * layers
        self.value_cache = [None] * layers

    def get_seq_length(self, layer_idx: int = 0) -> int:
        k = self.key_cache[layer_idx]
        return 0 if k is None else k.shape[-2]

    def update(self, k, v, layer_idx, cache_kwargs=None):
        if self.key_cache[layer_idx] is None:
            self.key_cache[layer_idx], self.value_cache[layer_idx] = k, v
        else:
            self.key_cache[layer_idx] = torch.cat([self.key_cache[layer_idx], k], dim=-2)
            self.value_cache[layer_idx] = torch.cat([self.value_cache[layer_idx], v], dim=-2)
        return self.key_cache[layer_idx], self.value_cache[layer_idx]


class Rotary(torch.nn.Module):
    def __init__(self, dim: int, theta: float, attention_scaling: float = 1.0):
        super().__init__()
        self.inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        self.attention_scaling = attention_scaling

    @torch.no_grad()
    def forward(self, x, position_ids):
        inv = self.inv_freq[None, :, None].float().expand(position_ids.shape[0], -1, 1)
        pos = position_ids[:, None, :].float()
        freqs = (inv @ pos).transpose(1, 2)
        emb = torch.cat((freqs, freqs), dim=-1)
        return (emb.cos() * self.attention_scaling).to(x.dtype), (emb.sin() * self.attention_scaling).to(x.dtype)


class TinyModel:
    def __init__(self, rotary):
        self.model = self
        self.rotary_emb = rotary


SCENARIOS = {
    # W workers, shared prompt of `prompt` tokens, worker caches of `own` tokens, S new tokens per step
    "bf16_s1": dict(W=3, Hkv=2, E=64, R=64, layers=2, prompt=37, own=[5, 9, 2], S=1, steps=3, theta=1e4, dtype="bfloat16"),
    "bf16_s4_masked": dict(W=2, Hkv=2, E=64, R=64, layers=1, prompt=50, own=[8, 3], S=4, steps=2, theta=5e5, dtype="bfloat16",
                           new_tokens=[[4, 2], [1, 4]]),
    "f16_partial_rotary": dict(W=2, Hkv=1, E=64, R=32, layers=1, prompt=20, own=[4, 4], S=2, steps=2, theta=1e4, dtype="float16"),
    "bf16_e128_w4": dict(W=4, Hkv=2, E=128, R=128, layers=1, prompt=100, own=[40, 17, 33, 8], S=1, steps=2, theta=5e5, dtype="bfloat16"),
    "f32_s2": dict(W=2, Hkv=2, E=32, R=32, layers=1, prompt=11, own=[3, 6], S=2, steps=2, theta=1e4, dtype="float32"),
}


def run_scenario(ref, name: str, cfg: dict, out: dict):
    g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
    dtype = getattr(torch, cfg["dtype"])
    W, Hkv, E, R, L, S = cfg["W"], cfg["Hkv"], cfg["E"], cfg["R"], cfg["layers"], cfg["S"]
    rotary = Rotary(R, cfg["theta"])
    model = TinyModel(rotary)

    def rnd(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)

    prompt = ListCache(L)
    workers = [ListCache(L) for _ in range(W)]
    for layer in range(L):
        prompt.update(rnd(1, Hkv, cfg["prompt"], E), rnd(1, Hkv, cfg["prompt"], E), layer)
        for w in range(W):
            workers[w].update(rnd(1, Hkv, cfg["own"][w], E), rnd(1, Hkv, cfg["own"][w], E), layer)
    # worker w: prompt, the other workers in index order, its own cache last
    structure = [[prompt] + [workers[o] for o in range(W) if o != w] + [workers[w]] for w in range(W)]
    cache = ref.HogwildCache(structure, model)
    segments0 = structure[0]
    out[f"{name}/order"] = np.array([[segments0.index(cs) for cs in structure[w]] for w in range(W)], dtype=np.int32)
    out[f"{name}/write_to"] = np.array([segments0.index(workers[w]) for w in range(W)], dtype=np.int32)
    out[f"{name}/inv_freq"] = rotary.inv_freq.numpy()
    for f, cs in enumerate(segments0):
        for layer in range(L):
            out[f"{name}/init/k{f}_l{layer}"] = cs.key_cache[layer][0].float().numpy()
            out[f"{name}/init/v{f}_l{layer}"] = cs.value_cache[layer][0].float().numpy()

    for step in range(cfg["steps"]):
        mask = None
        if "new_tokens" in cfg:
            n = cfg["new_tokens"][step]
            mask = torch.zeros(W, S, dtype=torch.int64)
            for w in range(W):
                mask[w, S - n[w]:] = 1
            out[f"{name}/step{step}/new_rows"] = np.array(n, dtype=np.int32)
        kw = cache.get_input_kwargs(torch.zeros(W, S, dtype=torch.int64), mask)
        pos_ids = kw["position_ids"]
        out[f"{name}/step{step}/position_ids"] = pos_ids.numpy().astype(np.int32)
        for layer in range(L):
            k_new, v_new = rnd(W, Hkv, S, E), rnd(W, Hkv, S, E)
            cos, sin = rotary(k_new, pos_ids)                       # what the model passes as position_embeddings
            k_rot = ref.apply_rotary_pos_emb(k_new, cos, sin)       # AttentionModule.forward, attention.py:315
            cs = cache.update(k_rot, v_new, layer, {"sin": sin, "cos": cos, "cache_position": None, "mask": mask})
            pre = f"{name}/step{step}/l{layer}"
            out[f"{pre}/k_new"] = k_new.float().numpy()
            out[f"{pre}/v_new"] = v_new.float().numpy()
            out[f"{pre}/key_cos"] = cos.float().numpy()
            out[f"{pre}/key_sin"] = sin.float().numpy()
            out[f"{pre}/k_rot"] = k_rot.float().numpy()
            for f in range(len(cs.keys)):
                out[f"{pre}/k{f}"] = cs.keys[f][0].float().numpy()
                out[f"{pre}/v{f}"] = cs.values[f][0].float().numpy()
            if layer == 0:
                out[f"{name}/step{step}/loc"] = cs.loc.numpy().astype(np.int32)
                out[f"{name}/step{step}/cos"] = cs.cos.numpy()
                out[f"{name}/step{step}/sin"] = cs.sin.numpy()
                out[f"{name}/step{step}/frags"] = cs.frags.numpy().astype(np.int32)

    # merge_caches: worker 1's cache re-rotated behind worker 0's (attention.py:251-257)
    target, source = workers[0], workers[1]
    out[f"{name}/merge/target_len"] = np.array([target.get_seq_length()], dtype=np.int32)
    ref.merge_caches(target, source, model)
    for layer in range(L):
        out[f"{name}/merge/k_l{layer}"] = target.key_cache[layer][0].float().numpy()
        out[f"{name}/merge/v_l{layer}"] = target.value_cache[layer][0].float().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    ref = load_reference(args.reference)
    torch._dynamo.graph_break = lambda: None        # the reference calls it for torch.compile's benefit; eager here
    out: dict = {}
    for name, cfg in SCENARIOS.items():
        run_scenario(ref, name, cfg, out)
    path = os.path.join(HERE, "cache_steps.npz")
    np.savez_compressed(path, **out)
    with open(os.path.join(HERE, "cache_steps.json"), "w") as fh:
        json.dump({"scenarios": SCENARIOS, "torch": torch.__version__, "arrays": len(out)}, fh, indent=1)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
