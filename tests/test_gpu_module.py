"""The attention layer (projections + cache update + fused attention + output projection) over a few decode
steps, against the same computation restated on the CPU with the oracles.

The attention result is compared BEFORE the output projection, at the op's own tolerance (16-bit output against
the fp32 oracle: max-abs <= 2e-2, mean-abs <= 2e-3; fp32: 1e-4), on the q/k/v the layer's own projections gave;
the projected output is compared as well, against the oracle's result sent through the same projection."""
import numpy as np
import pytest
import torch

from oracle import hogwild_cache_oracle as oc
from oracle import hogwild_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype,head_dim,tol,tol_mean", [(torch.bfloat16, 128, 2e-2, 2e-3), (torch.float16, 64, 2e-2, 2e-3),
                                                         (torch.float32, 64, 1e-4, 1e-5)])
def test_attention_layer_matches_the_cpu_restatement(dtype, head_dim, tol, tol_mean):
    from inference_lib_b200.cache import FragmentCache
    from inference_lib_b200.module import HogwildAttention
    torch.manual_seed(3)
    W, S, hidden, Hq, Hkv, layers, steps = 3, 1, 256, 8, 2, 2, 3
    lens = [45, 6, 9, 4]                                  # shared prompt + one fragment per worker
    order = [[0] + [1 + o for o in range(W) if o != w] + [1 + w] for w in range(W)]
    inv_freq = 1.0 / (1e4 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    g = torch.Generator().manual_seed(9)
    mods = [HogwildAttention(hidden, Hq, Hkv, head_dim, l, dtype=dtype, device=DEV) for l in range(layers)]
    cpu = [{n: p.detach().cpu() for n, p in m.named_parameters()} for m in mods]
    cache = FragmentCache(layers=layers, capacities=[n + steps * S + 8 for n in lens], Hkv=Hkv, E=head_dim, dtype=dtype,
                          device=DEV, order=order, inv_freq=inv_freq)
    frag_k = [[torch.randn(Hkv, n, head_dim, generator=g).to(dtype) for n in lens] for _ in range(layers)]
    frag_v = [[torch.randn(Hkv, n, head_dim, generator=g).to(dtype) for n in lens] for _ in range(layers)]
    for f in range(len(lens)):
        cache.load_fragment(f, [frag_k[l][f].to(DEV) for l in range(layers)], [frag_v[l][f].to(DEV) for l in range(layers)])
    own_len = [lens[1 + w] for w in range(W)]
    for step in range(steps):
        pos = np.stack([oc.own_positions(own_len[w], S, S) for w in range(W)])
        kcos, ksin = oc.rotary_tables(pos, inv_freq.numpy(), 1.0, dtype)
        kcos, ksin = kcos.to(dtype), ksin.to(dtype)
        h = torch.randn(W, S, hidden, generator=g).to(dtype)
        x_gpu, x_cpu = h.to(DEV), h
        for l in range(layers):
            y, weights = mods[l](x_gpu, (kcos.to(DEV), ksin.to(DEV)), None, cache, position_ids=torch.from_numpy(pos).to(DEV))
            assert weights is None
            # ---- the same layer on the CPU, from the q/k/v its projections gave ----
            p = cpu[l]
            lin = lambda x, w, b=None: torch.nn.functional.linear(x, w, b)
            q, k, v = (proj(x_gpu).view(W, S, -1, head_dim).transpose(1, 2).cpu()
                       for proj in (mods[l].q_proj, mods[l].k_proj, mods[l].v_proj))
            k_rot = oc.rotate_keys(k, kcos, ksin)
            for w in range(W):
                f = 1 + w
                frag_k[l][f], frag_v[l][f] = oc.append(frag_k[l][f], frag_v[l][f], k_rot[w], v[w])
            now = [t.shape[1] for t in frag_k[l]]
            loc = oc.step_locations(np.array(order, dtype=np.int32), now, S)
            cos, sin = oc.rotary_tables(loc, inv_freq.numpy(), 1.0, dtype)
            att, _ = oracle.fused(q.contiguous(), cos, sin, torch.from_numpy(loc), [t[None] for t in frag_k[l]],
                                  [t[None] for t in frag_v[l]], head_dim ** -0.5)
            torch.cuda.synchronize()
            assert int(cache.status.item()) == 0
            assert cache.frags(l).tolist() == now
            diff = (mods[l]._att.float().cpu() - att).abs()
            assert diff.max().item() <= tol and diff.mean().item() <= tol_mean, (step, l, diff.max().item(), diff.mean().item())
            y_ref = lin(att.to(dtype).transpose(1, 2).reshape(W, S, -1), p["o_proj.weight"])
            assert (y.float().cpu() - y_ref.float()).abs().max().item() <= 3 * tol
            x_gpu, x_cpu = y, y.cpu()                     # next layer continues from the GPU's output on both sides
        own_len = [n + S for n in own_len]
