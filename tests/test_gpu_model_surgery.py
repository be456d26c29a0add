"""``model_surgery`` on a small randomly initialised decoder, decoding a few steps on the GPU with several workers
that share fragments (reference: ``python/hogwild/attention.py:263-354``; its eager branch is the statement the
CPU side follows).

Per layer and step, the attention result BEFORE the output projection is compared at the op's tolerance (16-bit
output against the fp32 oracle: max-abs <= 2e-2, mean-abs <= 2e-3) on identical q/k/v, taken from the layer's own
projections.  The logits of the whole stack are compared against a CPU model that runs the same weights with the
oracle as its attention and never sees a GPU intermediate."""
import copy

import numpy as np
import pytest
import torch

from oracle import hogwild_cache_oracle as oc
from oracle import hogwild_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
transformers = pytest.importorskip("transformers")


class OracleCache:
    """Per layer a list of ``[Hkv,L,E]`` fragments grown by concatenation, and the step's query tables."""

    def __init__(self, layers, order, inv_freq, dtype):
        self.k = [[] for _ in range(layers)]
        self.v = [[] for _ in range(layers)]
        self.order, self.inv_freq, self.dtype = np.array(order, dtype=np.int32), inv_freq, dtype
        self.write_to = [o[-1] for o in order]
        self.loc = self.cos = self.sin = None


class OracleAttention(torch.nn.Module):
    """The reference's eager branch on the CPU: rotate the keys at their own positions, append, rotate the queries
    per fragment, attend over every fragment with the location mask (``attention.py:307-323``)."""

    def __init__(self, old, cfg):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = old.q_proj, old.k_proj, old.v_proj, old.o_proj
        self.layer_idx, self.Hq, self.Hkv = old.layer_idx, cfg.num_attention_heads, cfg.num_key_value_heads
        self.D = self.q_proj.out_features // self.Hq
        self.last_att = None
        self.given_qkv = None          # (q, k, v) to use instead of the projections

    def forward(self, hidden_states, position_embeddings, attention_mask=None, past_key_values=None, **kw):
        c, l = past_key_values, self.layer_idx
        W, S, _ = hidden_states.shape
        shape = (W, S, -1, self.D)
        if self.given_qkv is None:
            q = self.q_proj(hidden_states).view(shape).transpose(1, 2)
            k = self.k_proj(hidden_states).view(shape).transpose(1, 2)
            v = self.v_proj(hidden_states).view(shape).transpose(1, 2)
        else:
            q, k, v = self.given_qkv
        cos, sin = position_embeddings
        k_rot = oc.rotate_keys(k, cos, sin)
        rows = [None] * W if attention_mask is None else attention_mask.sum(dim=1).tolist()
        for w in range(W):
            f = c.write_to[w]
            c.k[l][f], c.v[l][f] = oc.append(c.k[l][f], c.v[l][f], k_rot[w], v[w], rows[w])
        if l == 0:
            c.loc = oc.step_locations(c.order, [t.shape[1] for t in c.k[0]], S)
            c.cos, c.sin = oc.rotary_tables(c.loc, c.inv_freq, 1.0, c.dtype)
        att, _ = oracle.fused(q.contiguous(), c.cos, c.sin, torch.from_numpy(c.loc), [t[None] for t in c.k[l]],
                              [t[None] for t in c.v[l]], self.D ** -0.5)
        self.last_att = att                                                   # fp32 [W,Hq,S,D]
        return self.o_proj(att.to(hidden_states.dtype).transpose(1, 2).reshape(W, S, -1)), None


def build(dtype, head_dim, layers=3, heads=4, kv_heads=2):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    torch.manual_seed(11)
    cfg = Qwen2Config(vocab_size=640, hidden_size=heads * head_dim, intermediate_size=2 * heads * head_dim,
                      num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
                      max_position_embeddings=8192)
    model = Qwen2ForCausalLM(cfg).eval().to(dtype)
    with torch.no_grad():
        for p in model.parameters():                 # livelier than the default init: attention that is not flat
            if p.dim() == 2:
                p.mul_(3.0)
    return model


@pytest.mark.parametrize("dtype,head_dim", [(torch.bfloat16, 128), (torch.float16, 64)])
@torch.no_grad()
def test_decoding_through_a_model_after_surgery(dtype, head_dim):
    from inference_lib_b200 import module as mod
    model_cpu = build(dtype, head_dim)
    model_gpu = copy.deepcopy(model_cpu).to(DEV)
    mod.model_surgery(model_gpu)
    cfg = model_cpu.model.config
    for layer in model_cpu.model.layers:
        layer.self_attn = OracleAttention(layer.self_attn, cfg)
    shadow = copy.deepcopy(model_cpu)              # a second CPU stack, fed the GPU layers' own q/k/v (see below)

    W, S_first, steps = 3, 4, 3
    L, Hkv = cfg.num_hidden_layers, cfg.num_key_value_heads
    lens = [70, 5, 0, 12]                                     # shared prompt, one fragment per worker (one empty)
    order = [[0] + [1 + o for o in range(W) if o != w] + [1 + w] for w in range(W)]
    inv_freq = model_cpu.model.rotary_emb.inv_freq.float().numpy()
    g = torch.Generator().manual_seed(5)
    cache = mod.cache_for_model(model_gpu, [n + S_first + steps + 8 for n in lens], order)
    cpu_caches = [OracleCache(L, order, inv_freq, dtype) for _ in range(2)]
    for f, n in enumerate(lens):
        ks = [torch.randn(Hkv, n, head_dim, generator=g).to(dtype) for _ in range(L)]
        vs = [torch.randn(Hkv, n, head_dim, generator=g).to(dtype) for _ in range(L)]
        cache.load_fragment(f, [k.to(DEV) for k in ks], [v.to(DEV) for v in vs])
        for c in cpu_caches:
            for l in range(L):
                c.k[l].append(ks[l].clone())
                c.v[l].append(vs[l].clone())

    # what each GPU layer projected: q/k/v for the shadow stack, so that its attention sees identical operands
    taken = {}

    def grab(module, args, kwargs):
        h = kwargs.get("hidden_states", args[0] if args else None)
        W_, S_, _ = h.shape
        shape = (W_, S_, -1, module.head_dim)
        taken[module.layer_idx] = tuple(p(h).view(shape).transpose(1, 2).float().cpu().to(dtype)
                                        for p in (module.q_proj, module.k_proj, module.v_proj))

    for layer in model_gpu.model.layers:
        layer.self_attn.register_forward_pre_hook(grab, with_kwargs=True)

    own = [lens[1 + w] for w in range(W)]
    worst = 0.0
    for step in range(steps + 1):
        S = S_first if step == 0 else 1
        if step == 0:                                         # a left-padded first input: 4, 2 and 3 real tokens
            mask = torch.tensor([[1, 1, 1, 1], [0, 0, 1, 1], [0, 1, 1, 1]])
        else:
            mask = None
        real = [S] * W if mask is None else mask.sum(dim=1).tolist()
        pos = torch.from_numpy(np.stack([oc.own_positions(own[w], real[w], S) for w in range(W)])).long()
        ids = torch.randint(0, cfg.vocab_size, (W, S), generator=g)
        logits_gpu = mod.decode_step(model_gpu, ids.to(DEV), pos.to(DEV), cache, None if mask is None else mask.to(DEV))
        torch.cuda.synchronize()
        assert int(cache.status.item()) == 0
        logits_cpu = mod.decode_step(model_cpu, ids, pos, cpu_caches[0], mask)

        # (1) per layer, before the output projection, identical operands
        for l, layer in enumerate(shadow.model.layers):
            layer.self_attn.given_qkv = taken[l]
        mod.decode_step(shadow, ids, pos, cpu_caches[1], mask)
        for l in range(L):
            got = model_gpu.model.layers[l].self_attn._att.float().cpu()
            ref = shadow.model.layers[l].self_attn.last_att
            live = torch.ones(W, 1, S, 1, dtype=torch.bool) if mask is None else mask.bool()[:, None, :, None]
            diff = ((got - ref).abs() * live)                 # padded positions carry no defined result
            assert torch.isfinite(got).all()
            assert diff.max().item() <= 2e-2 and diff.mean().item() <= 2e-3, (step, l, diff.max().item())
            assert cache.frags(l).tolist() == [t.shape[1] for t in cpu_caches[1].k[l]]
        # (2) the whole stack against a CPU stack that never saw a GPU intermediate
        live = torch.ones(W, S, dtype=torch.bool) if mask is None else mask.bool()
        d = (logits_gpu.float().cpu() - logits_cpu.float())[live]
        scale = logits_cpu.float()[live].abs().max().item()
        worst = max(worst, d.abs().max().item() / scale)
        assert d.abs().max().item() <= 0.06 * scale, (step, d.abs().max().item(), scale)
        own = [n + r for n, r in zip(own, real)]
    assert worst > 0.0
