"""``model_surgery`` on a small randomly initialised decoder (no GPU): which modules are swapped, that the
projections are adopted and not copied, and what the decoder hands to the swapped-in layer -- the contract
``HogwildAttention.forward`` is written against (reference: ``python/hogwild/attention.py:291-354``)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def tiny_model(layers=2, hidden=256, heads=4, kv_heads=2):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    torch.manual_seed(0)
    cfg = Qwen2Config(vocab_size=384, hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=layers,
                      num_attention_heads=heads, num_key_value_heads=kv_heads, max_position_embeddings=4096)
    return Qwen2ForCausalLM(cfg).eval()


def test_surgery_swaps_every_layer_and_adopts_the_projections():
    from inference_lib_b200.module import HogwildAttention, model_surgery
    model = tiny_model()
    before = [(l.self_attn.q_proj, l.self_attn.k_proj, l.self_attn.v_proj, l.self_attn.o_proj) for l in model.model.layers]
    n_params = sum(p.numel() for p in model.parameters())
    model_surgery(model)
    for i, layer in enumerate(model.model.layers):
        att = layer.self_attn
        assert isinstance(att, HogwildAttention) and att.layer_idx == i
        assert (att.q_proj, att.k_proj, att.v_proj, att.o_proj) == before[i]        # the same objects
        assert (att.num_heads, att.num_kv_heads, att.head_dim) == (4, 2, 64)
        assert att.scaling == 64 ** -0.5
    assert sum(p.numel() for p in model.parameters()) == n_params


def test_the_decoder_hands_the_layer_what_forward_expects(monkeypatch):
    """The decoder must pass the 2-D padding mask through untouched, the model's own rotary tables at
    ``position_ids``, and the cache object as ``past_key_values``."""
    from inference_lib_b200 import module as mod
    model = tiny_model()
    mod.model_surgery(model)
    seen = []

    def record(self, hidden_states, position_embeddings, attention_mask=None, past_key_values=None, position_ids=None,
               **kwargs):
        seen.append(dict(layer=self.layer_idx, hidden=hidden_states.shape, cos=position_embeddings[0],
                         mask=attention_mask, cache=past_key_values, pos=position_ids))
        return torch.zeros_like(hidden_states), None

    monkeypatch.setattr(mod.HogwildAttention, "forward", record)
    W, S = 3, 2
    ids = torch.randint(0, 384, (W, S))
    pos = torch.tensor([[7, 8], [0, 1], [40, 41]])
    mask = torch.tensor([[1, 1], [0, 1], [1, 1]])
    cache = object()
    logits = mod.decode_step(model, ids, pos, cache, attention_mask=mask)
    assert logits.shape == (W, S, 384)
    assert [s["layer"] for s in seen] == [0, 1]
    inv_freq = model.model.rotary_emb.inv_freq
    want = torch.cat([pos[..., None].float() * inv_freq] * 2, dim=-1).cos()
    for s in seen:
        assert s["cache"] is cache and s["mask"] is mask and torch.equal(s["pos"], pos)
        assert s["hidden"] == (W, S, 256)
        assert torch.allclose(s["cos"].float(), want, atol=1e-6)
    seen.clear()
    mod.decode_step(model, ids, pos, cache)
    assert all(s["mask"] is None for s in seen)


def test_forward_refuses_what_the_reference_asserts():
    from inference_lib_b200.module import HogwildAttention
    lin = lambda i, o, b: torch.nn.Linear(i, o, bias=b)
    att = HogwildAttention.from_projections(lin(32, 64, True), lin(32, 32, True), lin(32, 32, True), lin(64, 32, False),
                                            num_heads=4, num_kv_heads=2, layer_idx=0)
    h = torch.zeros(2, 1, 32)
    with pytest.raises(TypeError):
        att(h, (None, None), None, past_key_values=None)
