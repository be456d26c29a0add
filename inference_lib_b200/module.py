"""The attention layer around the op: the role of the reference's ``AttentionModule``
(``python/hogwild/attention.py:263-336``) on top of :class:`inference_lib_b200.cache.FragmentCache`.

``forward`` is the reference's sequence -- q/k/v projections, key rotation, cache update, fused attention over
all fragments, output projection -- with the eager pieces replaced: the key rotation and the append are one
kernel launch inside ``FragmentCache.update`` (the reference: ``apply_rotary_pos_emb`` + ``torch.cat`` per
worker), the per-step metadata one more at layer 0, and the attention is ``hogwild_fused``.  The projections
stay ``torch.nn.Linear`` (cuBLAS): they are plain GEMMs and not part of the path this package rebuilds.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
from torch import nn

from . import attention as ops
from .cache import FragmentCache


class HogwildAttention(nn.Module):
    """One decoder layer's attention for ``W`` workers that share ``cache``'s fragments.

    Same parameters as the reference's module (``q_proj`` / ``k_proj`` / ``v_proj`` with bias, ``o_proj``
    without, ``attention.py:278-289``); ``from_projections`` adopts the ``nn.Linear`` objects of an existing
    layer the way ``model_surgery`` does (``attention.py:339-347``).
    """

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, layer_idx: int,
                 dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.layer_idx, self.head_dim = layer_idx, head_dim
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.scaling = head_dim ** -0.5
        kw = dict(dtype=dtype, device=device)
        self.q_proj = nn.Linear(hidden_size, num_heads * head_dim, bias=True, **kw)
        self.k_proj = nn.Linear(hidden_size, num_kv_heads * head_dim, bias=True, **kw)
        self.v_proj = nn.Linear(hidden_size, num_kv_heads * head_dim, bias=True, **kw)
        self.o_proj = nn.Linear(num_heads * head_dim, hidden_size, bias=False, **kw)
        self._rq = self._att = None

    @classmethod
    def from_projections(cls, q_proj: nn.Linear, k_proj: nn.Linear, v_proj: nn.Linear, o_proj: nn.Linear, *,
                         num_heads: int, num_kv_heads: int, layer_idx: int) -> "HogwildAttention":
        head_dim = q_proj.out_features // num_heads
        m = cls.__new__(cls)
        nn.Module.__init__(m)
        m.layer_idx, m.head_dim, m.num_heads, m.num_kv_heads = layer_idx, head_dim, num_heads, num_kv_heads
        m.scaling = head_dim ** -0.5
        m.q_proj, m.k_proj, m.v_proj, m.o_proj = q_proj, k_proj, v_proj, o_proj
        m._rq = m._att = None
        return m

    def forward(self, hidden_states: torch.Tensor, position_embeddings: Tuple[torch.Tensor, torch.Tensor],
                attention_mask: Optional[torch.Tensor] = None, past_key_values: Optional[FragmentCache] = None,
                position_ids: Optional[torch.Tensor] = None, **kwargs) -> Tuple[torch.Tensor, None]:
        """The call a decoder layer makes (``attention.py:291-336``; the keyword names are those of the
        transformers release installed here, where the reference's ``past_key_value`` is ``past_key_values``).

        ``hidden_states [W,S,hidden]``; ``position_embeddings`` = (cos, sin) ``[W,S,R]`` at the tokens' own
        positions, as the model's ``rotary_emb`` computes them; ``attention_mask`` ``None`` or the ``[W,S]`` 0/1
        left-padding mask, passed through by the model untouched: only the last ``sum(mask[w])`` tokens of worker
        ``w`` enter the cache (``attention.py:148-154``).  Returns ``(attn_output, None)`` like the reference."""
        cache = past_key_values if past_key_values is not None else kwargs.get("past_key_value")
        if not isinstance(cache, FragmentCache):
            raise TypeError("HogwildAttention needs a FragmentCache as past_key_values")
        W, S, _ = hidden_states.shape
        if W != 1 and position_ids is None and "new_rows" not in kwargs:
            # the reference's assertion (attention.py:304-305): several workers never share default positions
            raise ValueError("when processing multiple workers, position_ids are mandatory")
        if position_ids is not None and tuple(position_ids.shape) != (W, S):
            raise ValueError(f"position_ids {tuple(position_ids.shape)} must match hidden_states {(W, S)}")
        new_rows = kwargs.get("new_rows")
        if attention_mask is not None:
            if attention_mask.dim() != 2 or tuple(attention_mask.shape) != (W, S):
                raise ValueError("attention_mask must be the [W,S] padding mask (left-padded), not an expanded one")
            new_rows = attention_mask.sum(dim=1).to(torch.int32)
        shape = (W, S, -1, self.head_dim)
        q = self.q_proj(hidden_states).view(shape).transpose(1, 2)          # [W,Hq,S,D] views, no copies
        k = self.k_proj(hidden_states).view(shape).transpose(1, 2)
        v = self.v_proj(hidden_states).view(shape).transpose(1, 2)
        cos, sin = position_embeddings
        cs = cache.update(k, v, self.layer_idx, cos, sin, new_rows)         # rotates the keys itself
        att = self._attend(q, cs)                                           # [W, all query heads, S, Ev]
        return self.o_proj(att.transpose(1, 2).reshape(W, S, -1)), None

    def _attend(self, q: torch.Tensor, cs) -> torch.Tensor:
        F = len(cs.keys)
        W, Hq, S, D = q.shape
        if self._rq is None or self._rq.shape != (F, W, Hq, S, D) or self._rq.dtype != q.dtype:
            self._rq = torch.empty((F, W, Hq, S, D), dtype=q.dtype, device=q.device)
            self._att = torch.empty((W, Hq, S, cs.values[0].shape[-1]), dtype=q.dtype, device=q.device)
        return ops.hogwild_fused_planned(q, cs.loc, cs.keys, cs.values, self.scaling, cs.frags, cs.cos, cs.sin,
                                         rotated_queries=self._rq, out=self._att, host_lengths=cs.host_lengths,
                                         stable_fragments=cs.stable)


class TensorParallel:
    """What the sharded layers of one rank share: rank, world size, and how the heads are gathered.

    ``peer_outputs`` (a :class:`inference_lib_b200.sharded.PeerOutputs` with at least two slots) selects the gather
    that is fused into the op: every rank's merge step stores its heads into all ranks' full-size outputs over
    NVLink, consecutive calls alternate between the slots.  Without it the heads are gathered by
    ``torch.distributed.all_gather_into_tensor`` on ``group`` (NCCL on GPUs; gloo in CPU tests)."""

    def __init__(self, rank: int, world: int, group=None, peer_outputs=None):
        if peer_outputs is not None and peer_outputs.slots < 2:
            raise ValueError("the fused gather needs two output slots: a rank may run one call ahead of its peers")
        self.rank, self.world, self.group, self.peer_outputs = rank, world, group, peer_outputs
        self.calls = 0

    def next_slot(self) -> int:
        slot = self.calls % self.peer_outputs.slots
        self.calls += 1
        return slot


class HogwildAttentionTP(HogwildAttention):
    """:class:`HogwildAttention` with its heads sharded over the GPUs of one node: rank ``r`` keeps the projection
    rows of query heads ``[r*Hq/G, (r+1)*Hq/G)`` and of kv heads ``[r*Hkv/G, (r+1)*Hkv/G)``, its cache holds those
    kv heads only, the attention results of all ranks are gathered along the head axis and feed a replicated
    ``o_proj``.  No counterpart in the reference (single device, ``src/kernels/kernel_v21.cuh:960``)."""

    @classmethod
    def from_full(cls, full: HogwildAttention, tp: TensorParallel) -> "HogwildAttentionTP":
        from . import sharded
        qs, ks = sharded.head_slices(full.num_heads, full.num_kv_heads, tp.rank, tp.world)
        D = full.head_dim

        def rows(lin: nn.Linear, heads: slice) -> nn.Linear:
            out = nn.Linear(lin.in_features, (heads.stop - heads.start) * D, bias=lin.bias is not None,
                            dtype=lin.weight.dtype, device=lin.weight.device)
            with torch.no_grad():
                out.weight.copy_(lin.weight[heads.start * D:heads.stop * D])
                if lin.bias is not None:
                    out.bias.copy_(lin.bias[heads.start * D:heads.stop * D])
            return out

        m = cls.from_projections(rows(full.q_proj, qs), rows(full.k_proj, ks), rows(full.v_proj, ks), full.o_proj,
                                 num_heads=qs.stop - qs.start, num_kv_heads=ks.stop - ks.start, layer_idx=full.layer_idx)
        m.head_dim, m.scaling = D, full.scaling          # (from_projections derived the same; kept explicit)
        m.tp, m.total_heads = tp, full.num_heads
        m._ws = m._bound = None
        return m

    def _attend_local(self, q: torch.Tensor, cs) -> torch.Tensor:
        return HogwildAttention._attend(self, q, cs)

    def _attend(self, q: torch.Tensor, cs) -> torch.Tensor:
        tp = self.tp
        if tp.peer_outputs is None:
            from . import sharded
            return sharded.gather_heads(self._attend_local(q, cs), tp.world, group=tp.group)
        # the gather fused into the op: the C ABI call with this rank's shard as the problem
        from . import _cabi
        F = len(cs.keys)
        W, Hq, S, D = q.shape
        if self._rq is None or self._rq.shape != (F, W, Hq, S, D) or self._rq.dtype != q.dtype:
            self._rq = torch.empty((F, W, Hq, S, D), dtype=q.dtype, device=q.device)
            self._att = torch.empty((W, Hq, S, cs.values[0].shape[-1]), dtype=q.dtype, device=q.device)
        slot = tp.next_slot()
        stream = torch.cuda.current_stream(q.device).cuda_stream
        bp = _cabi.bind(out=self._att, queries=q.contiguous(), locations=cs.loc, keys=cs.keys, values=cs.values,
                        scale=self.scaling, fragment_lengths=cs.frags, cos=cs.cos, sin=cs.sin, rq=self._rq,
                        host_lengths=cs.host_lengths, stable_fragments=cs.stable)
        need = _cabi.workspace_bytes(bp)
        if need == 0:
            raise RuntimeError("libhogatt_b200 refused the sharded problem")
        if self._ws is None or self._ws.numel() < need + 256:
            self._ws = torch.empty(need + 256, dtype=torch.uint8, device=q.device)
        ptr = self._ws.data_ptr() + (-self._ws.data_ptr()) % 256
        bp.struct.workspace, bp.struct.workspace_bytes = ptr, need
        rc = _cabi.launch_gather(bp, tp.peer_outputs.peers(slot), stream)
        if rc != 0:
            raise RuntimeError(f"hogatt_fused_launch_gather: {_cabi.status_string(rc)}")
        self._bound = bp                                   # keeps the argument arrays alive until the next call
        return tp.peer_outputs.output(slot)


def model_surgery(model, tp: Optional[TensorParallel] = None) -> None:
    """Swap every decoder layer's attention for :class:`HogwildAttention`, adopting its projections: the
    reference's ``model_surgery`` (``attention.py:339-354``).

    The reference also replaces the model's ``_update_causal_mask`` so that the 2-D padding mask reaches the
    layers as it is.  The transformers release installed here has no such hook: its decoder skips mask
    construction when ``attention_mask`` already is a dict of per-layer-type masks, which is what
    :func:`decode_step` passes.  With ``tp`` every layer becomes a :class:`HogwildAttentionTP`."""
    cfg = model.model.config
    for layer in model.model.layers:
        old = layer.self_attn
        layer.self_attn = HogwildAttention.from_projections(
            old.q_proj, old.k_proj, old.v_proj, old.o_proj, num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads, layer_idx=old.layer_idx)
        if tp is not None and tp.world > 1:        # heads sharded over the ranks, o_proj replicated
            layer.self_attn = HogwildAttentionTP.from_full(layer.self_attn, tp)


def decode_step(model, input_ids: torch.Tensor, position_ids: torch.Tensor, cache: FragmentCache,
                attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One forward of a model after :func:`model_surgery`: ``input_ids`` / ``position_ids`` ``[W,S]`` (one row per
    worker, positions = the row indices the tokens get in the worker's own fragment), ``attention_mask`` ``None``
    or the ``[W,S]`` left-padding mask.  Returns the logits ``[W,S,vocab]``.  Nothing is read back from the
    device: a step can be captured into a CUDA graph."""
    layer_types = set(getattr(model.model.config, "layer_types", None) or ["full_attention"])
    masks = {t: attention_mask for t in layer_types}
    hidden = model.model(input_ids=input_ids, position_ids=position_ids, attention_mask=masks, past_key_values=cache,
                         use_cache=True).last_hidden_state
    return model.lm_head(hidden)


def cache_for_model(model, capacities: Sequence[int], order: Sequence[Sequence[int]],
                    write_to: Optional[Sequence[int]] = None, world: int = 1) -> FragmentCache:
    """A :class:`FragmentCache` shaped for ``model``: layer count, kv heads, head size, the rotary frequencies and
    attention scaling of its ``rotary_emb`` (what the reference reads through ``HogwildCache(model=...)``,
    ``attention.py:113-121,199``).  ``world`` > 1: this rank's share of the kv heads."""
    cfg = model.model.config
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    rope = model.model.rotary_emb
    p = next(model.parameters())
    if cfg.num_key_value_heads % world:
        raise ValueError(f"{cfg.num_key_value_heads} kv heads cannot be split evenly over {world} ranks")
    return FragmentCache(layers=cfg.num_hidden_layers, capacities=capacities, Hkv=cfg.num_key_value_heads // world, E=head_dim,
                         dtype=p.dtype, device=p.device, order=order, write_to=write_to, inv_freq=rope.inv_freq,
                         attention_scaling=float(getattr(rope, "attention_scaling", 1.0)))
