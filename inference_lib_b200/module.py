"""The attention layer around the op: the role of the reference's ``AttentionModule``
(``python/hogwild/attention.py:263-336``) on top of :class:`inference_lib_b200.cache.FragmentCache`.

``forward`` is the reference's sequence -- q/k/v projections, key rotation, cache update, fused attention over
all fragments, output projection -- with the eager pieces replaced: the key rotation and the append are one
kernel launch inside ``FragmentCache.update`` (the reference: ``apply_rotary_pos_emb`` + ``torch.cat`` per
worker), the per-step metadata one more at layer 0, and the attention is ``hogwild_fused``.  The projections
stay ``torch.nn.Linear`` (cuBLAS): they are plain GEMMs and not part of the path this package rebuilds.
"""
from __future__ import annotations

from typing import Optional, Tuple

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
                cache: FragmentCache, new_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``hidden_states [W,S,hidden]``; ``position_embeddings`` = (cos, sin) ``[W,S,R]`` at the tokens' own
        positions, as the model computes them; ``new_rows [W]`` int32 device for left-masked inputs."""
        W, S, _ = hidden_states.shape
        shape = (W, S, -1, self.head_dim)
        q = self.q_proj(hidden_states).view(shape).transpose(1, 2)          # [W,Hq,S,D] views, no copies
        k = self.k_proj(hidden_states).view(shape).transpose(1, 2)
        v = self.v_proj(hidden_states).view(shape).transpose(1, 2)
        cos, sin = position_embeddings
        cs = cache.update(k, v, self.layer_idx, cos, sin, new_rows)         # rotates the keys itself
        F = len(cs.keys)
        if self._rq is None or self._rq.shape != (F, W, self.num_heads, S, self.head_dim):
            self._rq = torch.empty((F, W, self.num_heads, S, self.head_dim), dtype=q.dtype, device=q.device)
            self._att = torch.empty((W, self.num_heads, S, cs.values[0].shape[-1]), dtype=q.dtype, device=q.device)
        att = ops.hogwild_fused_planned(q, cs.loc, cs.keys, cs.values, self.scaling, cs.frags, cs.cos, cs.sin,
                                        rotated_queries=self._rq, out=self._att, host_lengths=cs.host_lengths,
                                        stable_fragments=cs.stable)
        return self.o_proj(att.transpose(1, 2).reshape(W, S, -1))
