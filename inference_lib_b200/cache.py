"""Device-resident fragment cache: the role of the reference's ``HogwildCache``
(``python/hogwild/attention.py:112-257``) around the attention op, without its per-step host work.

The reference keeps one growing tensor per fragment and layer (``torch.cat`` on every append, ``.contiguous()``
on every read), rebuilds ``locations`` / ``cos`` / ``sin`` with Python loops and the model's ``rotary_emb`` at
layer 0 of every step, and rotates the new keys with eager elementwise ops.  Here

* every fragment is a preallocated slab ``[Hkv, capacity, E]`` per layer: pointers never change, the current
  lengths live in a device tensor (two buffers per layer, flipped by every append), so a whole decode step can
  be enqueued without reading anything back;
* ``update`` = one ``hogatt_append_launch`` (key rotation at the tokens' own positions + append of keys and
  values) and, at layer 0, one ``hogatt_step_plan_launch`` (locations and rotary tables for the queries);
* ``merge`` = ``merge_caches``: one append per layer whose single table row (the target's length as a constant
  position) is broadcast over the source's rows.

``update`` returns the same bundle the reference's does (``CacheStructure``: keys, values, frags, cos, sin,
loc), ready for :func:`inference_lib_b200.attention.hogwild_fused`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from . import _cabi


@dataclass
class CacheStructure:
    keys: List[torch.Tensor]      # per fragment [Hkv, capacity, E] slabs (only the first frags[f] rows are valid)
    values: List[torch.Tensor]
    frags: torch.Tensor           # [F] int32 device: current lengths
    cos: torch.Tensor             # [F,W,S,R] fp32: tables to rotate the queries with
    sin: torch.Tensor
    loc: torch.Tensor             # [F,W,S] int32
    host_lengths: Optional[List[int]] = None   # per fragment: an upper bound of frags[f] that the host knows
    stable: int = 0               # leading fragments that no worker appends to


class FragmentCache:
    """``order[w]`` lists the fragment ids in worker ``w``'s sequence order (its own fragment last);
    ``write_to[w]`` is the fragment worker ``w`` appends to (default: the last of its order)."""

    def __init__(self, *, layers: int, capacities: Sequence[int], Hkv: int, E: int, Ev: Optional[int] = None,
                 dtype=torch.bfloat16, device="cuda", order: Sequence[Sequence[int]], write_to: Optional[Sequence[int]] = None,
                 inv_freq: torch.Tensor, attention_scaling: float = 1.0, round_tables_to_model_dtype: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("FragmentCache needs a CUDA device: there is no CPU path")
        self.device = torch.device(device)
        self.layers, self.F, self.W = layers, len(capacities), len(order)
        self.Hkv, self.E, self.Ev, self.dtype = Hkv, E, Ev or E, dtype
        self.capacities = [int(c) for c in capacities]
        self.keys = [[torch.zeros((Hkv, c, E), dtype=dtype, device=self.device) for c in self.capacities] for _ in range(layers)]
        self.values = [[torch.zeros((Hkv, c, self.Ev), dtype=dtype, device=self.device) for c in self.capacities] for _ in range(layers)]
        # lengths[layer][flip]: the buffer index `cur[layer]` holds the valid lengths
        self.lengths = [[torch.zeros(self.F, dtype=torch.int32, device=self.device) for _ in range(2)] for _ in range(layers)]
        self.cur = [0] * layers
        # what the host knows without reading anything back: an upper bound of every length (appends add at most S)
        self.host_lengths = [[0] * self.F for _ in range(layers)]
        rows = [list(o) + [-1] * (self.F - len(o)) for o in order]
        self.order = torch.tensor(rows, dtype=torch.int32, device=self.device)
        self.write_to = [int(x) for x in (write_to if write_to is not None else [o[-1] for o in order])]
        self.inv_freq = inv_freq.to(device=self.device, dtype=torch.float32).contiguous()
        self.attention_scaling = float(attention_scaling)
        self.round_to = _cabi.dtype_code(dtype) if round_tables_to_model_dtype else _cabi.F32
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.loc = self.cos = self.sin = None

    # ---- filling -----------------------------------------------------------------------------------------
    def load_fragment(self, f: int, keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor]):
        """Prefill fragment ``f`` from per-layer ``[Hkv, L, E]`` tensors whose keys are already rotated."""
        for layer in range(self.layers):
            L = keys[layer].shape[-2]
            self.keys[layer][f][:, :L].copy_(keys[layer])
            self.values[layer][f][:, :L].copy_(values[layer])
            self.lengths[layer][self.cur[layer]][f] = L
            self.host_lengths[layer][f] = int(L)

    def frags(self, layer: int = 0) -> torch.Tensor:
        return self.lengths[layer][self.cur[layer]]

    # ---- one layer of a decode step --------------------------------------------------------------------------
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer: int, cos: torch.Tensor, sin: torch.Tensor,
               new_rows: Optional[torch.Tensor] = None) -> CacheStructure:
        """``key_states`` / ``value_states`` ``[W,Hkv,S,E]`` (any strides, e.g. the transposed view of a projection
        output), un-rotated; ``cos`` / ``sin`` ``[W,S,R]`` for the tokens' own positions, fp32 or the model's type
        (the latter reproduces the reference's arithmetic, ``attention.py:315``).  ``new_rows [W]`` int32 device:
        only the last ``new_rows[w]`` tokens of worker ``w`` are real (left-masked input, ``attention.py:139-145``)."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        S = key_states.shape[2]
        src, dst = self.lengths[layer][self.cur[layer]], self.lengths[layer][1 - self.cur[layer]]
        rc = _cabi.append(keys=key_states, values=value_states, cosines=cos, sines=sin, write_to=self.write_to,
                          key_fragments=self.keys[layer], value_fragments=self.values[layer], lengths_in=src,
                          lengths_out=dst, new_rows=new_rows, status=self.status, stream=stream)
        if rc != 0:
            raise RuntimeError(f"hogatt_append_launch: {_cabi.status_string(rc)}")
        self.cur[layer] = 1 - self.cur[layer]
        for f in self.write_to:
            self.host_lengths[layer][f] = min(self.capacities[f], self.host_lengths[layer][f] + S)
        if layer == 0:
            R = 2 * self.inv_freq.numel()
            if self.loc is None or self.loc.shape[2] != S:
                self.loc = torch.empty((self.F, self.W, S), dtype=torch.int32, device=self.device)
                self.cos = torch.empty((self.F, self.W, S, R), dtype=torch.float32, device=self.device)
                self.sin = torch.empty_like(self.cos)
            rc = _cabi.step_plan(order=self.order, fragment_lengths=dst, inv_freq=self.inv_freq, S=S, locations=self.loc,
                                 cosines=self.cos, sines=self.sin, attention_scaling=self.attention_scaling,
                                 round_tables_to=self.round_to, stream=stream)
            if rc != 0:
                raise RuntimeError(f"hogatt_step_plan_launch: {_cabi.status_string(rc)}")
        return CacheStructure(keys=self.keys[layer], values=self.values[layer], frags=dst, cos=self.cos, sin=self.sin,
                              loc=self.loc, host_lengths=list(self.host_lengths[layer]), stable=min(self.write_to))

    # ---- merge_caches ----------------------------------------------------------------------------------------
    def merge(self, target: int, source: int):
        """Append fragment ``source`` to fragment ``target`` in every layer, its keys re-rotated by the target's
        current length as one constant position, tables in the model's type (``merge_caches``,
        ``python/hogwild/attention.py:251-257``).  The source keeps its contents."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        t_len = self.frags(0)[target:target + 1].to(torch.float32)          # stays on the device
        angle = t_len * self.inv_freq
        emb = torch.cat([angle, angle])
        cos = (emb.cos() * self.attention_scaling).to(self.dtype)
        sin = (emb.sin() * self.attention_scaling).to(self.dtype)
        for layer in range(self.layers):
            src, dst = self.lengths[layer][self.cur[layer]], self.lengths[layer][1 - self.cur[layer]]
            cap = self.capacities[source]
            k = self.keys[layer][source].view(1, self.Hkv, cap, self.E)
            v = self.values[layer][source].view(1, self.Hkv, cap, self.Ev)
            # the source is a slab itself: its first lengths[source] rows are taken, the count stays on the device
            rc = _cabi.append(keys=k, values=v, cosines=cos, sines=sin, write_to=[target], key_fragments=self.keys[layer],
                              value_fragments=self.values[layer], lengths_in=src, lengths_out=dst,
                              new_rows=src[source:source + 1], take_leading=True, status=self.status, stream=stream)
            if rc != 0:
                raise RuntimeError(f"hogatt_append_launch: {_cabi.status_string(rc)}")
            self.cur[layer] = 1 - self.cur[layer]
            self.host_lengths[layer][target] = min(self.capacities[target],
                                                   self.host_lengths[layer][target] + self.host_lengths[layer][source])
