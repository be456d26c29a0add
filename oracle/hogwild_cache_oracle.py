"""CPU restatement of the steps either side of the attention op.  TEST INFRASTRUCTURE ONLY: nothing in
the product imports this module; tests compare the CUDA path against it.

Restates, in plain numpy / torch-CPU:

* the per-step metadata built by ``HogwildCache.update`` at layer 0 (``python/hogwild/attention.py:164-204``):
  ``step_locations``, ``rotary_tables``;
* the positions a worker's new tokens get in its own fragment (``get_input_kwargs``, ``:233-244``):
  ``own_positions``;
* the key rotation of ``AttentionModule.forward`` (``:315``, ``apply_rotary_pos_emb`` ``:84-90``) and the
  append of ``HogwildCache.update`` (``:139-158``): ``rotate_keys``, ``append``;
* ``merge_caches`` (``:251-257``): ``merge``.

Parity is pinned: ``tests/test_cache_oracle.py`` checks every function against
``tests/golden/cache_steps.npz``, which ``tests/golden/make_cache_golden.py`` produced by running the
reference's own ``HogwildCache`` / ``apply_rotary_pos_emb`` / ``merge_caches``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch


def step_locations(order: np.ndarray, lengths: Sequence[int], S: int) -> np.ndarray:
    """``[F,W,S]`` int32.  ``order[w]`` lists fragment ids in worker ``w``'s sequence order (-1 = unused slot);
    ``lengths`` already include the ``S`` tokens of this step.  Walking the order backwards, ``pos`` is the
    distance from the end of the worker's sequence to the start of the fragment; the new tokens sit at
    ``pos - S .. pos - 1`` (attention.py:173-181).  Fragments a worker does not have get -1."""
    W = order.shape[0]
    F = len(lengths)
    loc = np.full((F, W, S), -1, dtype=np.int32)
    for w in range(W):
        pos = 0
        for f in reversed([int(x) for x in order[w] if x >= 0]):
            pos += int(lengths[f])
            loc[f, w] = np.arange(pos - S, pos, dtype=np.int32)
    return loc


def rotary_tables(locations: np.ndarray, inv_freq: np.ndarray, attention_scaling: float = 1.0,
                  model_dtype: Optional[torch.dtype] = None):
    """cos/sin ``[..., R]`` fp32 for integer positions: fp32 ``position * inv_freq``, both halves equal, times
    ``attention_scaling``; if ``model_dtype`` is given the values pass through that type first, as when
    ``rotary_emb`` returns them in the model's type and the caller converts back to float (attention.py:191-193)."""
    pos = torch.from_numpy(np.asarray(locations)).to(torch.float32)
    freqs = pos[..., None] * torch.from_numpy(np.asarray(inv_freq, dtype=np.float32))
    emb = torch.cat([freqs, freqs], dim=-1)
    cos, sin = emb.cos() * attention_scaling, emb.sin() * attention_scaling
    if model_dtype is not None:
        cos, sin = cos.to(model_dtype), sin.to(model_dtype)
    return cos.to(torch.float32), sin.to(torch.float32)


def own_positions(own_length: int, new_rows: int, S: int) -> np.ndarray:
    """Positions of a worker's ``S`` input tokens in its own fragment, of which the last ``new_rows`` are real
    (left-masked): they end at ``own_length + new_rows`` (attention.py:233-244)."""
    e = own_length + new_rows
    return np.arange(e - S, e, dtype=np.int32)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def rotate_keys(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x [W,Hkv,S,E]``, tables ``[W,S,R]`` (fp32 or ``x``'s type): ``x*cos + rotate_half(x)*sin`` on the first
    ``R`` channels in torch's own promotion and rounding rules, result in ``x``'s type (attention.py:84-90)."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    R = cos.shape[-1]
    rot, rest = x[..., :R], x[..., R:]
    emb = (rot * cos) + (rotate_half(rot) * sin)
    return torch.cat((emb, rest), dim=-1).to(x.dtype)


def append(frag_k: torch.Tensor, frag_v: torch.Tensor, k_rot: torch.Tensor, v_new: torch.Tensor, new_rows: Optional[int] = None):
    """Fragment ``[Hkv,L,E]`` grown by the last ``new_rows`` rows of ``[Hkv,S,E]`` (attention.py:148-158)."""
    n = k_rot.shape[-2] if new_rows is None else int(new_rows)
    if n == 0:
        return frag_k, frag_v
    return torch.cat([frag_k, k_rot[:, -n:]], dim=-2), torch.cat([frag_v, v_new[:, -n:]], dim=-2)


def merge(target_k: List[torch.Tensor], target_v: List[torch.Tensor], source_k: List[torch.Tensor],
          source_v: List[torch.Tensor], inv_freq: np.ndarray, attention_scaling: float = 1.0):
    """Per layer: the source's keys re-rotated by the constant position ``len(target)`` (tables in the keys'
    type) and appended, values appended as they are (attention.py:251-257).  Lists of ``[Hkv,L,E]`` per layer."""
    t_len = target_k[0].shape[-2]
    s_len = source_k[0].shape[-2]
    loc = np.full((1, s_len), t_len, dtype=np.int32)
    cos, sin = rotary_tables(loc, inv_freq, attention_scaling, source_k[0].dtype)
    cos, sin = cos.to(source_k[0].dtype), sin.to(source_k[0].dtype)
    out_k, out_v = [], []
    for tk, tv, sk, sv in zip(target_k, target_v, source_k, source_v):
        k_rot = rotate_keys(sk[None], cos, sin)[0]
        out_k.append(torch.cat([tk, k_rot], dim=-2))
        out_v.append(torch.cat([tv, sv], dim=-2))
    return out_k, out_v
