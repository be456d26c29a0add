"""Host-side mirror of the reference's operator wrappers (``python/hogwild/attention.py:12-90``).

Same function names, argument order and meaning as the reference, so code written against
``hogwild.attention`` can import this module instead.  Every function ends in a
``torch.ops.libhogatt.*`` call that is served by the CUDA library of this package; there is no
eager / CPU implementation here (the reference's ``hogwild_sdpa_pt`` lives on as the test oracle
only), and importing this module fails loudly when the compiled library cannot be loaded.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
TORCH_LIB = os.path.join(_PKG, "hogatt.abi3.so")


def _load_ops() -> None:
    if hasattr(torch.ops, "libhogatt") and hasattr(torch.ops.libhogatt, "hogwild_fused"):
        return
    if not os.path.exists(TORCH_LIB):
        raise ImportError(f"{TORCH_LIB} is missing: run `python -m inference_lib_b200._build` (no fallback exists)")
    torch.ops.load_library(TORCH_LIB)


_load_ops()


def hogwild_fused(queries: torch.Tensor, locations: torch.Tensor, keys: List[torch.Tensor], values: List[torch.Tensor],
                  scale: float, fragment_lengths: torch.Tensor, cosines: torch.Tensor, sines: torch.Tensor, *,
                  rotated_queries: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Query RoPE per fragment + attention over all fragments (``attention.py:19-23``).

    ``queries [W,Hq,S,E]`` un-rotated; ``rotated_queries [F,W,Hq,S,E]`` and ``out [W,Hq,S,Ev]`` are
    caller-owned buffers that are overwritten.
    """
    torch.ops.libhogatt.hogwild_fused(out, rotated_queries, scale, locations, queries.contiguous(), fragment_lengths,
                                      keys, values, cosines, sines)
    return out


def hogwild_fused_planned(queries: torch.Tensor, locations: torch.Tensor, keys: List[torch.Tensor],
                          values: List[torch.Tensor], scale: float, fragment_lengths: torch.Tensor, cosines: torch.Tensor,
                          sines: torch.Tensor, *, rotated_queries: torch.Tensor, out: torch.Tensor,
                          host_lengths: List[int], stable_fragments: int = 0) -> torch.Tensor:
    """:func:`hogwild_fused` for fragments kept in preallocated slabs ``[Hkv, capacity, E]`` (no copies are made;
    the slabs must be contiguous).  ``host_lengths[f]`` is an upper bound, known on the host, of fragment ``f``'s
    current length (the true lengths stay on the device in ``fragment_lengths``); ``stable_fragments`` leading
    fragments are not written by work enqueued before this call, e.g. the shared prompt.  With both, the kernel
    starts streaming keys and values without reading anything from device memory first.  No counterpart in the
    reference, whose fragment tensors always end at the fragment's length."""
    torch.ops.libhogatt.hogwild_fused_planned(out, rotated_queries, scale, locations, queries.contiguous(),
                                              fragment_lengths, keys, values, cosines, sines,
                                              [int(x) for x in host_lengths], int(stable_fragments))
    return out


def hogwild_sdpa(queries: torch.Tensor, locations: torch.Tensor, keys: List[torch.Tensor], values: List[torch.Tensor],
                 scale: float, fragment_lengths: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention over fragments with already-rotated ``queries [F,W,Hq,S,E]`` (``attention.py:26-35``)."""
    if out is None:
        out = torch.empty((queries.size(1), queries.size(2), queries.size(3), values[0].size(-1)),
                          dtype=queries.dtype, device=queries.device)
    if fragment_lengths is None:
        fragment_lengths = torch.tensor([k.size(-2) for k in keys], dtype=torch.int32, device=queries.device)
    keys = [k.contiguous() for k in keys]
    values = [v.contiguous() for v in values]
    torch.ops.libhogatt.hogwild_sdpa(out, scale, locations, queries.contiguous(), fragment_lengths, keys, values)
    return out


def hogwild_rope(queries: torch.Tensor, cosines: torch.Tensor, sines: torch.Tensor,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[W,Hq,S,E]`` queries -> ``[F,W,Hq,S,E]``, one rotation per fragment (``attention.py:70-74``)."""
    if out is None:
        out = torch.empty((cosines.size(0), queries.size(0), queries.size(1), queries.size(2), queries.size(3)),
                          dtype=queries.dtype, device=queries.device)
    torch.ops.libhogatt.hogwild_rope(out, queries, cosines, sines)
    return out


def hogwild_paged_sdpa(queries: torch.Tensor, locations: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                       block_table: torch.Tensor, scale: float, fragment_lengths: torch.Tensor,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged attention: ``queries [F,W,Hq,S,E]`` (rotated), worker ``w`` reads the paged sequence
    ``block_table[w]`` of ``key_cache / value_cache [NumBlocks,Hkv,bs,E]``.  The reference registers this
    operator (``src/binding.cu:368-369``) but ships no Python wrapper for it."""
    if out is None:
        out = torch.empty((queries.size(1), queries.size(2), queries.size(3), value_cache.size(3)),
                          dtype=queries.dtype, device=queries.device)
    torch.ops.libhogatt.hogwild_paged_sdpa(out, scale, locations, queries.contiguous(), fragment_lengths, key_cache,
                                           value_cache, block_table)
    return out


def hogwild_varlen_paged_sdpa(queries: torch.Tensor, locations: torch.Tensor, key_cache: torch.Tensor,
                              value_cache: torch.Tensor, block_table: torch.Tensor, scale: float,
                              fragment_lengths: torch.Tensor, cu_seqlens_q: torch.Tensor,
                              cu_seqlens_k: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed-query paged attention: ``queries [F,total_q,Hq,E]``, ``locations [F,total_q]``,
    ``fragment_lengths [F,W]``, ``cu_seqlens_q [W+1]`` (``src/binding.cu:372-374``)."""
    if out is None:
        out = torch.empty((queries.size(1), queries.size(2), value_cache.size(3)), dtype=queries.dtype, device=queries.device)
    if cu_seqlens_k is None:
        cu_seqlens_k = cu_seqlens_q
    torch.ops.libhogatt.hogwild_varlen_paged_sdpa(out, scale, locations, queries.contiguous(), fragment_lengths, key_cache,
                                                  value_cache, block_table, cu_seqlens_q, cu_seqlens_k)
    return out


def copy_to_blocks(key_states: torch.Tensor, value_states: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                   block_table: torch.Tensor, seq_lengths: torch.Tensor) -> None:
    """Append ``key_states / value_states [B,Hkv,S_new,E]`` to the paged caches at ``seq_lengths[b] + t``
    (``src/binding.cu:370-371``)."""
    torch.ops.libhogatt.copy_to_blocks(key_states.contiguous(), value_states.contiguous(), key_cache, value_cache,
                                       block_table, seq_lengths)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``attention.py:77-81``."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary_pos_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, unsqueeze_dim: int = 1) -> torch.Tensor:
    """Key-side RoPE used when new keys are written to a fragment (``attention.py:84-90``, call site ``:315``)."""
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    r = cos.shape[-1]
    head, tail = x[..., :r], x[..., r:]
    return torch.cat(((head * cos) + (rotate_half(head) * sin), tail), dim=-1).to(x.dtype)
