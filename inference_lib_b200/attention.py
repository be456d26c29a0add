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
