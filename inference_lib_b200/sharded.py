"""KV-head sharding of the op across the GPUs of one node.

Heads are independent (a CTA never mixes kv heads and the softmax is per query head), so rank ``r`` of
``G`` keeps kv heads ``[r*Hkv/G, (r+1)*Hkv/G)`` of every fragment plus the matching ``Hq/G`` query heads,
and runs the unchanged single-GPU op on them; locations, tables and lengths are replicated.  The only
exchange is the all-gather of the output along the head axis.  The reference has no multi-device path
(device 0 is hard-coded, ``src/kernels/kernel_v21.cuh:960``).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def head_slices(Hq: int, Hkv: int, rank: int, world: int):
    if Hkv % world:
        raise ValueError(f"{Hkv} kv heads cannot be split evenly over {world} ranks")
    hk = Hkv // world
    g = Hq // Hkv
    return slice(rank * hk * g, (rank + 1) * hk * g), slice(rank * hk, (rank + 1) * hk)


def shard_inputs(queries: torch.Tensor, keys: List[torch.Tensor], values: List[torch.Tensor], rank: int, world: int):
    """This rank's query heads and kv heads (contiguous copies; done once when the cache is placed)."""
    Hq, Hkv = queries.shape[1], keys[0].shape[-3]
    qs, ks = head_slices(Hq, Hkv, rank, world)
    return (queries[:, qs].contiguous(), [k[..., ks, :, :].contiguous() for k in keys],
            [v[..., ks, :, :].contiguous() for v in values])


def gather_heads(out_local: torch.Tensor, world: int, *, gather_buffer: Optional[torch.Tensor] = None,
                 group=None) -> torch.Tensor:
    """All-gather ``[W, Hq/G, S, Ev]`` per rank into ``[W, Hq, S, Ev]`` on every rank.

    The collective lands rank-major (``[G, W, Hq/G, S, Ev]``); the head axis is not the leading one, so
    one permute-copy puts the result in operator layout.
    """
    W, hq, S, Ev = out_local.shape
    if gather_buffer is None:
        gather_buffer = torch.empty((world, W, hq, S, Ev), dtype=out_local.dtype, device=out_local.device)
    # concatenated form along dim 0 (accepted by every backend); the buffer is [G, W, ...] in memory
    dist.all_gather_into_tensor(gather_buffer.view(world * W, hq, S, Ev), out_local.contiguous(), group=group)
    return gather_buffer.permute(1, 0, 2, 3, 4).reshape(W, world * hq, S, Ev)
