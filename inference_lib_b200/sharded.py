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


class PeerOutputs:
    """Peer-mapped buffers for the all-gather that is fused into the op (``hogatt_fused_launch_gather``).

    ``slots`` full-size outputs ``[W, Hq_total, S, Ev]`` plus one flag array per slot live in symmetric
    memory (``torch.distributed._symmetric_memory``: every rank allocates the same sizes and maps the
    others' allocations into its own address space).  The merge step of each rank stores its heads into
    ALL ranks' outputs through those mappings; no collective library call is involved, so a step that
    uses it can be captured into a CUDA graph.  Use a different slot for calls whose outputs are alive
    at the same time (e.g. one per layer, or two alternating).
    """

    def __init__(self, group, world: int, rank: int, slots: int, shape_full, dtype, device):
        import torch.distributed._symmetric_memory as symm
        self.world, self.rank, self.slots = world, rank, slots
        self.out = symm.empty((slots,) + tuple(shape_full), dtype=dtype, device=device)
        self.flags = symm.empty((slots, world + 1), dtype=torch.int32, device=device)
        self.out.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(device)
        h_out = symm.rendezvous(self.out, group)
        h_flags = symm.rendezvous(self.flags, group)
        self._handles = (h_out, h_flags)          # keep the mappings alive
        self._out_ptrs = [int(p) for p in h_out.buffer_ptrs]
        self._flag_ptrs = [int(p) for p in h_flags.buffer_ptrs]
        self._out_stride = self.out[0].numel() * self.out.element_size()
        self._flag_stride = (world + 1) * 4
        dist.barrier(group=group if not isinstance(group, str) else None)

    def peers(self, slot: int):
        """The ``hogatt_peers`` table for one slot."""
        from . import _cabi
        p = _cabi.Peers()
        p.world, p.rank = self.world, self.rank
        for r in range(self.world):
            p.out_full[r] = self._out_ptrs[r] + slot * self._out_stride
            p.flags[r] = self._flag_ptrs[r] + slot * self._flag_stride
        return p

    def output(self, slot: int) -> torch.Tensor:
        """This rank's full-size output of a slot (complete once the call's stream work has finished)."""
        return self.out[slot]
