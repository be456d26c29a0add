"""Seeded synthetic problems for the Hogwild! fragmented-KV attention op.

A *problem* is one call of the op: ``W`` workers each issue ``S`` query tokens against the
same list of ``F`` KV fragments, every worker seeing the fragments in its own order (so at
its own position offsets).  The tensors follow the operator contract of the reference
(``src/binding.cu:39-108`` for shapes, ``python/hogwild/attention.py:164-204`` for how the
cache builds ``locations`` / ``cos`` / ``sin`` / ``frags``):

* ``queries``      ``[W, Hq, S, E]``   un-rotated
* ``keys[f]``      ``[1, Hkv, L_f, E]``  already rotated at fragment-local positions 0..L_f-1
* ``values[f]``    ``[1, Hkv, L_f, Ev]``
* ``locations``    ``[F, W, S]`` int32   key ``l`` of fragment ``f`` is visible to ``(w, s)``
  iff ``l <= locations[f, w, s]``
* ``cos`` / ``sin`` ``[F, W, S, R]`` fp32  rotation of worker ``w``'s query for fragment ``f``
* ``fragment_lengths`` ``[F]`` int32

Everything is generated on the CPU from ``torch.Generator().manual_seed(seed)`` in a fixed
draw order (queries, then per fragment keys followed by values), so the same problem can be
rebuilt bit-identically on any machine.  No dataset is involved.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Sequence

import torch

__all__ = [
    "Problem", "make_problem", "rope_tables", "rotate_keys", "hogwild_locations",
    "BASELINE_CONFIGS", "EDGE_CASES", "baseline_problem", "edge_problem",
]


def rope_tables(positions: torch.Tensor, rotary_dim: int, theta: float):
    """cos/sin tables in the duplicated-halves layout used by HF rotary embeddings.

    ``positions`` is any integer tensor; the result has one trailing axis of length
    ``rotary_dim`` with ``table[..., i] == table[..., i + rotary_dim // 2]``.
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    angle = positions.to(torch.float32)[..., None] * inv_freq
    angle = torch.cat([angle, angle], dim=-1)
    return angle.cos(), angle.sin()


def rotate_keys(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on the leading ``cos.shape[-1]`` channels of ``x`` (fp32 math).

    Same convention as ``apply_rotary_pos_emb`` of the reference
    (``python/hogwild/attention.py:84-90``): channel ``e`` pairs with ``e +- R/2``.
    """
    r = cos.shape[-1]
    xr, xp = x[..., :r].to(torch.float32), x[..., r:]
    half = r // 2
    swapped = torch.cat([-xr[..., half:], xr[..., :half]], dim=-1)
    out = xr * cos + swapped * sin
    return torch.cat([out.to(x.dtype), xp], dim=-1)


def hogwild_locations(lengths: Sequence[int], orders: Sequence[Sequence[int]], S: int) -> torch.Tensor:
    """Query positions relative to each fragment (``attention.py:173-181`` semantics).

    ``orders[w]`` lists the fragments worker ``w`` sees, first to last; its own fragment
    (the one holding its ``S`` newest tokens) is last.  A fragment missing from the order
    is invisible to that worker and gets location ``-1``.
    """
    F, W = len(lengths), len(orders)
    loc = torch.full((F, W, S), -1, dtype=torch.int32)
    for w, order in enumerate(orders):
        pos = 0
        for f in reversed(list(order)):
            pos += int(lengths[f])
            loc[f, w] = torch.arange(pos - S, pos, dtype=torch.int32)
    return loc


@dataclass
class Problem:
    name: str
    queries: torch.Tensor
    keys: List[torch.Tensor]
    values: List[torch.Tensor]
    locations: torch.Tensor
    cos: torch.Tensor
    sin: torch.Tensor
    fragment_lengths: torch.Tensor
    scale: float
    theta: float
    meta: Dict = field(default_factory=dict)

    # ---- shape helpers -------------------------------------------------------------
    @property
    def F(self): return len(self.keys)
    @property
    def W(self): return self.queries.shape[0]
    @property
    def Hq(self): return self.queries.shape[1]
    @property
    def S(self): return self.queries.shape[2]
    @property
    def E(self): return self.queries.shape[3]
    @property
    def Hkv(self): return self.keys[0].shape[-3]
    @property
    def Ev(self): return self.values[0].shape[-1]
    @property
    def dtype(self): return self.queries.dtype

    def to(self, device) -> "Problem":
        mv = lambda t: t.to(device)
        return replace(self, queries=mv(self.queries), keys=[mv(k) for k in self.keys],
                       values=[mv(v) for v in self.values], locations=mv(self.locations),
                       cos=mv(self.cos), sin=mv(self.sin), fragment_lengths=mv(self.fragment_lengths))

    def shard(self, rank: int, world: int) -> "Problem":
        """KV-head shard ``rank`` of ``world``: heads are independent, metadata is replicated."""
        if self.Hkv % world:
            raise ValueError(f"Hkv={self.Hkv} is not divisible by world size {world}")
        hk = self.Hkv // world
        g = self.Hq // self.Hkv
        ks, qs = slice(rank * hk, (rank + 1) * hk), slice(rank * hk * g, (rank + 1) * hk * g)
        return replace(self, name=f"{self.name}[kv-shard {rank}/{world}]",
                       queries=self.queries[:, qs].contiguous(),
                       keys=[k[..., ks, :, :].contiguous() for k in self.keys],
                       values=[v[..., ks, :, :].contiguous() for v in self.values])

    def visible_lengths(self) -> List[int]:
        """Per fragment, how many leading keys at least one query row can see."""
        top = self.locations.reshape(self.F, -1).max(dim=1).values + 1
        return [int(min(max(int(t), 0), int(l))) for t, l in zip(top, self.fragment_lengths)]

    def algorithmic_bytes(self) -> int:
        """KV read once + un-rotated Q once + O once (what the roofline fraction is taken of)."""
        sz = self.queries.element_size()
        kv = sum(self.Hkv * v * (self.E + self.Ev) * sz for v in self.visible_lengths())
        return kv + self.W * self.Hq * self.S * (self.E + self.Ev) * sz

    def flops(self) -> int:
        return 2 * self.W * self.Hq * self.S * sum(self.visible_lengths()) * (self.E + self.Ev)


def make_problem(name: str, *, W: int, Hq: int, Hkv: int, E: int, S: int, lengths: Sequence[int],
                 theta: float, dtype: torch.dtype, seed: int = 0, Ev: Optional[int] = None,
                 rotary_dim: Optional[int] = None, orders: Optional[Sequence[Sequence[int]]] = None,
                 locations: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> Problem:
    """Build one seeded problem.

    Default fragment layout is the Hogwild! one: fragment 0 is the shared prompt and fragment
    ``1 + w`` belongs to worker ``w``; worker ``w`` sees *prompt, the other workers in index
    order, then its own fragment*.  ``orders`` / ``locations`` override that for edge cases.
    """
    Ev = E if Ev is None else Ev
    R = E if rotary_dim is None else rotary_dim
    F = len(lengths)
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(W, Hq, S, E, generator=gen)
    keys, values = [], []
    for L in lengths:
        k = torch.randn(1, Hkv, L, E, generator=gen)
        v = torch.randn(1, Hkv, L, Ev, generator=gen)
        c, s = rope_tables(torch.arange(L)[None], R, theta)           # [1, L, R] -> broadcast over heads
        keys.append(rotate_keys(k, c, s).to(dtype))
        values.append(v.to(dtype))
    if locations is None:
        if orders is None:
            if F != W + 1:
                raise ValueError("default Hogwild! layout needs F == W + 1 fragments")
            orders = [[0] + [1 + o for o in range(W) if o != w] + [1 + w] for w in range(W)]
        locations = hogwild_locations(lengths, orders, S)
    locations = locations.to(torch.int32).contiguous()
    cos, sin = rope_tables(locations, R, theta)                        # [F, W, S, R]
    return Problem(name=name, queries=q.to(dtype), keys=keys, values=values, locations=locations,
                   cos=cos.contiguous(), sin=sin.contiguous(),
                   fragment_lengths=torch.tensor(list(lengths), dtype=torch.int32),
                   scale=float(E ** -0.5 if scale is None else scale), theta=theta,
                   meta=dict(W=W, Hq=Hq, Hkv=Hkv, E=E, Ev=Ev, S=S, R=R, lengths=list(lengths), seed=seed,
                             dtype=str(dtype).replace("torch.", "")))


# ---------------------------------------------------------------------------------------
# The benchmark shapes.  cfg1..cfg5 are the five named configurations; "target" is the
# shape the >=70 %-of-peak goal is stated on (Llama-3-8B heads, 4 workers, 16,384 tokens).
# ---------------------------------------------------------------------------------------
BASELINE_CONFIGS: Dict[str, Dict] = {
    "cfg1": dict(W=2, Hq=8, Hkv=2, E=64, S=1, lengths=[256, 64, 64], theta=1e4, dtype=torch.float32),
    "cfg2": dict(W=2, Hq=32, Hkv=8, E=128, S=1, lengths=[4096, 2048, 2048], theta=5e5, dtype=torch.bfloat16),
    "cfg3": dict(W=4, Hq=40, Hkv=8, E=128, S=1, lengths=[8192] + [2048] * 4, theta=1e6, dtype=torch.bfloat16),
    "cfg4": dict(W=2, Hq=32, Hkv=8, E=128, S=1, lengths=[131072, 4096, 4096], theta=5e5, dtype=torch.bfloat16),
    "cfg5": dict(W=8, Hq=64, Hkv=8, E=128, S=16, lengths=[16384] + [1024] * 8, theta=5e5, dtype=torch.bfloat16),
    "target": dict(W=4, Hq=32, Hkv=8, E=128, S=1, lengths=[8192] + [2048] * 4, theta=5e5, dtype=torch.bfloat16),
    # the target's workers and lengths at the one head layout the reference's CUDA kernel accepts (16 query heads per
    # kv head, src/kernels/kernel_v21.cuh:982): the shape both implementations can be timed on side by side
    "gqa16": dict(W=4, Hq=32, Hkv=2, E=128, S=1, lengths=[8192] + [2048] * 4, theta=5e5, dtype=torch.bfloat16),
}


def baseline_problem(name: str, seed: int = 0, **overrides) -> Problem:
    cfg = dict(BASELINE_CONFIGS[name]); cfg.update(overrides)
    return make_problem(name, seed=seed, **cfg)


def _loc(rows):  # helper: nested list [F][W][S] -> int32 tensor
    return torch.tensor(rows, dtype=torch.int32)


# Small problems that exercise what the big shapes do not: ragged lengths, hidden fragments,
# partially visible fragments, rows that see nothing, causal chunks, partial rotary dim,
# GQA 1 / 5 / 16, a single KV head, E != Ev, fp16, empty fragments.
EDGE_CASES: Dict[str, Dict] = {
    "ragged_bf16": dict(W=3, Hq=8, Hkv=2, E=128, S=1, lengths=[37, 1, 9, 130], theta=1e4, dtype=torch.bfloat16),
    "ragged_f16": dict(W=2, Hq=6, Hkv=2, E=128, S=1, lengths=[71, 8, 33], theta=1e4, dtype=torch.float16),
    "ragged_f32": dict(W=2, Hq=4, Hkv=2, E=64, S=1, lengths=[45, 7, 19], theta=1e4, dtype=torch.float32),
    "gqa1_bf16": dict(W=2, Hq=4, Hkv=4, E=128, S=1, lengths=[100, 20, 20], theta=5e5, dtype=torch.bfloat16),
    "gqa5_bf16": dict(W=4, Hq=10, Hkv=2, E=128, S=1, lengths=[300, 17, 18, 19, 20], theta=1e6, dtype=torch.bfloat16),
    "gqa16_bf16": dict(W=2, Hq=32, Hkv=2, E=128, S=1, lengths=[257, 63, 65], theta=5e5, dtype=torch.bfloat16),
    "one_kv_head_bf16": dict(W=2, Hq=4, Hkv=1, E=128, S=1, lengths=[513, 31, 33], theta=5e5, dtype=torch.bfloat16),
    "d64_bf16": dict(W=2, Hq=8, Hkv=2, E=64, S=1, lengths=[200, 40, 41], theta=1e4, dtype=torch.bfloat16),
    "causal_chunk_bf16": dict(W=2, Hq=8, Hkv=2, E=128, S=5, lengths=[90, 12, 23], theta=5e5, dtype=torch.bfloat16),
    "causal_chunk_f32": dict(W=2, Hq=4, Hkv=2, E=64, S=4, lengths=[50, 9, 11], theta=1e4, dtype=torch.float32),
    "partial_rotary_bf16": dict(W=2, Hq=8, Hkv=2, E=128, S=1, lengths=[64, 16, 16], theta=1e4,
                                dtype=torch.bfloat16, rotary_dim=64),
    "ev_differs_f32": dict(W=2, Hq=4, Hkv=2, E=64, Ev=32, S=1, lengths=[40, 8, 8], theta=1e4, dtype=torch.float32),
    "ev_differs_bf16": dict(W=2, Hq=8, Hkv=2, E=128, Ev=64, S=2, lengths=[70, 10, 10], theta=1e4,
                            dtype=torch.bfloat16),
    # worker 1 does not see fragment 1 at all (-1); worker 0 sees only the first 10 keys of the
    # prompt; fragment 2 is fully visible to both; fragment 3 is empty.
    "hidden_and_partial_bf16": dict(W=2, Hq=8, Hkv=2, E=128, S=1, lengths=[64, 20, 30, 0], theta=1e4,
                                    dtype=torch.bfloat16,
                                    locations=_loc([[[9], [200]], [[40], [-1]], [[60], [29]], [[5], [5]]])),
    # worker 1 sees nothing anywhere: its rows must come out as zeros.
    "blind_worker_bf16": dict(W=2, Hq=4, Hkv=2, E=128, S=1, lengths=[33, 12], theta=1e4, dtype=torch.bfloat16,
                              locations=_loc([[[32], [-1]], [[11], [-1]]])),
    "blind_worker_f32": dict(W=2, Hq=4, Hkv=2, E=64, S=1, lengths=[33, 12], theta=1e4, dtype=torch.float32,
                             locations=_loc([[[32], [-1]], [[11], [-1]]])),
    # many workers: 40 query rows per KV head, more than one 32-row tile
    "many_rows_bf16": dict(W=5, Hq=16, Hkv=2, E=128, S=1, lengths=[150, 10, 11, 12, 13, 14], theta=5e5,
                           dtype=torch.bfloat16),
    # 96 rows per KV head: more than one row block of the tensor-core kernel
    "row_blocks_bf16": dict(W=3, Hq=8, Hkv=2, E=128, S=8, lengths=[120, 16, 24, 32], theta=5e5,
                            dtype=torch.bfloat16),
    # long enough that every SM gets several tiles and heads are split many ways
    "split_many_bf16": dict(W=2, Hq=8, Hkv=2, E=128, S=1, lengths=[20000, 3000, 3001], theta=5e5,
                            dtype=torch.bfloat16),
    "split_many_f32": dict(W=2, Hq=4, Hkv=2, E=64, S=1, lengths=[6000, 700, 701], theta=1e4, dtype=torch.float32),
    # many query rows per kv head (token chunks): 128-row query blocks.  G*S = 128: a block is one worker ...
    "dense_chunk_bf16": dict(W=2, Hq=16, Hkv=2, E=128, S=16, lengths=[300, 40, 150], theta=5e5, dtype=torch.bfloat16),
    # ... G*S = 32: a block is four workers ...
    "dense_small_gs_bf16": dict(W=8, Hq=8, Hkv=2, E=128, S=8, lengths=[200, 20, 21, 22, 23, 24, 25, 26, 129], theta=5e5,
                                dtype=torch.bfloat16),
    # ... G*S = 256: a worker is two blocks (fp16) ...
    "dense_big_gs_f16": dict(W=2, Hq=16, Hkv=1, E=128, S=16, lengths=[260, 33, 47], theta=1e4, dtype=torch.float16),
    # ... and 192 rows: the second block is half empty; one fragment is invisible to worker 0, one is empty
    "dense_partial_block_bf16": dict(W=3, Hq=8, Hkv=2, E=128, S=16, lengths=[131, 17, 64, 0, 30], theta=5e5,
                                     dtype=torch.bfloat16,
                                     orders=[[0, 2, 4, 1], [0, 1, 4, 2], [0, 1, 2, 4]]),
}


def edge_problem(name: str, seed: int = 1234) -> Problem:
    return make_problem(name, seed=seed, **EDGE_CASES[name])


# ---- paged decode (operators hogwild_paged_sdpa / copy_to_blocks) -------------------------------------------------
PAGED_CONFIGS = {
    # 8 sequences of 16,384 keys in 16-row blocks, 32 query / 2 kv heads of size 128 (the head layout the reference's
    # paged kernel is instantiated for, src/kernels/kernel_v21.cuh:1025), one token per sequence and step
    "paged_gqa16": dict(W=8, Hq=32, Hkv=2, E=128, S=1, F=1, block_size=16, length=16384, dtype=torch.bfloat16),
}


def paged_problem(name: str = "paged_gqa16", seed: int = 0) -> dict:
    """Seeded inputs of a paged decode call: ``queries [F,W,Hq,S,E]`` (already rotated), ``locations [F,W,S]``,
    ``fragment_lengths [F]``, ``key_cache`` / ``value_cache [blocks,Hkv,block_size,E]``, ``block_table [W,max_blocks]``
    (a random permutation of the blocks), ``scale``; ``bytes`` = every visible key and value once, queries, output."""
    c = PAGED_CONFIGS[name]
    g = torch.Generator().manual_seed(1000 + seed)
    W, Hq, Hkv, E, S, F, bs, L, dtype = (c[k] for k in ("W", "Hq", "Hkv", "E", "S", "F", "block_size", "length", "dtype"))
    max_blocks = (L + bs - 1) // bs
    nblk = W * max_blocks
    kc = torch.randn(nblk, Hkv, bs, E, generator=g).to(dtype)
    vc = torch.randn(nblk, Hkv, bs, E, generator=g).to(dtype)
    table = torch.randperm(nblk, generator=g).to(torch.int32).reshape(W, max_blocks).contiguous()
    rq = torch.randn(F, W, Hq, S, E, generator=g).to(dtype)
    loc = torch.full((F, W, S), L - 1, dtype=torch.int32)
    lens = torch.full((F,), L, dtype=torch.int32)
    esz = 2 if dtype != torch.float32 else 4
    nbytes = W * Hkv * L * 2 * E * esz + rq.numel() * esz + W * Hq * S * E * esz
    return dict(name=name, queries=rq, locations=loc, fragment_lengths=lens, key_cache=kc, value_cache=vc, block_table=table,
                scale=E ** -0.5, bytes=nbytes, meta=dict(c, dtype=str(dtype).replace("torch.", "")))
