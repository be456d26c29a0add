"""CPU oracle for the Hogwild! attention op.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch CPU ops, the algorithm of the reference's own
PyTorch path.  It is the checker the CUDA kernels are compared against; nothing in the
shipped package imports it, and it must never be used as a fallback for the CUDA path.
Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark use it.

Parity pin: the reference ships no golden vectors or tests for this path, so the oracle is
pinned against outputs of the reference itself.  ``tests/golden/make_golden.py`` imports the
reference's ``python/hogwild/attention.py``, runs
``hogwild_sdpa_pt`` / ``apply_rotary_pos_emb`` on the seeded problems of
``inference_lib_b200.workloads`` and stores the results under ``tests/golden/``;
``tests/test_oracle.py`` checks every function below against those files.  The paged
variants have no Python/CPU implementation in the reference at all: their oracle is by
construction (gather the blocks into contiguous fragments, then the function below); it is
pinned on the GPU instead, against the reference's own CUDA kernels recompiled for sm_100a
at the one head layout they accept (``tests/test_gpu_reference_cuda.py``,
``oracle/ref_cuda_runner.py``).

Which reference lines each function follows:

* ``rotate_half`` / ``apply_rope``      -> ``python/hogwild/attention.py:77-90``
* ``rope_rows`` (scalar loops, numpy)   -> ``src/q_rope.h:3-35`` (``rope_cpu``)
* ``sdpa``                              -> ``python/hogwild/attention.py:38-67`` (``hogwild_sdpa_pt``)
* ``fused``                             -> ``python/hogwild/attention.py:320-323`` (eager branch)
* ``paged_*``                           -> addressing of ``src/kernels/kernel_v21.cuh:402-411``,
                                           ``:726-757`` and ``src/cache.cuh:6-49``
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch


# ---------------------------------------------------------------------------------------
# RoPE
# ---------------------------------------------------------------------------------------
def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(x1, x2) -> (-x2, x1) on the last axis (``attention.py:77-81``)."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, unsqueeze_dim: int = 1) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin`` on the first ``cos.shape[-1]`` channels, rest passed through,
    computed in the promoted dtype and rounded back to ``x.dtype`` (``attention.py:84-90``)."""
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    r = cos.shape[-1]
    head, tail = x[..., :r], x[..., r:]
    rotated = (head * cos) + (rotate_half(head) * sin)
    return torch.cat((rotated, tail), dim=-1).to(x.dtype)


def rotate_queries(queries: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``[W,Hq,S,E]`` un-rotated queries -> ``[F,W,Hq,S,E]``, one rotation per fragment
    (the tile + rope of ``attention.py:321-322``; also what the ``hogwild_rope`` op returns)."""
    F = cos.shape[0]
    tiled = queries.unsqueeze(0).expand(F, *queries.shape)
    return apply_rope(tiled, cos, sin, unsqueeze_dim=2)


def rope_rows(queries: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Scalar-loop restatement of ``rope_cpu`` (``src/q_rope.h:3-35``) on fp32 numpy arrays.

    ``queries [W,Hq,S,E]``, ``cos/sin [F,W,S,R]`` -> ``[F,W,Hq,S,E]``.  The second half of a
    pair reads the table at its own index ``e + R/2`` (``q_rope.h:23-24``).  Small inputs only.
    """
    W, Hq, S, E = queries.shape
    F, _, _, R = cos.shape
    out = np.empty((F, W, Hq, S, E), dtype=np.float32)
    half = R // 2
    for f in range(F):
        for w in range(W):
            for h in range(Hq):
                for s in range(S):
                    q = queries[w, h, s]
                    c, sn = cos[f, w, s], sin[f, w, s]
                    for e in range(half):
                        x1, x2 = np.float32(q[e]), np.float32(q[e + half])
                        out[f, w, h, s, e] = np.float32(x1 * c[e]) - np.float32(x2 * sn[e])
                        out[f, w, h, s, e + half] = np.float32(x2 * c[e + half]) + np.float32(x1 * sn[e + half])
                    out[f, w, h, s, R:] = q[R:]
    return out


# ---------------------------------------------------------------------------------------
# Attention over fragments
# ---------------------------------------------------------------------------------------
def sdpa(rotated_queries: torch.Tensor, locations: torch.Tensor, keys: Sequence[torch.Tensor],
         values: Sequence[torch.Tensor], scale: float, return_intermediate: bool = False):
    """One softmax over the concatenation of all fragments (``attention.py:38-67``).

    ``rotated_queries [F,W,Hq,S,E]``; ``keys[f] [1,Hkv,L_f,E]`` (or ``[Hkv,L_f,E]``).  Scores and the
    weighted sum are fp32.  The result is fp32 ``[W,Hq,S,Ev]``; a row that sees no key at all is
    NaN here (softmax over nothing), exactly as in the reference -- the CUDA op defines such rows
    as zero, so callers compare them separately.
    """
    F, W, Hq, S, E = rotated_queries.shape
    scores, vals = [], []
    for f in range(F):
        k = keys[f][0] if keys[f].dim() == 4 else keys[f]                    # [Hkv, L, E]
        v = values[f][0] if values[f].dim() == 4 else values[f]              # [Hkv, L, Ev]
        Hkv, L = k.shape[0], k.shape[1]
        G = Hq // Hkv
        # grouped-query heads: query head h reads kv head h // G  (repeat_interleave, :47-48)
        q = rotated_queries[f].to(torch.float32).reshape(W, Hkv, G, S, E)
        kt = k.to(torch.float32).transpose(-1, -2)                           # [Hkv, E, L]
        att = torch.matmul(q, kt[None, :, None])                             # [W,Hkv,G,S,L]
        key_pos = torch.arange(L, dtype=torch.int32)
        hidden = key_pos[None, None, None, None, :] > locations[f][:, None, None, :, None]   # (:50-54)
        att = att.masked_fill(hidden, float("-inf"))
        scores.append(att)
        vals.append(v.to(torch.float32))
    qk = torch.cat(scores, dim=-1)                                           # [W,Hkv,G,S,sum L]
    vv = torch.cat(vals, dim=-2)                                             # [Hkv, sum L, Ev]
    att = torch.softmax(scale * qk, dim=-1)
    out = torch.matmul(att, vv[None, :, None])                               # [W,Hkv,G,S,Ev]
    out = out.reshape(W, Hq, S, -1)
    if return_intermediate:
        return out, qk.reshape(W, Hq, S, -1), att.reshape(W, Hq, S, -1)
    return out


def fused(queries: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, locations: torch.Tensor,
          keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor], scale: float):
    """Per-fragment query rotation followed by ``sdpa`` -- the eager branch of the reference's
    attention module (``attention.py:320-323``).  Returns ``(out fp32 [W,Hq,S,Ev], rq [F,W,Hq,S,E])``."""
    rq = rotate_queries(queries, cos, sin)
    return sdpa(rq, locations, keys, values, scale), rq


def blind_rows(locations: torch.Tensor, fragment_lengths: torch.Tensor) -> torch.Tensor:
    """``[W,S]`` bool: rows that can see no key of any fragment (oracle gives NaN, the op gives 0)."""
    sees = (locations >= 0) & (fragment_lengths[:, None, None] > 0)
    return ~sees.any(dim=0)


# ---------------------------------------------------------------------------------------
# Paged variants (no reference CPU path exists; oracle by construction)
# ---------------------------------------------------------------------------------------
def gather_pages(cache: torch.Tensor, block_table_row: torch.Tensor, length: int) -> torch.Tensor:
    """``cache [NumBlocks,Hkv,bs,D]`` + one sequence's block list -> contiguous ``[1,Hkv,length,D]``
    (address rule of ``kernel_v21.cuh:405-411``: token ``l`` lives in block ``table[l // bs]`` at
    row ``l % bs``)."""
    bs = cache.shape[2]
    nblk = (length + bs - 1) // bs
    blocks = cache[block_table_row[:nblk].long()]            # [nblk, Hkv, bs, D]
    seq = blocks.permute(1, 0, 2, 3).reshape(cache.shape[1], nblk * bs, cache.shape[3])
    return seq[None, :, :length]


def paged_sdpa(rotated_queries: torch.Tensor, locations: torch.Tensor, fragment_lengths: torch.Tensor,
               key_cache: torch.Tensor, value_cache: torch.Tensor, block_table: torch.Tensor, scale: float):
    """Oracle for ``hogwild_paged_sdpa``.  In the reference kernel the block table is indexed by the
    worker only (``kernel_v21.cuh:405``), so each worker attends to *its own* paged sequence and
    every fragment index ``f`` re-reads that same sequence with its own query rotation, location
    and length.  Worker by worker this is ``sdpa`` with W=1."""
    F, W, Hq, S, E = rotated_queries.shape
    outs = []
    for w in range(W):
        ks, vs = [], []
        for f in range(F):
            L = int(fragment_lengths[f])
            ks.append(gather_pages(key_cache, block_table[w], L))
            vs.append(gather_pages(value_cache, block_table[w], L))
        outs.append(sdpa(rotated_queries[:, w:w + 1], locations[:, w:w + 1], ks, vs, scale))
    return torch.cat(outs, dim=0)


def varlen_paged_sdpa(rotated_queries: torch.Tensor, locations: torch.Tensor, fragment_lengths: torch.Tensor,
                      key_cache: torch.Tensor, value_cache: torch.Tensor, block_table: torch.Tensor,
                      cu_seqlens_q: torch.Tensor, scale: float):
    """Oracle for ``hogwild_varlen_paged_sdpa``: packed queries ``[F,total_q,Hq,E]``, locations
    ``[F,total_q]``, lengths ``[F,W]`` (``kernel_v21.cuh:695,726``); result ``[total_q,Hq,Ev]``."""
    F, total_q, Hq, E = rotated_queries.shape
    W = cu_seqlens_q.numel() - 1
    out = None
    for w in range(W):
        a, b = int(cu_seqlens_q[w]), int(cu_seqlens_q[w + 1])
        if a == b:
            continue
        ks, vs = [], []
        for f in range(F):
            L = int(fragment_lengths[f, w])
            ks.append(gather_pages(key_cache, block_table[w], L))
            vs.append(gather_pages(value_cache, block_table[w], L))
        q = rotated_queries[:, a:b].permute(0, 2, 1, 3)[:, None]            # [F,1,Hq,s,E]
        loc = locations[:, a:b][:, None]                                    # [F,1,s]
        o = sdpa(q, loc, ks, vs, scale)[0].permute(1, 0, 2)                  # [s,Hq,Ev]
        if out is None:
            out = torch.zeros(total_q, Hq, o.shape[-1], dtype=torch.float32)
        out[a:b] = o
    return out


def copy_to_blocks(key_states: torch.Tensor, value_states: torch.Tensor, key_cache: torch.Tensor,
                   value_cache: torch.Tensor, block_table: torch.Tensor, seq_lengths: torch.Tensor):
    """Oracle for ``copy_to_blocks`` (``src/cache.cuh:6-49``): append ``S_new`` rows per (batch, kv head)
    at positions ``seq_lengths[b] + t`` through the block table.  In place, python loops, small only."""
    B, Hkv, S_new, _ = key_states.shape
    bs = key_cache.shape[2]
    for b in range(B):
        for t in range(S_new):
            pos = int(seq_lengths[b]) + t
            blk = int(block_table[b, pos // bs])
            key_cache[blk, :, pos % bs] = key_states[b, :, t]
            value_cache[blk, :, pos % bs] = value_states[b, :, t]
    return key_cache, value_cache
