"""KV-head sharding on CPU ranks (gloo, world size 2): per-rank results, all-gathered, equal the
unsharded result.  The per-rank compute here is the oracle; what is under test is the host logic
(slicing, gather layout), which is what the GPU path uses unchanged."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from inference_lib_b200 import sharded
from inference_lib_b200 import workloads as wl


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, name, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import hogwild_oracle as oracle
        torch.set_num_threads(2)
        p = wl.edge_problem(name)
        qs, ks, vs = sharded.shard_inputs(p.queries, p.keys, p.values, rank, world)
        # same shard through the Problem helper
        ps = p.shard(rank, world)
        assert torch.equal(ps.queries, qs) and all(torch.equal(a, b) for a, b in zip(ps.keys, ks))
        local, _ = oracle.fused(qs, p.cos, p.sin, p.locations, ks, vs, p.scale)
        full = sharded.gather_heads(local, world)
        q.put((rank, full.numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", ["gqa5_bf16", "causal_chunk_f32"])
def test_two_cpu_ranks_reassemble_the_unsharded_result(golden, name):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, name, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    ref = golden[f"{name}/out"]
    for r in range(world):
        assert results[r].shape == ref.shape
        assert np.abs(results[r] - ref).max() <= 3e-5, "every rank must hold the full output"


def test_head_slices_cover_all_heads_once():
    for Hq, Hkv, world in [(32, 8, 1), (32, 8, 2), (32, 8, 8), (40, 8, 4), (64, 8, 8)]:
        qcover, kcover = [], []
        for r in range(world):
            qs, ks = sharded.head_slices(Hq, Hkv, r, world)
            qcover += list(range(Hq))[qs]
            kcover += list(range(Hkv))[ks]
        assert qcover == list(range(Hq)) and kcover == list(range(Hkv))
    with pytest.raises(ValueError):
        sharded.head_slices(32, 8, 0, 3)


# ---- the attention layer with its heads sharded (inference_lib_b200.module.HogwildAttentionTP) --------------------
def _layer_problem():
    W, S, hidden, Hq, Hkv, D = 3, 2, 96, 8, 4, 16
    g = torch.Generator().manual_seed(21)
    lens = [11, 4, 0, 7]
    keys = [torch.randn(Hkv, n + S, D, generator=g) for n in lens]
    values = [torch.randn(Hkv, n + S, D, generator=g) for n in lens]
    order = [[0] + [1 + o for o in range(W) if o != w] + [1 + w] for w in range(W)]
    hidden_states = torch.randn(W, S, hidden, generator=g)
    return W, S, hidden, Hq, Hkv, D, lens, keys, values, order, hidden_states


def _layer_rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from inference_lib_b200 import module as mod
        from inference_lib_b200.cache import CacheStructure, FragmentCache
        from oracle import hogwild_cache_oracle as oc
        from oracle import hogwild_oracle as oracle
        torch.set_num_threads(2)
        W, S, hidden, Hq, Hkv, D, lens, keys, values, order, h = _layer_problem()
        torch.manual_seed(4)
        full = mod.HogwildAttention(hidden, Hq, Hkv, D, layer_idx=0, dtype=torch.float32, device="cpu")
        loc = oc.step_locations(np.array(order, dtype=np.int32), [n + S for n in lens], S)
        inv_freq = (1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).numpy()
        cos, sin = oc.rotary_tables(loc, inv_freq, 1.0, torch.float32)

        class StubCache(FragmentCache):
            """Hands out fixed fragments (the rank's kv heads of them); the new keys and values are ignored."""
            def __init__(self, heads):
                self.heads, self.seen = heads, None

            def update(self, k, v, layer, kcos, ksin, new_rows=None):
                self.seen = (tuple(k.shape), tuple(v.shape))
                return CacheStructure(keys=[t[self.heads] for t in keys], values=[t[self.heads] for t in values],
                                      frags=None, cos=cos, sin=sin, loc=torch.from_numpy(loc))

        def attend(self, qq, cs):                       # the op, restated: what runs on a GPU is libhogatt
            out, _ = oracle.fused(qq.contiguous(), cs.cos, cs.sin, cs.loc, [t[None] for t in cs.keys],
                                  [t[None] for t in cs.values], self.scaling)
            return out

        tp = mod.TensorParallel(rank, world)
        layer = mod.HogwildAttentionTP.from_full(full, tp)
        layer._attend_local = attend.__get__(layer)
        _, ks = sharded.head_slices(Hq, Hkv, rank, world)
        cache = StubCache(ks)
        pos = torch.zeros(W, S, dtype=torch.long)
        tables = (torch.ones(W, S, D), torch.zeros(W, S, D))
        with torch.no_grad():
            y, _ = layer(h, tables, None, cache, position_ids=pos)
            # the unsharded layer on the same inputs
            full._attend = attend.__get__(full)
            y_full, _ = full(h, tables, None, StubCache(slice(0, Hkv)), position_ids=pos)
        q.put((rank, y.numpy(), y_full.numpy(), cache.seen, [tuple(p.shape) for p in layer.parameters()]))
    finally:
        dist.destroy_process_group()


def test_sharded_attention_layer_on_two_cpu_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_layer_rank_main, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    W, S, hidden, Hq, Hkv, D = _layer_problem()[:6]
    for rank, y, y_full, seen, shapes in results:
        assert y.shape == (W, S, hidden)
        assert np.abs(y - y_full).max() <= 2e-5, "every rank must produce the unsharded layer's output"
        assert seen == ((W, Hkv // world, S, D), (W, Hkv // world, S, D)), "the cache gets this rank's kv heads only"
        # q rows halved, k / v rows halved, o_proj replicated
        assert (Hq // world * D, hidden) in shapes and (Hkv // world * D, hidden) in shapes and (hidden, Hq * D) in shapes
