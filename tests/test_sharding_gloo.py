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
