"""Two GPUs: KV-head sharding with the output all-gather fused into the op (peer stores + flag
exchange) against the NCCL all-gather and the reference output.  Needs two devices; skipped
otherwise.  Ranks run as child processes, one per GPU, NVLS off."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, name, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from inference_lib_b200 import _cabi, sharded, workloads as wl
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        p = wl.baseline_problem(name) if name in wl.BASELINE_CONFIGS else wl.edge_problem(name)
        d = p.shard(rank, world).to(dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        out_local = torch.empty((d.W, d.Hq, d.S, d.Ev), dtype=d.dtype, device=dev)
        bp = _cabi.bind(out=out_local, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values,
                        scale=d.scale, fragment_lengths=d.fragment_lengths, cos=d.cos, sin=d.sin, status=status)
        stream = torch.cuda.current_stream(dev).cuda_stream
        _cabi.attach_workspace(bp, dev, stream)
        # (1) NCCL baseline
        assert _cabi.launch(bp, stream) == 0
        nccl_full = sharded.gather_heads(out_local, world)
        # (2) fused gather, three calls over two alternating slots
        po = sharded.PeerOutputs(dist.group.WORLD, world, rank, 2, (p.W, p.Hq, p.S, p.Ev), p.dtype, dev)
        fused = []
        for call in range(3):
            slot = call % 2
            peers = po.peers(slot)
            rc = _cabi.launch_gather(bp, peers, stream)
            assert rc == 0, _cabi.status_string(rc)
            torch.cuda.synchronize(dev)
            dist.barrier()                      # nobody reuses a slot while a peer may still read it
            fused.append(po.output(slot).clone())
        q.put((rank, nccl_full.float().cpu().numpy(), [f.float().cpu().numpy() for f in fused], int(status.item())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", ["cfg2", "gqa5_bf16", "causal_chunk_bf16"])
def test_fused_gather_equals_nccl_gather_on_two_gpus(golden, name):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from tests.gpu_util import check_against
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, name, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    ref = golden[f"{name}/out"]
    for rank, nccl_full, fused, status in results:
        assert status == 0
        check_against(torch.from_numpy(nccl_full), ref, torch.bfloat16, what=f"{name} nccl rank {rank}")
        for f in fused:
            assert np.array_equal(f, nccl_full), "fused gather must deliver exactly what the NCCL gather delivers"
