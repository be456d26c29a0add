"""A bounded wait inside a kernel that actually runs out: the kernel gives up, says so in the caller's status word and
returns; nothing hangs, nothing faults, and the next call is fine.

The failure is made on the host side of the protocol: a fused-gather call for a world of two ranks is issued on ONE
GPU, with the second rank's output and flag buffers being ordinary local allocations that no second rank ever writes
to.  This rank's rows are delivered everywhere, its own count is published, and the exchange kernel then watches a
flag that nothing sets -- for HOGATT_WAIT_LIMIT_MS (read once per process, hence the child) instead of a second.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))

SCRIPT = r"""
import sys, time, numpy as np, torch
sys.path.insert(0, {root!r})
from inference_lib_b200 import _cabi, workloads as wl
dev = torch.device("cuda:0")
golden = np.load({root!r} + "/tests/golden/reference_outputs.npz")
for name, kernel in (("cfg2", _cabi.KERNEL_AUTO), ("ragged_bf16", _cabi.KERNEL_MMA), ("gqa5_bf16", _cabi.KERNEL_MMA_CLUSTER)):
    p = wl.baseline_problem(name) if name in wl.BASELINE_CONFIGS else wl.edge_problem(name)
    world = 2
    d = p.shard(0, world).to(dev)                      # rank 0's kv heads
    full = [torch.zeros((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device=dev) for _ in range(world)]
    flags = [torch.zeros(world + 1, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out_local = torch.empty((d.W, d.Hq, d.S, d.Ev), dtype=p.dtype, device=dev)     # gives the shard's dims; not written by a gather call
    bp = _cabi.bind(out=out_local, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values, scale=d.scale,
                    fragment_lengths=d.fragment_lengths, cos=d.cos, sin=d.sin, status=status, kernel=kernel)
    _cabi.attach_workspace(bp, dev)
    peers = _cabi.Peers()
    peers.world, peers.rank = world, 0
    for r in range(world):
        peers.out_full[r], peers.flags[r] = full[r].data_ptr(), flags[r].data_ptr()
    t0 = time.perf_counter()
    rc = _cabi.launch_gather(bp, peers, torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert rc == 0, _cabi.status_string(rc)
    assert int(status.item()) == 32, int(status.item())        # STATUS_WAIT_PEER_TIMEOUT, and only that
    assert 0.04 < dt < 2.0, dt                                   # it waited for the shortened limit, not for a second
    hq = p.Hq // world
    ref = golden[name + "/out"][:, :hq]
    for r in range(world):                                       # this rank's rows were delivered to both outputs
        got = full[r][:, :hq].float().cpu().numpy()
        assert np.abs(got - ref).max() <= 2e-2, (name, r)
        assert (full[r][:, hq:] == 0).all()
    assert flags[0].tolist()[:3] == [1, 0, 1] and flags[1].tolist()[0] == 1, (flags[0].tolist(), flags[1].tolist())
    # the context is intact: an ordinary call right after it
    status.zero_()
    out = torch.empty((d.W, d.Hq, d.S, d.Ev), dtype=p.dtype, device=dev)
    bp2 = _cabi.bind(out=out, queries=d.queries, locations=d.locations, keys=d.keys, values=d.values, scale=d.scale,
                     fragment_lengths=d.fragment_lengths, cos=d.cos, sin=d.sin, status=status)
    _cabi.attach_workspace(bp2, dev)
    assert _cabi.launch(bp2, torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and np.abs(out.float().cpu().numpy() - ref).max() <= 2e-2
print("WAIT_LIMIT_OK")
"""


def test_a_peer_that_never_reports_makes_the_wait_give_up():
    env = dict(os.environ, HOGATT_WAIT_LIMIT_MS="60")
    res = subprocess.run([sys.executable, "-c", SCRIPT.format(root=ROOT)], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "WAIT_LIMIT_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
