"""Run the REFERENCE's own CUDA extension (``oracle/_ref/hogatt_ref.so``, built by ``build_oracle.build_ref_cuda``)
in a process of its own.  TEST INFRASTRUCTURE ONLY: the checker of the paged operators and a timed competitor.

It must be a separate process: the reference registers the same ``libhogatt`` operator names as this package, keeps
static device buffers and launches on the default stream.  Its launchers only take head size 128 with 16 query heads
per kv head (``src/kernels/kernel_v21.cuh:982-986,1025,1074``) and its paged bindings check nothing
(``src/binding.cu:110-181``), so every job is validated on the host first and anything else is refused here.

    python oracle/ref_cuda_runner.py check  <jobs.pt> <results.pt>
    python oracle/ref_cuda_runner.py time   --workload gqa16 --layers 32 --steps 20 --warmup 5

``check``: ``jobs.pt`` is a ``torch.save``d dict of CPU tensors, one entry per operator (``fragment``, ``paged``,
``varlen``, ``copy``); the outputs go to ``results.pt``.  ``time``: prints one JSON line with the microseconds per
``hogwild_fused`` call, layers with distinct KV called back to back, CUDA events on the default stream.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "_ref", "hogatt_ref.so")


def load():
    if not os.path.exists(LIB):
        raise SystemExit(f"{LIB} is missing (oracle/build_oracle.py builds it where a reference checkout is present)")
    torch.ops.load_library(LIB)
    return torch.ops.libhogatt


def _require(cond, what):
    if not cond:
        raise SystemExit(f"refused: {what}")


def _check_heads(Hq, Hkv, E, Ev):
    _require(E == 128 and Ev == 128 and Hq == 16 * Hkv, "the reference kernel takes head size 128 and 16 query heads per kv head only")


def _check_paged(loc, lens, kc, vc, table, W):
    nblk, Hkv, bs, E = kc.shape
    _require(vc.shape[:3] == kc.shape[:3] and table.shape[0] == W, "cache / block-table shapes")
    _require(int(table.min()) >= 0 and int(table.max()) < nblk, "block ids outside the cache")
    _require(int(lens.max()) <= table.shape[1] * bs and int(lens.min()) >= 0, "lengths beyond the block table")


def run_checks(jobs):
    ops = load()
    dev = torch.device("cuda:0")
    out = {}
    mv = lambda t: t.to(dev).contiguous()
    if "fragment" in jobs:
        j = jobs["fragment"]
        q, keys, vals = j["queries"], j["keys"], j["values"]
        W, Hq, S, E = q.shape
        _check_heads(Hq, keys[0].shape[-3], E, vals[0].shape[-1])
        F = len(keys)
        o = torch.zeros((W, Hq, S, vals[0].shape[-1]), dtype=q.dtype, device=dev)
        rq = torch.zeros((F, W, Hq, S, E), dtype=q.dtype, device=dev)
        ops.hogwild_fused(o, rq, float(j["scale"]), mv(j["locations"]), mv(q), mv(j["fragment_lengths"]),
                          [mv(k) for k in keys], [mv(v) for v in vals], mv(j["cos"]), mv(j["sin"]))
        torch.cuda.synchronize()
        out["fragment"] = {"out": o.cpu(), "rq": rq.cpu()}
    if "paged" in jobs:
        j = jobs["paged"]
        rq, kc, vc = j["queries"], j["key_cache"], j["value_cache"]
        F, W, Hq, S, E = rq.shape
        _check_heads(Hq, kc.shape[1], E, vc.shape[3])
        _check_paged(j["locations"], j["fragment_lengths"], kc, vc, j["block_table"], W)
        o = torch.zeros((W, Hq, S, vc.shape[3]), dtype=rq.dtype, device=dev)
        ops.hogwild_paged_sdpa(o, float(j["scale"]), mv(j["locations"]), mv(rq), mv(j["fragment_lengths"]), mv(kc), mv(vc),
                               mv(j["block_table"]))
        torch.cuda.synchronize()
        out["paged"] = {"out": o.cpu()}
    if "varlen" in jobs:
        j = jobs["varlen"]
        rq, kc, vc, cu = j["queries"], j["key_cache"], j["value_cache"], j["cu_seqlens_q"]
        F, total_q, Hq, E = rq.shape
        W = cu.numel() - 1
        _check_heads(Hq, kc.shape[1], E, vc.shape[3])
        _check_paged(j["locations"], j["fragment_lengths"], kc, vc, j["block_table"], W)
        _require(int(cu[0]) == 0 and int(cu[-1]) == total_q and bool((cu[1:] > cu[:-1]).all()), "cu_seqlens_q must be strictly increasing from 0")
        o = torch.zeros((total_q, Hq, vc.shape[3]), dtype=rq.dtype, device=dev)
        ops.hogwild_varlen_paged_sdpa(o, float(j["scale"]), mv(j["locations"]), mv(rq), mv(j["fragment_lengths"]), mv(kc), mv(vc),
                                      mv(j["block_table"]), mv(cu), mv(cu))
        torch.cuda.synchronize()
        out["varlen"] = {"out": o.cpu()}
    if "copy" in jobs:
        j = jobs["copy"]
        ks, vs, kc, vc, table, seq = j["key_states"], j["value_states"], j["key_cache"], j["value_cache"], j["block_table"], j["seq_lengths"]
        B, Hkv, S_new, E = ks.shape
        bs = kc.shape[2]
        _require(S_new * max(E, vs.shape[3]) <= 1024, "the reference launches S_new x max(E, Ev) threads per block")
        _require(int(table.min()) >= 0 and int(table.max()) < kc.shape[0], "block ids outside the cache")
        _require(int(seq.max()) + S_new <= table.shape[1] * bs, "appended rows beyond the block table")
        dk, dv = mv(kc), mv(vc)
        ops.copy_to_blocks(mv(ks), mv(vs), dk, dv, mv(table), mv(seq))
        torch.cuda.synchronize()
        out["copy"] = {"key_cache": dk.cpu(), "value_cache": dv.cpu()}
    return out


def run_timing(args):
    sys.path.insert(0, ROOT)
    from inference_lib_b200 import workloads as wl
    ops = load()
    dev = torch.device("cuda:0")
    if args.workload in wl.PAGED_CONFIGS:
        return run_paged_timing(args, ops, dev, wl)
    p = wl.baseline_problem(args.workload)
    _check_heads(p.Hq, p.Hkv, p.E, p.Ev)
    d = p.to(dev)
    layers = []
    for i in range(args.layers):               # every layer its own K/V memory: calls read their KV cold, as in bench.py
        layers.append(([torch.roll(k, shifts=i, dims=2) for k in d.keys], [torch.roll(v, shifts=i, dims=2) for v in d.values]))
    out = torch.zeros((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device=dev)
    rq = torch.zeros((p.F, p.W, p.Hq, p.S, p.E), dtype=p.dtype, device=dev)

    def step():
        for keys, vals in layers:
            ops.hogwild_fused(out, rq, p.scale, d.locations, d.queries, d.fragment_lengths, keys, vals, d.cos, d.sin)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.steps * args.layers)
    print(json.dumps({"impl": "reference CUDA kernel (kernel_v21, recompiled for sm_100a)", "workload": args.workload,
                      "us_per_call": round(us, 3), "value_TBps": round(p.algorithmic_bytes() / us / 1e6, 4),
                      "layers_per_step": args.layers, "steps": args.steps, "launch": "eager, default stream (the reference "
                      "copies a pointer table from host memory in every call and cannot be captured into a graph)"}), flush=True)


def run_paged_timing(args, ops, dev, wl):
    """``hogwild_paged_sdpa`` of the reference on a paged decode workload; ``--layers`` distinct caches in turn."""
    pp = wl.paged_problem(args.workload)
    rq, kc, vc, table = pp["queries"], pp["key_cache"], pp["value_cache"], pp["block_table"]
    F, W, Hq, S, E = rq.shape
    _check_heads(Hq, kc.shape[1], E, vc.shape[3])
    _check_paged(pp["locations"], pp["fragment_lengths"], kc, vc, table, W)
    d = {k: (v.to(dev).contiguous() if torch.is_tensor(v) else v) for k, v in pp.items()}
    caches = [(torch.roll(d["key_cache"], i, 2), torch.roll(d["value_cache"], i, 2)) for i in range(args.layers)]
    out = torch.zeros((W, Hq, S, vc.shape[3]), dtype=rq.dtype, device=dev)

    def step():
        for k, v in caches:
            ops.hogwild_paged_sdpa(out, float(pp["scale"]), d["locations"], d["queries"], d["fragment_lengths"], k, v,
                                   d["block_table"])

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.steps * args.layers)
    print(json.dumps({"impl": "reference CUDA paged kernel (kernel_v21, recompiled for sm_100a)", "workload": args.workload,
                      "us_per_call": round(us, 3), "value_TBps": round(pp["bytes"] / us / 1e6, 4),
                      "caches_in_turn": args.layers, "steps": args.steps, "launch": "eager, default stream"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("check")
    c.add_argument("jobs")
    c.add_argument("results")
    t = sub.add_parser("time")
    t.add_argument("--workload", default="gqa16")
    t.add_argument("--layers", type=int, default=32)
    t.add_argument("--steps", type=int, default=20)
    t.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    if args.cmd == "check":
        torch.save(run_checks(torch.load(args.jobs)), args.results)
    else:
        run_timing(args)


if __name__ == "__main__":
    main()
