#!/usr/bin/env python
"""Benchmark of the Hogwild! fragmented-KV attention op on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload target|cfg2|cfg3|cfg4|cfg5] [--impl reference]

One *step* is one decode step's worth of attention: ``--layers`` (default 32) calls of the fused
RoPE + attention op, one per transformer layer, each layer with its own KV fragments.  The layers'
KV sets together (2 GiB for the default workload) are far larger than the 126 MB L2, so every call
reads its KV cold from HBM.  ``value`` is the achieved algorithmic bandwidth of the whole job
(KV once + Q + O bytes of every call / time); ``us_per_call`` is the time of one call.

With ``--gpus N`` (launched under torchrun, one rank per GPU) the same workload is sharded by KV
head; every rank computes its heads and the outputs are all-gathered over NCCL.  Timing is on the
device (CUDA events on the launching stream), max over ranks.

``--impl reference`` times the reference's CPU algorithm (its PyTorch path, restated in
``oracle/``) on the host cores for the same workload, metric and unit.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from inference_lib_b200 import workloads as wl  # noqa: E402

METRIC = "hogwild attn achieved HBM TB/s (us/call in us_per_call)"
UNIT = "TB/s"
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum of the attention kernel divided by its algorithmic bytes, per workload,
# from the ncu captures summarised under profiles/ (mma_attention_kernel_target.md, ..._cfg2_cfg3_cfg4.md).  Only a
# single-GPU run of a captured shape at its full length reports `traffic`; everything else reports null.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {"target": 1.0072, "cfg2": 1.0017, "cfg3": 1.0191, "cfg4": 1.0082}
FALLBACK_HBM_GBS = 6650.0


FALLBACK_BF16_TFLOPS_SUSTAINED = 1400.0


def measured_peak(key="hbm_gbs", fallback=FALLBACK_HBM_GBS):
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)[key]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return fallback, "fallback"


def job_config(args, meta, world, fused_gather=True, graph=True):
    """What the job is, identical for both arms (the reference arm times the same workload on the host cores)."""
    lengths = meta["lengths"]
    sz = 4 if meta["dtype"] == "float32" else 2
    kv_bytes = meta["Hkv"] * sum(lengths) * (meta["E"] + meta["Ev"]) * sz
    return {"workload": args.workload, **{k: v for k, v in meta.items() if k not in ("seed",)},
            "layers_per_step": args.layers, "kv_bytes_resident": int(kv_bytes * args.layers),
            "l2": "inputs larger than L2 (one distinct KV set per layer); isolated call uses an L2 flush",
            "parallelism": (f"kv-head shard x{world}, output all-gather " +
                            ("fused into the merge step (peer stores)" if fused_gather else "by NCCL")) if world > 1
                           else "single GPU",
            "cuda_graph": graph}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# workload
# ------------------------------------------------------------------------------------------------
def layer_problems(name: str, layers: int, rank: int, world: int, device):
    """``layers`` device-resident problems.  Layer 0 is the seeded problem itself; the other layers
    reuse its queries and metadata with their own KV memory (layer i's KV = layer 0's values rolled
    by i rows), so the layers occupy distinct HBM without spending minutes in the CPU generator."""
    base = wl.baseline_problem(name)
    if LENGTH_SCALE != 1.0:       # context-length sweeps: same heads and workers, every fragment scaled
        lengths = [max(base.S, int(l * LENGTH_SCALE)) for l in wl.BASELINE_CONFIGS[name]["lengths"]]
        base = wl.baseline_problem(name, lengths=lengths)
    if world > 1:
        base = base.shard(rank, world)
    elif EMULATE_SHARD > 1:       # what rank 0 of an N-way kv-head split computes, alone on this GPU (no gather)
        base = base.shard(0, EMULATE_SHARD)
    d0 = base.to(device)
    probs = [d0]
    for i in range(1, layers):
        keys = [torch.roll(k, shifts=i, dims=2) for k in d0.keys]
        vals = [torch.roll(v, shifts=i, dims=2) for v in d0.values]
        probs.append(wl.Problem(**{**d0.__dict__, "keys": keys, "values": vals}))
    return base, probs


KERNEL_CHOICE = 0          # hogatt_kernel_choice passed to every call (--kernel)
LENGTH_SCALE = 1.0         # --scale-lengths
EMULATE_SHARD = 1          # --emulate-shard
HOST_PLAN = True           # --plan: the host passes the fragment lengths it knows (the tensors' row counts)
STABLE_FRAGMENTS = 1       # --stable: the shared prompt (fragment 0) is not written during a decode step


def parity_against_stored_reference(name: str, out: torch.Tensor):
    """Layer 0 of every workload is the seeded problem itself: compare the output every rank ends up with against
    the reference's own output for that problem (``tests/golden``; tolerance of the parity gate: max-abs <= 2e-2,
    mean-abs <= 2e-3 for 16-bit outputs).  Returns None for length-scaled or otherwise unstored problems."""
    import numpy as np
    if LENGTH_SCALE != 1.0 or EMULATE_SHARD > 1:
        return None
    try:
        if name == "cfg5":
            ref = np.load(os.path.join(ROOT, "tests", "golden", "cfg5_g0_full.npz"))["out"]
        else:
            ref = np.load(os.path.join(ROOT, "tests", "golden", "reference_outputs.npz"))[f"{name}/out"]
    except Exception:
        return None
    got = out.detach().float().cpu().numpy()
    if got.shape != ref.shape:
        return {"checked": True, "ok": False, "why": f"shape {got.shape} != {ref.shape}"}
    diff = np.abs(got - ref)
    mx, mean = float(diff.max()), float(diff.mean())
    return {"checked": True, "ok": bool(np.isfinite(got).all() and mx <= 2e-2 and mean <= 2e-3), "max_abs": round(mx, 6),
            "mean_abs": round(mean, 7), "against": "reference output stored in tests/golden (layer 0 of the step)"}


class CabiCall:
    """One pre-bound C-ABI call (pointers fixed, so the step can be captured into a CUDA graph)."""

    def __init__(self, p: wl.Problem, device, workspace=None, want_rq=True):
        from inference_lib_b200 import _cabi
        self._cabi = _cabi
        self.out = torch.empty((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device=device)
        self.rq = torch.empty((p.F, p.W, p.Hq, p.S, p.E), dtype=p.dtype, device=device) if want_rq else None
        self.bp = _cabi.bind(out=self.out, queries=p.queries, locations=p.locations, keys=p.keys, values=p.values,
                             scale=p.scale, fragment_lengths=p.fragment_lengths, cos=p.cos, sin=p.sin, rq=self.rq,
                             kernel=KERNEL_CHOICE, host_lengths="rows" if HOST_PLAN else None,
                             stable_fragments=STABLE_FRAGMENTS)
        # 1 when the attention kernel merges its split-K partials itself, 2 when merge_kernel follows
        self.kernels_per_call = _cabi.launch_shape(self.bp)["kernels_per_call"]
        need = _cabi.workspace_bytes(self.bp)
        if need == 0:
            raise RuntimeError("libhogatt_b200 refused the workload")
        self.ws = workspace if workspace is not None else torch.empty(need + 256, dtype=torch.uint8, device=device)
        off = (-self.ws.data_ptr()) % 256
        self.bp.struct.workspace, self.bp.struct.workspace_bytes = self.ws.data_ptr() + off, need

    def launch(self, stream: int):
        rc = self._cabi.launch(self.bp, stream)
        if rc != 0:
            raise RuntimeError(f"hogatt launch failed: {self._cabi.status_string(rc)}")

    def launch_gather(self, peers, stream: int):
        rc = self._cabi.launch_gather(self.bp, peers, stream)
        if rc != 0:
            raise RuntimeError(f"hogatt gather launch failed: {self._cabi.status_string(rc)}")


def time_steps(step_fn, steps: int, warmup: int, barrier):
    torch.cuda.synchronize()
    barrier()                     # ranks enter the warm-up together (their kernels wait for each other, bounded)
    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    # one event per step boundary: the total is what the line reports, the per-step spread goes beside it
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        step_fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    barrier()
    per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(steps))
    pick = lambda q: per[min(len(per) - 1, int(q * len(per)))]
    STEP_SPREAD.update(median_ms=round(pick(0.5), 5), p10_ms=round(pick(0.1), 5), p90_ms=round(pick(0.9), 5))
    return ev[0].elapsed_time(ev[steps]) / 1e3      # seconds


STEP_SPREAD = {}       # per-step times of the most recent time_steps() on this rank


def run_ours(args):
    rank = int(os.environ.get("RANK", 0)); world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback for the op")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    barrier = (lambda: dist.barrier()) if dist else (lambda: None)

    from inference_lib_b200 import _build
    _build.build_all()
    stream = torch.cuda.Stream(device)

    def measure(workload, layers, steps, warmup, primary):
        """Build `layers` device-resident problems of a workload, time `steps` steps (gather included at
        N > 1), plus the attention-only leg at N > 1 and, for the primary workload, the isolated cold call."""
        full, probs = layer_problems(workload, layers, rank, world, device)
        whole = wl.baseline_problem(workload) if world > 1 else full
        bytes_per_call = whole.algorithmic_bytes()                   # whole job, all ranks
        calls = [CabiCall(p, device, want_rq=not args.no_rq) for p in probs]

        gathered = peer_out = peer_tables = None
        fused_gather = bool(dist) and args.gather == "fused"
        if dist:
            from inference_lib_b200 import sharded
            if fused_gather:
                # one full-size output + flag array per layer in symmetric memory; the merge step of every rank
                # stores its heads into all ranks' outputs over NVLink, no collective call in the step
                ok = torch.ones(1, dtype=torch.int32, device=device)
                try:
                    peer_out = sharded.PeerOutputs(dist.group.WORLD, world, rank, len(calls),
                                                   (whole.W, whole.Hq, whole.S, whole.Ev), whole.dtype, device)
                    peer_tables = [peer_out.peers(i) for i in range(len(calls))]
                except Exception as exc:                  # noqa: BLE001  (no peer mapping on this box: use NCCL)
                    print(f"[bench] rank {rank}: symmetric memory unavailable ({exc}); gathering with NCCL", file=sys.stderr)
                    ok.zero_()
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)       # all ranks take the same path
                fused_gather = bool(int(ok.item()))
            if not fused_gather:
                gathered = [torch.empty((world,) + tuple(c.out.shape), dtype=c.out.dtype, device=device) for c in calls]

        def step_body(sid):
            for i, c in enumerate(calls):
                if fused_gather:
                    c.launch_gather(peer_tables[i], sid)
                else:
                    c.launch(sid)
                    if dist:       # every rank ends up with the full [W,Hq,S,Ev] output of the layer
                        sharded.gather_heads(c.out, world, gather_buffer=gathered[i])

        launches_per_step = sum(c.kernels_per_call + (1 if fused_gather else 0) for c in calls)

        def capture(body):
            """The step is launch-bound from Python, so it is replayed as a CUDA graph (only steps without
            collectives); falls back to eager launches if capture is refused."""
            if args.no_graph:
                return None
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    body(torch.cuda.current_stream().cuda_stream)
                return g
            except Exception as exc:                      # noqa: BLE001
                if rank == 0:
                    print(f"[bench] graph capture failed, running eagerly: {exc}", file=sys.stderr)
                torch.cuda.synchronize()
                return None

        graph = None
        with torch.cuda.stream(stream):
            step_body(stream.cuda_stream)
            torch.cuda.synchronize()
            barrier()
            # what this rank holds for layer 0 after one step (at N > 1: the gathered, full-size output)
            if fused_gather:
                first_out = peer_out.output(0)
            elif dist:
                first_out = gathered[0].permute(1, 0, 2, 3, 4).reshape(whole.W, whole.Hq, whole.S, whole.Ev)
            else:
                first_out = calls[0].out
            parity = parity_against_stored_reference(workload, first_out)
            if dist and parity is not None:          # every rank must hold the right answer
                flag = torch.tensor([1 if parity["ok"] else 0], dtype=torch.int32, device=device)
                worst = torch.tensor([parity.get("max_abs", 1e9)], dtype=torch.float64, device=device)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                dist.all_reduce(worst, op=dist.ReduceOp.MAX)
                parity.update(ok=bool(int(flag.item())), max_abs=round(float(worst.item()), 6), ranks_checked=world)
            # NCCL collectives stay outside graphs: capturing them stalled this benchmark on a 2-GPU box
            graph = None if (dist and not fused_gather) else capture(step_body)

            def step():
                if graph is not None:
                    graph.replay()
                else:
                    step_body(torch.cuda.current_stream().cuda_stream)

            sampler = ClockSampler(local)
            if rank == 0 and primary:
                sampler.start()
            secs = time_steps(step, steps, warmup, barrier)
            spread = dict(STEP_SPREAD)
            if primary:
                # The timed region lasts 0.1-0.2 s, two samples of the 100 ms clock query at most: every rank keeps
                # replaying the same steps, untimed, until 0.7 s of this load have been sampled.
                per_step = torch.tensor([secs / steps], dtype=torch.float64, device=device)
                if dist:
                    dist.all_reduce(per_step, op=dist.ReduceOp.MAX)
                for _ in range(int(min(max(0.0, 0.7 - secs) / float(per_step.item()), 20000))):
                    step()
                torch.cuda.synchronize()
                barrier()
            clocks = sampler.stop() if (rank == 0 and primary) else None
            if clocks is not None:
                clocks["window"] = "warm-up, the timed steps and an untimed continuation of the same steps (0.7 s of load in all)"

            # attention-only time at N > 1 (no gather), for the split the scaling discussion needs
            secs_attn = None
            if dist:
                def attn_body(sid):
                    for c in calls:
                        c.launch(sid)
                g_attn = capture(attn_body)

                def step_attn():
                    if g_attn is not None:
                        g_attn.replay()
                    else:
                        attn_body(torch.cuda.current_stream().cuda_stream)
                secs_attn = time_steps(step_attn, steps, warmup, barrier)

            # isolated, cold call: one launch between events, L2 flushed by a 256 MiB write before it
            flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
            iso = []
            for i in range(0 if (args.no_isolated or not primary) else 12):
                flush.fill_(i)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); calls[i % len(calls)].launch(torch.cuda.current_stream().cuda_stream); e1.record()
                torch.cuda.synchronize()
                iso.append(e0.elapsed_time(e1) * 1e3)
            iso_us = statistics.median(iso[2:]) if iso else float("nan")

        t = torch.tensor([secs, secs_attn or 0.0], dtype=torch.float64, device=device)
        if dist:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res = dict(secs=float(t[0]), secs_attn=float(t[1]) or None, n_calls=steps * len(calls), bytes_per_call=bytes_per_call,
                   launches_per_step=launches_per_step, graph=graph is not None, fused_gather=fused_gather, iso_us=iso_us,
                   clocks=clocks, full=full, layers=len(calls), kv_resident=int(sum(p.algorithmic_bytes() for p in probs)),
                   parity=parity, spread=spread)
        del calls, probs, graph, gathered, peer_out, peer_tables
        torch.cuda.empty_cache()
        return res

    m = measure(args.workload, args.layers, args.steps, args.warmup, True)
    secs, secs_attn, n_calls, bytes_per_call = m["secs"], m["secs_attn"], m["n_calls"], m["bytes_per_call"]
    full, iso_us, clocks, graph_used, fused_gather = m["full"], m["iso_us"], m["clocks"], m["graph"], m["fused_gather"]
    launches_per_step = m["launches_per_step"]
    extra = None
    if not args.no_extra:
        # every other named shape beside the headline one, each with its own roofline fraction: the HBM-bound ones
        # against the measured copy bandwidth, the dense chunked one (cfg5: its four groups are the four calls of a
        # step) against the measured sustained bf16 tensor throughput
        hbm_peak, _ = measured_peak()
        tf_peak, _ = measured_peak("bf16_tflops_sustained", FALLBACK_BF16_TFLOPS_SUSTAINED)
        extra = {}
        for name, layers, steps, warm in (("cfg2", 32, 100, 10), ("cfg3", 32, 100, 10), ("target", 32, 100, 10),
                                          ("cfg4", 4, 30, 5), ("cfg5", 4, 10, 3), ("gqa16", 32, 100, 10)):
            if name == args.workload or (world > 1 and wl.BASELINE_CONFIGS[name]["Hkv"] % world):
                continue
            x = measure(name, layers, steps, warm, False)
            t_call = x["secs"] / x["n_calls"]
            t_kernel = (x["secs_attn"] or x["secs"]) / x["n_calls"]
            e = {"us_per_call": round(t_call * 1e6, 3),
                 "value_TBps": round(x["bytes_per_call"] / t_call / 1e12, 4),
                 "attention_only_us_per_call": round(x["secs_attn"] / x["n_calls"] * 1e6, 3) if x["secs_attn"] else None,
                 "us_per_call_spread": {k.replace("_ms", ""): round(v * 1e3 / x["layers"], 3) for k, v in x["spread"].items()},
                 "layers_per_step": x["layers"], "steps": steps, "bytes_per_call": x["bytes_per_call"],
                 "parity": x["parity"]}
            if name == "cfg5":
                flops = wl.baseline_problem(name).flops()
                e.update({"bound": "tensor", "flops_per_call": flops,
                          "achieved_TFLOPs_per_gpu": round(flops / world / t_kernel / 1e12, 1),
                          "frac": round(flops / world / t_kernel / 1e12 / tf_peak, 4), "peak_TFLOPs": tf_peak})
            else:
                r = NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(name) if world == 1 else None
                e.update({"bound": "hbm", "frac": round(x["bytes_per_call"] / world / t_kernel / 1e9 / hbm_peak, 4),
                          "traffic": int(x["bytes_per_call"] * r) if r else None})
            if name == "gqa16" and world == 1:
                # the one head layout the reference's own CUDA kernel accepts: race it on the same GPU, same inputs
                e["reference_cuda_kernel"] = race_reference_kernel(name, layers)
            extra[name] = e
        if world == 1:
            try:
                extra["paged_gqa16"] = measure_paged(device)
            except Exception as exc:                      # noqa: BLE001
                extra["paged_gqa16"] = {"unavailable": str(exc)[:200]}
    us_per_call = secs / n_calls * 1e6
    value = bytes_per_call * n_calls / secs / 1e12

    e2e = None if args.no_e2e else measure_e2e(args, full, device, dist, world)

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return
    peak, peak_src = measured_peak()
    per_gpu_bytes = bytes_per_call / world
    achieved = per_gpu_bytes / ((secs_attn or secs) / n_calls) / 1e9
    tensor_bound = args.workload == "cfg5"          # ~1,000 flop per K/V byte: bounded by the tensor pipe, not by HBM
    if tensor_bound:
        tf_peak, tf_src = measured_peak("bf16_tflops_sustained", FALLBACK_BF16_TFLOPS_SUSTAINED)
        tf = wl.baseline_problem(args.workload).flops() / world / ((secs_attn or secs) / n_calls) / 1e12
    ratio = NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(args.workload) if world == 1 and LENGTH_SCALE == 1.0 else None
    traffic = int(per_gpu_bytes * ratio) if ratio else None
    traffic_src = (f"ncu capture of this shape (profiles/): {ratio} x algorithmic bytes" if ratio
                   else "no ncu capture of this shape / shard")
    line = {
        "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(secs / args.steps * 1e3, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": str(full.dtype).replace("torch.", "") + " in, fp32 accumulate",
        "data": "synthetic (seeded N(0,1) q/k/v, keys pre-rotated)",
        "config": job_config(args, wl.baseline_problem(args.workload).meta if world > 1 else full.meta, world,
                             fused_gather or world == 1, graph_used),
        "us_per_call": round(us_per_call, 3),
        "us_per_call_spread": {k.replace("_ms", ""): round(v * 1e3 / (n_calls / args.steps), 3) for k, v in m["spread"].items()},
        "us_per_call_isolated_cold": round(iso_us, 3),
        "pct_of_nominal_8TBps": round(100 * value * 1e3 / (NOMINAL_HBM_GBS * world), 2),
        "gpu_launches": launches_per_step * args.steps,
        "parity_checked": bool(m["parity"] and m["parity"]["ok"]), "parity": m["parity"],
        "clocks": clocks,
        "e2e": e2e,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": traffic,
                     "traffic_source": traffic_src, "peak_source": peak_src,
                     "kernel": "mma_attention_kernel (+ merge_kernel in the same interval)",
                     "bytes_per_launch": int(per_gpu_bytes)},
    }
    if tensor_bound:
        line["roofline"] = {"bound": "tensor", "achieved": round(tf, 1), "peak": tf_peak, "unit": "TFLOP/s",
                            "frac": round(tf / tf_peak, 4), "traffic": None, "peak_source": tf_src + ", sustained bf16",
                            "kernel": "dense_attention_kernel (+ rope_kernel and merge_kernel in the same interval)",
                            "flops_per_launch": int(wl.baseline_problem(args.workload).flops() / world)}
    if extra:
        line["other_workloads"] = extra
    if secs_attn:
        line["attention_only_us_per_call"] = round(secs_attn / n_calls * 1e6, 3)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.workload, budget_s=20.0)
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def measure_e2e(args, p: wl.Problem, device, dist, world):
    """The same metric through the public Python API with HOST inputs: every call copies the step's
    tensors (queries, tables, locations and the KV fragments) from pinned host memory, runs
    ``hogwild_fused`` and reads the output back."""
    import inference_lib_b200.attention as A
    pin = lambda t: t.contiguous().pin_memory()
    hq, hcos, hsin, hloc, hlen = pin(p.queries), pin(p.cos), pin(p.sin), pin(p.locations), pin(p.fragment_lengths)
    hk, hv = [pin(k) for k in p.keys], [pin(v) for v in p.values]
    dq, dcos, dsin, dloc, dlen = [torch.empty_like(t, device=device) for t in (hq, hcos, hsin, hloc, hlen)]
    dk, dv = [torch.empty_like(t, device=device) for t in hk], [torch.empty_like(t, device=device) for t in hv]
    rq = torch.empty((p.F, p.W, p.Hq, p.S, p.E), dtype=p.dtype, device=device)
    out = torch.empty((p.W, p.Hq, p.S, p.Ev), dtype=p.dtype, device=device)
    hout = torch.empty((p.W, p.Hq * world, p.S, p.Ev), dtype=out.dtype).pin_memory()
    gathered = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=device) if dist else None
    h2d = sum(t.numel() * t.element_size() for t in [hq, hcos, hsin, hloc, hlen] + hk + hv)
    d2h = hout.numel() * hout.element_size()

    def call():
        for d, h in zip([dq, dcos, dsin, dloc, dlen] + dk + dv, [hq, hcos, hsin, hloc, hlen] + hk + hv):
            d.copy_(h, non_blocking=True)
        A.hogwild_fused(dq, dloc, dk, dv, p.scale, dlen, dcos, dsin, rotated_queries=rq, out=out)
        res = out
        if dist:
            from inference_lib_b200 import sharded
            res = sharded.gather_heads(out, world, gather_buffer=gathered)
        hout.copy_(res, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def call_resident():
        # what a decode step pays: the KV cache stays on the device, only the step's queries and metadata come in
        for d, h in zip([dq, dcos, dsin, dloc, dlen], [hq, hcos, hsin, hloc, hlen]):
            d.copy_(h, non_blocking=True)
        A.hogwild_fused(dq, dloc, dk, dv, p.scale, dlen, dcos, dsin, rotated_queries=rq, out=out)
        res = out
        if dist:
            from inference_lib_b200 import sharded
            res = sharded.gather_heads(out, world, gather_buffer=gathered)
        hout.copy_(res, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def median_time(fn, n):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        ts = []
        for _ in range(n):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        tt = torch.tensor([statistics.median(ts)], dtype=torch.float64, device=device)
        if dist:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt[0])

    n = 60
    dt = median_time(call, n)
    dt_res = median_time(call_resident, n)
    whole_bytes = wl.baseline_problem(args.workload).algorithmic_bytes() if world > 1 else p.algorithmic_bytes()
    h2d_small = sum(t.numel() * t.element_size() for t in [hq, hcos, hsin, hloc, hlen])
    return {"value": round(whole_bytes / dt / 1e12, 5), "unit": UNIT, "us_per_call": round(dt * 1e6, 1),
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "calls": n, "statistic": "median",
            "what": "pinned host -> device copy of q/cos/sin/loc/lengths and all KV fragments, hogwild_fused, output back to host",
            "kv_resident": {"value": round(whole_bytes / dt_res / 1e12, 5), "us_per_call": round(dt_res * 1e6, 1),
                            "h2d_bytes_per_step": int(h2d_small), "d2h_bytes_per_step": int(d2h),
                            "what": "KV cache resident on the device; only q/cos/sin/loc/lengths are copied in, output back to host"}}


def measure_paged(device, name="paged_gqa16", copies=3, steps=20, warmup=5, race=True):
    """The paged operator (``hogatt_paged_sdpa_launch``) at a decode shape: tensor-core kernel and CUDA-core kernel of
    this library, and the reference's own paged kernel in a process of its own.  ``copies`` distinct caches are used
    in turn (more than L2 in total), calls replayed from a CUDA graph, CUDA events around ``steps`` replays."""
    from inference_lib_b200 import _cabi
    pp = wl.paged_problem(name)
    d = {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in pp.items()}
    caches = [(torch.roll(d["key_cache"], i, 2), torch.roll(d["value_cache"], i, 2)) for i in range(copies)]
    out = torch.empty((d["queries"].shape[1], d["queries"].shape[2], d["queries"].shape[3], d["value_cache"].shape[3]),
                      dtype=d["queries"].dtype, device=device)
    res = {"bytes_per_call": pp["bytes"], "config": pp["meta"]}
    hbm_peak, _ = measured_peak()
    outs = {}
    for label, kernel in (("tensor_core_kernel", _cabi.KERNEL_MMA), ("cuda_core_kernel", _cabi.KERNEL_FMA)):
        bound = [_cabi.bind_paged(out=out, queries=d["queries"], locations=d["locations"], fragment_lengths=d["fragment_lengths"],
                                  key_cache=kc, value_cache=vc, block_table=d["block_table"], scale=d["scale"], kernel=kernel)
                 for kc, vc in caches]
        stream = torch.cuda.Stream(device)
        with torch.cuda.stream(stream):
            for p, _ in bound:
                assert _cabi.launch_paged(p, stream.cuda_stream) == 0
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for p, _ in bound:
                    _cabi.launch_paged(p, torch.cuda.current_stream().cuda_stream)
            for _ in range(warmup):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                g.replay()
            e1.record()
            stream.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (steps * copies)
        res[label] = {"us_per_call": round(us, 2), "value_TBps": round(pp["bytes"] / us / 1e6, 4),
                      "frac": round(pp["bytes"] / us / 1e3 / hbm_peak, 4)}
        outs[label] = out.float().clone()
    diff = (outs["tensor_core_kernel"] - outs["cuda_core_kernel"]).abs()
    res["kernels_agree"] = {"max_abs": round(float(diff.max().item()), 6), "ok": bool(diff.max().item() <= 2e-2)}
    if race:
        res["reference_cuda_kernel"] = race_reference_kernel(name, copies)
    return res


# ------------------------------------------------------------------------------------------------
# CPU legs (the only places that run the oracle)
# ------------------------------------------------------------------------------------------------
def race_reference_kernel(workload: str, layers: int):
    """Time the reference's own CUDA kernels (``oracle/_ref/hogatt_ref.so``: ``kernel_v21`` recompiled for sm_100a) on
    the same workload in a process of their own (same operator names, static device buffers, default stream).  Only
    head size 128 with 16 query heads per kv head can run there (``kernel_v21.cuh:982-986``)."""
    runner = os.path.join(ROOT, "oracle", "ref_cuda_runner.py")
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "hogatt_ref.so")):
        return {"unavailable": "the reference's CUDA extension was not built (no reference checkout at build time)"}
    try:
        res = subprocess.run([sys.executable, runner, "time", "--workload", workload, "--layers", str(layers), "--steps", "20",
                              "--warmup", "5"], capture_output=True, text=True, timeout=300)
        if res.returncode != 0:
            return {"unavailable": (res.stderr.strip().splitlines() or ["failed"])[-1][:200]}
        return json.loads(res.stdout.strip().splitlines()[-1])
    except Exception as exc:                              # noqa: BLE001
        return {"unavailable": str(exc)[:200]}


def reference_runner(p: wl.Problem):
    """One call of the op on the host cores: the reference's own ``hogwild_sdpa_pt`` fed by its
    ``apply_rotary_pos_emb`` (python/hogwild/attention.py:38-67, :84-90, i.e. the eager branch :320-323) when the
    module was staged under ``oracle/_ref``, else the restatement in ``oracle/`` (``kind: "port"``)."""
    torch.set_num_threads(os.cpu_count() or 1)
    from oracle import build_oracle
    ref = build_oracle.load_reference_python()
    if ref is not None:
        def run():
            tiled = torch.tile(torch.unsqueeze(p.queries, 0), (p.cos.size(0), 1, 1, 1, 1))
            rq = ref.apply_rotary_pos_emb(tiled, p.cos, p.sin, unsqueeze_dim=2)
            return ref.hogwild_sdpa_pt(rq, p.locations, p.keys, p.values, p.scale)
        return run, "reference", "the reference's hogwild_sdpa_pt + apply_rotary_pos_emb (python/hogwild/attention.py)"
    from oracle import hogwild_oracle as oracle
    return (lambda: oracle.fused(p.queries, p.cos, p.sin, p.locations, p.keys, p.values, p.scale), "port",
            "the reference's PyTorch algorithm restated in oracle/ (the reference module was not staged)")


def cpu_baseline(workload: str, budget_s: float, reps_cap: int = 5):
    p = wl.baseline_problem(workload)
    run, kind, what = reference_runner(p)
    t0 = time.perf_counter(); run(); first = time.perf_counter() - t0
    reps = max(1, min(reps_cap, int(budget_s / max(first, 1e-3)) - 1))
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter(); run(); ts.append(time.perf_counter() - t0)
    dt = statistics.median(ts)
    return {"value": round(p.algorithmic_bytes() / dt / 1e12, 7), "unit": UNIT, "us_per_call": round(dt * 1e6, 1),
            "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{reps} full calls of the '{workload}' problem (one layer) after 1 warm-up, median; {what}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", 1))
    p = wl.baseline_problem(args.workload)
    run, kind, what = reference_runner(p)
    steps, warmup = args.steps, args.warmup       # a step here is ONE call on one layer's tensors: a bounded sample
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    value = p.algorithmic_bytes() / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 7), "unit": UNIT,
        "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": str(p.dtype).replace("torch.", "") + " in, fp32 accumulate", "data": "synthetic (seeded N(0,1) q/k/v, keys pre-rotated)",
        "config": job_config(args, p.meta, world),
        "us_per_call": round(dt * 1e6, 1),
        "cpu_baseline": {"value": round(value, 7), "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
                         "sample": f"{steps} timed steps, each ONE call of the '{args.workload}' problem on one layer's tensors "
                                   f"(a bounded sample of the {args.layers}-call step; value is per-call throughput); {what}"},
        "e2e": {"value": round(value, 7), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="target", choices=["target", "cfg2", "cfg3", "cfg4", "cfg5", "gqa16"])
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the additional long-context (cfg4) measurement")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: how the per-rank outputs are all-gathered (fused = peer stores from the merge kernel)")
    ap.add_argument("--kernel", default="auto", choices=["auto", "persistent", "cluster"],
                    help="launch shape of the tensor-core kernel (auto = the library's own choice)")
    ap.add_argument("--scale-lengths", type=float, default=1.0,
                    help="multiply every fragment length of the workload (context-length sweeps; not the headline number)")
    ap.add_argument("--emulate-shard", type=int, default=1,
                    help="single GPU only: run rank 0's share of an N-way kv-head split (kernel tuning; not the headline number)")
    ap.add_argument("--plan", default="host", choices=["host", "device"],
                    help="host: the call carries the fragment lengths the host knows, tiles are cut from them; "
                         "device: tiles are derived on the device from locations / fragment_lengths")
    ap.add_argument("--stable", type=int, default=1,
                    help="leading fragments marked as not written by earlier work of the stream (the shared prompt)")
    ap.add_argument("--pdl", default=None, choices=["0", "1"],
                    help="programmatic dependent launch between the kernels of consecutive calls (default: the library's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-rq", action="store_true", help="do not ask for the rotated-query side output")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-isolated", action="store_true", help="skip the isolated cold-call leg (profiling runs)")
    ap.add_argument("--paged-only", action="store_true",
                    help="only the paged-operator leg (one GPU): prints its JSON object and exits (profiling runs)")
    ap.add_argument("--no-reference-race", action="store_true", help="do not time the reference's own CUDA kernels")
    args = ap.parse_args()
    if args.paged_only:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the op has no CPU path")
        print(json.dumps(measure_paged(torch.device("cuda:0"), steps=min(args.steps, 20), warmup=min(args.warmup, 5),
                                       race=not args.no_reference_race)), flush=True)
        return
    global KERNEL_CHOICE, LENGTH_SCALE, EMULATE_SHARD, HOST_PLAN, STABLE_FRAGMENTS
    HOST_PLAN = args.plan == "host"
    STABLE_FRAGMENTS = args.stable
    if args.pdl is not None:
        os.environ["HOGATT_PDL"] = args.pdl          # read by the library when it is first used
    LENGTH_SCALE = args.scale_lengths
    EMULATE_SHARD = args.emulate_shard
    KERNEL_CHOICE = {"auto": 0, "persistent": 2, "cluster": 3}[args.kernel]
    if args.workload == "cfg4":
        args.layers = min(args.layers, 4)          # 570 MB of KV per layer
    if args.workload == "cfg5":
        args.layers = min(args.layers, 4)          # the four independent groups of that configuration (105 MB each)
        args.steps = min(args.steps, 20)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
