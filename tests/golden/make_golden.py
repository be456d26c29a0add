"""Generate golden outputs by running the REFERENCE's own PyTorch path.

Needs a checkout of the reference (nothing at test time does):

    python tests/golden/make_golden.py --reference /path/to/reference [--only name,name]

For every seeded problem of ``inference_lib_b200.workloads`` it calls the reference's
``apply_rotary_pos_emb`` + ``hogwild_sdpa_pt(..., return_intermediate_results=True)``
(``python/hogwild/attention.py:38-90``, i.e. the eager branch ``:320-323``) and stores the fp32
result in ``tests/golden/reference_outputs.npz``:

* ``<name>/out``  fp32 ``[W,Hq,S,Ev]`` (for cfg5, whose output is 4 MiB per group, the rows
  ``[:, ::8, ::4, :]`` only; four groups, seeds 0..3; every row of group 0 goes to ``cfg5_g0_full.npz``)
* ``<name>/rq``   rotated queries ``[F,W,Hq,S,E]`` as fp32, for a few small problems

The reference module imports as shipped except for one thing: it looks up an installed
``hogwild`` distribution and only catches ``OSError``; a thin wrapper around
``importlib.metadata.distribution`` turns the "not installed" error into that ``OSError`` so
the module takes its own "no compiled kernel, eager path" branch.  No reference file is edited
or copied.
"""
from __future__ import annotations

import argparse
import importlib.metadata as md
import json
import os
import sys
import time
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from inference_lib_b200 import workloads as wl  # noqa: E402

RQ_CASES = {"cfg1", "ragged_f16", "ragged_bf16", "partial_rotary_bf16", "causal_chunk_bf16", "ragged_f32"}
CFG5_SLICE = (slice(None), slice(None, None, 8), slice(None, None, 4), slice(None))


def load_reference(path: str):
    warnings.simplefilter("ignore")
    real = md.distribution

    def shim(name):
        if name == "hogwild":
            raise OSError("hogwild wheel is not installed here")
        return real(name)

    md.distribution = shim
    sys.path.insert(0, os.path.join(path, "python"))
    try:
        import hogwild.attention as ref
    finally:
        md.distribution = real
    return ref


def reference_run(ref, p: wl.Problem):
    tiled = torch.tile(torch.unsqueeze(p.queries, 0), (p.cos.size(0), 1, 1, 1, 1))
    rq = ref.apply_rotary_pos_emb(tiled, p.cos, p.sin, unsqueeze_dim=2)
    out, _, _ = ref.hogwild_sdpa_pt(rq, p.locations, p.keys, p.values, p.scale, True)
    return out, rq


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("HOGWILD_REFERENCE"), required="HOGWILD_REFERENCE" not in os.environ,
                    help="checkout of choyakawa/inference_lib (or set HOGWILD_REFERENCE)")
    ap.add_argument("--only", default="")
    ap.add_argument("--skip-big", action="store_true", help="skip cfg4 (20 s, ~10 GB RSS)")
    args = ap.parse_args()
    ref = load_reference(args.reference)
    only = set(filter(None, args.only.split(",")))
    path = os.path.join(HERE, "reference_outputs.npz")
    store = dict(np.load(path)) if (only and os.path.exists(path)) else {}

    jobs = [(n, lambda n=n: wl.baseline_problem(n)) for n in ("cfg1", "cfg2", "cfg3", "target", "cfg4", "gqa16")]
    jobs += [(f"cfg5_g{g}", lambda g=g: wl.baseline_problem("cfg5", seed=g)) for g in range(4)]
    jobs += [(n, lambda n=n: wl.edge_problem(n)) for n in wl.EDGE_CASES]
    for name, build in jobs:
        if only and name not in only:
            continue
        if args.skip_big and name == "cfg4":
            continue
        t = time.time()
        p = build()
        out, rq = reference_run(ref, p)
        out = out.to(torch.float32)
        if name == "cfg5_g0":
            np.savez_compressed(os.path.join(HERE, "cfg5_g0_full.npz"), out=out.contiguous().numpy())
        if name.startswith("cfg5"):
            out = out[CFG5_SLICE]
        store[f"{name}/out"] = out.contiguous().numpy()
        if name in RQ_CASES:
            store[f"{name}/rq"] = rq.to(torch.float32).numpy()
        print(f"{name:28s} out{tuple(out.shape)} {time.time() - t:6.1f}s", flush=True)

    np.savez_compressed(path, **store)
    with open(os.path.join(HERE, "reference_outputs.json"), "w") as fh:
        json.dump({"generator": "tests/golden/make_golden.py", "torch": torch.__version__,
                   "reference_functions": ["apply_rotary_pos_emb (attention.py:84-90)",
                                           "hogwild_sdpa_pt (attention.py:38-67)"],
                   "entries": sorted(store.keys())}, fh, indent=1)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
