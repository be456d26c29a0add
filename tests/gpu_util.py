"""Helpers for the GPU parity tests: drive the C ABI with torch-owned device memory."""
from __future__ import annotations

import numpy as np
import torch

from inference_lib_b200 import _cabi
from inference_lib_b200 import workloads as wl

CANARY = 0x5A          # around the buffers: any overrun shows
WS_FILL = 0xFF         # inside the workspace: every fp32 word is a NaN, so a slot that is read without having been
                       # written (or multiplied by zero instead of being selected away) poisons the result


class Result:
    def __init__(self, out, rq, status, rc):
        self.out, self.rq, self.status, self.rc = out, rq, status, rc


def run_cabi(p: wl.Problem, *, fused: bool = True, want_rq: bool = False, kernel=_cabi.KERNEL_AUTO, max_ctas: int = 0,
             device: str = "cuda:0", pre_rotated=None, host_lengths=None, stable_fragments: int = 0, keys=None,
             values=None) -> Result:
    """One call through ``hogatt_fused_launch`` / ``hogatt_sdpa_launch`` with canaries around the
    output and the workspace.  ``p`` holds CPU tensors; ``pre_rotated`` is the [F,W,Hq,S,E] query
    tensor for the sdpa entry point; ``keys`` / ``values`` replace the problem's device fragments
    (already on the device); ``host_lengths`` / ``stable_fragments`` as in ``_cabi.bind``."""
    dev = torch.device(device)
    d = p.to(dev)
    W, Hq, S, Ev = p.W, p.Hq, p.S, p.Ev
    pad = 64
    out_buf = torch.full((W * Hq * S * Ev + 2 * pad,), float("nan"), dtype=p.dtype, device=dev)
    out = out_buf[pad:-pad].view(W, Hq, S, Ev)
    rq = torch.zeros((p.F, W, Hq, S, p.E), dtype=p.dtype, device=dev) if (fused and want_rq) else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    if fused:
        q, cos, sin = d.queries, d.cos, d.sin
    else:
        q, cos, sin = pre_rotated.to(dev).contiguous(), None, None
    bp = _cabi.bind(out=out, queries=q, locations=d.locations, keys=keys if keys is not None else d.keys,
                    values=values if values is not None else d.values, scale=p.scale,
                    fragment_lengths=d.fragment_lengths, cos=cos, sin=sin, rq=rq, status=status, kernel=kernel,
                    max_ctas=max_ctas, host_lengths=host_lengths, stable_fragments=stable_fragments)
    need = _cabi.workspace_bytes(bp)
    assert need > 0, "library refused the problem"
    ws_buf = torch.full((need + 512,), CANARY, dtype=torch.uint8, device=dev)
    off = (-ws_buf.data_ptr()) % 256
    ws = ws_buf[off:off + need]
    ws.fill_(WS_FILL)
    bp.struct.workspace, bp.struct.workspace_bytes = ws.data_ptr(), need
    rc = _cabi.launch(bp, torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize(dev)
    if rc == 0:
        assert torch.isnan(out_buf[:pad].float()).all() and torch.isnan(out_buf[-pad:].float()).all(), "output overrun"
        assert (ws_buf[:off] == CANARY).all() and (ws_buf[off + need:] == CANARY).all(), "workspace overrun"
    return Result(out.clone(), rq, int(status.item()), rc)


def check_against(out: torch.Tensor, ref: np.ndarray, dtype, *, what: str = ""):
    """Tolerances of the parity gate: 16-bit outputs against an fp32 reference max-abs <= 2e-2 and
    mean-abs <= 2e-3; fp32 outputs max-abs <= 1e-4.  Rows that see no key are NaN in the reference
    and must be exactly zero here."""
    got = out.detach().float().cpu().numpy()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    blind = np.isnan(ref)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    if blind.any():
        assert (got[blind] == 0).all(), f"{what}: rows without visible keys must be zero"
    diff = np.abs(got - np.where(blind, 0, ref))[~blind]
    if diff.size == 0:
        return 0.0, 0.0
    mx, mean = float(diff.max()), float(diff.mean())
    if dtype == torch.float32:
        assert mx <= 1e-4, f"{what}: max-abs {mx}"
    else:
        assert mx <= 2e-2, f"{what}: max-abs {mx}"
        assert mean <= 2e-3, f"{what}: mean-abs {mean}"
    return mx, mean
