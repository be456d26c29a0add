"""ctypes view of the C ABI in ``include/hogatt.h`` (``libhogatt_b200.so``).

Used by the tests and the benchmark to drive the library exactly as a non-torch host would:
raw device pointers, a caller-provided workspace and a stream handle.  There is no fallback: if
the shared object is missing, :func:`load` raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libhogatt_b200.so")

F32, F16, BF16 = 0, 1, 2
KERNEL_AUTO, KERNEL_FMA, KERNEL_MMA, KERNEL_MMA_CLUSTER, KERNEL_DENSE = 0, 1, 2, 3, 4
MAX_FRAGMENTS = 128

EXPORTS = ["hogatt_abi_version", "hogatt_status_string", "hogatt_last_cuda_error", "hogatt_workspace_bytes",
           "hogatt_sdpa_launch", "hogatt_fused_launch", "hogatt_fused_launch_static", "hogatt_fused_launch_gather", "hogatt_rope_launch",
           "hogatt_paged_workspace_bytes", "hogatt_paged_sdpa_launch", "hogatt_copy_to_blocks_launch", "hogatt_plan_describe",
           "hogatt_plan_ranges", "hogatt_launch_shape", "hogatt_step_plan_launch", "hogatt_append_launch"]


class Problem(C.Structure):
    _fields_ = [
        ("F", C.c_int32), ("W", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("E", C.c_int32),
        ("Ev", C.c_int32), ("S", C.c_int32), ("rotary_dim", C.c_int32), ("dtype", C.c_int32), ("scale", C.c_float),
        ("out", C.c_void_p), ("rq", C.c_void_p), ("queries", C.c_void_p), ("cosines", C.c_void_p),
        ("sines", C.c_void_p), ("locations", C.c_void_p), ("fragment_lengths", C.c_void_p),
        ("key_fragments", C.POINTER(C.c_void_p)), ("value_fragments", C.POINTER(C.c_void_p)),
        ("fragment_rows", C.POINTER(C.c_int32)),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("device_status", C.c_void_p),
        ("kernel", C.c_int32), ("max_ctas", C.c_int32),
        ("host_lengths", C.POINTER(C.c_int32)), ("stable_fragments", C.c_int32), ("reserved_", C.c_int32),
    ]


class PagedProblem(C.Structure):
    _fields_ = [
        ("F", C.c_int32), ("W", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("E", C.c_int32), ("Ev", C.c_int32),
        ("S", C.c_int32), ("total_q_tokens", C.c_int32), ("block_size", C.c_int32), ("max_blocks_per_seq", C.c_int32),
        ("dtype", C.c_int32), ("scale", C.c_float),
        ("out", C.c_void_p), ("queries", C.c_void_p), ("locations", C.c_void_p), ("fragment_lengths", C.c_void_p),
        ("key_cache", C.c_void_p), ("value_cache", C.c_void_p), ("block_table", C.c_void_p), ("cu_seqlens_q", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("kernel", C.c_int32), ("reserved_", C.c_int32),
    ]


MAX_PEERS = 8


class Peers(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("out_full", C.c_void_p * MAX_PEERS),
                ("flags", C.c_void_p * MAX_PEERS)]


_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m inference_lib_b200._build` "
                               "(there is no fallback implementation)")
        lib = C.CDLL(LIB_PATH)
        lib.hogatt_abi_version.restype = C.c_int
        lib.hogatt_status_string.restype = C.c_char_p
        lib.hogatt_status_string.argtypes = [C.c_int]
        lib.hogatt_last_cuda_error.restype = C.c_int
        lib.hogatt_workspace_bytes.restype = C.c_size_t
        lib.hogatt_workspace_bytes.argtypes = [C.POINTER(Problem)]
        for name in ("hogatt_sdpa_launch", "hogatt_fused_launch", "hogatt_fused_launch_static"):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(Problem), C.c_void_p]
        lib.hogatt_fused_launch_gather.restype = C.c_int
        lib.hogatt_fused_launch_gather.argtypes = [C.POINTER(Problem), C.POINTER(Peers), C.c_void_p]
        lib.hogatt_rope_launch.restype = C.c_int
        lib.hogatt_rope_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int32] * 7 + [C.c_void_p]
        lib.hogatt_paged_workspace_bytes.restype = C.c_size_t
        lib.hogatt_paged_workspace_bytes.argtypes = [C.POINTER(PagedProblem)]
        lib.hogatt_paged_sdpa_launch.restype = C.c_int
        lib.hogatt_paged_sdpa_launch.argtypes = [C.POINTER(PagedProblem), C.c_void_p]
        lib.hogatt_copy_to_blocks_launch.restype = C.c_int
        lib.hogatt_copy_to_blocks_launch.argtypes = [C.c_void_p] * 6 + [C.c_int32] * 8 + [C.c_void_p]
        lib.hogatt_step_plan_launch.restype = C.c_int
        lib.hogatt_step_plan_launch.argtypes = [C.POINTER(StepPlan), C.c_void_p]
        lib.hogatt_append_launch.restype = C.c_int
        lib.hogatt_append_launch.argtypes = [C.POINTER(Append), C.c_void_p]
        lib.hogatt_launch_shape.restype = C.c_int
        lib.hogatt_launch_shape.argtypes = [C.POINTER(Problem), C.POINTER(C.c_int32)]
        lib.hogatt_plan_describe.restype = C.c_int
        lib.hogatt_plan_describe.argtypes = [C.POINTER(Problem), C.POINTER(C.c_int32), C.c_int32, C.POINTER(C.c_int32)]
        lib.hogatt_plan_ranges.restype = C.c_int
        lib.hogatt_plan_ranges.argtypes = [C.c_int32] * 5 + [C.POINTER(C.c_int64)]
        _lib = lib
    return _lib


def status_string(rc: int) -> str:
    return load().hogatt_status_string(rc).decode()


def dtype_code(torch_dtype) -> int:
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[torch_dtype]


def shape_problem(*, F, W, Hq, Hkv, E, Ev, S, dtype, rotary_dim=0, scale=1.0, kernel=KERNEL_AUTO, max_ctas=0) -> Problem:
    """A problem with dims only (enough for the plan / workspace queries)."""
    p = Problem()
    p.F, p.W, p.Hq, p.Hkv, p.E, p.Ev, p.S = F, W, Hq, Hkv, E, Ev, S
    p.rotary_dim, p.dtype, p.scale, p.kernel, p.max_ctas = rotary_dim, dtype, scale, kernel, max_ctas
    return p


class StepPlan(C.Structure):
    _fields_ = [
        ("F", C.c_int32), ("W", C.c_int32), ("S", C.c_int32), ("rotary_dim", C.c_int32),
        ("order", C.c_void_p), ("fragment_lengths", C.c_void_p), ("inv_freq", C.c_void_p),
        ("attention_scaling", C.c_float), ("round_tables_to", C.c_int32),
        ("locations", C.c_void_p), ("cosines", C.c_void_p), ("sines", C.c_void_p),
    ]


MAX_APPEND_SOURCES = 64


class Append(C.Structure):
    _fields_ = [
        ("W", C.c_int32), ("Hkv", C.c_int32), ("E", C.c_int32), ("Ev", C.c_int32), ("S", C.c_int32),
        ("rotary_dim", C.c_int32), ("dtype", C.c_int32), ("table_dtype", C.c_int32),
        ("keys", C.c_void_p), ("key_strides", C.c_int64 * 3),
        ("values", C.c_void_p), ("value_strides", C.c_int64 * 3),
        ("cosines", C.c_void_p), ("sines", C.c_void_p), ("table_strides", C.c_int64 * 2),
        ("new_rows", C.c_void_p), ("write_to", C.POINTER(C.c_int32)),
        ("F", C.c_int32), ("take_leading", C.c_int32),
        ("key_fragments", C.POINTER(C.c_void_p)), ("value_fragments", C.POINTER(C.c_void_p)),
        ("fragment_rows", C.POINTER(C.c_int32)),
        ("lengths_in", C.c_void_p), ("lengths_out", C.c_void_p), ("device_status", C.c_void_p),
    ]


class BoundProblem:
    """A ``Problem`` struct together with the Python objects that keep its pointers alive."""

    def __init__(self, struct: Problem, keep: Sequence):
        self.struct = struct
        self._keep = list(keep)


def bind(*, out, queries, locations, keys, values, scale, fragment_lengths=None, cos=None, sin=None, rq=None,
         workspace=None, status=None, kernel=KERNEL_AUTO, max_ctas=0, host_lengths=None,
         stable_fragments=0) -> BoundProblem:
    """Fill a ``Problem`` from torch CUDA tensors (pointers only; nothing is copied).

    ``queries`` is ``[W,Hq,S,E]`` with ``cos``/``sin`` given (fused entry point) or ``[F,W,Hq,S,E]``
    already rotated.  Fragments may be ``[Hkv,L,E]`` or ``[1,Hkv,L,E]``.  ``host_lengths``: a list of
    F ints (upper bounds of the visible lengths that the host knows) or ``"rows"`` for the tensors'
    own row counts; ``stable_fragments``: leading fragments nothing enqueued earlier still writes.
    """
    F = len(keys)
    W, Hq, S, Ev = out.shape
    E = queries.shape[-1]
    Hkv = keys[0].shape[-3]
    p = shape_problem(F=F, W=W, Hq=Hq, Hkv=Hkv, E=E, Ev=Ev, S=S, dtype=dtype_code(out.dtype),
                      rotary_dim=(cos.shape[-1] if cos is not None else 0), scale=float(scale), kernel=kernel,
                      max_ctas=max_ctas)
    kp = (C.c_void_p * F)(*[k.data_ptr() for k in keys])
    vp = (C.c_void_p * F)(*[v.data_ptr() for v in values])
    rows = (C.c_int32 * F)(*[int(k.shape[-2]) for k in keys])
    p.out, p.queries, p.locations = out.data_ptr(), queries.data_ptr(), locations.data_ptr()
    p.rq = rq.data_ptr() if rq is not None else None
    p.cosines = cos.data_ptr() if cos is not None else None
    p.sines = sin.data_ptr() if sin is not None else None
    p.fragment_lengths = fragment_lengths.data_ptr() if fragment_lengths is not None else None
    p.key_fragments = C.cast(kp, C.POINTER(C.c_void_p))
    p.value_fragments = C.cast(vp, C.POINTER(C.c_void_p))
    p.fragment_rows = C.cast(rows, C.POINTER(C.c_int32))
    p.device_status = status.data_ptr() if status is not None else None
    hl = None
    if host_lengths is not None:
        vals = [int(k.shape[-2]) for k in keys] if isinstance(host_lengths, str) else [int(x) for x in host_lengths]
        assert len(vals) == F
        hl = (C.c_int32 * F)(*vals)
        p.host_lengths = C.cast(hl, C.POINTER(C.c_int32))
    p.stable_fragments = int(stable_fragments)
    if workspace is not None:
        p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    return BoundProblem(p, [hl, kp, vp, rows, out, queries, locations, keys, values, fragment_lengths, cos, sin, rq,
                            workspace, status])


def workspace_bytes(bp: BoundProblem) -> int:
    return int(load().hogatt_workspace_bytes(C.byref(bp.struct)))


def describe(bp: BoundProblem, num_sms: int) -> dict:
    """``hogatt_plan_describe`` for a bound problem, taking every row of every fragment as visible."""
    F = bp.struct.F
    vis = (C.c_int32 * F)(*[bp.struct.fragment_rows[f] for f in range(F)])
    plan = (C.c_int32 * 8)()
    rc = int(load().hogatt_plan_describe(C.byref(bp.struct), vis, num_sms, plan))
    if rc != 0:
        raise ValueError(status_string(rc))
    keys = ("tile_tokens", "rows_per_block", "row_blocks", "tiles_per_unit", "units", "ctas", "parts_per_unit", "kernel")
    return dict(zip(keys, list(plan)))


def launch_shape(bp: BoundProblem) -> dict:
    """``hogatt_launch_shape``: what one launch of this problem enqueues on the current device."""
    shape = (C.c_int32 * 4)()
    rc = int(load().hogatt_launch_shape(C.byref(bp.struct), shape))
    if rc != 0:
        raise ValueError(status_string(rc))
    return dict(zip(("kernel", "ctas", "cluster", "kernels_per_call"), list(shape)))


def attach_workspace(bp: BoundProblem, device, stream: int = 0):
    """Allocate (torch), align and bind the scratch a problem needs; returns the tensor that owns the
    memory (also kept alive by ``bp``)."""
    import torch
    need = workspace_bytes(bp)
    if need == 0:
        raise ValueError("libhogatt_b200 refused the problem")
    ws = torch.empty(need + 256, dtype=torch.uint8, device=device)
    ptr = ws.data_ptr() + (-ws.data_ptr()) % 256
    bp.struct.workspace, bp.struct.workspace_bytes = ptr, need
    bp._keep.append(ws)
    return ws


STATIC_SCRATCH_BYTES = 8 << 20


def launch_static(bp: BoundProblem, stream: int = 0) -> int:
    """``hogatt_fused_launch_static``: like :func:`launch` for a fused problem, but the split-K
    scratch is the library's own fixed device array, so no workspace has to be bound."""
    return int(load().hogatt_fused_launch_static(C.byref(bp.struct), C.c_void_p(stream)))


def launch_gather(bp: BoundProblem, peers: Peers, stream: int = 0) -> int:
    """``hogatt_fused_launch_gather``: this rank's shard, output rows stored into every rank's full output."""
    return int(load().hogatt_fused_launch_gather(C.byref(bp.struct), C.byref(peers), C.c_void_p(stream)))


def launch(bp: BoundProblem, stream: int = 0) -> int:
    """Enqueue one call; returns the library's status code (0 = ok)."""
    lib = load()
    fn = lib.hogatt_fused_launch if bp.struct.cosines else lib.hogatt_sdpa_launch
    return int(fn(C.byref(bp.struct), C.c_void_p(stream)))


def step_plan(*, order, fragment_lengths, inv_freq, S, locations, cosines, sines, attention_scaling=1.0,
              round_tables_to=F32, stream: int = 0) -> int:
    """``hogatt_step_plan_launch`` on torch CUDA tensors: ``order [W,F]`` int32, ``fragment_lengths [F]`` int32,
    ``inv_freq [R/2]`` fp32; fills ``locations [F,W,S]`` int32 and ``cosines`` / ``sines [F,W,S,R]`` fp32."""
    p = StepPlan()
    W, F_ = order.shape
    p.F, p.W, p.S, p.rotary_dim = F_, W, S, 2 * inv_freq.numel()
    p.order, p.fragment_lengths, p.inv_freq = order.data_ptr(), fragment_lengths.data_ptr(), inv_freq.data_ptr()
    p.attention_scaling, p.round_tables_to = float(attention_scaling), int(round_tables_to)
    p.locations, p.cosines, p.sines = locations.data_ptr(), cosines.data_ptr(), sines.data_ptr()
    return int(load().hogatt_step_plan_launch(C.byref(p), C.c_void_p(stream)))


def append(*, keys, values, cosines, sines, write_to, key_fragments, value_fragments, lengths_in, lengths_out,
           new_rows=None, take_leading=False, status=None, stream: int = 0) -> int:
    """``hogatt_append_launch`` on torch CUDA tensors.  ``keys`` / ``values`` are ``[W,Hkv,S,E]`` views with any
    strides whose last axis is contiguous; ``cosines`` / ``sines`` are ``[W,S,R]`` (or ``[1,1,R]`` / ``[R]`` to
    broadcast one row), fp32 or the tensors' own type; fragments are ``[Hkv,capacity,E]`` slabs.  ``new_rows [W]``
    int32 device: how many rows of each source are real, counted from its end (``take_leading``: from its start)."""
    W, Hkv, S, E = keys.shape
    Ev = values.shape[-1]
    assert keys.stride(-1) == 1 and values.stride(-1) == 1 and cosines.stride(-1) == 1 and sines.stride(-1) == 1
    p = Append()
    p.W, p.Hkv, p.E, p.Ev, p.S = W, Hkv, E, Ev, S
    p.rotary_dim, p.dtype, p.table_dtype = cosines.shape[-1], dtype_code(keys.dtype), dtype_code(cosines.dtype)
    p.keys, p.values = keys.data_ptr(), values.data_ptr()
    p.key_strides = (C.c_int64 * 3)(keys.stride(0), keys.stride(1), keys.stride(2))
    p.value_strides = (C.c_int64 * 3)(values.stride(0), values.stride(1), values.stride(2))
    p.cosines, p.sines = cosines.data_ptr(), sines.data_ptr()
    if cosines.dim() == 3 and cosines.shape[0] == W and cosines.shape[1] == S:
        ts = (cosines.stride(0), cosines.stride(1))
        assert (sines.stride(0), sines.stride(1)) == ts
    else:
        assert cosines.numel() == cosines.shape[-1], "tables are [W,S,R] or a single row"
        ts = (0, 0)
    p.table_strides = (C.c_int64 * 2)(*ts)
    p.new_rows = new_rows.data_ptr() if new_rows is not None else None
    p.take_leading = 1 if take_leading else 0
    wt = (C.c_int32 * W)(*[int(x) for x in write_to])
    p.write_to = C.cast(wt, C.POINTER(C.c_int32))
    F_ = len(key_fragments)
    kp = (C.c_void_p * F_)(*[k.data_ptr() for k in key_fragments])
    vp = (C.c_void_p * F_)(*[v.data_ptr() for v in value_fragments])
    rows = (C.c_int32 * F_)(*[int(k.shape[-2]) for k in key_fragments])
    p.F = F_
    p.key_fragments, p.value_fragments = C.cast(kp, C.POINTER(C.c_void_p)), C.cast(vp, C.POINTER(C.c_void_p))
    p.fragment_rows = C.cast(rows, C.POINTER(C.c_int32))
    p.lengths_in, p.lengths_out = lengths_in.data_ptr(), lengths_out.data_ptr()
    p.device_status = status.data_ptr() if status is not None else None
    return int(load().hogatt_append_launch(C.byref(p), C.c_void_p(stream)))


def bind_paged(*, out, queries, locations, fragment_lengths, key_cache, value_cache, block_table, scale,
               cu_seqlens_q=None, kernel=KERNEL_AUTO):
    """Fill a ``PagedProblem`` from torch CUDA tensors (fixed layout: ``queries [F,W,Hq,S,E]``, ``out [W,Hq,S,Ev]``;
    packed layout with ``cu_seqlens_q``: ``queries [F,total_q,Hq,E]``, ``out [total_q,Hq,Ev]``) and give it a
    workspace allocated with torch.  Returns ``(problem, keepalive)``; ``problem`` is ``None`` when the library
    refuses the shape."""
    import torch
    p = PagedProblem()
    packed = cu_seqlens_q is not None
    if packed:
        p.F, total_q, p.Hq, p.E = queries.shape
        p.W, p.S, p.total_q_tokens = cu_seqlens_q.numel() - 1, 0, total_q
    else:
        p.F, p.W, p.Hq, p.S, p.E = queries.shape
    p.Hkv, p.block_size, p.Ev = key_cache.shape[1], key_cache.shape[2], value_cache.shape[3]
    p.max_blocks_per_seq = block_table.shape[1]
    p.dtype, p.scale, p.kernel = dtype_code(out.dtype), float(scale), int(kernel)
    p.out, p.queries, p.locations = out.data_ptr(), queries.data_ptr(), locations.data_ptr()
    p.fragment_lengths, p.key_cache, p.value_cache = fragment_lengths.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr()
    p.block_table = block_table.data_ptr()
    p.cu_seqlens_q = cu_seqlens_q.data_ptr() if packed else None
    need = int(load().hogatt_paged_workspace_bytes(C.byref(p)))
    if need == 0:
        return None, None
    ws = torch.empty(need + 256, dtype=torch.uint8, device=out.device)
    p.workspace, p.workspace_bytes = ws.data_ptr() + (-ws.data_ptr()) % 256, need
    return p, [ws, out, queries, locations, fragment_lengths, key_cache, value_cache, block_table, cu_seqlens_q]


def launch_paged(problem: PagedProblem, stream: int = 0) -> int:
    """``hogatt_paged_sdpa_launch``: enqueue one call; returns the library's status code."""
    return int(load().hogatt_paged_sdpa_launch(C.byref(problem), C.c_void_p(stream)))


def paged_sdpa(*, stream: int = 0, **kw):
    """:func:`bind_paged` + :func:`launch_paged`; returns ``(status, keepalive)`` -- keep the second alive until the
    work has run."""
    p, keep = bind_paged(**kw)
    if p is None:
        return -1, None
    return launch_paged(p, stream), keep
