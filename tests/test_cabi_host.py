"""CPU-only checks of the C ABI: the library loads, exports what the header declares, and the
split-K decomposition covers every tile exactly once for any grid."""
import ctypes as C
import os
import re

import pytest

from inference_lib_b200 import _build, _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    _build.build_cabi()
    return _cabi.load()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "hogatt.h")).read()
    declared = set(re.findall(r"\b(hogatt_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_cabi.EXPORTS) | (declared - set(_cabi.EXPORTS))
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/hogatt.h but not exported"
    assert lib.hogatt_abi_version() == int(re.search(r"#define HOGATT_ABI_VERSION (\d+)", header).group(1))


def test_status_strings(lib):
    assert _cabi.status_string(0) == "ok"
    for rc in range(-11, 0):
        assert _cabi.status_string(rc) not in ("ok", "unknown status")
    assert _cabi.status_string(-99) == "unknown status"


def test_struct_layout_matches_the_header(lib):
    # 10 x 4-byte scalars, 7 pointers, 3 host-array pointers, workspace ptr + size, status ptr, 2 ints,
    # host_lengths pointer, stable_fragments + one reserved int
    assert C.sizeof(_cabi.Problem) == 40 + 8 * 7 + 8 * 3 + 16 + 8 + 8 + 8 + 8


def _describe(lib, visible, sms=148, **dims):
    p = _cabi.shape_problem(**dims)
    vis = (C.c_int32 * len(visible))(*visible)
    plan = (C.c_int32 * 8)()
    rc = lib.hogatt_plan_describe(C.byref(p), vis, sms, plan)
    return rc, list(plan)


def test_plan_for_the_headline_shapes(lib):
    rc, plan = _describe(lib, [8192, 2048, 2048, 2048, 2048], F=5, W=4, Hq=32, Hkv=8, E=128, Ev=128, S=1, dtype=_cabi.BF16)
    assert rc == 0
    tile, rows, row_blocks, th, units, ctas, parts, kernel = plan
    # 1,024 tiles: 128 CTAs of exactly 8 tiles (8 divides the 64 + 4 x 16 tiles of a unit), so that no CTA's range
    # crosses a fragment or kv-head boundary; the workspace keeps room for 148 // 8 + 2 partials per unit
    assert (tile, rows, row_blocks, th, units, ctas, parts, kernel) == (128, 16, 1, 128, 8, 128, 148 // 8 + 2, _cabi.KERNEL_MMA)
    # ragged lengths: no common tile count, balanced ranges over all SMs
    rc, plan = _describe(lib, [8192, 2000, 2100, 1500, 2048], F=5, W=4, Hq=32, Hkv=8, E=128, Ev=128, S=1, dtype=_cabi.BF16)
    assert rc == 0 and plan[5] == 148
    # the cluster launch shape only on request: one cluster of up to 16 CTAs per kv head, merged inside the kernel
    rc, plan = _describe(lib, [8192, 2048, 2048, 2048, 2048], F=5, W=4, Hq=32, Hkv=8, E=128, Ev=128, S=1, dtype=_cabi.BF16,
                         kernel=_cabi.KERNEL_MMA_CLUSTER)
    assert rc == 0 and plan[5] == 128 and plan[6] == 16 and plan[7] == _cabi.KERNEL_MMA_CLUSTER
    # long context: persistent grid over all SMs
    rc, plan = _describe(lib, [131072, 4096, 4096], F=3, W=2, Hq=32, Hkv=8, E=128, Ev=128, S=1, dtype=_cabi.BF16)
    assert rc == 0 and plan[3] == 1088 and plan[5] == 148 and plan[7] == _cabi.KERNEL_MMA   # 1088 tiles per head >= 64 chunks per head
    # the cluster shape needs at least two CTAs per unit
    rc, plan = _describe(lib, [1024], F=1, W=8, Hq=64, Hkv=8, E=128, Ev=128, S=16, dtype=_cabi.BF16, kernel=_cabi.KERNEL_MMA_CLUSTER)
    assert rc == -9
    rc, plan = _describe(lib, [256, 64, 64], F=3, W=2, Hq=8, Hkv=2, E=64, Ev=64, S=1, dtype=_cabi.F32)
    assert rc == 0 and plan[7] == _cabi.KERNEL_FMA and plan[0] == 32
    rc, plan = _describe(lib, [16384] + [1024] * 8, F=9, W=8, Hq=64, Hkv=8, E=128, Ev=128, S=16, dtype=_cabi.BF16)
    # 1,024 query rows per kv head: the tcgen05 kernel, 128-row blocks, 192 tiles of 128 keys per unit
    assert rc == 0 and plan[7] == _cabi.KERNEL_DENSE and plan[0] == 128 and plan[1] == 128 and plan[2] == 8 and plan[3] == 192 and plan[4] == 64
    rc, plan = _describe(lib, [16384] + [1024] * 8, F=9, W=8, Hq=64, Hkv=8, E=128, Ev=128, S=16, dtype=_cabi.BF16, kernel=_cabi.KERNEL_MMA)
    assert rc == 0 and plan[1] == 64 and plan[2] == 16 and plan[4] == 128


def test_plan_refuses_bad_problems(lib):
    assert _describe(lib, [8], F=1, W=1, Hq=3, Hkv=2, E=128, Ev=128, S=1, dtype=_cabi.BF16)[0] == -2
    assert _describe(lib, [8], F=1, W=1, Hq=2, Hkv=2, E=24, Ev=24, S=1, dtype=_cabi.BF16)[0] == -3
    assert _describe(lib, [8], F=1, W=1, Hq=2, Hkv=2, E=128, Ev=128, S=1, dtype=7)[0] == -4
    assert _describe(lib, [8] * 200, F=200, W=1, Hq=2, Hkv=2, E=128, Ev=128, S=1, dtype=_cabi.BF16)[0] == -5
    assert _describe(lib, [8], F=1, W=1, Hq=2, Hkv=2, E=128, Ev=128, S=1, dtype=_cabi.F32, kernel=_cabi.KERNEL_MMA)[0] == -9


@pytest.mark.parametrize("th,units,grid", [(1, 1, 148), (3, 2, 148), (256, 8, 148), (2176, 8, 148), (7, 128, 148),
                                           (13, 5, 4), (1, 200, 148), (19, 8, 148), (100, 3, 7), (5, 5, 25), (64, 1, 148)])
def test_ranges_tile_the_work_exactly_once(lib, th, units, grid):
    n = th * units
    ctas = min(grid, n)
    parts_bound = grid // units + 2
    rng = (C.c_int64 * 4)()
    covered = 0
    owners = {}
    for c in range(ctas):
        assert lib.hogatt_plan_ranges(th, units, ctas, c, 0, rng) == 0
        a, b = rng[0], rng[1]
        assert a == covered and b > a, "ranges must be contiguous and non-empty"
        covered = b
        for u in range(a // th, (b - 1) // th + 1):
            owners.setdefault(u, []).append(c)
    assert covered == n
    for u in range(units):
        assert lib.hogatt_plan_ranges(th, units, ctas, 0, u, rng) == 0
        first, count = rng[2], rng[3]
        assert owners[u] == list(range(first, first + count)), "partial slots must match the CTAs that touch the unit"
        assert count <= parts_bound, "more partials than the workspace reserves"


def test_cache_step_structs_match_the_header_and_refuse_bad_arguments(lib):
    # hogatt_step_plan: 4 ints, 3 pointers, float + int, 3 pointers; hogatt_append: 8 ints, 2 x (pointer + 3 strides),
    # 2 table pointers + 2 strides, 2 pointers, 2 ints, 3 host-array pointers, 3 pointers
    assert C.sizeof(_cabi.StepPlan) == 16 + 24 + 8 + 24
    assert C.sizeof(_cabi.Append) == 32 + 2 * (8 + 24) + 16 + 16 + 16 + 8 + 24 + 24
    assert lib.hogatt_step_plan_launch(None, None) == -1
    assert lib.hogatt_append_launch(None, None) == -1
    sp = _cabi.StepPlan()
    assert lib.hogatt_step_plan_launch(C.byref(sp), None) == -1          # no pointers at all
    ap = _cabi.Append()
    assert lib.hogatt_append_launch(C.byref(ap), None) == -1


def test_ctypes_mirrors_agree_with_the_compiler(tmp_path):
    """Every struct of include/hogatt.h, field by field, as a C compiler lays it out against its ctypes mirror: a
    plain C program that includes the header prints ``sizeof`` and every ``offsetof``."""
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    pairs = [("hogatt_problem", _cabi.Problem), ("hogatt_paged_problem", _cabi.PagedProblem), ("hogatt_peers", _cabi.Peers),
             ("hogatt_step_plan", _cabi.StepPlan), ("hogatt_append", _cabi.Append)]
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "hogatt.h"', "int main(void) {"]
    for cname, mirror in pairs:
        lines.append(f'  printf("{cname} sizeof %zu\\n", sizeof({cname}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([cc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    seen = {}
    for ln in out.splitlines():
        cname, field, value = ln.split()
        seen[(cname, field)] = int(value)
    for cname, mirror in pairs:
        assert seen[(cname, "sizeof")] == C.sizeof(mirror), cname
        for field, _ in mirror._fields_:
            assert seen[(cname, field)] == getattr(mirror, field).offset, (cname, field)


def test_short_calls_with_few_kv_heads_get_smaller_row_blocks(lib):
    """64 query rows per kv head, 2 kv heads: as one 64-row block a CTA would get 1.7 tiles behind the largest
    start-up; the plan cuts the rows into four 16-row blocks (8 units, 6.9 tiles per CTA).  Long contexts and shapes
    where the larger block wins keep it."""
    dims = dict(F=5, W=4, Hq=32, Hkv=2, E=128, Ev=128, S=1, dtype=_cabi.BF16)
    rc, plan = _describe(lib, [8192, 2048, 2048, 2048, 2048], **dims)
    assert rc == 0 and plan[7] == _cabi.KERNEL_MMA and (plan[1], plan[2], plan[4]) == (16, 4, 8)
    rc, plan = _describe(lib, [8 * 8192] + [8 * 2048] * 4, **dims)                  # 1,024 tiles per unit: every key once
    assert rc == 0 and (plan[1], plan[2], plan[4]) == (64, 1, 2)
    # 20 rows over 8 kv heads (GQA 5): one 32-row block stays faster than two of 16
    rc, plan = _describe(lib, [8192, 2048, 2048, 2048, 2048], F=5, W=4, Hq=40, Hkv=8, E=128, Ev=128, S=1, dtype=_cabi.BF16)
    assert rc == 0 and (plan[1], plan[2], plan[4]) == (32, 1, 8)
    # ... but not when the kv heads are spread over 8 GPUs (one head here: under one tile per CTA)
    rc, plan = _describe(lib, [8192, 2048, 2048, 2048, 2048], F=5, W=4, Hq=5, Hkv=1, E=128, Ev=128, S=1, dtype=_cabi.BF16)
    assert rc == 0 and (plan[1], plan[2], plan[4]) == (16, 2, 2)


@pytest.mark.parametrize("lengths,dims", [
    ([8192, 2048, 2048, 2048, 2048], dict(F=5, W=4, Hq=32, Hkv=8, E=128, Ev=128, S=1)),        # the north-star shape
    ([4096, 2048, 2048], dict(F=3, W=2, Hq=32, Hkv=8, E=128, Ev=128, S=1)),                    # cfg2
    ([8192, 2048, 2048, 2048, 2048], dict(F=5, W=4, Hq=16, Hkv=4, E=128, Ev=128, S=1)),        # one of two ranks' share
])
def test_aligned_ranges_stay_inside_one_fragment_of_one_unit(lib, lengths, dims):
    rc, plan = _describe(lib, lengths, dtype=_cabi.BF16, **dims)
    assert rc == 0
    tile, th, units, ctas = plan[0], plan[3], plan[4], plan[5]
    assert ctas < 148 and (th * units) % ctas == 0, "a whole number of tiles per CTA"
    bounds, acc = [], 0
    for n in lengths:
        acc += -(-n // tile)
        bounds.append(acc)
    rng = (C.c_int64 * 4)()
    for c in range(ctas):
        assert lib.hogatt_plan_ranges(th, units, ctas, c, 0, rng) == 0
        a, b = rng[0], rng[1] - 1                                   # first and last tile of the range
        assert a // th == b // th, "a range must not run on into the next kv head"
        seg = lambda t: next(i for i, e in enumerate(bounds) if t % th < e)
        assert seg(a) == seg(b), "a range must not run on into the next fragment"
