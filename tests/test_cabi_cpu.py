"""The C-ABI library loads without a GPU and exports every symbol its header declares."""
import ctypes
import os
import re

import pytest

from tensorcomprehensions_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tcb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tcb200_[a-z0-9_]+)\s*\(", text)))


def test_exports_every_declared_symbol():
    L = cabi.lib()
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(L, n), "libtcb200.so does not export " + n
    assert set(cabi.SYMBOLS) <= set(names)
    assert L.tcb200_abi_version() == 3


def test_strerror_and_argument_checks():
    L = cabi.lib()
    assert cabi.strerror(0) == "success"
    assert "no kernel" in cabi.strerror(-2)
    n = ctypes.c_int(0)
    assert L.tcb200_query(None, None, 0, ctypes.byref(n)) == -1
    bad = cabi.Problem()
    bad.family = 99
    assert L.tcb200_query(ctypes.byref(bad), None, 0, ctypes.byref(n)) == -1
    h = ctypes.c_void_p()
    assert L.tcb200_plan_create(ctypes.byref(bad), None, 0, ctypes.byref(h)) == -1 and not h


def test_query_and_plan_without_gpu():
    p = cabi.tensordot_problem(32, 512, 8, 2, 784)
    tiles = cabi.query(p)
    assert tiles and tiles[0].variant == cabi.VARIANT_SIMT and tiles[0].bm > 0
    assert tiles[0].stages >= 2                      # persistent bulk-copy kernel first
    plan = cabi.Plan(p, tiles[0])
    grid, block = plan.geometry()
    assert grid == (148, 1, 1) and block == (256, 1, 1)
    direct = [t for t in tiles if t.stages == 0 and t.bm > 0][0]
    grid, block = cabi.Plan(p, direct).geometry()
    assert grid[2] == 32 and block[0] * block[1] <= 256
    assert "tensordot" in plan.describe()
    # tensordot with an epilogue is not a kernel of the library: hard error, no fallback
    p.epilogue = cabi.EPI_BIAS
    with pytest.raises(cabi.Tcb200Error) as e:
        cabi.Plan(p)
    assert e.value.status == -2

    q = cabi.contraction_problem(500, 26, 26, 72, a_k_major=True, b_k_major=False)
    variants = [t.variant for t in cabi.query(q)]
    assert cabi.VARIANT_SIMT_SMALL in variants and cabi.VARIANT_SIMT in variants
    c = cabi.group_conv_problem(32, 32, 16, 16, 16, 16, 3, 3)
    plan = cabi.Plan(c)
    grid, block = plan.geometry()
    assert grid == (148, 1, 1) and block == (512, 1, 1)   # default: persistent tensor-core kernel, filter rows as accumulator rows
    assert "variant=tcgen05_ts tile=128x128x8 stages=3" in plan.describe()
    item = [t for t in cabi.query(c) if t.variant == cabi.VARIANT_SIMT and t.stages == 4 and t.threads == 128][0]
    grid, block = cabi.Plan(c, item).geometry()
    assert grid == (1024, 1, 1) and block == (128, 1, 1)  # item kernel: one CTA per (n, g), 2 channels per thread
    rows = [t for t in cabi.query(c) if t.variant == cabi.VARIANT_SIMT and t.bk == 2][0]
    assert cabi.Plan(c, rows).geometry()[0][:2] == (32, 16)  # rows kernel: one CTA per (g, pair of n)
    tcv = [t for t in cabi.query(c) if t.variant == cabi.VARIANT_TCGEN05_TS and t.stages == 4][0]
    pt = cabi.Plan(c, tcv)
    assert pt.geometry() == ((148, 1, 1), (448, 1, 1)) and "tcgen05_ts" in pt.describe()  # implicit GEMM, pixels x F
    rows = [t for t in cabi.query(c) if t.variant == cabi.VARIANT_TCGEN05_TS and t.stages == 3][0]
    pr = cabi.Plan(c, rows)   # filters stationary in tensor memory, filter rows as accumulator rows
    assert pr.geometry() == ((148, 1, 1), (512, 1, 1)) and "tile=128x128x8" in pr.describe()
    band = [t for t in cabi.query(c) if t.variant == cabi.VARIANT_SIMT and t.bk == 0 and t.stages == 0][0]
    assert cabi.Plan(c, band).geometry()[0][0] == 32 * 32


def test_reduction_plans_and_the_static_scratch_limit_without_a_device():
    """Planning needs no GPU; the no-allocation launch refuses an oversize plan (and a plan of another family)
    on the sizes alone, before any CUDA call."""
    p = cabi.reduction_problem(1, 1 << 26, 1)
    plan = cabi.Plan(p)
    grid, block = plan.geometry()
    assert block == (256, 1, 1) and grid[0] == 1 and grid[1] > 1          # one output tile, many segments
    assert "tcb200::reduction sum A=1 C=67108864 B=1" in plan.describe() and "stages=4" in plan.describe()
    assert cabi.Plan(cabi.reduction_problem(16384, 4096, 1)).geometry()[0][1] == 1  # warp per row: no segments
    odd = cabi.Plan(cabi.reduction_problem(3, 1001, 7))                    # no 128-bit loads possible
    assert "stages=1" in odd.describe()
    t = cabi.Tile()
    t.variant, t.bm, t.bn, t.stages = cabi.VARIANT_SIMT, 32, 512, 1
    big = cabi.Plan(cabi.reduction_problem(64, 1 << 16, 1024), t)          # 2048 tiles x 512 segments x 32 columns
    L = cabi.lib()
    null = ctypes.c_void_p(8)  # never dereferenced: the call must fail first
    assert L.tcb200_reduce_launch_static(big._h, null, null, None) == -7    # TCB200_ERR_TOO_LARGE
    other = cabi.Plan(cabi.contraction_problem(1, 64, 64, 64))
    assert L.tcb200_reduce_launch_static(other._h, null, null, None) == -1  # not a reduction plan
    bad = cabi.reduction_problem(0, 5, 1)
    with pytest.raises(cabi.Tcb200Error):
        cabi.Plan(bad)
