"""The CPU checker against ATen-CPU and against itself (no GPU)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tensorcomprehensions_b200 import workloads as wl


@pytest.mark.parametrize("name", list(wl.ALL))
def test_loop_nest_matches_aten(name):
    w = wl.ALL[name](**wl.SMALL[name])
    ins = wl.make_inputs(w)
    loop = orc.as_list(orc.LOOP[name](*ins))
    loop64 = orc.as_list(orc.LOOP[name](*ins, double=True))
    aten = orc.as_list(orc.ATEN[name](*ins))
    for a, d, b, L in zip(loop, loop64, aten, w.reduction):
        assert a.shape == tuple(b.shape)
        # both fp32 evaluations sit within the rounding budget of the fp64-accumulated one
        for x in (a, b):
            ok, err = orc.check_rtol_baseline(x, d, L, rtol=1e-6)
            assert ok, (name, err)


def test_loop_nest_tiny_by_hand():
    # 1x2x2x1x1 * 1x2x1x1x1 tensordot, values chosen so the answer is exact
    I0 = np.array([1, 2, 3, 4], np.float32).reshape(1, 2, 2, 1, 1)
    I1 = np.array([10, 100], np.float32).reshape(1, 2, 1, 1, 1)
    O = orc.loop_tensordot(I0, I1)
    assert O.reshape(-1).tolist() == [210.0, 430.0]
    # valid convolution extents: (H-KH)+1 (test/test_inference.cc:190-212)
    I = np.ones((1, 1, 1, 4, 5), np.float32)
    W = np.ones((1, 1, 1, 3, 2), np.float32)
    O = orc.loop_group_conv(I, W, np.array([[0.5]], np.float32))
    assert O.shape == (1, 1, 1, 2, 4) and np.all(O == 6.5)
    # fmax(x, 0) after the bias statement
    O = orc.loop_fcrelu(np.array([[1.0, -2.0]], np.float32), np.array([[1.0, 1.0], [-1.0, -1.0]], np.float32),
                        np.array([0.25, 0.25], np.float32))
    assert O.tolist() == [[0.0, 1.25]]


def test_pass_criteria_forms():
    ref = np.array([1.0, -4.0], np.float32)
    out = ref + np.array([0.0, 1e-4], np.float32)
    ok, e = orc.check_rtol_baseline(out, ref, 8)
    assert ok and abs(e - 2.5e-5) < 1e-6
    ok, e = orc.check_rtol_baseline(out, ref, 1)
    assert not ok
    ok, d, bound = orc.check_rtol_reference(out, ref, [ref], 8, 5e-7)
    assert not ok and bound == pytest.approx(8 * 5e-7 * 4.0)
