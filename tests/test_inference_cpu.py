"""Size binding, range inference and output shapes (what replaces tc2halide's bounds inference).
Known answers follow the rules the reference's inference tests pin (test/test_inference.cc:70-533):
a valid convolution has extent (H-KH)+1, a strided read A(i*s) has extent ceil(N/s), a shifted read
A(i+c) keeps the extent and moves the minimum to -c, later statements see the bounds of earlier
outputs."""
import pytest

from tensorcomprehensions_b200 import tclib
from tensorcomprehensions_b200 import workloads as wl


def shapes(tc, entry, ins, **kw):
    return tclib.infer_output_shapes(tc, entry, [list(s) for s in ins], **kw)


def test_benchmark_output_shapes():
    for name, expect in [("tensordot", [[32, 512, 2, 28, 28]]), ("batchmatmul", [[500, 26, 26]]),
                         ("tmm", [[128, 16384]]), ("group_conv", [[32, 32, 16, 14, 14]]),
                         ("mlp3", [[16384, 1024], [16384, 512], [16384, 256]])]:
        w = wl.ALL[name]()
        assert shapes(w.tc, w.entry, w.shapes) == expect


@pytest.mark.parametrize("tc,ins,expect", [
    ("def f(float(N, M) A) -> (O) { O(i, j) = A(i, j) }", [(5, 7)], [[5, 7]]),                    # copy
    ("def f(float(N, M) A) -> (O) { O(j, i) = A(i, j) }", [(5, 7)], [[7, 5]]),                    # transpose
    ("def f(float(N) A) -> (O) { O(i) = A(i * 123) }", [(1000,)], [[9]]),                         # scale: (N+122)/123
    ("def f(float(N) A) -> (O) { O(i) = A(i + 3) }", [(10,)], None),                              # shift: min -3, extent N
    ("def f(float(N) A) -> (O) { O(i) = A(i - 3) }", [(10,)], None),                              # shift: min 3, extent N
    ("def f(float(N, C, H, W) I, float(F, C, KH, KW) Wt) -> (O) { O(n, f, h, w) +=! I(n, c, h + kh, w + kw) * Wt(f, c, kh, kw) }",
     [(2, 3, 16, 12), (5, 3, 3, 5)], [[2, 5, 14, 8]]),                                            # conv: (H-KH)+1
    ("def f(float(N, C, H, W) I, float(F, C, KH, KW) Wt) -> (O) { O(n, f, h, w) +=! I(n, c, 2 * h + kh, 2 * w + kw) * Wt(f, c, kh, kw) }",
     [(1, 1, 9, 9), (1, 1, 3, 3)], [[1, 1, 4, 4]]),                                               # strided conv
    ("def f(float(N) A, float(M) B) -> (O) { O(i) = A(i) + B(i) }", [(8,), (5,)], [[5]]),         # intersection
    ("def f(float(N) A) -> (O) { O(i) = A(i) where i in 2:6 }", [(10,)], None),
    ("def f(float(N, K) A) -> (O, P) { O(i) +=! A(i, k)\n P(i) = O(i) * 2 }", [(4, 6)], [[4], [4]]),  # later stmt sees O
    ("def f(float(M, K) I, float(K, N) W1, float(N, P) W2) -> (O1, O2) { O1(m, n) +=! I(m, r_k) * W1(r_k, n)\n O2(m, p) +=! O1(m, r_n) * W2(r_n, p) }",
     [(3, 4), (4, 5), (5, 6)], [[3, 5], [3, 6]]),                                                 # two matmuls
    ("def f(float(N) A) -> (O) { O +=! A(i) }", [(9,)], [[]]),                                    # full reduction
])
def test_output_extents(tc, ins, expect):
    if expect is None:
        # ranges that do not start at 0: extent is max - min + 1 of the left-hand-side index
        a = tclib.analyze(tc, "f", [list(s) for s in ins])
        r = a["statements"][0]["ranges"]["i"]
        assert r in ((-3, 7), (3, 13), (2, 6))   # half-open; Shift1D / Shift1D2 of the reference
        assert a["outputs"][0][1] == [r[1] - r[0]]
        return
    assert shapes(tc, "f", ins) == expect


def test_ranges_of_group_convolution():
    a = tclib.analyze(wl.GROUP_CONV_TC, "group_convolution", [[32, 32, 16, 16, 16], [32, 16, 16, 3, 3], [32, 16]])
    r = a["statements"][0]["ranges"]
    assert r["h"] == (0, 14) and r["w"] == (0, 14) and r["r_kh"] == (0, 3) and r["r_c"] == (0, 16)
    assert a["statements"][0]["reduction"] == ["r_c", "r_kh", "r_kw"]
    assert a["sizes"] == {"N": 32, "G": 32, "C": 16, "H": 16, "W": 16, "F": 16, "KH": 3, "KW": 3}


@pytest.mark.parametrize("tc,ins,fragment", [
    ("def f(float(N, M) A, float(M, K) B) -> (O) { O(i, j) +=! A(i, k) * B(k, j) }", [(3, 4), (5, 6)], "Mismatched sizes for dimension M"),
    ("def f(float(N, 4) A) -> (O) { O(i) +=! A(i, j) }", [(3, 5)], "Constant dimension expected size 4 but found 5"),
    ("def f(float(N) A) -> (O) { O(i) = A(i) }", [(3,), (4,)], "expected 1 inputs but got 2"),
    ("def f(float(N, M) A) -> (O) { O(i) = A(i, 0) }", [(3,)], "expected a tensor with 2 dimensions but found 1"),
    ("def f(float(N) A, float(M) B) -> (O) { O(i) +=! A(j) * B(j + i) }", [(4,), (2,)], "Inferred an empty range"),
    ("def f(float(N) A) -> (O) { O(i, j) = A(i + j) }", [(4,)], "Could not infer ranges for free variables"),
])
def test_errors(tc, ins, fragment):
    with pytest.raises(tclib.ErrorReport) as e:
        shapes(tc, "f", ins)
    assert fragment in str(e.value)


def test_unchecked_precondition_warns_or_throws():
    tc = "def f(float(N) A) -> (O) { O(i) = A(i) + A(7) }"
    assert shapes(tc, "f", [(10,)]) == [[10]]           # 7 < 10: nothing to report
    with pytest.raises(tclib.ErrorReport, match="Required precondition will not be checked at runtime"):
        tclib.analyze(tc, "f", [[5]], [], True)          # throwWarnings


def test_dtype_propagation():
    tc = "def f(double(N) A, int32(N) B) -> (O, P) { O(i) = A(i) * B(i)\n P(i) = B(i) + 1 }"
    a = tclib.analyze(tc, "f", [[4], [4]], ["float64", "int32"])
    assert [(o[0], o[2]) for o in a["outputs"]] == [("O", "double"), ("P", "int32")]
