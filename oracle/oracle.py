"""Python face of the CPU checker.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the cpu_baseline / reference legs of the benchmark may
import this module; the product never does.

Two independent references per comprehension:
  * loop_*  : the C loop-nest restatement (tc_oracle.c; cites the reference lines it follows),
  * aten_*  : ATen on CPU, the library the reference's own harness compares against
              (X.bmm(Y) tc/benchmarks/batchmatmul.cc:67; A.mm(B.t()) tc/benchmarks/tmm.cc:66;
              I.mm(W.t()).add(B).clamp_min(0) tc/benchmarks/MLP_model.cc:537-541; grouped conv
              == Caffe2 Conv(group=G) tc/benchmarks/group_convolution.cc:83-101).  Tensordot has
              no ATen reference in the repo (python/tests/test_tc.py:512-517): einsum is used.
and the two forms of the pass criterion:
  * check_rtol_reference : test/test_harness_aten.h:36-54  (max|diff| < nOps * eps * max|inputs|)
  * check_rtol_baseline  : max|out-ref| / max|ref| <= 1e-5 * reduction length
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "libtc_oracle.so")
        if not os.path.exists(path):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_oracle_build", os.path.join(HERE, "build.py"))
            m = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(m)
            m.build_oracle()
        _lib = ctypes.CDLL(path)
    return _lib


def _np(t):
    if hasattr(t, "detach"):
        t = t.detach().cpu().numpy()
    return np.ascontiguousarray(t, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


_i64 = ctypes.c_int64


def loop_tensordot(I0, I1, double=False):
    I0, I1 = _np(I0), _np(I1)
    N, C1, C2, H, W = I0.shape
    C3 = I1.shape[2]
    assert I1.shape == (N, C2, C3, H, W)
    O = np.empty((N, C1, C3, H, W), np.float32)
    lib().oracle_tensordot_f32(_p(I0), _p(I1), _p(O), _i64(N), _i64(C1), _i64(C2), _i64(C3), _i64(H),
                               _i64(W), int(double))
    return O


def loop_batchmatmul(X, Y, double=False):
    X, Y = _np(X), _np(Y)
    B, N, M = X.shape
    K = Y.shape[2]
    assert Y.shape == (B, M, K)
    Z = np.empty((B, N, K), np.float32)
    lib().oracle_batchmatmul_f32(_p(X), _p(Y), _p(Z), _i64(B), _i64(N), _i64(M), _i64(K), int(double))
    return Z


def loop_tmm(A, B, double=False):
    A, B = _np(A), _np(B)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape == (N, K)
    C = np.empty((M, N), np.float32)
    lib().oracle_tmm_f32(_p(A), _p(B), _p(C), _i64(M), _i64(N), _i64(K), int(double))
    return C


def loop_group_conv(I, W1, Bias=None, double=False, stride=(1, 1)):
    I, W1 = _np(I), _np(W1)
    Bias = _np(Bias) if Bias is not None else None
    N, G, C, H, W = I.shape
    _, F, _, KH, KW = W1.shape
    assert W1.shape == (G, F, C, KH, KW)
    SH, SW = stride
    O = np.empty((N, G, F, (H - KH) // SH + 1, (W - KW) // SW + 1), np.float32)
    lib().oracle_group_conv_strided_f32(_p(I), _p(W1), _p(Bias), _p(O), _i64(N), _i64(G), _i64(C), _i64(F),
                                        _i64(H), _i64(W), _i64(KH), _i64(KW), _i64(SH), _i64(SW), int(double))
    return O


def loop_reduce(I, double=False):
    """Sum over the middle axis of a 3-D [A, C, B] array (the family's canonical view)."""
    I = _np(I)
    A, C, B = I.shape
    O = np.empty((A, B), np.float32)
    lib().oracle_reduce_f32(_p(I), _p(O), _i64(A), _i64(C), _i64(B), int(double))
    return O


def loop_reduce_op(I, op):
    """max (1), min (2) or product (3) over the middle axis of a 3-D [A, C, B] array, accumulated in double."""
    I = _np(I)
    A, C, B = I.shape
    O = np.empty((A, B), np.float32)
    lib().oracle_reduce_op_f32(_p(I), _p(O), _i64(A), _i64(C), _i64(B), int(op))
    return O


def loop_fcrelu(I, W1, Bias=None, relu=True, double=False):
    I, W1 = _np(I), _np(W1)
    Bias = _np(Bias) if Bias is not None else None
    B, M = I.shape
    N = W1.shape[0]
    assert W1.shape == (N, M)
    O = np.empty((B, N), np.float32)
    lib().oracle_fcrelu_f32(_p(I), _p(W1), _p(Bias), _p(O), _i64(B), _i64(N), _i64(M), int(relu),
                            int(double))
    return O


def loop_mlp3(I, W2, B2, W3, B3, W4, B4, double=False):
    O2 = loop_fcrelu(I, W2, B2, True, double)
    O3 = loop_fcrelu(O2, W3, B3, True, double)
    O4 = loop_fcrelu(O3, W4, B4, True, double)
    return O2, O3, O4


# ---- ATen CPU ---------------------------------------------------------------------------

def aten_tensordot(I0, I1):
    import torch
    return torch.einsum("nakhw,nkchw->nachw", I0, I1)


def aten_batchmatmul(X, Y):
    return X.bmm(Y)


def aten_tmm(A, B):
    return A.mm(B.t())


def aten_group_conv(I, W1, Bias=None, stride=(1, 1)):
    import torch
    N, G, C, H, W = I.shape
    _, F, _, KH, KW = W1.shape
    out = torch.nn.functional.conv2d(I.reshape(N, G * C, H, W), W1.reshape(G * F, C, KH, KW),
                                     Bias.reshape(G * F) if Bias is not None else None, stride=stride, groups=G)
    return out.reshape(N, G, F, (H - KH) // stride[0] + 1, (W - KW) // stride[1] + 1)


def aten_mlp3(I, W2, B2, W3, B3, W4, B4):
    O2 = I.mm(W2.t()).add(B2).clamp_min(0)
    O3 = O2.mm(W3.t()).add(B3).clamp_min(0)
    O4 = O3.mm(W4.t()).add(B4).clamp_min(0)
    return O2, O3, O4


LOOP = {"tensordot": loop_tensordot, "batchmatmul": loop_batchmatmul, "tmm": loop_tmm,
        "group_conv": loop_group_conv, "mlp3": loop_mlp3}
ATEN = {"tensordot": aten_tensordot, "batchmatmul": aten_batchmatmul, "tmm": aten_tmm,
        "group_conv": aten_group_conv, "mlp3": aten_mlp3,
        "sum1d": lambda A: A.sum(), "sum2d": lambda A: A.sum(1), "colsum": lambda A: A.sum(0)}


def as_list(x):
    return list(x) if isinstance(x, (tuple, list)) else [x]


# ---- pass criteria ------------------------------------------------------------------------

def rel_err_baseline(out, ref):
    out, ref = _np(out).astype(np.float64), _np(ref).astype(np.float64)
    denom = np.abs(ref).max()
    return float(np.abs(out - ref).max() / (denom if denom > 0 else 1.0))


def check_rtol_baseline(out, ref, reduction_length, rtol=1e-5):
    """max|out - ref| / max|ref| <= rtol * reduction length."""
    e = rel_err_baseline(out, ref)
    return e <= rtol * reduction_length, e


def check_rtol_reference(out, ref, inputs, n_operations, precision):
    """test/test_harness_aten.h:36-54: max|diff| < nOperations * precision * max over inputs of max|input|."""
    out, ref = _np(out).astype(np.float64), _np(ref).astype(np.float64)
    max_value = max(float(np.abs(_np(t)).max()) for t in inputs)
    max_diff = float(np.abs(out - ref).max())
    return max_diff < n_operations * precision * max_value, max_diff, n_operations * precision * max_value
