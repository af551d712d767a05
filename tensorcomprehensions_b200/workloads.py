"""The five benchmark comprehensions: TC text, shapes, seeded synthetic inputs, work counts.

Shapes come from the reference's own benchmark / test cases (tensordot:
test/cuda/test_tc_mapper.cc:282-300; batchmatmul: tc/benchmarks/batchmatmul.cc:122-126;
transposed matmul: tc/benchmarks/tmm.cc:138-142; group convolution and MLP3 follow
tc/benchmarks/group_convolution.cc:124-132 and tc/benchmarks/MLP_model.cc:547-560 at
the sizes this build is measured on).  Inputs are synthetic, drawn from a seeded CPU
generator so the CPU checker and the GPU see identical bits.
"""
import math
from collections import namedtuple

TENSORDOT_TC = """
def tensordot(float(N, C1, C2, H, W) I0, float(N, C2, C3, H, W) I1) -> (O) {
    O(n, c1, c3, h, w) +=! I0(n, c1, r_c2, h, w) * I1(n, r_c2, c3, h, w)
}
"""

BATCHMATMUL_TC = """
def batch_matmul(float(B, N, M) X, float(B, M, K) Y) -> (Z) {
    Z(b, n, k) +=! X(b, n, r_m) * Y(b, r_m, k)
}
"""

TMM_TC = """
def tmm(float(M, K) A, float(N, K) B) -> (C) {
    C(m, n) +=! A(m, r_k) * B(n, r_k)
}
"""

GROUP_CONV_TC = """
def group_convolution(float(N, G, C, H, W) I, float(G, F, C, KH, KW) W1, float(G, F) B) -> (O) {
    O(n, g, f, h, w) +=! I(n, g, r_c, h + r_kh, w + r_kw) * W1(g, f, r_c, r_kh, r_kw)
    O(n, g, f, h, w)  = O(n, g, f, h, w) + B(g, f)
}
"""

MLP3_TC = """
def mlp3(float(B, N) I, float(O, N) W2, float(O) B2, float(P, O) W3, float(P) B3,
         float(Q, P) W4, float(Q) B4) -> (O2, O3, O4) {
    O2(b, o) +=! I(b, n) * W2(o, n)
    O2(b, o)  = O2(b, o) + B2(o)
    O2(b, o)  = fmax(O2(b, o), 0)
    O3(b, p) +=! O2(b, o) * W3(p, o)
    O3(b, p)  = O3(b, p) + B3(p)
    O3(b, p)  = fmax(O3(b, p), 0)
    O4(b, q) +=! O3(b, p) * W4(q, p)
    O4(b, q)  = O4(b, q) + B4(q)
    O4(b, q)  = fmax(O4(b, q), 0)
}
"""

# shard_inputs: per input, the dimension that is split across GPUs (None = replicated);
# shard_outputs: per output, the dimension the shards concatenate along.
Workload = namedtuple("Workload", "name index tc entry shapes dist shard_inputs shard_outputs reduction bytes flops bound")


def _prod(s):
    r = 1
    for x in s:
        r *= x
    return r


def tensordot(N=32, C1=512, C2=8, C3=2, H=28, W=28):
    shapes = [(N, C1, C2, H, W), (N, C2, C3, H, W)]
    out = N * C1 * C3 * H * W
    return Workload("tensordot", 1, TENSORDOT_TC, "tensordot", shapes, ["uniform", "uniform"], [0, 0], [0], [C2],
                    4 * (_prod(shapes[0]) + _prod(shapes[1]) + out), 2 * out * C2, "hbm")


def batchmatmul(B=500, N=26, M=72, K=26):
    shapes = [(B, N, M), (B, M, K)]
    out = B * N * K
    return Workload("batchmatmul", 2, BATCHMATMUL_TC, "batch_matmul", shapes, ["normal", "normal"], [0, 0], [0], [M],
                    4 * (_prod(shapes[0]) + _prod(shapes[1]) + out), 2 * out * M, "hbm")


def tmm(M=128, N=16384, K=4096):
    shapes = [(M, K), (N, K)]
    out = M * N
    # N is the sharded index: B's rows are sharded (dim 0), A is replicated (None)
    return Workload("tmm", 3, TMM_TC, "tmm", shapes, ["normal", "normal"], [None, 0], [1], [K],
                    4 * (_prod(shapes[0]) + _prod(shapes[1]) + out), 2 * out * K, "tensor")


def group_conv(N=32, G=32, C=16, F=16, H=16, W=16, KH=3, KW=3):
    shapes = [(N, G, C, H, W), (G, F, C, KH, KW), (G, F)]
    out = N * G * F * (H - KH + 1) * (W - KW + 1)
    return Workload("group_conv", 4, GROUP_CONV_TC, "group_convolution", shapes,
                    ["uniform", "uniform", "uniform"], [0, None, None], [0], [C * KH * KW],
                    4 * (sum(_prod(s) for s in shapes) + out), 2 * out * C * KH * KW + out, "hbm")


def mlp3(B=16384, N=2048, O=1024, P=512, Q=256):
    shapes = [(B, N), (O, N), (O,), (P, O), (P,), (Q, P), (Q,)]
    dist = ["normal", ("normal", 1 / math.sqrt(N)), ("normal", 1 / math.sqrt(N)),
            ("normal", 1 / math.sqrt(O)), ("normal", 1 / math.sqrt(O)),
            ("normal", 1 / math.sqrt(P)), ("normal", 1 / math.sqrt(P))]
    outs = B * (O + P + Q)
    return Workload("mlp3", 5, MLP3_TC, "mlp3", shapes, dist, [0, None, None, None, None, None, None], [0, 0, 0],
                    [N, O, P], 4 * (sum(_prod(s) for s in shapes) + outs),
                    2 * B * (N * O + O * P + P * Q), "tensor")


ALL = {"tensordot": tensordot, "batchmatmul": batchmatmul, "tmm": tmm, "group_conv": group_conv,
       "mlp3": mlp3}

# Reductions (not part of the five-comprehension suite; `bench.py --workload <name>` measures one alone):
# the reference's sum1D / sum2D (test/test_tc_mapper_harness-inl.h:60-146) at sizes that stream 256 MB,
# and the column-sum form.
SUM1D_TC = """
def sum1D(float(M) A) -> (C) {
    C +=! A(r_m)
}
"""
SUM2D_TC = """
def sum2D(float(M, N) A) -> (C) {
    C(m) +=! A(m, r_n)
}
"""
COLSUM_TC = """
def colsum(float(M, N) A) -> (C) {
    C(n) +=! A(r_m, n)
}
"""


def sum1d(M=1 << 26):
    return Workload("sum1d", 6, SUM1D_TC, "sum1D", [(M,)], ["uniform"], [None], [None], [M], 4 * (M + 1), M, "hbm")


def sum2d(M=16384, N=4096):
    return Workload("sum2d", 7, SUM2D_TC, "sum2D", [(M, N)], ["uniform"], [0], [0], [N], 4 * (M * N + M), M * N, "hbm")


def colsum(M=16384, N=4096):
    return Workload("colsum", 8, COLSUM_TC, "colsum", [(M, N)], ["uniform"], [None], [None], [M], 4 * (M * N + N), M * N,
                    "hbm")


EXTRA = {"sum1d": sum1d, "sum2d": sum2d, "colsum": colsum}

# The size argument of each factory that is split across GPUs (the output index that also indexes the large
# operand): a rank's shard of a comprehension is the same comprehension at a smaller extent.
SHARD_ARG = {"tensordot": "N", "batchmatmul": "B", "tmm": "N", "group_conv": "N", "mlp3": "B"}


def shard_of(name, world, rank):
    """The Workload a rank of a `world`-GPU run compiles: extent / world of the sharded index, the remainder
    on the first ranks (500 matrices over 8 GPUs -> 63, 63, 63, 63, 62, 62, 62, 62)."""
    full = ALL[name]()
    if world == 1:
        return full
    dim = next(d for d in full.shard_inputs if d is not None)
    big = next(s for s, d in zip(full.shapes, full.shard_inputs) if d is not None)
    base, rem = divmod(big[dim], world)
    return ALL[name](**{SHARD_ARG[name]: base + (1 if rank < rem else 0)})
BY_NAME = dict(ALL, **EXTRA)

# Small instances of the same comprehensions for quick parity checks (odd sizes on purpose).
SMALL = {
    "tensordot": dict(N=3, C1=20, C2=8, C3=2, H=6, W=10),
    "batchmatmul": dict(B=7, N=26, M=72, K=26),
    "tmm": dict(M=70, N=200, K=132),
    "group_conv": dict(N=2, G=3, C=16, F=16, H=16, W=16),
    "mlp3": dict(B=130, N=96, O=80, P=48, Q=24),
}


def make_inputs(w, seed=None, device="cpu"):
    """Seeded CPU draws (seed 20240 + workload index), optionally copied to `device`."""
    import torch
    g = torch.Generator().manual_seed(20240 + w.index if seed is None else seed)
    out = []
    for shape, d in zip(w.shapes, w.dist):
        scale = 1.0
        if isinstance(d, tuple):
            d, scale = d
        if d == "uniform":
            t = torch.rand(shape, generator=g, dtype=torch.float32)
        else:
            t = torch.randn(shape, generator=g, dtype=torch.float32)
        if scale != 1.0:
            t = t * scale
        out.append(t.to(device) if device != "cpu" else t)
    return out


def make_shard_inputs(name, world, rank):
    """Seeded inputs of one rank's shard.  Every tensor is drawn from its own generator: a replicated operand
    (weights, the A of the transposed matmul) gets the same bits on every rank, a sharded operand a
    rank-specific draw of its shard shape.  Returns (shard workload, tensors)."""
    import torch
    w = shard_of(name, world, rank)
    out = []
    for k, (shape, d, sd) in enumerate(zip(w.shapes, w.dist, w.shard_inputs)):
        g = torch.Generator().manual_seed(20240 + 100 * w.index + k + (1000 * rank if sd is not None else 0))
        scale = 1.0
        if isinstance(d, tuple):
            d, scale = d
        t = torch.rand(shape, generator=g) if d == "uniform" else torch.randn(shape, generator=g)
        out.append(t * scale if scale != 1.0 else t)
    return w, out
