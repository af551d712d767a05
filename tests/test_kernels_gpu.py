"""Parity of the CUDA kernels (through the C ABI) with the CPU checker.  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tensorcomprehensions_b200 import cabi
from tensorcomprehensions_b200 import workloads as wl

from helpers import STRICT, assert_close, run_plan

pytestmark = pytest.mark.gpu


def _rand(shape, seed, dist="normal"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn if dist == "normal" else torch.rand)(shape, generator=g, dtype=torch.float32)


# ---------------------------------------------------------------- tensordot (K2)

@pytest.mark.parametrize("dims", [
    (3, 20, 8, 2, 6, 10),    # vec4 kernel, ragged c1 chunk
    (2, 5, 8, 2, 28, 28),    # benchmark inner sizes
    (16, 8, 16, 2, 17, 25),  # README sizes: P=425 odd -> generic kernel
    (4, 9, 7, 3, 16, 14),    # C2=7, C3=3 -> generic kernel
    (2, 5, 11, 16, 10, 10),  # large C3
    (1, 1, 1, 1, 1, 1),      # degenerate
    (2, 33, 4, 4, 2, 2),     # P4 = 1
])
def test_tensordot_small(cuda, dims):
    N, C1, C2, C3, H, W = dims
    I0, I1 = _rand((N, C1, C2, H, W), 1, "uniform"), _rand((N, C2, C3, H, W), 2, "uniform")
    ref = orc.loop_tensordot(I0, I1)
    p = cabi.tensordot_problem(N, C1, C2, C3, H * W)
    for tile in [None] + cabi.query(p):
        out, plan = run_plan(p, [I0.to(cuda), I1.to(cuda)], ref.shape, tile)
        assert_close(out, ref, C2, [I0, I1], STRICT["tensordot"], plan.describe())


def test_tensordot_unaligned_views(cuda):
    N, C1, C2, C3, H, W = 2, 6, 8, 2, 4, 4
    I0, I1 = _rand((N, C1, C2, H, W), 3), _rand((N, C2, C3, H, W), 4)
    ref = orc.loop_tensordot(I0, I1)
    buf = torch.empty(I0.numel() + 1, device=cuda)
    v = buf[1:].view(I0.shape)  # 4-byte aligned only
    v.copy_(I0)
    p = cabi.tensordot_problem(N, C1, C2, C3, H * W)
    out, plan = run_plan(p, [v, I1.to(cuda)], ref.shape)
    assert_close(out, ref, C2, what="unaligned I0")


def test_tensordot_full_size(cuda):
    w = wl.tensordot()
    I0, I1 = wl.make_inputs(w)
    p = cabi.tensordot_problem(32, 512, 8, 2, 784)
    out, plan = run_plan(p, [I0.to(cuda), I1.to(cuda)], (32, 512, 2, 28, 28))
    ref = orc.loop_tensordot(I0, I1)
    assert_close(out, ref, 8, [I0, I1], STRICT["tensordot"], plan.describe())
    assert_close(out, orc.aten_tensordot(I0, I1), 8, what="vs einsum")
    # linearity in I0 (size-independent property): f(2*I0) == 2*f(I0) exactly in binary fp
    out2, _ = run_plan(p, [(2 * I0).to(cuda), I1.to(cuda)], (32, 512, 2, 28, 28))
    assert torch.equal(out2, 2 * out)


# ---------------------------------------------------------------- contraction (K1), SIMT variants

def _contraction_ref(A, B, a_k, b_k):
    # logical A(b,m,k), B(b,n,k)
    Al = A if a_k else A.transpose(-1, -2)
    Bl = B if b_k else B.transpose(-1, -2)
    return torch.matmul(Al.double(), Bl.double().transpose(-1, -2)).float()


@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("shape", [(1, 70, 200, 132), (3, 65, 63, 17), (2, 4, 4, 1), (1, 128, 256, 64)])
def test_contraction_simt_forms(cuda, a_k, b_k, shape):
    b, M, N, K = shape
    A = _rand((b, M, K) if a_k else (b, K, M), 5)
    B = _rand((b, N, K) if b_k else (b, K, N), 6)
    ref = _contraction_ref(A, B, a_k, b_k)
    p = cabi.contraction_problem(b, M, N, K, a_k, b_k)
    t = cabi.Tile()
    t.variant = cabi.VARIANT_SIMT
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (b, M, N), t)
    assert_close(out, ref, K, [A, B], 3e-7, plan.describe())


def test_batchmatmul_all_tiles(cuda):
    w = wl.batchmatmul()
    X, Y = wl.make_inputs(w)
    ref = orc.loop_batchmatmul(X, Y)
    p = cabi.contraction_problem(500, 26, 26, 72, a_k_major=True, b_k_major=False)
    tiles = cabi.query(p)
    assert tiles[0].variant == cabi.VARIANT_SIMT_SMALL
    for tile in [None] + tiles:
        out, plan = run_plan(p, [X.to(cuda), Y.to(cuda)], (500, 26, 26), tile)
        assert_close(out, ref, 72, [X, Y], STRICT["batchmatmul"], plan.describe())
        assert_close(out, orc.aten_batchmatmul(X, Y), 72, what="vs bmm")


@pytest.mark.parametrize("shape", [(7, 26, 26, 72), (5, 15, 21, 40), (3, 1, 1, 1), (4, 33, 31, 7)])
def test_batchmatmul_small_kernel_ragged(cuda, shape):
    b, M, N, K = shape
    X, Y = _rand((b, M, K), 7), _rand((b, K, N), 8)
    ref = orc.loop_batchmatmul(X, Y)
    p = cabi.contraction_problem(b, M, N, K, True, False)
    t = cabi.Tile()
    t.variant = cabi.VARIANT_SIMT_SMALL
    out, plan = run_plan(p, [X.to(cuda), Y.to(cuda)], (b, M, N), t)
    assert_close(out, ref, K, [X, Y], 3e-7, plan.describe())


@pytest.mark.parametrize("epi", [cabi.EPI_NONE, cabi.EPI_BIAS, cabi.EPI_BIAS_RELU, cabi.EPI_RELU])
def test_contraction_simt_epilogues_and_accumulate(cuda, epi):
    M, N, K = 50, 72, 96
    I, W, b = _rand((M, K), 9), _rand((N, K), 10), _rand((N,), 11)
    has_bias = epi in (cabi.EPI_BIAS, cabi.EPI_BIAS_RELU)
    ref = orc.loop_fcrelu(I, W, b if has_bias else None, relu=epi in (cabi.EPI_BIAS_RELU, cabi.EPI_RELU))
    p = cabi.contraction_problem(1, M, N, K, True, True, epilogue=epi)
    t = cabi.Tile()
    t.variant = cabi.VARIANT_SIMT
    ins = [I.to(cuda), W.to(cuda)] + ([b.to(cuda)] if has_bias else [])
    out, plan = run_plan(p, ins, (M, N), t)
    assert_close(out, ref, K, what=plan.describe())
    if epi == cabi.EPI_NONE:
        # "+=" keeps what the output holds (test/cuda/test_compile_and_run.cc:181-200)
        p2 = cabi.contraction_problem(1, M, N, K, True, True, accumulate=True)
        init = _rand((M, N), 12).to(cuda)
        out2, _ = run_plan(p2, ins, (M, N), t, out_init=init)
        assert_close(out2, ref + init.cpu().numpy(), K, what="accumulate")


def test_contraction_shared_operand_and_padded_ld(cuda):
    # stride 0: every batch entry multiplies the same B; padded leading dimensions
    b, M, N, K = 3, 20, 24, 36
    A = _rand((b, M, K + 4), 13)
    B = _rand((N, K + 8), 14)
    ref = torch.matmul(A[:, :, :K].double(), B[:, :K].double().t()).float()
    p = cabi.contraction_problem(b, M, N, K, True, True, lda=K + 4, ldb=K + 8, ldc=N,
                                 stride_a=M * (K + 4), stride_b=0, stride_c=M * N)
    t = cabi.Tile()
    t.variant = cabi.VARIANT_SIMT
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (b, M, N), t)
    assert_close(out, ref, K, what=plan.describe())


# ---------------------------------------------------------------- group convolution (K3)

@pytest.mark.parametrize("dims", [
    (2, 3, 16, 16, 16, 16, 3, 3),
    (3, 2, 8, 12, 16, 16, 3, 3),    # item kernel: C=8, F=12
    (2, 2, 4, 4, 16, 16, 1, 3),     # item kernel: one filter row, 16 output rows
    (1, 2, 4, 16, 16, 16, 5, 2),    # item kernel: 12 output rows, 15 output columns -> not eligible (rows kernel)
    (1, 2, 4, 4, 56, 56, 3, 3),     # reference benchmark shape family, large image -> row bands
    (2, 2, 3, 5, 9, 7, 3, 3),       # F not a multiple of 4, odd sizes
    (1, 1, 1, 1, 3, 3, 3, 3),       # single output pixel
    (2, 2, 8, 4, 6, 6, 1, 1),       # 1x1 filter
    (1, 2, 4, 8, 8, 10, 5, 2),      # non-square filter
    (3, 2, 8, 16, 12, 20, 3, 3),    # tensor-core form: C=8, wide rows
    (2, 2, 16, 32, 10, 8, 5, 2),    # tensor-core form: F=32, non-square filter
    (5, 3, 16, 16, 9, 12, 1, 1),    # tensor-core form: 1x1 filter, odd item count
    (1, 1, 16, 16, 24, 20, 3, 3),   # tensor-core form: four pixel tiles
    (3, 2, 8, 8, 16, 16, 3, 3),     # filter-row tensor-core form: C = F = 8
    (5, 3, 16, 8, 11, 16, 3, 2),    # ... 11 input rows (two units, the second short), 15 output columns
    (4, 2, 8, 16, 8, 16, 3, 1),     # ... one unit per item, one filter column
    (9, 50, 16, 8, 12, 16, 3, 2),   # ... three items per CTA, group changes inside a CTA's run
    (37, 32, 8, 8, 16, 16, 3, 3),   # ... eight items per CTA: every ring of the kernel wraps several times
])
@pytest.mark.parametrize("bias", [True, False])
def test_group_conv_small(cuda, dims, bias):
    N, G, C, F, H, W, KH, KW = dims
    I, W1, B = _rand((N, G, C, H, W), 15, "uniform"), _rand((G, F, C, KH, KW), 16, "uniform"), _rand((G, F), 17)
    ref = orc.loop_group_conv(I, W1, B if bias else None)
    p = cabi.group_conv_problem(*dims, epilogue=cabi.EPI_BIAS if bias else cabi.EPI_NONE)
    ins = [I.to(cuda), W1.to(cuda)] + ([B.to(cuda)] if bias else [])
    for tile in [None] + cabi.query(p):
        out, plan = run_plan(p, ins, ref.shape, tile)
        assert_close(out, ref, C * KH * KW, [I, W1], STRICT["group_conv"], plan.describe())


@pytest.mark.parametrize("dims,stride", [
    ((2, 3, 4, 8, 11, 11, 3, 3), (2, 2)),
    ((2, 1, 3, 4, 10, 9, 3, 3), (3, 2)),     # ragged: the last rows / columns of the image are never read
    ((1, 2, 16, 16, 16, 16, 3, 3), (2, 1)),  # item-kernel shape, but strided: band kernel only
    ((1, 2, 8, 5, 40, 64, 5, 5), (2, 2)),    # several bands per image, F not a multiple of 4
    ((3, 2, 4, 4, 7, 7, 7, 7), (4, 4)),      # filter as large as the image: one output pixel
])
def test_group_conv_strided(cuda, dims, stride):
    """I(.., SH*h+kh, SW*w+kw): the strides of tc/library/convolution.h:27-31 against the loop nest and
    against conv2d."""
    N, G, C, F, H, W, KH, KW = dims
    I, W1, B = _rand((N, G, C, H, W), 35, "uniform"), _rand((G, F, C, KH, KW), 36, "uniform"), _rand((G, F), 37)
    ref = orc.loop_group_conv(I, W1, B, stride=stride)
    p = cabi.group_conv_problem(*dims, stride=stride)
    tiles = cabi.query(p)
    assert all(t.variant == cabi.VARIANT_SIMT and t.bk == 0 for t in tiles)  # band kernel only
    for tile in [None] + tiles:
        out, plan = run_plan(p, [I.to(cuda), W1.to(cuda), B.to(cuda)], ref.shape, tile)
        assert "stride=" in plan.describe()
        assert_close(out, ref, C * KH * KW, [I, W1], STRICT["group_conv"], plan.describe())
    assert_close(out, orc.aten_group_conv(I, W1, B, stride=stride), C * KH * KW, what="vs conv2d")


@pytest.mark.parametrize("bias", [True, False])
def test_group_conv_accumulate(cuda, bias):
    """`+=` without `!`: O = epilogue(O_in + conv) for every tile the family lists."""
    dims = (2, 3, 16, 16, 16, 16, 3, 3)
    N, G, C, F, H, W, KH, KW = dims
    I, W1, B = _rand((N, G, C, H, W), 25, "uniform"), _rand((G, F, C, KH, KW), 26, "uniform"), _rand((G, F), 27)
    init = _rand((N, G, F, H - KH + 1, W - KW + 1), 28)
    ref = orc.loop_group_conv(I, W1, None) + init.numpy() + (B.numpy()[None, :, :, None, None] if bias else 0)
    p = cabi.group_conv_problem(*dims, epilogue=cabi.EPI_BIAS if bias else cabi.EPI_NONE, accumulate=True)
    ins = [I.to(cuda), W1.to(cuda)] + ([B.to(cuda)] if bias else [])
    for tile in [None] + cabi.query(p):
        out, plan = run_plan(p, ins, ref.shape, tile, out_init=init.to(cuda))
        assert_close(out, ref, C * KH * KW, what=plan.describe())


@pytest.mark.parametrize("dims", [
    (40, 16, 8, 12, 16, 16, 3, 3),    # 640 items: five per CTA, three channel quads, ragged last CTA
    (37, 17, 4, 4, 16, 16, 1, 3),     # filter height read at run time, 16 output rows, runs that cross a group
    (32, 32, 16, 16, 16, 16, 3, 3),   # the benchmark shape: seven items per CTA
])
def test_group_conv_multi_item_kernel(cuda, dims):
    """A run of items per CTA (a sweep tile from about four items per SM on): threads numbered densely over
    (item, channel quad, row), filters of up to two groups per CTA, output through bulk copies."""
    N, G, C, F, H, W, KH, KW = dims
    I, W1, B = _rand((N, G, C, H, W), 55, "uniform"), _rand((G, F, C, KH, KW), 56, "uniform"), _rand((G, F), 57)
    ref = orc.aten_group_conv(I, W1, B)
    for bias in (True, False):
        p = cabi.group_conv_problem(*dims, epilogue=cabi.EPI_BIAS if bias else cabi.EPI_NONE)
        ins = [I.to(cuda), W1.to(cuda)] + ([B.to(cuda)] if bias else [])
        tiles = [t for t in cabi.query(p) if t.stages == 5]
        assert len(tiles) == 2, "the multi-item tiles are listed for this many items"
        out, plan = run_plan(p, ins, ref.shape, tiles[0 if bias else 1])
        assert "stages=5" in plan.describe(), plan.describe()
        if bias:
            assert_close(out, ref, C * KH * KW, [I, W1], STRICT["group_conv"], plan.describe())
        else:
            assert_close(out, orc.aten_group_conv(I, W1, None), C * KH * KW, [I, W1], STRICT["group_conv"], plan.describe())
        out2, _ = run_plan(p, ins, ref.shape, tiles[0 if bias else 1])
        assert torch.equal(out, out2)


def test_group_conv_views_at_a_4_byte_offset(cuda):
    """Dense input / filter tensors that start 4 bytes into a larger buffer: the default (item) kernel
    stages with 16-byte copies, so such a launch must run on a kernel that does not need the alignment."""
    dims = (2, 3, 16, 16, 16, 16, 3, 3)
    N, G, C, F, H, W, KH, KW = dims
    I, W1, B = _rand((N, G, C, H, W), 45, "uniform"), _rand((G, F, C, KH, KW), 46, "uniform"), _rand((G, F), 47)
    ref = orc.loop_group_conv(I, W1, B)

    def offset_view(t):
        buf = torch.empty(t.numel() + 1, device=cuda)
        v = buf[1:].view(t.shape)
        v.copy_(t)
        assert v.data_ptr() % 16 == 4
        return v

    p = cabi.group_conv_problem(*dims)
    for views in ((True, False), (False, True), (True, True)):
        ins = [offset_view(I) if views[0] else I.to(cuda), offset_view(W1) if views[1] else W1.to(cuda), B.to(cuda)]
        out, plan = run_plan(p, ins, ref.shape)
        assert_close(out, ref, C * KH * KW, [I, W1], STRICT["group_conv"], plan.describe())


def test_group_conv_full_size(cuda):
    w = wl.group_conv()
    I, W1, B = wl.make_inputs(w)
    p = cabi.group_conv_problem(32, 32, 16, 16, 16, 16, 3, 3)
    out, plan = run_plan(p, [I.to(cuda), W1.to(cuda), B.to(cuda)], (32, 32, 16, 14, 14))
    assert_close(out, orc.loop_group_conv(I, W1, B), 144, [I, W1, B], STRICT["group_conv"], plan.describe())
    assert_close(out, orc.aten_group_conv(I, W1, B), 144, what="vs conv2d")
    assert "tcgen05_ts" in plan.describe() and "stages=3" in plan.describe()   # the family default for this shape
    out2, _ = run_plan(p, [I.to(cuda), W1.to(cuda), B.to(cuda)], (32, 32, 16, 14, 14))
    assert torch.equal(out, out2)   # fixed order of additions: the same bits on every run


# ---------------------------------------------------------------- TMM / MLP3 through whatever the default tile is

def test_tmm_full_size_default_tile(cuda):
    w = wl.tmm()
    A, B = wl.make_inputs(w)
    p = cabi.contraction_problem(1, 128, 16384, 4096, True, True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (128, 16384))
    ref = orc.aten_tmm(A, B)
    assert_close(out, ref, 4096, [A, B], STRICT["tmm"], plan.describe(), strict_is_gate=False)
    # a sample of rows against the loop nest (the full nest is 8.6 GMAC)
    rows = [0, 63, 127]
    loop = orc.loop_tmm(A[rows], B)
    assert_close(out[rows], loop, 4096, what="vs loop nest rows")


def test_mlp3_full_size_default_tile(cuda):
    w = wl.mlp3()
    ins = wl.make_inputs(w)
    I, W2, B2, W3, B3, W4, B4 = [t.to(cuda) for t in ins]
    refs = orc.aten_mlp3(*ins)
    x = I
    outs = []
    for Wt, Bt, L in ((W2, B2, 2048), (W3, B3, 1024), (W4, B4, 512)):
        p = cabi.contraction_problem(1, x.shape[0], Wt.shape[0], x.shape[1], True, True,
                                     epilogue=cabi.EPI_BIAS_RELU)
        out, plan = run_plan(p, [x, Wt, Bt], (x.shape[0], Wt.shape[0]))
        outs.append((out, L, plan.describe()))
        x = out
    for (out, L, what), ref in zip(outs, refs):
        assert_close(out, ref, L, ins, STRICT["mlp3"], what, strict_is_gate=False)
    # loop nest on a slice of the batch
    sl = slice(1000, 1016)
    loop = orc.loop_mlp3(*([ins[0][sl]] + ins[1:]))
    for (out, L, what), ref in zip(outs, loop):
        assert_close(out[sl], ref, L, what="vs loop nest rows " + what)
