"""The reduction family (sums of one tensor over adjacent indices) against the loop nest and ATen.
Shapes follow the reference's mapper tests (test/cuda/test_tc_mapper.cc:47-177: sum1D, sum2D and its
stress sizes) plus sizes at which the split over segments, the ticket hand-off and both kernels run."""
import pytest
import torch

import tensorcomprehensions_b200 as tc
from oracle import oracle as orc
from tensorcomprehensions_b200 import cabi

from helpers import assert_close, run_plan

pytestmark = pytest.mark.gpu
PREC = 5e-7  # checkRtol precision of the reference's reduction tests (test_tc_mapper_harness-inl.h:104,137)


def _rand(shape, seed):
    return torch.rand(shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float32)


@pytest.mark.parametrize("dims", [
    (1, 100, 1), (1, 1, 1), (7, 9, 1), (4, 7, 1), (11, 5, 1), (16, 9, 1), (8, 11, 1), (111, 7, 1), (130, 1, 1),
    (1, 7, 9), (3, 5, 2), (2, 12, 30), (32, 1000, 77), (5, 33, 257), (1, 3, 1000), (4, 1, 5),
    (600, 1030, 1),      # warp per row, rows not a multiple of four floats
    (600, 1024, 1),      # warp per row, 128-bit loads
    (64, 100000, 1),     # rows split over segments
    (1, 3000001, 1),     # sum1D over every SM, ragged last segment
    (1, 5000, 4096),     # column sums, segments
    (2, 70000, 3),       # narrow trailing dimension, segments
])
def test_reduce_every_tile(cuda, dims):
    A, C, B = dims
    I = _rand((A, C, B), 71)
    ref = orc.loop_reduce(I, double=True)
    p = cabi.reduction_problem(A, C, B)
    for tile in [None] + cabi.query(p):
        out, plan = run_plan(p, [I.to(cuda)], (A, B), tile)
        assert_close(out, ref, C, [I], PREC, plan.describe())
        out2, _ = run_plan(p, [I.to(cuda)], (A, B), tile)
        assert torch.equal(out, out2), plan.describe()  # segment order is fixed: the same bits every run
    assert_close(out, I.double().sum(1).float(), C, what="vs ATen sum")


def test_reduce_explicit_segments_and_reuse_of_the_scratch(cuda):
    """One plan launched repeatedly: the tickets must be back at zero after every launch."""
    A, C, B = 3, 40000, 5
    p = cabi.reduction_problem(A, C, B)
    t = cabi.Tile()
    t.variant, t.bm, t.bn = cabi.VARIANT_SIMT, 8, 37
    plan = cabi.Plan(p, t)
    assert plan.geometry()[0] == (3, 37, 1)
    for seed in range(4):
        I = _rand((A, C, B), 80 + seed).to(cuda)
        out = torch.full((A, B), float("nan"), device=cuda)
        plan.launch([I], [out])
        torch.cuda.synchronize()
        assert_close(out, orc.loop_reduce(I.cpu(), double=True), C, [I.cpu()], PREC, plan.describe())


def test_first_launch_of_a_split_plan_on_a_fresh_stream(cuda):
    """The ticket counters of a plan's scratch are zeroed on the launch stream: a first launch on a
    non-blocking stream (every torch.cuda.Stream) must see them zero."""
    A, C, B = 2, 300000, 3
    I = _rand((A, C, B), 91).to(cuda)
    ref = orc.loop_reduce(I.cpu(), double=True)
    for _ in range(3):
        plan = cabi.Plan(cabi.reduction_problem(A, C, B))
        assert plan.geometry()[0][1] > 1, "the case must split the reduced range"
        stream = torch.cuda.Stream()
        out = torch.full((A, B), float("nan"), device=cuda)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            plan.launch([I], [out])
            plan.launch([I], [out])
        stream.synchronize()
        assert_close(out, ref, C, [I.cpu()], PREC, plan.describe())


def test_reduce_accumulates_into_the_output(cuda):
    for dims in ((5, 300, 1), (1, 200000, 1), (2, 9000, 40)):
        I = _rand(dims, 90)
        init = _rand((dims[0], dims[2]), 91)
        p = cabi.reduction_problem(*dims, accumulate=True)
        for tile in [None] + cabi.query(p):
            out, plan = run_plan(p, [I.to(cuda)], (dims[0], dims[2]), tile, out_init=init.to(cuda))
            assert_close(out, orc.loop_reduce(I, double=True) + init.numpy(), dims[1], what=plan.describe())


@pytest.mark.parametrize("op", [cabi.REDUCE_MAX, cabi.REDUCE_MIN, cabi.REDUCE_PROD])
@pytest.mark.parametrize("dims", [(1, 100, 1), (7, 9, 1), (111, 7, 1), (3, 5, 2), (5, 33, 257), (600, 1024, 1),
                                  (64, 100000, 1), (1, 300001, 1), (1, 5000, 4096), (2, 70000, 3)])
def test_max_min_product_every_tile(cuda, dims, op):
    """max=!, min=! and *=! of one operand (tc/lang/tree.h TK_MAX_EQ_B ...): exact for max / min; the product
    of values near 1 against a float64 product."""
    A, C, B = dims
    g = torch.Generator().manual_seed(73)
    if op == cabi.REDUCE_PROD:
        I = 1.0 + (torch.rand((A, C, B), generator=g) - 0.5) * (2.0 / C ** 0.5)  # keeps the product O(1)
    else:
        I = torch.randn((A, C, B), generator=g)
    ref = orc.loop_reduce_op(I, op)
    p = cabi.reduction_problem(A, C, B, op=op)
    for tile in [None] + cabi.query(p):
        out, plan = run_plan(p, [I.to(cuda)], (A, B), tile)
        if op == cabi.REDUCE_PROD:
            assert_close(out, ref, C, what=plan.describe())
        else:
            assert torch.equal(out.cpu(), torch.from_numpy(ref)), plan.describe()
    # without '!' the old output takes part
    init = torch.randn((A, B), generator=g) if op != cabi.REDUCE_PROD else 1.0 + torch.rand((A, B), generator=g)
    pa = cabi.reduction_problem(A, C, B, accumulate=True, op=op)
    out, plan = run_plan(pa, [I.to(cuda)], (A, B), None, out_init=init.to(cuda))
    r = torch.from_numpy(ref)
    expect = torch.maximum(r, init) if op == cabi.REDUCE_MAX else torch.minimum(r, init) if op == cabi.REDUCE_MIN else r * init
    assert_close(out, expect, C, what=plan.describe() + " accumulate")


def test_max_min_product_through_the_api(cuda):
    T = tc.define("def rowmax(float(M, N) A) -> (C) { C(m) max=! A(m, r_n) }\n"
                  "def colmin(float(M, N) A) -> (C) { C(n) min=! A(r_m, n) }\n"
                  "def prod(float(M) A) -> (C) { C *=! A(r_m) }", tc.make_naive_options_factory())
    A = torch.randn(513, 77, device=cuda)
    assert torch.equal(T.rowmax(A), A.max(1).values) and torch.equal(T.colmin(A), A.min(0).values)
    v = 1.0 + (torch.rand(4000, device=cuda) - 0.5) * 0.02
    assert_close(T.prod(v).reshape(1), v.double().prod().float().reshape(1).cpu(), 4000)


@pytest.mark.parametrize("body", ["C() +=! A(r_m)", "C +=! A(r_m)", "C(i) +=! A(r_m) where i in 0:1"])
def test_sum1d_forms_through_the_api(cuda, body):
    A = torch.rand(1000003, device=cuda)
    T = tc.define("def sum1D(float(M) A) -> (C) { %s }" % body, tc.make_naive_options_factory())
    out = T.sum1D(A)
    ref = A.double().sum().float().cpu()
    assert_close(out.reshape(-1), ref.reshape(-1), A.numel(), [A.cpu()], PREC, body)


def test_sum2d_and_general_forms_through_the_api(cuda):
    A = torch.rand(130, 17, device=cuda)
    T = tc.define("def sum2D(float(M, N) A) -> (C) { C(m) +=! A(m, r_n) }\n"
                  "def cols(float(M, N) A) -> (C) { C(n) +=! A(r_m, n) }\n"
                  "def mid(float(N, C, D, H, W) I) -> (O) { O(n, h, w) +=! I(n, c, d, h, w) }",
                  tc.make_naive_options_factory())
    assert_close(T.sum2D(A), A.double().sum(1).float().cpu(), 17, [A.cpu()], PREC)
    assert_close(T.cols(A), A.double().sum(0).float().cpu(), 130, [A.cpu()], PREC)
    I = torch.rand(3, 5, 7, 6, 4, device=cuda)
    assert_close(T.mid(I), I.double().sum((1, 2)).float().cpu(), 35, [I.cpu()], PREC)
    best = tc.autotune("def sum2D(float(M, N) A) -> (C) { C(m) +=! A(m, r_n) }", "sum2D", A, starting_options="naive")
    assert best.to_tile() is not None
