"""The public API end to end on a B200: tc.compile / tc.define / autotune -> C++ host -> kernels,
checked against the CPU checker.  Mirrors how the reference's tests drive it
(test/cuda/test_tc_mapper.cc, python/tests/test_tc.py)."""
import pytest
import torch

import tensorcomprehensions_b200 as tc
from oracle import oracle as orc
from tensorcomprehensions_b200 import tclib
from tensorcomprehensions_b200 import workloads as wl

from helpers import STRICT, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", list(wl.ALL))
def test_small_instances_through_define(cuda, name):
    w = wl.ALL[name](**wl.SMALL[name])
    ins = wl.make_inputs(w)
    T = tc.define(w.tc, tc.make_naive_options_factory())
    outs = getattr(T, w.entry)(*[t.to(cuda) for t in ins])
    outs = list(outs) if isinstance(outs, tuple) else [outs]
    refs = orc.as_list(orc.LOOP[name](*ins))
    assert len(outs) == len(refs)
    for o, r, L in zip(outs, refs, w.reduction):
        assert_close(o, r, L, ins, STRICT[name], name, strict_is_gate=True)
    # second call hits the per-shape executor cache and gives the same bits
    outs2 = getattr(T, w.entry)(*[t.to(cuda) for t in ins])
    outs2 = list(outs2) if isinstance(outs2, tuple) else [outs2]
    for a, b in zip(outs, outs2):
        assert torch.equal(a, b)


@pytest.mark.parametrize("name", list(wl.ALL))
def test_full_size_through_compile(cuda, name):
    w = wl.ALL[name]()
    ins = wl.make_inputs(w)
    dev_ins = [t.to(cuda) for t in ins]
    exe = tc.compile(w.tc, w.entry, "naive", *dev_ins)
    outs = [torch.full(s, float("nan"), device=cuda) for s in exe.output_shapes()]
    res = exe(*dev_ins, outputs=tuple(outs))
    torch.cuda.synchronize()
    refs = orc.as_list(orc.ATEN[name](*ins))
    # the family defaults meet the reference's own checkRtol (test/test_harness_aten.h:36-54) at its
    # benchmark precisions on these inputs, not only the benchmark criterion
    for o, r, L in zip(outs, refs, w.reduction):
        assert_close(o, r, L, ins, STRICT[name], exe.compiled_source, strict_is_gate=True)
    prof = exe.profile(*dev_ins, outputs=outs)
    assert prof["kernel_runtime_us"] > 0


def test_tensordot_example_flow(cuda):
    """tc/examples/tensordot.cc:41-69: tune from naive options, compile with the best, run, reuse the
    options on two other sizes."""
    tcs = wl.TENSORDOT_TC
    I0, I1 = torch.rand(16, 8, 16, 17, 25, device=cuda), torch.rand(16, 16, 2, 17, 25, device=cuda)
    best = tc.autotune(tcs, "tensordot", I0, I1, starting_options="naive")
    assert isinstance(best, tc.MappingOptions) and best.to_tile() is not None
    exe = tc.compile(tcs, "tensordot", best, I0, I1)
    out = exe(I0, I1)
    assert_close(out, orc.loop_tensordot(I0.cpu(), I1.cpu()), 16, what=exe.compiled_source)
    for s0, s1 in (((4, 9, 7, 16, 14), (4, 7, 3, 16, 14)), ((8, 5, 11, 10, 10), (8, 11, 16, 10, 10))):
        A, B = torch.rand(s0, device=cuda), torch.rand(s1, device=cuda)
        exe = tc.compile(tcs, "tensordot", best, A, B)
        assert_close(exe(A, B), orc.loop_tensordot(A.cpu(), B.cpu()), s0[2], what=exe.compiled_source)


def test_tune_returns_best_first_and_every_option_compiles(cuda):
    w = wl.batchmatmul()
    X, Y = [t.to(cuda) for t in wl.make_inputs(w)]
    ranked = tclib.tune_report(w.tc, w.entry, [X, Y])
    assert len(ranked) >= 2
    times = [r[1] for r in ranked]
    assert times == sorted(times)
    ref = orc.loop_batchmatmul(X.cpu(), Y.cpu())
    for options, us, desc in ranked:
        exe = tc.compile(w.tc, w.entry, options, X, Y)
        assert exe.tiles()[0] == options.to_tile()
        assert_close(exe(X, Y), ref, 72, what=desc)


@pytest.mark.parametrize("name", ["tensordot", "group_conv", "tmm"])
def test_tune_sweeps_every_tile_the_family_lists(cuda, name):
    """The sweep must not lose a candidate because the plan filled in fields the listed tile left open
    (the family default, e.g. the bulk-copy tensordot kernel, has to be among the timed ones)."""
    w = wl.ALL[name](**wl.SMALL[name])
    ins = [t.to(cuda) for t in wl.make_inputs(w)]
    ranked = tclib.tune_report(w.tc, w.entry, ins)
    default = tc.compile(w.tc, w.entry, "naive", *ins).tiles()[0]
    swept = [options.to_tile() for options, _, _ in ranked]
    assert default in swept, (default, swept)
    assert len(swept) >= 2


def test_library_convolution_with_strides(cuda):
    """makeConvolution2DTc(sh, sw) of tc/library/convolution.h:33-41 through compile / run."""
    t = ("def convolution(float(N,C,H,W) I, float(M,C,KH,KW) W1, float(M) B) -> (O) {\n"
         " O(n, m, h, w) +=! I(n, c, %d * h + kh, %d * w + kw) * W1(m, c, kh, kw)\n"
         " O(n, m, h, w) = O(n, m, h, w) + B(m)\n}")
    I, W1, B = torch.rand(4, 8, 33, 30, device=cuda), torch.rand(16, 8, 3, 3, device=cuda), torch.rand(16, device=cuda)
    for sh, sw in ((1, 1), (2, 2), (2, 3)):
        exe = tc.compile(t % (sh, sw), "convolution", "naive", I, W1, B)
        out = exe(I, W1, B)
        ref = torch.nn.functional.conv2d(I.cpu().double(), W1.cpu().double(), B.cpu().double(), stride=(sh, sw)).float()
        assert list(out.shape) == list(ref.shape)
        assert_close(out, ref, 72, what=exe.compiled_source)


def test_autotune_stores_to_and_loads_from_a_cache_file(cuda, tmp_path):
    """python/tests/test_tc.py:485-506 of the reference: tune with a cache file, then compile from it."""
    w = wl.batchmatmul()
    X, Y = [t.to(cuda) for t in wl.make_inputs(w)]
    path = str(tmp_path / "bmm.cuda.options")
    best = tc.autotune(w.tc, w.entry, X, Y, starting_options="naive", cache_filename=path, store_to_cache=True)
    assert tc.MappingOptionsCache(path).load(w.tc, w.entry, [X, Y]) == [best]
    assert tc.autotune(w.tc, w.entry, X, Y, cache_filename=path, load_from_cache=True) == best
    T = tc.define(w.tc, tc.make_load_from_cache_options_factory(path))
    assert_close(getattr(T, w.entry)(X, Y), orc.loop_batchmatmul(X.cpu(), Y.cpu()), 72)
    # a second tuning run on other sizes merges into the same file
    X2, Y2 = X[:100].contiguous(), Y[:100].contiguous()
    tc.Tuner(w.tc, path).tune(w.entry, [X2, Y2], tc.MappingOptions("naive"))
    cache = tc.MappingOptionsCache(path)
    assert len(cache) == 2 and cache.load(w.tc, w.entry, [X, Y]) == [best] and len(cache.load(w.tc, w.entry, [X2, Y2])) == 1


def test_make_autograd_with_matmul_gradients(cuda):
    """tc.make_autograd (tensor_comprehensions/__init__.py:513-601) with the matmul gradients of
    python/benchmarks/python_overhead.py:40-50: all three comprehensions are contractions."""
    T = tc.define("""
def matmul(float(M, K) A, float(K, N) B) -> (C) { C(m, n) +=! A(m, r_k) * B(r_k, n) }
def matmul_agrad(float(K, N) B, float(M, N) d_C) -> (d_A) { d_A(m, k) +=! d_C(m, r_n) * B(k, r_n) }
def matmul_bgrad(float(M, K) A, float(M, N) d_C) -> (d_B) { d_B(k, n) +=! d_C(r_m, n) * A(r_m, k) }
""", tc.make_naive_options_factory())

    def backward(A, B, d_C):
        return T.matmul_agrad(B, d_C), T.matmul_bgrad(A, d_C)

    fn = tc.make_autograd(T.matmul, backward)
    A = torch.randn(70, 40, device=cuda, requires_grad=True)
    B = torch.randn(40, 50, device=cuda, requires_grad=True)
    w = torch.randn(70, 50, device=cuda)
    (fn(A, B) * w).sum().backward()
    A2, B2 = A.detach().clone().requires_grad_(), B.detach().clone().requires_grad_()
    ((A2.double() @ B2.double()).float() * w).sum().backward()
    assert_close(A.grad, A2.grad.cpu(), 50, what="d_A")
    assert_close(B.grad, B2.grad.cpu(), 70, what="d_B")
    assert tc.debug_tc_mapper(True) is True and tc.dump_cuda(False) is False  # accepted, no effect


def test_make_autograd_with_the_convolution_example(cuda):
    """The reference's own make_autograd example (tensor_comprehensions/__init__.py:558-601,
    python/tests/test_tc.py:383-443): a 1x1 convolution with bias and its gradients, written with index
    differences (h - r_kh, r_h - kh) that are the plain index for 1-wide filter ranges.  The input gradient is a
    contraction over which the filter is shared by all images, the weight gradient a contraction that also reduces
    over the image index, the bias "gradient" of the example a whole-tensor copy.  Forward and both real gradients
    are compared with torch.autograd on conv2d."""
    conv = """
def convolution(float(N,C,H,W) I, float(M,C,KH,KW) W1, float(M) Bias) -> (O) {
    O(n, m, h, w) +=! I(n, r_c, h + r_kh, w + r_kw) * W1(m, r_c, r_kh, r_kw)
    O(n, m, h, w)  = O(n, m, h, w) + Bias(m)
}
def convolution_igrad(float(M,C,KH,KW) W1, float(N,M,H,W) d_O) -> (d_I) {
    d_I(n, c, h, w) +=! d_O(  n, r_m, h - r_kh, w - r_kw) * W1(r_m, c, r_kh, r_kw)
}
def convolution_wgrad(float(N,C,H,W) I, float(N,M,H,W) d_O) -> (d_W1) {
    d_W1(m, c, kh, kw) +=! d_O(r_n,   m, r_h - kh, r_w - kw) *  I(r_n, c,  r_h,  r_w)
}
def convolution_biasgrad(float(M) Bias) -> (d_Bias) {
    d_Bias(m) = Bias(m)
}
"""
    N, C, H, W, O, kH, kW = 32, 4, 56, 56, 16, 1, 1
    T = tc.define(conv, tc.make_naive_options_factory())
    g = torch.Generator().manual_seed(11)
    I = torch.randn(N, C, H, W, generator=g).to(cuda).requires_grad_()
    Wt = torch.randn(O, C, kH, kW, generator=g).to(cuda).requires_grad_()
    Bias = torch.randn(O, generator=g).to(cuda).requires_grad_()
    weight = torch.randn(N, O, H, W, generator=g).to(cuda)

    def convolution_backward(I, W1, Bias, d_O):
        return T.convolution_igrad(W1, d_O), T.convolution_wgrad(I, d_O), T.convolution_biasgrad(Bias)

    fn = tc.make_autograd(T.convolution, convolution_backward)
    out = fn(I, Wt, Bias)
    (out * weight).sum().backward()
    out2 = fn(I, Wt, Bias)          # the second call reuses the compiled executors
    assert torch.equal(out, out2)

    I2, W2, B2 = (t.detach().clone().double().requires_grad_() for t in (I, Wt, Bias))
    ref = torch.nn.functional.conv2d(I2, W2, B2)
    (ref * weight.double()).sum().backward()
    assert_close(out.detach(), ref.detach().float().cpu(), C * kH * kW, what="forward")
    assert_close(I.grad, I2.grad.float().cpu(), O, what="d_I")
    assert_close(Wt.grad, W2.grad.float().cpu(), N * H * W, what="d_W1")
    assert torch.equal(Bias.grad, Bias.detach())  # what the example's biasgrad comprehension computes: a copy


def test_batch_reduced_contraction_and_copy_through_the_c_abi(cuda):
    """C(m,n) = sum_b sum_k A(b,m,k) B(b,n,k) for every contraction tile, against float64; the copy family."""
    b, M, N, K = 5, 130, 96, 256
    g = torch.Generator().manual_seed(12)
    A, B = torch.randn(b, M, K, generator=g), torch.randn(b, N, K, generator=g)
    ref = torch.einsum("bmk,bnk->mn", A.double(), B.double()).float()
    from tensorcomprehensions_b200 import cabi
    from helpers import run_plan
    p = cabi.contraction_problem(b, M, N, K, True, True, batch_reduce=True)
    for tile in [None] + cabi.query(p):
        out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (M, N), tile)
        assert "(reduced)" in plan.describe()
        assert_close(out, ref, b * K, what=plan.describe())
    init = torch.randn(M, N, generator=g)
    p = cabi.contraction_problem(b, M, N, K, True, True, batch_reduce=True, accumulate=True, epilogue=cabi.EPI_RELU)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (M, N), None, out_init=init.to(cuda))
    assert_close(out, torch.clamp_min(ref + init, 0), b * K, what=plan.describe())
    pc = cabi.Problem()
    pc.family = cabi.FAMILY_COPY
    pc.red[0] = 1001
    src = torch.randn(1001, generator=g).to(cuda)
    out, plan = run_plan(pc, [src], (1001,))
    assert torch.equal(out, src) and "copy" in plan.describe()


def test_trivial_copies_of_the_corner_case_suite_run(cuda):
    """test/cuda/test_corner_cases.cc E2 and E4: a one-element copy and a zero-dimensional one."""
    a = torch.randn(1, device=cuda)
    assert torch.equal(tc.compile("def f(float(1) a) -> (b) { b(i) = a(i) }", "f", "naive", a)(a), a)
    s = torch.randn((), device=cuda)
    out = tc.compile("def f(float a) -> (b) { b = a }", "f", "naive", s)(s)
    assert out.shape == s.shape and torch.equal(out, s)
    m = torch.randn(37, 21, device=cuda)
    assert torch.equal(tc.compile("def f(float(N, M) a) -> (b) { b(i, j) = a(i, j) }", "f", "naive", m)(m), m)


def test_accumulating_reduction_keeps_output(cuda):
    """'+=' without '!' adds to what the output holds (test/cuda/test_compile_and_run.cc:181-200)."""
    tcs = "def mm(float(M,K) A, float(K,N) B) -> (C) { C(m,n) += A(m,k) * B(k,n) }"
    A, B = torch.randn(33, 20, device=cuda), torch.randn(20, 17, device=cuda)
    exe = tc.compile(tcs, "mm", "naive", A, B)
    C = torch.ones(33, 17, device=cuda)
    exe(A, B, outputs=(C,))
    assert_close(C, (A.double() @ B.double()).float().cpu() + 1, 20, what="+=")


def test_run_checks_shapes_and_types(cuda):
    w = wl.tmm(M=64, N=64, K=64)
    A, B = [t.to(cuda) for t in wl.make_inputs(w)]
    exe = tc.compile(w.tc, w.entry, "naive", A, B)
    with pytest.raises(tclib.ErrorReport, match="expected size"):
        exe(A[:32].contiguous(), B)
    with pytest.raises(tclib.ErrorReport, match="expected 2 "):
        exe(A)
    with pytest.raises(tclib.ErrorReport, match="float"):
        exe(A.double(), B)
    # the unchecked path takes raw pointers
    C = torch.empty(64, 64, device=cuda)
    exe(A, B, outputs=(C,), unchecked=True)
    assert_close(C, (A.double() @ B.double().t()).float().cpu(), 64)


def test_runs_on_the_callers_stream(cuda):
    w = wl.tmm(M=128, N=256, K=128)
    A, B = [t.to(cuda) for t in wl.make_inputs(w)]
    exe = tc.compile(w.tc, w.entry, "naive", A, B)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        C = exe(A, B)
    s.synchronize()
    assert_close(C, (A.double() @ B.double().t()).float().cpu(), 128)


def test_host_staged_executor_matches_direct_run(cuda):
    """Host buffers in / out through three streams and two buffer sets: same bits as a direct run."""
    w = wl.tmm(M=128, N=512, K=256)
    exe = tc.compile(w.tc, w.entry, "naive", *[torch.empty(s, device=cuda) for s in w.shapes])
    staged = tc.HostStagedExecutor(exe, cuda, depth=2)
    batches = []
    for seed in range(5):
        ins = [t.pin_memory() for t in wl.make_inputs(w, seed=100 + seed)]
        out = torch.empty(128, 512).pin_memory()
        batches.append((ins, out))
        staged.submit(ins, [out])
    staged.synchronize()
    for ins, out in batches:
        ref = exe(*[t.to(cuda) for t in ins]).cpu()
        assert torch.equal(out, ref)
