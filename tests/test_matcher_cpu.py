"""Pattern matcher: TC statements -> kernel-family problems; compile-time behaviour of the API without
a GPU (the compile path needs no device, like the reference's no-SDK build flavour)."""
import pytest
import torch

import tensorcomprehensions_b200 as tc
from tensorcomprehensions_b200 import tclib
from tensorcomprehensions_b200 import workloads as wl


def match(tcs, entry, ins):
    return tclib.match(tcs, entry, [list(s) for s in ins])


def test_benchmark_comprehensions():
    m = match(wl.TENSORDOT_TC, "tensordot", wl.tensordot().shapes)
    assert len(m) == 1 and m[0]["family"] == "tensordot" and m[0]["td"] == [32, 512, 8, 2, 784]
    m = match(wl.BATCHMATMUL_TC, "batch_matmul", wl.batchmatmul().shapes)[0]
    assert (m["family"], m["batch"], m["M"], m["N"], m["K"], m["a_k_major"], m["b_k_major"]) == \
        ("contraction", 500, 26, 26, 72, 1, 0)
    m = match(wl.TMM_TC, "tmm", wl.tmm().shapes)[0]
    assert (m["batch"], m["M"], m["N"], m["K"], m["a_k_major"], m["b_k_major"], m["ldc"]) == (1, 128, 16384, 4096, 1, 1, 16384)
    m = match(wl.GROUP_CONV_TC, "group_convolution", wl.group_conv().shapes)
    assert len(m) == 1 and m[0]["conv"] == [32, 32, 16, 16, 16, 16, 3, 3] and m[0]["epilogue"] == 1
    assert m[0]["statements"] == [0, 1] and m[0]["inputs"] == [0, 1, 2]
    m = match(wl.MLP3_TC, "mlp3", wl.mlp3().shapes)
    assert [x["epilogue"] for x in m] == [2, 2, 2]
    assert [x["inputs"] for x in m] == [[0, 1, 2], [7, 3, 4], [8, 5, 6]] and [x["output"] for x in m] == [7, 8, 9]
    assert [(x["M"], x["N"], x["K"]) for x in m] == [(16384, 1024, 2048), (16384, 512, 1024), (16384, 256, 512)]


def test_matching_is_structural_not_by_name():
    a = "def t(float(N, C1, C2, H, W) I0, float(N, C2, C3, H, W) I1) -> (O) { O(n, c1, c3, h, w) +=! I0(n, c1, c2, h, w) * I1(n, c2, c3, h, w) }"
    b = "def t(float(N, C1, C2, H, W) I0, float(N, C2, C3, H, W) I1) -> (O) { O(a, b, c, d, e) +=! I1(a, z, c, d, e) * I0(a, b, z, d, e) }"
    sh = [(2, 3, 4, 5, 6), (2, 4, 7, 5, 6)]
    ma, mb = match(a, "t", sh)[0], match(b, "t", sh)[0]
    assert ma["td"] == mb["td"] == [2, 3, 4, 7, 30]
    assert ma["inputs"] == [0, 1] and mb["inputs"] == [0, 1]   # operands re-ordered so I0 plays "A"


@pytest.mark.parametrize("tcs,ins,expect", [
    # the four transpose forms of tc/library/matmul.h
    ("def mm(float(M,K) A, float(K,N) B) -> (C) { C(m,n) +=! A(m,k) * B(k,n) }", [(5, 7), (7, 9)], (5, 9, 7, 1, 0)),
    ("def mm(float(K,M) A, float(K,N) B) -> (C) { C(m,n) +=! A(k,m) * B(k,n) }", [(7, 5), (7, 9)], (5, 9, 7, 0, 0)),
    ("def mm(float(M,K) A, float(N,K) B) -> (C) { C(m,n) +=! A(m,k) * B(n,k) }", [(5, 7), (9, 7)], (5, 9, 7, 1, 1)),
    ("def mm(float(K,M) A, float(N,K) B) -> (C) { C(m,n) +=! A(k,m) * B(n,k) }", [(7, 5), (9, 7)], (5, 9, 7, 0, 1)),
    # transposed output: operands swap roles
    ("def mm(float(M,K) A, float(N,K) B) -> (C) { C(n,m) +=! A(m,k) * B(n,k) }", [(5, 7), (9, 7)], (9, 5, 7, 1, 1)),
    # matrix-vector
    ("def mv(float(M,K) A, float(K) x) -> (y) { y(m) +=! A(m,k) * x(k) }", [(5, 7), (7,)], (5, 1, 7, 1, 1)),
    # row index shared with a leading index of only one operand flattens into M
    ("def f(float(B,M,K) A, float(N,K) W) -> (O) { O(b,m,n) +=! A(b,m,k) * W(n,k) }", [(3, 5, 7), (9, 7)], (15, 9, 7, 1, 1)),
])
def test_contraction_forms(tcs, ins, expect):
    m = match(tcs, tcs.split("(")[0].split()[1], ins)[0]
    assert m["family"] == "contraction"
    assert (m["M"], m["N"], m["K"], m["a_k_major"], m["b_k_major"]) == expect


def test_bias_on_rows_and_relu_only():
    t = "def f(float(M,K) A, float(N,K) B, float(M) b) -> (C) { C(m,n) +=! A(m,k) * B(n,k)\n C(m,n) = C(m,n) + b(m) }"
    m = match(t, "f", [(4, 6), (5, 6), (4,)])[0]
    assert m["epilogue"] == 1 and m["bias_on_m"] == 1
    t = "def f(float(M,K) A, float(N,K) B) -> (C) { C(m,n) +=! A(m,k) * B(n,k)\n C(m,n) = fmax(C(m,n), 0) }"
    assert match(t, "f", [(4, 6), (5, 6)])[0]["epilogue"] == 3


def test_sum_reductions():
    """sum1D / sum2D of the reference's mapper tests (test/test_tc_mapper_harness-inl.h:60-146) and the
    general form: one operand, the reduced indices adjacent, the kept ones in the operand's order."""
    for body in ("C() +=! A(r_m)", "C +=! A(r_m)", "C(i) +=! A(r_m) where i in 0:1"):
        m = match("def sum1D(float(M) A) -> (C) { %s }" % body, "sum1D", [(100,)])
        assert len(m) == 1 and m[0]["family"] == "reduction" and m[0]["red"] == [1, 100, 1] and m[0]["inputs"] == [0]
    m = match("def sum2D(float(M, N) A) -> (C) { C(m) +=! A(m, r_n) }", "sum2D", [(7, 9)])[0]
    assert m["red"] == [7, 9, 1] and m["accumulate"] == 0
    m = match("def cols(float(M, N) A) -> (C) { C(n) += A(r_m, n) }", "cols", [(7, 9)])[0]
    assert m["red"] == [1, 7, 9] and m["accumulate"] == 1
    m = match("def f(float(N, C, D, H, W) I) -> (O) { O(n, h, w) +=! I(n, c, d, h, w) }", "f", [(2, 3, 4, 5, 6)])[0]
    assert m["red"] == [2, 12, 30]
    exe = tc.compile("def sum2D(float(M, N) A) -> (C) { C(m) +=! A(m, r_n) }", "sum2D", "naive", torch.empty(7, 9))
    assert exe.output_shapes() == [[7]] and "tcb200::reduction sum A=7 C=9 B=1" in exe.compiled_source
    # the other reduction assignments of the language, for one operand
    for assign, op, acc in (("max=!", 1, 0), ("min=!", 2, 0), ("*=!", 3, 0), ("max=", 1, 1), ("*=", 3, 1)):
        m = match("def r(float(M, N) A) -> (C) { C(m) %s A(m, r_n) }" % assign, "r", [(7, 9)])[0]
        assert (m["family"], m["red"], m["reduce_op"], m["accumulate"]) == ("reduction", [7, 9, 1], op, acc)


def test_ungrouped_convolution_is_group_conv_with_one_group():
    t = "def c(float(N,C,H,W) I, float(F,C,KH,KW) W1) -> (O) { O(n,f,h,w) +=! I(n,c,h+kh,w+kw) * W1(f,c,kh,kw) }"
    m = match(t, "c", [(2, 3, 8, 9), (4, 3, 3, 2)])[0]
    assert m["family"] == "group_conv" and m["conv"] == [2, 1, 3, 4, 8, 9, 3, 2]


def test_strided_convolution_of_the_library():
    """tc/library/convolution.h:27-31 and group_convolution.h:26-44 substitute the strides as literal
    factors; the output extent is the largest that keeps SH*h+kh inside the image."""
    t = ("def convolution(float(N,C,H,W) I, float(M,C,KH,KW) W1, float(M) B) -> (O) {\n"
         " O(n, m, h, w) +=! I(n, c, %d * h + kh, %d * w + kw) * W1(m, c, kh, kw)\n"
         " O(n, m, h, w) = O(n, m, h, w) + B(m)\n}")
    m = match(t % (1, 1), "convolution", [(2, 3, 10, 9), (4, 3, 3, 3), (4,)])[0]
    assert m["conv"] == [2, 1, 3, 4, 10, 9, 3, 3] and m["conv_stride"] == [1, 1] and m["epilogue"] == 1
    m = match(t % (3, 2), "convolution", [(2, 3, 10, 9), (4, 3, 3, 3), (4,)])[0]
    assert m["conv"] == [2, 1, 3, 4, 10, 9, 3, 3] and m["conv_stride"] == [3, 2]
    exe = tc.compile(t % (3, 2), "convolution", "naive", torch.empty(2, 3, 10, 9), torch.empty(4, 3, 3, 3), torch.empty(4))
    assert exe.output_shapes() == [[2, 4, 3, 4]] and "stride=3x2" in exe.compiled_source
    g = ("def gc(float(N,G,C,H,W) I, float(G,F,C,KH,KW) W1) -> (O) "
         "{ O(n,g,f,h,w) +=! I(n,g,c,2*h+kh,2*w+kw) * W1(g,f,c,kh,kw) }")
    m = match(g, "gc", [(2, 3, 4, 11, 11), (3, 8, 4, 3, 3)])[0]
    assert m["conv"] == [2, 3, 4, 8, 11, 11, 3, 3] and m["conv_stride"] == [2, 2] and m["epilogue"] == 0


@pytest.mark.parametrize("tcs,ins,fragment", [
    ("def f(float(N) A, float(N) B) -> (C) { C(i) = A(i) + B(i) }", [(4,), (4,)], "elementwise statement"),
    ("def f(float(N,M) A) -> (O) { O(i) +=! exp(A(i,j)) }", [(4, 5)], "not a product of two tensor accesses"),
    ("def f(float(N,M,K) A) -> (O) { O(m) +=! A(n,m,k) }", [(4, 5, 6)], "not adjacent dimensions"),
    ("def f(float(N,M) A, float(M) B) -> (O) { O(i) max=! A(i,j) * B(j) }", [(4, 5), (5,)], "only sum reductions"),
    ("def f(float(N,M,K) A) -> (O) { O(m) min=! A(n,m,k) }", [(4, 5, 6)], "not adjacent dimensions"),
    # dilated filter taps: strides are covered (next test), dilation is not
    ("def f(float(N,C,H,W) I, float(F,C,KH,KW) W1) -> (O) { O(n,f,h,w) +=! I(n,c,h+2*kh,w+2*kw) * W1(f,c,kh,kw) }",
     [(1, 1, 9, 9), (1, 1, 3, 3)], "not a plain index variable"),
    ("def f(float(M,K) A, float(N,K) B) -> (C) { C(m,n) +=! A(m,k) * B(n,k)\n C(m,n) = C(m,n) * 2 }", [(4, 6), (5, 6)], "epilogue"),
    ("def f(double(M,K) A, double(N,K) B) -> (C) { C(m,n) +=! A(m,k) * B(n,k) }", [(4, 6), (5, 6)], "float32"),
])
def test_unmatched_is_a_hard_error(tcs, ins, fragment):
    with pytest.raises(tclib.ErrorReport) as e:
        if "double" in tcs:
            tc.compile(tcs, "f", "naive", *[torch.empty(s, dtype=torch.float64) for s in ins])
        else:
            match(tcs, "f", ins)
    assert "no kernel family" in str(e.value) and fragment in str(e.value)


def test_compile_without_a_device_and_compiled_source():
    w = wl.tmm()
    exe = tc.compile(w.tc, w.entry, tc.MappingOptions("naive"), *[torch.empty(s) for s in w.shapes])
    src = exe.compiled_source
    assert "tcb200::contraction" in src and "variant=tcgen05" in src and exe.num_launches == 1
    assert exe.output_shapes() == [[128, 16384]]
    assert exe.grid == [128, 1, 1] and exe.block == [608, 1, 1]  # C^T = B A^T on 64 CTA pairs (256 x 128 tiles)
    w = wl.mlp3()
    assert tc.compile(w.tc, w.entry, "mlp", *[torch.empty(s) for s in w.shapes]).num_launches == 3


def test_compile_time_input_checks():
    t = wl.TMM_TC
    with pytest.raises(tclib.ErrorReport, match="expected 2 inputs but got 1"):
        tc.compile(t, "tmm", "naive", torch.empty(4, 4))
    with pytest.raises(tclib.ErrorReport, match="expected type float but found int32"):
        tc.compile(t, "tmm", "naive", torch.empty(4, 4, dtype=torch.int32), torch.empty(4, 4))
    with pytest.raises(tclib.ErrorReport, match="expected a tensor with 2 dimensions but found 3"):
        tc.compile(t, "tmm", "naive", torch.empty(4, 4, 1), torch.empty(4, 4))
    with pytest.raises(tclib.InvalidStrideException, match="invalid strides"):
        tc.compile(t, "tmm", "naive", torch.empty(8, 4).t(), torch.empty(4, 8))
    with pytest.raises(RuntimeError, match="undefined function"):
        tc.compile(t, "nope", "naive", torch.empty(4, 4), torch.empty(4, 4))


def test_mapping_options_roundtrip_and_tile_encoding():
    naive = tc.MappingOptions("naive")
    assert naive.to_tile() is None and "tiling" in str(naive)
    o = tc.MappingOptions.from_tile(3, 128, 128, 32, 2, 192, 3)
    assert o.to_tile() == (3, 128, 128, 32, 2, 192, 3, 0)
    assert tc.MappingOptions.from_tile(5, 256, 128, 32, 8, 608, 3, 4).to_tile() == (5, 256, 128, 32, 8, 608, 3, 4)
    assert tc.MappingOptions(o.serialize()) == o and tc.MappingOptions(naive.serialize()) == naive
    assert naive != o
    # a tuned tile is honoured where a launch accepts it and ignored elsewhere
    w = wl.tmm()
    exe = tc.compile(w.tc, w.entry, o, *[torch.empty(s) for s in w.shapes])
    assert exe.tiles()[0][:4] == (3, 128, 128, 32) and exe.tiles()[0][5:] == (448, 3, 1)
    w = wl.tensordot()
    exe = tc.compile(w.tc, w.entry, o, *[torch.empty(s) for s in w.shapes])
    assert exe.tiles()[0][0] == 1  # tensordot has no tcgen05 variant: family default


def test_options_cache_file(tmp_path):
    cache = tc.MappingOptionsCache(str(tmp_path / "opts.cuda.options"))
    ins = [torch.empty(4, 6), torch.empty(5, 6)]
    o = tc.MappingOptions.from_tile(1, 64, 64, 16, 0, 256, 0)
    slow = tc.MappingOptions.from_tile(1, 32, 32, 16, 0, 128, 0)
    assert cache.load(wl.TMM_TC, "tmm", ins) == [] and len(cache) == 0
    cache.store(wl.TMM_TC, "tmm", ins, slow, runtime_us=90)
    cache.store(wl.TMM_TC, "tmm", ins, o, runtime_us=30)
    cache.store(wl.TMM_TC, "tmm", ins, o, runtime_us=50)     # a second runtime of the same options
    assert len(cache) == 2
    assert cache.load(wl.TMM_TC, "tmm", ins) == [o]          # fastest median first
    assert cache.load(wl.TMM_TC, "tmm", ins, 5) == [o, slow]
    assert cache.load(wl.TMM_TC, "tmm", [torch.empty(4, 7), torch.empty(5, 7)]) == []
    # the key is the canonical TC: renaming the indices finds the entry, another comprehension does not
    renamed = wl.TMM_TC.replace("r_k", "q")
    assert renamed != wl.TMM_TC and cache.load(renamed, "tmm", ins) == [o]
    other = "def tmm(float(M,K) A, float(N,K) B) -> (C) { C(m,n) +=! A(m,k) * B(n,k) * 2 }"
    assert cache.load(other, "tmm", ins) == []
    fac = tc.make_load_from_cache_options_factory(str(tmp_path / "opts.cuda.options"))
    assert fac(wl.TMM_TC, "tmm", *ins) == o
