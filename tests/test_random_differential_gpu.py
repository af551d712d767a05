"""Randomised differential tests, the reference's own test style (its numeric tests draw random inputs and
compare with ATen: test/cuda/test_tc_mapper.cc, test/test_harness_aten.h) with a fixed seed: random
comprehensions of every family the matcher takes, random sizes, through tc.define, against torch in
float64."""
import random
import string

import pytest
import torch

import tensorcomprehensions_b200 as tc

from helpers import assert_close

pytestmark = pytest.mark.gpu


def _names(rng, n, taken):
    out = []
    while len(out) < n:
        v = "x" + rng.choice(string.ascii_lowercase) + rng.choice("0123456789")  # (bare y1, j0, ... are TC built-ins)
        if v not in taken:
            taken.add(v)
            out.append(v)
    return out


def _decl(name, idx, size_of):
    return "float(%s) %s" % (", ".join(size_of[i] for i in idx), name)


def _contraction_case(rng, large=False):
    """O(batch..., m..., n...) +=! A(batch..., m.. | k..) * B(batch..., n.. | k..) with either group first.
    large: extents that reach the tensor-core tiles (two indices per group at most, 8..48 each)."""
    taken = set()
    nb, nm, nn, nk = rng.randint(0, 2), rng.randint(1, 2), rng.randint(0, 2), rng.randint(1, 2)
    if large:
        nb, nn = rng.randint(0, 1), rng.randint(1, 2)
    b, m, n, k = (_names(rng, c, taken) for c in (nb, nm, nn, nk))
    ext = {v: rng.randint(1, 24) for v in b + m + n + k}
    if large:
        ext = {v: (rng.randint(1, 3) if v in b else 4 * rng.randint(2, 12)) for v in ext}
    size_of = {v: "S" + v.upper() for v in ext}
    k_last = 0.85 if large else 0.5  # the tensor-core tiles take operands whose reduction index is innermost
    a_idx = b + (m + k if rng.random() < k_last else k + m)
    b_idx = b + (n + k if rng.random() < k_last else k + n)
    o_idx = b + m + n
    ops = [("A", a_idx), ("B", b_idx)]
    if rng.random() < 0.5:
        ops.reverse()  # multiplication commutes: either operand may come first
    text = "def f(%s, %s) -> (O) {\n  O(%s) +=! %s(%s) * %s(%s)\n}" % (
        _decl("A", a_idx, size_of), _decl("B", b_idx, size_of), ", ".join(o_idx),
        ops[0][0], ", ".join(ops[0][1]), ops[1][0], ", ".join(ops[1][1]))
    letters = {v: string.ascii_letters[i] for i, v in enumerate(ext)}
    spec = "%s,%s->%s" % tuple("".join(letters[v] for v in idx) for idx in (a_idx, b_idx, o_idx))
    shapes = [[ext[v] for v in a_idx], [ext[v] for v in b_idx]]
    red = 1
    for v in k:
        red *= ext[v]
    return text, shapes, lambda A, B: torch.einsum(spec, A, B), red


def _tensordot_case(rng):
    """Shared trailing indices: O(n, a, c, p...) +=! I0(n, a, r, p...) * I1(n, r, c, p...)."""
    N, A, R, C = rng.randint(1, 4), rng.randint(1, 40), rng.randint(1, 9), rng.randint(1, 5)
    trail = [rng.randint(1, 12) for _ in range(rng.randint(1, 2))]
    t_sz = ", ".join("P%d" % i for i in range(len(trail)))
    t_ix = ", ".join("p%d" % i for i in range(len(trail)))
    text = ("def f(float(N, A, R, %s) I0, float(N, R, C, %s) I1) -> (O) {\n  O(n, a, c, %s) +=! I0(n, a, r, %s) * I1(n, r, c, %s)\n}"
            % (t_sz, t_sz, t_ix, t_ix, t_ix))
    tl = "xyz"[:len(trail)]
    spec = "nar%s,nrc%s->nac%s" % (tl, tl, tl)
    return text, [[N, A, R] + trail, [N, R, C] + trail], lambda a, b: torch.einsum(spec, a, b), R


def _conv_case(rng):
    grouped = rng.random() < 0.5
    N, G, C, F = rng.randint(1, 3), rng.randint(1, 3) if grouped else 1, rng.randint(1, 9), rng.randint(1, 9)
    KH, KW, SH, SW = rng.randint(1, 4), rng.randint(1, 4), rng.randint(1, 3), rng.randint(1, 3)
    H, W = KH + rng.randint(0, 14), KW + rng.randint(0, 14)
    g_sz, g_ix = ("G, ", "g, ") if grouped else ("", "")
    text = ("def f(float(N, %sC, H, W) I, float(%sF, C, KH, KW) W1, float(%sF) B) -> (O) {\n"
            "  O(n, %sf, h, w) +=! I(n, %sc, %d * h + kh, %d * w + kw) * W1(%sf, c, kh, kw)\n"
            "  O(n, %sf, h, w) = O(n, %sf, h, w) + B(%sf)\n}" % (g_sz, g_sz, g_sz, g_ix, g_ix, SH, SW, g_ix, g_ix, g_ix, g_ix))
    i_shape = [N] + ([G] if grouped else []) + [C, H, W]
    w_shape = ([G] if grouped else []) + [F, C, KH, KW]
    b_shape = ([G] if grouped else []) + [F]

    def ref(I, W1, B):
        out = torch.nn.functional.conv2d(I.reshape(N, G * C, H, W), W1.reshape(G * F, C, KH, KW), B.reshape(G * F),
                                         stride=(SH, SW), groups=G)
        return out.reshape([N] + ([G] if grouped else []) + [F] + list(out.shape[2:]))
    return text, [i_shape, w_shape, b_shape], ref, C * KH * KW


def _reduction_case(rng):
    lead, mid, trail = rng.randint(0, 2), rng.randint(1, 2), rng.randint(0, 2)
    ext = [rng.randint(1, 30) for _ in range(lead + mid + trail)]
    ix = ["i%d" % d for d in range(len(ext))]
    kept = ix[:lead] + ix[lead + mid:]
    text = "def f(float(%s) I) -> (O) {\n  O%s +=! I(%s)\n}" % (
        ", ".join("D%d" % d for d in range(len(ext))), "(%s)" % ", ".join(kept) if kept else "", ", ".join(ix))
    dims = tuple(range(lead, lead + mid))
    red = 1
    for d in dims:
        red *= ext[d]
    return text, [ext], lambda I: I.sum(dims), red


CASES = {"contraction": (_contraction_case, 40), "contraction_large": (lambda rng: _contraction_case(rng, True), 16), "tensordot": (_tensordot_case, 12), "conv": (_conv_case, 20),
         "reduction": (_reduction_case, 20)}


@pytest.mark.parametrize("family", list(CASES))
def test_random_comprehensions_against_torch(cuda, family):
    make, count = CASES[family]
    rng = random.Random(20240 + len(family))
    g = torch.Generator().manual_seed(99)
    for case in range(count):
        text, shapes, ref, red = make(rng)
        ins = [torch.randn(s, generator=g, dtype=torch.float32) for s in shapes]
        T = tc.define(text, tc.make_naive_options_factory())
        out = T.f(*[t.to(cuda) for t in ins])
        expect = ref(*[t.double() for t in ins]).float()
        assert list(out.shape) == list(expect.shape), (text, shapes)
        assert_close(out, expect, red, ins, 1e-6, "%s case %d: %s %s" % (family, case, text, shapes))
