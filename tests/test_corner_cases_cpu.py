"""The reference's corner cases at the compile boundary (test/cuda/test_corner_cases.cc:84-160): the error fragments
its tests look for come out of the re-written front-end and compliance checks; the two trivial copies it expects to
succeed match the copy family; what it runs through its generic code generator (pointwise broadcasts, comparisons)
is a hard `no kernel family` error here, never a fallback."""
import pytest
import torch

import tensorcomprehensions_b200 as tc
from tensorcomprehensions_b200 import tclib


def F(*s):
    return torch.empty(*s) if s else torch.empty(())


def I(*s):
    return torch.empty(*s, dtype=torch.int32) if s else torch.empty((), dtype=torch.int32)


@pytest.mark.parametrize("fragment,text,inputs", [
    ("expected (", " def f{} {}", []),                                                              # E1
    ("expected 2 inputs", "def f(float a, float c) -> (b) { b(i) = a where i in 0:10 }", [F()]),      # E7
    ("expected type int32", "def f(int32 a) -> (b) { b(i) = a where i in 0:10 }", [F()]),            # E8
    ("expected a tensor with 0", "def f(int32 a) -> (b) { b(i) = a where i in 0:10 }", [I(1, 2)]),   # E9
    ("expected integral type", "def f(int32(N) a) -> (b) { b(i) = a(i + .5) }", [I(10)]),            # E11
    ("tensor accesses cannot be used in this context",
     "def f(int32 a, float(N) b) -> (c) { c(i) += b(i + j) where j in 0:a, i in 0:10 }", [I(), F(12)]),  # E12
    ("tensor accesses cannot be used in this context",
     "def f(int32 a, float(N) b) -> (c) { c(i) += b(i + j) where j in 0:a }", [I(), F(12)]),          # E13
])
def test_failures_carry_the_reference_fragments(fragment, text, inputs):
    with pytest.raises(tclib.ErrorReport) as e:
        tc.compile(text, "f", "naive", *inputs)
    assert fragment in str(e.value), str(e.value)


@pytest.mark.parametrize("text,inputs,elements", [
    ("def f(float(1) a) -> (b) { b(i) = a(i) }", [F(1)], 1),          # E2
    ("def f(float a) -> (b) { b = a }", [F()], 1),                     # E4: zero-dimensional tensors
    ("def f(float(N, M) a) -> (b) { b(i, j) = a(i, j) }", [F(5, 7)], 35),
])
def test_whole_tensor_copies_match_the_copy_family(text, inputs, elements):
    exe = tc.compile(text, "f", "naive", *inputs)
    launches = exe.launches()
    assert len(launches) == 1 and launches[0]["family"] == "copy" and launches[0]["elements"] == elements
    assert exe.output_shapes() == [list(inputs[0].shape)]


@pytest.mark.parametrize("text,inputs", [
    ("def f(float a) -> (b) { b(i) = a where i in 0:10 }", [F()]),                              # E6: broadcast
    ("def f(float a, float b) -> (c) { c(i) = float(a <= b) where i in 0:1 }", [F(), F()]),    # E15: comparison
    ("def f(float(N) a) -> (b) { b(i) = a(i) * 2 }", [F(4)]),                                   # pointwise arithmetic
    ("def f(float(N, M) a) -> (b) { b(j, i) = a(i, j) }", [F(3, 4)]),                           # a transposing copy
])
def test_pointwise_comprehensions_are_a_hard_error(text, inputs):
    with pytest.raises(tclib.ErrorReport, match="no kernel family"):
        tc.compile(text, "f", "naive", *inputs)
