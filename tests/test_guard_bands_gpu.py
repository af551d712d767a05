"""Out-of-bounds writes, caught without a sanitizer: every output sits between two guard bands of a known bit
pattern inside a larger allocation, on shapes that are not multiples of any tile; after the launch the bands must
still hold the pattern (and the output the right values).  One case per kernel of every family, tile edges included:
ragged rows / columns / k-blocks for the tensor-core tiles (their TMA stores clip at the tensor's edge, their direct
stores are predicated), split reductions with their second passes, the channel-split and multi-item convolutions."""
import pytest
import torch

from tensorcomprehensions_b200 import cabi

from helpers import assert_close

pytestmark = pytest.mark.gpu
GUARD = 4096  # floats on each side
PATTERN = -12345.6789


def guarded(shape, device, offset=0):
    """A view of `shape` inside a buffer with a guard band on each side (offset: extra floats in front, to break the
    16-byte alignment of the view)."""
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((GUARD + offset + n + GUARD,), PATTERN, device=device)
    view = buf[GUARD + offset:GUARD + offset + n].view(shape)
    view.fill_(float("nan"))
    return buf, view


def bands_intact(buf, n, offset=0):
    front = buf[:GUARD + offset]
    back = buf[GUARD + offset + n:]
    return bool((front == PATTERN).all()) and bool((back == PATTERN).all())


def tile(variant, bn=0, split_tf32=0, split_k=0, stages=0, bk=0, threads=0, bm=0):
    t = cabi.Tile()
    t.variant, t.bm, t.bn, t.bk, t.stages, t.threads, t.split_tf32, t.split_k = variant, bm, bn, bk, stages, threads, split_tf32, split_k
    return t


def rnd(shape, seed):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed))


CONTRACTIONS = [
    # (batch, M, N, K, a_k, b_k, epilogue, tile)
    (1, 130, 100, 132, True, True, cabi.EPI_BIAS_RELU, tile(cabi.VARIANT_TCGEN05_TS, 128, 3)),
    (1, 130, 100, 132, True, True, cabi.EPI_NONE, tile(cabi.VARIANT_TCGEN05_TS, 64, 3)),
    (1, 70, 230, 260, True, True, cabi.EPI_BIAS, tile(cabi.VARIANT_TCGEN05_TS, 112, 3)),
    (2, 300, 136, 96, True, True, cabi.EPI_NONE, tile(cabi.VARIANT_TCGEN05_PAIR, 128, 3)),
    (1, 100, 1000, 520, True, True, cabi.EPI_NONE, tile(cabi.VARIANT_TCGEN05_PAIR, 128, 3)),   # pair tiles written transposed
    (1, 300, 200, 1000, True, True, cabi.EPI_BIAS_RELU, tile(cabi.VARIANT_TCGEN05_TS, 64, 3, split_k=5)),
    (1, 5000, 500, 1800, True, True, cabi.EPI_BIAS_RELU, None),   # pair tiles with a split tail
    (1, 130, 100, 132, True, True, cabi.EPI_NONE, tile(cabi.VARIANT_TCGEN05, 128, 3)),
    (3, 70, 45, 33, True, False, cabi.EPI_NONE, tile(cabi.VARIANT_SIMT)),
    (3, 70, 45, 33, False, True, cabi.EPI_RELU, tile(cabi.VARIANT_SIMT)),
    (7, 26, 26, 72, True, False, cabi.EPI_NONE, None),             # batchmatmul default
    (7, 26, 26, 72, True, False, cabi.EPI_NONE, tile(cabi.VARIANT_SIMT_SMALL, 26, bk=4, bm=26)),  # 4x4 tiles, split reduction
    (5, 25, 22, 36, True, False, cabi.EPI_NONE, None),             # ragged small matrices
]


@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("case", CONTRACTIONS)
def test_contraction_outputs_stay_inside(cuda, case, offset):
    b, M, N, K, ak, bk, epi, t = case
    A = rnd((b, M, K) if ak else (b, K, M), 1)
    B = rnd((b, N, K) if bk else (b, K, N), 2)
    bias = rnd((N,), 3)
    a2 = A if ak else A.transpose(1, 2)
    b2 = B if bk else B.transpose(1, 2)
    ref = torch.matmul(a2.double(), b2.double().transpose(1, 2))
    if epi in (cabi.EPI_BIAS, cabi.EPI_BIAS_RELU):
        ref = ref + bias.double()
    if epi in (cabi.EPI_RELU, cabi.EPI_BIAS_RELU):
        ref = ref.clamp_min(0)
    p = cabi.contraction_problem(b, M, N, K, ak, bk, epilogue=epi)
    plan = cabi.Plan(p, t)
    buf, out = guarded((b, M, N), cuda, offset)
    ins = [A.to(cuda), B.to(cuda)] + ([bias.to(cuda)] if epi in (cabi.EPI_BIAS, cabi.EPI_BIAS_RELU) else [])
    plan.launch(ins, [out])
    torch.cuda.synchronize()
    assert bands_intact(buf, b * M * N, offset), plan.describe()
    assert_close(out, ref.float(), K, what=plan.describe())


@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("dims,stages", [
    ((3, 5, 16, 16, 16, 16, 3, 3), 3),     # tensor-core kernel, filter rows as accumulator rows (8-byte stores)
    ((9, 20, 16, 8, 11, 16, 3, 2), 3),     # ... odd row length (scalar stores), a short second unit, runs of items
    ((3, 5, 16, 16, 16, 16, 3, 3), 4),     # item kernel
    ((3, 5, 16, 16, 16, 16, 3, 3), 6),     # channel-split item kernel
    ((40, 16, 8, 12, 16, 16, 3, 3), 5),    # multi-item kernel, ragged last CTA
    ((2, 3, 5, 6, 11, 9, 3, 2), 0),        # band kernel, nothing a multiple of anything
    ((2, 2, 8, 8, 12, 12, 3, 3), None),    # whatever the default is
])
def test_group_conv_outputs_stay_inside(cuda, dims, stages, offset):
    N, G, C, F, H, W, KH, KW = dims
    I, W1, Bv = torch.rand((N, G, C, H, W)), torch.rand((G, F, C, KH, KW)), torch.rand((G, F))
    ref = torch.nn.functional.conv2d(I.reshape(N, G * C, H, W).double(), W1.reshape(G * F, C, KH, KW).double(),
                                     Bv.reshape(G * F).double(), groups=G).reshape(N, G, F, H - KH + 1, W - KW + 1)
    p = cabi.group_conv_problem(*dims)
    t = None
    if stages is not None:
        variant = cabi.VARIANT_TCGEN05_TS if stages == 3 else cabi.VARIANT_SIMT
        cands = [c for c in cabi.query(p) if c.variant == variant and c.stages == stages and (stages or c.bk == 0)]
        assert cands, "the tile this case is about is not listed"
        t = cands[0]
    plan = cabi.Plan(p, t)
    shape = tuple(ref.shape)
    buf, out = guarded(shape, cuda, offset)
    plan.launch([I.to(cuda), W1.to(cuda), Bv.to(cuda)], [out])
    torch.cuda.synchronize()
    assert bands_intact(buf, out.numel(), offset), plan.describe()
    assert_close(out, ref.float(), C * KH * KW, what=plan.describe())


@pytest.mark.parametrize("offset", [0, 1])
def test_tensordot_and_reduction_outputs_stay_inside(cuda, offset):
    I0, I1 = torch.rand((3, 21, 8, 5, 12)), torch.rand((3, 8, 2, 5, 12))
    ref = torch.einsum("nakhw,nkchw->nachw", I0.double(), I1.double())
    plan = cabi.Plan(cabi.tensordot_problem(3, 21, 8, 2, 60))
    buf, out = guarded(tuple(ref.shape), cuda, offset)
    plan.launch([I0.to(cuda), I1.to(cuda)], [out])
    torch.cuda.synchronize()
    assert bands_intact(buf, out.numel(), offset), plan.describe()
    assert_close(out, ref.float(), 8, what=plan.describe())
    for dims in [(5, 70001, 3), (1, 300007, 1), (37, 129, 1), (2, 33, 1000)]:
        A, C, B = dims
        X = torch.rand(dims)
        plan = cabi.Plan(cabi.reduction_problem(A, C, B))
        buf, out = guarded((A, B), cuda, offset)
        try:
            plan.launch([X.to(cuda)], [out])
        except cabi.Tcb200Error as e:
            # a tile that stores 128 bits at a time refuses an output view that is not 16-byte aligned (status, no
            # launch); the plain-float tile of the same family takes it
            assert offset == 1 and e.status == -4, plan.describe()
            plain = [t for t in cabi.query(cabi.reduction_problem(A, C, B)) if t.stages == 1][-1]
            plan = cabi.Plan(cabi.reduction_problem(A, C, B), plain)
            plan.launch([X.to(cuda)], [out])
        torch.cuda.synchronize()
        assert bands_intact(buf, A * B, offset), plan.describe()
        assert_close(out, X.double().sum(1).float(), C, what=plan.describe())
