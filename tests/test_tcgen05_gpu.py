"""The tcgen05/TMEM contraction kernel (explicit tiles) against the CPU checker.  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tensorcomprehensions_b200 import cabi
from tensorcomprehensions_b200 import workloads as wl

from helpers import STRICT, assert_close, run_plan

pytestmark = pytest.mark.gpu


def _rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32)


def tc_tile(bn, split, ts=False, pair=False):
    t = cabi.Tile()
    variant = cabi.VARIANT_TCGEN05_PAIR if pair else cabi.VARIANT_TCGEN05_TS if ts else cabi.VARIANT_TCGEN05
    t.variant, t.bn, t.split_tf32 = variant, bn, split
    return t


def ref64(A, B):
    return torch.matmul(A.double(), B.double().transpose(-1, -2)).float()


@pytest.mark.parametrize("bn", [128, 64, 256])
@pytest.mark.parametrize("split", [1, 3])
@pytest.mark.parametrize("shape", [(1, 128, 256, 128), (1, 256, 384, 512), (1, 70, 200, 132), (3, 130, 96, 256)])
def test_tcgen05_tiles(cuda, bn, split, shape):
    b, M, N, K = shape
    A, B = _rand((b, M, K), 21), _rand((b, N, K), 22)
    ref = ref64(A, B)
    p = cabi.contraction_problem(b, M, N, K, True, True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (b, M, N), tc_tile(bn, split))
    # one TF32 pass keeps 10 mantissa bits per operand: only the benchmark criterion applies;
    # the 3xTF32 split must also meet the reference's own checkRtol at 3e-7.
    assert_close(out, ref, K, [A, B], 3e-7 if split == 3 else None, plan.describe())


@pytest.mark.parametrize("bn", [128, 112, 64])
@pytest.mark.parametrize("shape", [(1, 128, 256, 128), (1, 256, 384, 512), (1, 70, 200, 132), (3, 130, 96, 256),
                                   (1, 300, 128, 4096)])
def test_tcgen05_ts_tiles(cuda, bn, shape):
    """A operand staged in tensor memory: must meet the reference's own checkRtol too."""
    b, M, N, K = shape
    A, B = _rand((b, M, K), 31), _rand((b, N, K), 32)
    p = cabi.contraction_problem(b, M, N, K, True, True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (b, M, N), tc_tile(bn, 3, ts=True))
    assert "tcgen05_ts" in plan.describe()
    assert_close(out, ref64(A, B), K, [A, B], 3e-7, plan.describe())


@pytest.mark.parametrize("shape", [(1, 256, 128, 128), (1, 512, 384, 512), (1, 70, 200, 132), (3, 130, 96, 256),
                                   (1, 300, 128, 4096), (2, 700, 300, 1056), (1, 4096, 256, 64)])
def test_tcgen05_pair_tiles(cuda, shape):
    """CTA pairs (cta_group::2): 256-row tiles, each CTA stages half of B; ragged rows/columns, batches,
    odd numbers of k-blocks, tiles where the second CTA of the pair has no rows at all."""
    b, M, N, K = shape
    A, B = _rand((b, M, K), 41), _rand((b, N, K), 42)
    p = cabi.contraction_problem(b, M, N, K, True, True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (b, M, N), tc_tile(128, 3, pair=True))
    assert "tcgen05_pair" in plan.describe()
    assert_close(out, ref64(A, B), K, [A, B], 3e-7, plan.describe())
    out2, _ = run_plan(p, [A.to(cuda), B.to(cuda)], (b, M, N), tc_tile(128, 3, pair=True))
    assert torch.equal(out, out2)  # one accumulator per issuer: the same bits on every run


@pytest.mark.parametrize("epi", [cabi.EPI_NONE, cabi.EPI_BIAS, cabi.EPI_BIAS_RELU, cabi.EPI_RELU])
@pytest.mark.parametrize("N", [384, 100])  # 100: ragged columns -> scalar stores
@pytest.mark.parametrize("kind", ["ss", "ts", "pair"])
def test_tcgen05_epilogues(cuda, epi, N, kind):
    tile = lambda: tc_tile(128 if N >= 128 else 64, 3, ts=kind == "ts", pair=kind == "pair")
    if kind == "pair" and N < 128:
        tile = lambda: tc_tile(128, 3, pair=True)
    M, K = 200, 320
    I, W, b = _rand((M, K), 23), _rand((N, K), 24), _rand((N,), 25)
    has_bias = epi in (cabi.EPI_BIAS, cabi.EPI_BIAS_RELU)
    ref = orc.loop_fcrelu(I, W, b if has_bias else None, relu=epi in (cabi.EPI_BIAS_RELU, cabi.EPI_RELU),
                          double=True)
    p = cabi.contraction_problem(1, M, N, K, True, True, epilogue=epi)
    ins = [I.to(cuda), W.to(cuda)] + ([b.to(cuda)] if has_bias else [])
    out, plan = run_plan(p, ins, (M, N), tile())
    assert_close(out, ref, K, [I, W], 3e-7, plan.describe())
    if epi == cabi.EPI_NONE:
        p2 = cabi.contraction_problem(1, M, N, K, True, True, accumulate=True)
        init = _rand((M, N), 26).to(cuda)
        out2, _ = run_plan(p2, ins, (M, N), tile(), out_init=init)
        assert_close(out2, ref + init.cpu().numpy(), K, what="accumulate")


def test_tcgen05_shared_operand(cuda):
    b, M, N, K = 4, 128, 128, 128
    A, B = _rand((b, M, K), 27), _rand((N, K), 28)
    ref = ref64(A, B)
    p = cabi.contraction_problem(b, M, N, K, True, True, stride_b=0)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (b, M, N), tc_tile(128, 3))
    assert_close(out, ref, K, [A, B], 3e-7, plan.describe())


@pytest.mark.parametrize("kind", ["ts", "pair"])
def test_tcgen05_ts_and_pair_corner_forms(cuda, kind):
    """Forms the matcher produces besides the plain ones: an operand shared by all batch entries, bias
    indexed by the row, K that is not a multiple of the k-block, padded leading dimensions, narrow N."""
    tile = lambda: tc_tile(128, 3, ts=kind == "ts", pair=kind == "pair")
    # shared B (stride 0) over 3 batches, K = 132 (4 k-blocks + 4 columns)
    b, M, N, K = 3, 260, 160, 132
    A, B = _rand((b, M, K), 51), _rand((N, K), 52)
    p = cabi.contraction_problem(b, M, N, K, True, True, stride_b=0)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (b, M, N), tile())
    assert_close(out, ref64(A, B), K, [A, B], 3e-7, plan.describe())
    # bias along the rows (O(m,n) + Bias(m)) with ReLU
    M, N, K = 300, 200, 256
    A, B, bias = _rand((M, K), 53), _rand((N, K), 54), _rand((M,), 55)
    ref = np.maximum((A.double() @ B.double().t() + bias.double()[:, None]).numpy(), 0)
    p = cabi.contraction_problem(1, M, N, K, True, True, epilogue=cabi.EPI_BIAS_RELU, bias_on_m=True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda), bias.to(cuda)], (M, N), tile())
    assert_close(out, ref, K, [A, B], 3e-7, plan.describe())
    # padded leading dimensions of all three tensors (views into wider buffers), N narrower than a tile
    M, N, K = 384, 96, 512
    Ab, Bb = _rand((M, K + 8), 56), _rand((N, K + 4), 57)
    A, B = Ab[:, :K], Bb[:, :K]
    Ad, Bd = Ab.to(cuda), Bb.to(cuda)
    Cd = torch.full((M, N + 4), float("nan"), device=cuda)
    p = cabi.contraction_problem(1, M, N, K, True, True, lda=K + 8, ldb=K + 4, ldc=N + 4)
    plan = cabi.Plan(p, tile())
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    plan.launch_ptrs([Ad.data_ptr(), Bd.data_ptr()], [Cd.data_ptr()],
                     stream=torch.cuda.current_stream().cuda_stream, dev_status=status.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_close(Cd[:, :N].cpu(), ref64(A, B), K, [A, B], 3e-7, plan.describe())
    assert torch.isnan(Cd[:, N:]).all()  # the padding columns are not written


@pytest.mark.parametrize("kind,limit", [("ts", 3.2e-6), ("pair", 6.4e-6)])
def test_tcgen05_all_positive_operands(cuda, kind, limit):
    """The tensor core truncates when it adds into its fp32 accumulator, so with all-positive operands
    (the reference's own U[0,1) benchmark data) the error has a sign.  Draining the accumulators into
    round-to-nearest adds every 4 (single CTA) / 8 (CTA pair) k-blocks bounds it: relative error of a
    K = 2048 sum below 3.2e-6 / 6.4e-6 (measured 2.7e-6 / 5.2e-6), i.e. inside the 1e-6 * (K + 1) * max|in|
    bound of the reference's MLP1 / C3 checks (tc/benchmarks/MLP_model.cc:413-417,469-473) for the
    single-CTA kernel."""
    M, N, K = 256, 256, 2048
    g = torch.Generator().manual_seed(61)
    A, B = torch.rand((M, K), generator=g), torch.rand((N, K), generator=g)
    ref = A.double() @ B.double().t()
    p = cabi.contraction_problem(1, M, N, K, True, True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (M, N), tc_tile(128, 3, ts=kind == "ts", pair=kind == "pair"))
    err = (out.cpu().double() - ref).abs().max().item()
    assert err / ref.max().item() < limit, (err, plan.describe())
    if kind == "ts":
        assert err < 1e-6 * (K + 1) * 1.0


def test_tcgen05_rejects_what_it_cannot_take(cuda):
    # K not a multiple of 4 breaks the 16-byte row pitch TMA needs: the plan is refused
    p = cabi.contraction_problem(1, 128, 128, 130, True, True)
    with pytest.raises(cabi.Tcb200Error) as e:
        cabi.Plan(p, tc_tile(128, 3))
    assert e.value.status == -2
    p = cabi.contraction_problem(1, 128, 128, 128, True, False)
    with pytest.raises(cabi.Tcb200Error):
        cabi.Plan(p, tc_tile(128, 3))


@pytest.mark.parametrize("bn,split,ts", [(128, 3, True), (112, 3, True), (128, 3, False), (256, 3, False), (128, 1, False)])
def test_tmm_full_size_tcgen05(cuda, bn, split, ts):
    w = wl.tmm()
    A, B = wl.make_inputs(w)
    p = cabi.contraction_problem(1, 128, 16384, 4096, True, True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (128, 16384), tc_tile(bn, split, ts))
    # gate on the reference's own checkRtol for the A-in-tensor-memory tiles (the family default among them);
    # the plain SS tiles with one long accumulation per tile only log it
    assert_close(out, orc.aten_tmm(A, B), 4096, [A, B], STRICT["tmm"] if split == 3 else None, plan.describe(),
                 strict_is_gate=ts)


def test_mlp3_full_size_tcgen05(cuda):
    w = wl.mlp3()
    ins = wl.make_inputs(w)
    I, W2, B2, W3, B3, W4, B4 = [t.to(cuda) for t in ins]
    refs = orc.aten_mlp3(*ins)
    x = I
    for (Wt, Bt, L), ref in zip(((W2, B2, 2048), (W3, B3, 1024), (W4, B4, 512)), refs):
        p = cabi.contraction_problem(1, x.shape[0], Wt.shape[0], x.shape[1], True, True,
                                     epilogue=cabi.EPI_BIAS_RELU)
        out, plan = run_plan(p, [x, Wt, Bt], (x.shape[0], Wt.shape[0]), tc_tile(128, 3))
        assert_close(out, ref, L, ins, STRICT["mlp3"], plan.describe(), strict_is_gate=False)
        x = out
