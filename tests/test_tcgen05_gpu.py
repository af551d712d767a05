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
    if bn == 256 and split == 3:
        # one accumulation over the whole K: offered as a one-pass TF32 tile only
        with pytest.raises(cabi.Tcb200Error):
            cabi.Plan(cabi.contraction_problem(b, M, N, K, True, True), tc_tile(bn, split))
        return
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


@pytest.mark.parametrize("bn,split,ts", [(128, 3, True), (112, 3, True), (128, 3, False), (256, 1, False), (128, 1, False)])
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


def split_tile(bn, split_k, pair=False):
    t = tc_tile(bn, 3, ts=not pair, pair=pair)
    t.split_k = split_k
    return t


@pytest.mark.parametrize("case", [
    # (M, N, K, tile width, pair, split_k)
    (128, 2048, 4096, 128, False, 9),    # a 1/8 shard of the transposed matmul: 16 tiles x 9 splits, ragged last split
    (128, 2048, 4096, 112, False, 7),    # 19 tiles x 7 splits
    (2048, 512, 1024, 128, True, 2),     # MLP layer 2 on a 2048-row shard, CTA pairs
    (2048, 256, 512, 128, True, 4),      # MLP layer 3 on a 2048-row shard
    (300, 200, 1000, 64, False, 5),      # ragged everything, K not a multiple of the k-block
    (130, 130, 132, 128, False, 5),      # more splits than k-blocks that hold data: the last splits add zeros
])
@pytest.mark.parametrize("epi", [cabi.EPI_NONE, cabi.EPI_BIAS_RELU])
def test_split_k_tiles(cuda, case, epi):
    """The reduction split over several CTAs per output tile: partial sums in the plan's scratch, added in a
    fixed order by the second-pass kernel together with bias / ReLU.  Same criterion as the unsplit tiles, the
    same bits on every run, and the scratch is reused by later launches of the plan."""
    M, N, K, bn, pair, S = case
    A, B, bias = _rand((M, K), 61), _rand((N, K), 62), _rand((N,), 63)
    has_bias = epi == cabi.EPI_BIAS_RELU
    ref = orc.loop_fcrelu(A, B, bias if has_bias else None, relu=has_bias, double=True) if M * N * K < 2 ** 28 else None
    if ref is None:
        r = A.double() @ B.double().t()
        ref = (torch.clamp_min(r + bias.double(), 0) if has_bias else r).float()
    p = cabi.contraction_problem(1, M, N, K, True, True, epilogue=epi)
    ins = [A.to(cuda), B.to(cuda)] + ([bias.to(cuda)] if has_bias else [])
    out, plan = run_plan(p, ins, (M, N), split_tile(bn, S, pair))
    assert plan.tile().split_k == S
    assert_close(out, ref, K, [A, B], 3e-7, plan.describe())
    outs = []
    for _ in range(2):  # one plan, launched again: same scratch, same bits
        o = torch.full((M, N), float("nan"), device=cuda)
        plan.launch(ins, [o])
        torch.cuda.synchronize()
        outs.append(o)
    assert torch.equal(outs[0], out) and torch.equal(outs[1], out)


def test_split_k_accumulates_and_takes_odd_outputs(cuda):
    """`+=` through the second pass, and an output view at a 4-byte offset (scalar second pass)."""
    M, N, K, S = 128, 384, 2048, 4
    A, B = _rand((M, K), 64), _rand((N, K), 65)
    init = _rand((M, N), 66)
    ref = (A.double() @ B.double().t() + init.double()).float()
    p = cabi.contraction_problem(1, M, N, K, True, True, accumulate=True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (M, N), split_tile(128, S), out_init=init.to(cuda))
    assert_close(out, ref, K, what=plan.describe())
    p = cabi.contraction_problem(1, M, N, K, True, True)
    buf = torch.full((M * N + 1,), float("nan"), device=cuda)
    view = buf[1:].view(M, N)
    plan = cabi.Plan(p, split_tile(128, S))
    plan.launch([A.to(cuda), B.to(cuda)], [view])
    torch.cuda.synchronize()
    assert_close(view, (A.double() @ B.double().t()).float(), K, [A, B], 3e-7, plan.describe())


def test_shard_shapes_get_a_split_by_default(cuda):
    """What the family default is on the 1/8 shards of the benchmark contractions: the transposed matmul's
    2048-column shard and the last two MLP layers on 2048 rows split their reductions, the full-size
    problems do not."""
    full = cabi.Plan(cabi.contraction_problem(1, 128, 16384, 4096, True, True))
    assert full.tile().split_k <= 1
    shard = cabi.Plan(cabi.contraction_problem(1, 128, 2048, 4096, True, True))
    assert shard.tile().split_k > 1, shard.describe()
    g = shard.geometry()[0][0]
    assert 120 <= g <= 148, shard.describe()
    l3 = cabi.Plan(cabi.contraction_problem(1, 2048, 256, 512, True, True, epilogue=cabi.EPI_BIAS_RELU))
    assert l3.tile().split_k > 1, l3.describe()
    A, B, bias = _rand((2048, 512), 67), _rand((256, 512), 68), _rand((256,), 69)
    out = torch.full((2048, 256), float("nan"), device=cuda)
    l3.launch([A.to(cuda), B.to(cuda), bias.to(cuda)], [out])
    torch.cuda.synchronize()
    ref = torch.clamp_min(A.double() @ B.double().t() + bias.double(), 0).float()
    assert_close(out, ref, 512, [A, B], 3e-7, l3.describe())


@pytest.mark.parametrize("case", [
    # (M, N, K, tile width, pair)
    (128, 2048, 4096, 112, False),   # the transposed matmul of tc/benchmarks/tmm.cc:63-64 on its own rand() data
    (128, 2048, 4096, 128, False),
    (1024, 1024, 2048, 128, True),   # a fully connected layer of tc/benchmarks/MLP_model.cc:524-530 on rand() data
    (512, 256, 512, 128, True),
])
def test_strict_accumulation_tiles_meet_the_reference_bound_on_all_positive_data(cuda, case):
    """split_tf32 = 4: the accumulators are drained after every k-block.  On U[0,1) operands, where the
    truncating accumulation of the tensor core has a sign, the result is inside the reference's own
    checkRtol bound 3e-7 * K * max|input| (test/test_harness_aten.h:36-54), which the default tiles miss at
    K = 4096 (2.8e-3 against 1.2e-3); the default tiles' error is printed beside it."""
    M, N, K, bn, pair = case
    g = torch.Generator().manual_seed(71)
    A, B = torch.rand((M, K), generator=g), torch.rand((N, K), generator=g)
    ref = A.double() @ B.double().t()
    p = cabi.contraction_problem(1, M, N, K, True, True)
    errs = {}
    for split in (4, 3):
        out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (M, N), tc_tile(bn, split, ts=not pair, pair=pair))
        assert plan.tile().split_tf32 == split
        errs[split] = (out.cpu().double() - ref).abs().max().item()
    bound = 3e-7 * K * 1.0
    print("K=%d bound %.3e: strict tile %.3e, default tile %.3e" % (K, bound, errs[4], errs[3]))
    assert errs[4] < bound, (errs, bound)


@pytest.mark.parametrize("case", [
    # (M, N, K): CTA-pair tiles that do not fill the last round of the 74 pairs
    (5120, 512, 2048),     # 80 tiles: one full round and 6 tail tiles split 4 ways
    (5000, 500, 1800),     # the same with ragged rows, columns and k-blocks
    (8192, 1024, 2048),    # MLP layer 1 on an 8192-row shard: 256 tiles, 34 tail tiles split in two
])
@pytest.mark.parametrize("epi", [cabi.EPI_NONE, cabi.EPI_BIAS_RELU])
def test_pair_tiles_with_a_split_tail(cuda, case, epi):
    """The last, partly filled round of the persistent CTA pairs runs as units of 1 / S of the reduction whose
    partial tiles a second kernel adds: same criterion as the plain pair tiles, same bits on every run, and
    the default for these shapes."""
    M, N, K = case
    A, B, bias = _rand((M, K), 81), _rand((N, K), 82), _rand((N,), 83)
    has_bias = epi == cabi.EPI_BIAS_RELU
    r = A.double() @ B.double().t()
    ref = (torch.clamp_min(r + bias.double(), 0) if has_bias else r).float()
    p = cabi.contraction_problem(1, M, N, K, True, True, epilogue=epi)
    ins = [A.to(cuda), B.to(cuda)] + ([bias.to(cuda)] if has_bias else [])
    out, plan = run_plan(p, ins, (M, N))
    assert plan.tile().variant == cabi.VARIANT_TCGEN05_PAIR and "tail_split" in plan.describe(), plan.describe()
    assert_close(out, ref, K, [A, B], 3e-7, plan.describe())
    out2 = torch.full((M, N), float("nan"), device=cuda)
    plan.launch(ins, [out2])
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    # the plain pair tile gives the same values up to the order of the additions in the tail
    plain = tc_tile(128, 3, pair=True)
    plain.split_k = 1
    out3, plan3 = run_plan(p, ins, (M, N), plain)
    assert "tail_split" not in plan3.describe()
    assert_close(out3, ref, K, [A, B], 3e-7, plan3.describe())


def test_pair_tail_split_accumulates_and_takes_odd_outputs(cuda):
    M, N, K = 5120, 512, 1792
    A, B, init = _rand((M, K), 84), _rand((N, K), 85), _rand((M, N), 86)
    ref = (A.double() @ B.double().t() + init.double()).float()
    p = cabi.contraction_problem(1, M, N, K, True, True, accumulate=True)
    out, plan = run_plan(p, [A.to(cuda), B.to(cuda)], (M, N), out_init=init.to(cuda))
    assert "tail_split" in plan.describe()
    assert_close(out, ref, K, what=plan.describe())
    # an output view at a 4-byte offset: direct stores for the whole tiles, scalar second pass for the tail
    p = cabi.contraction_problem(1, M, N, K, True, True)
    buf = torch.full((M * N + 1,), float("nan"), device=cuda)
    view = buf[1:].view(M, N)
    plan = cabi.Plan(p)
    plan.launch([A.to(cuda), B.to(cuda)], [view])
    torch.cuda.synchronize()
    assert_close(view, (A.double() @ B.double().t()).float(), K, [A, B], 3e-7, plan.describe())


@pytest.mark.parametrize("case", [
    # (M, N, K, ldc offset): at most 128 rows, so the CTA-pair kernel runs C^T = B A^T and writes its tiles transposed
    (128, 1024, 512, 0),      # four pair tiles, everything aligned: staged tiles, TMA stores
    (100, 1000, 520, 0),      # ragged rows, columns and k-blocks: the stores clip
    (128, 16384, 4096, 0),    # the transposed matmul of the benchmark: 64 pair tiles
    (77, 600, 256, 1),        # an output view at a 4-byte offset: strided direct stores
])
def test_pair_tiles_with_a_transposed_output(cuda, case):
    _transposed_case(cuda, case, 1)


@pytest.mark.parametrize("case,split", [
    ((128, 2048, 4096, 0), 8),    # the 1/8 shard of the transposed matmul: 8 pair tiles, the reduction split 8 ways
    ((100, 1000, 520, 0), 3),     # ragged everything, k-blocks that do not divide by the split
    ((128, 512, 1024, 1), 4),     # the second pass writes an output view at a 4-byte offset
])
def test_pair_tiles_with_a_transposed_output_and_a_split_reduction(cuda, case, split):
    """The partial planes are written transposed as well, i.e. in the output's own orientation, and the same
    second pass as for every other split adds them."""
    _transposed_case(cuda, case, split)
    M, N, K, _ = case
    if (M, N, K) == (128, 2048, 4096):   # what the family lists first for that shard
        first = cabi.query(cabi.contraction_problem(1, M, N, K, True, True))[0]
        assert first.variant == cabi.VARIANT_TCGEN05_PAIR and first.split_k > 1


def _transposed_case(cuda, case, split):
    M, N, K, off = case
    A, B = _rand((M, K), 91), _rand((N, K), 92)
    ref = (A.double() @ B.double().t()).float()
    p = cabi.contraction_problem(1, M, N, K, True, True)
    t = tc_tile(128, 3, pair=True)
    t.split_k = split
    plan = cabi.Plan(p, t)
    assert plan.tile().variant == cabi.VARIANT_TCGEN05_PAIR and plan.geometry()[0][0] == 2 * min(74, -(-N // 256) * split)
    buf = torch.full((M * N + off,), float("nan"), device=cuda)
    out = buf[off:].view(M, N)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    plan.launch([A.to(cuda), B.to(cuda)], [out], dev_status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_close(out, ref, K, [A, B], 3e-7, plan.describe())
    out2 = torch.full((M, N), float("nan"), device=cuda)
    plan.launch([A.to(cuda), B.to(cuda)], [out2])
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    # an epilogue or "+=" keeps the kernel's own orientation (one CTA of each pair idles on these shapes)
    pe = cabi.contraction_problem(1, M, N, K, True, True, accumulate=True)
    init = _rand((M, N), 93)
    out3, plan3 = run_plan(pe, [A.to(cuda), B.to(cuda)], (M, N), t, out_init=init.to(cuda))
    assert_close(out3, (A.double() @ B.double().t() + init.double()).float(), K, what=plan3.describe())
