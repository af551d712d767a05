"""tcb200_reduce_launch_static: the reduction launch whose scratch (tickets + partial sums) is a fixed
array of the library image instead of memory the plan allocates.  Compared with tcb200_launch on the
same plans: the kernel and the order of the additions are the same, so the bits must be equal.  This
file is collected last on purpose: the array is shared by every call of the process, so the checks must
hold whatever ran before, and when the file runs alone."""
import pytest
import torch

from oracle import oracle as orc
from tensorcomprehensions_b200 import cabi

from helpers import assert_close

pytestmark = pytest.mark.gpu

# shapes whose default plan splits the reduced range (scratch in use), one that does not
SPLIT = [(1, 3000001, 1), (64, 100000, 1), (1, 5000, 4096), (2, 70000, 3)]


def _rand(shape, seed):
    return torch.rand(shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float32)


@pytest.mark.parametrize("dims", SPLIT + [(600, 1024, 1)])
def test_static_scratch_launch_matches_the_allocating_launch_twice_in_a_row(cuda, dims):
    A, C, B = dims
    plan = cabi.Plan(cabi.reduction_problem(A, C, B))
    if dims in SPLIT:
        assert plan.geometry()[0][1] > 1, plan.describe()  # several segments: partial sums and tickets are used
    for call in range(2):  # the second call finds the tickets the first one left: they must be zero again
        I = _rand((A, C, B), 300 + call).to(cuda)
        ref = torch.full((A, B), float("nan"), device=cuda)
        out = torch.full((A, B), float("nan"), device=cuda)
        plan.launch([I], [ref])
        plan.launch_static(I, out)
        torch.cuda.synchronize()
        assert torch.equal(out, ref), (call, plan.describe())
        assert_close(out, orc.loop_reduce(I.cpu(), double=True), C, [I.cpu()], 5e-7, plan.describe())


def test_static_scratch_is_shared_between_plans_on_one_stream(cuda):
    """Different plans, back to back on one stream, no synchronisation in between: stream order keeps
    their use of the one array apart."""
    cases = []
    for k, dims in enumerate(SPLIT):
        I = _rand(dims, 400 + k).to(cuda)
        plan = cabi.Plan(cabi.reduction_problem(*dims))
        out = torch.full((dims[0], dims[2]), float("nan"), device=cuda)
        cases.append((plan, I, out))
    for _ in range(2):
        for plan, I, out in cases:
            plan.launch_static(I, out)
    torch.cuda.synchronize()
    for plan, I, out in cases:
        ref = torch.empty_like(out)
        plan.launch([I], [ref])
        torch.cuda.synchronize()
        assert torch.equal(out, ref), plan.describe()


def test_static_scratch_accumulating_form(cuda):
    dims = (1, 200000, 1)
    I, init = _rand(dims, 500).to(cuda), _rand((1, 1), 501).to(cuda)
    plan = cabi.Plan(cabi.reduction_problem(*dims, accumulate=True))
    ref, out = init.clone(), init.clone()
    plan.launch([I], [ref])
    plan.launch_static(I, out)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


def test_static_scratch_refuses_what_does_not_fit(cuda):
    """A tile whose partial sums exceed the fixed array is refused before anything is launched; so is a
    plan of another family."""
    A, C, B = 64, 1 << 16, 1024
    t = cabi.Tile()
    t.variant, t.bm, t.bn, t.stages = cabi.VARIANT_SIMT, 32, 512, 1   # 64 * 32 tiles: 2048 tickets, 33.5 M partial sums
    plan = cabi.Plan(cabi.reduction_problem(A, C, B), t)
    I = torch.zeros(8, device=cuda)  # never read: the call must fail on the sizes alone
    out = torch.full((8,), 7.0, device=cuda)
    with pytest.raises(cabi.Tcb200Error) as e:
        plan.launch_static(I, out)
    assert e.value.status == -7  # TCB200_ERR_TOO_LARGE
    other = cabi.Plan(cabi.contraction_problem(1, 64, 64, 64, True, True))
    with pytest.raises(cabi.Tcb200Error) as e:
        other.launch_static(I, out)
    assert e.value.status == -1
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())


def test_static_scratch_launch_takes_no_device_memory(cuda):
    """The reason the entry point exists: a plan that has never gone through the allocating launch runs
    through the static one without the device's free memory moving.  (One earlier call of the entry point,
    with another plan, has loaded the kernels and looked the array up: what the driver takes for code when a
    module is first used is not this call's doing.)"""
    warm_dims = (1, 300000, 1)
    warm = cabi.Plan(cabi.reduction_problem(*warm_dims))
    warm.launch_static(_rand(warm_dims, 599).to(cuda), torch.empty((1, 1), device=cuda))
    dims = (1, 2500000, 1)
    I = _rand(dims, 600).to(cuda)
    out = torch.full((1, 1), float("nan"), device=cuda)
    plan = cabi.Plan(cabi.reduction_problem(*dims))
    assert plan.geometry()[0][1] > 1
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):
        plan.launch_static(I, out)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert_close(out, orc.loop_reduce(I.cpu(), double=True), dims[1], [I.cpu()], 5e-7, plan.describe())
