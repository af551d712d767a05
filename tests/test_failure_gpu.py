"""Failure reporting without a fault: a device-side wait that runs out is recorded in the status word, reaches
the host as TCB200_ERR_DEVICE_TIMEOUT, and leaves the context usable.  The wait that runs out is the library's
own self-test (one warp waiting on a barrier nothing arrives on, with a short limit); no kernel is made to
trap, fault or hang."""
import ctypes

import pytest
import torch

import tensorcomprehensions_b200 as tc
from oracle import oracle as orc
from tensorcomprehensions_b200 import cabi
from tensorcomprehensions_b200 import workloads as wl

from helpers import STRICT, assert_close

pytestmark = pytest.mark.gpu
ERR_DEVICE_TIMEOUT = -5


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(cuda):
    L = cabi.lib()
    status = ctypes.c_void_p()
    cabi.check(L.tcb200_status_create(ctypes.byref(status)), "tcb200_status_create")
    stream = torch.cuda.current_stream().cuda_stream
    code = ctypes.c_int(-1)
    try:
        assert L.tcb200_status_check(status, stream, ctypes.byref(code)) == cabi.OK and code.value == 0
        # limits the kernels never use are refused on the host
        assert L.tcb200_selftest_wait(0, status, stream) == -1
        assert L.tcb200_selftest_wait(10 ** 12, status, stream) == -1
        # about half a millisecond of waiting, then the warp gives up and records its code
        cabi.check(L.tcb200_selftest_wait(1000000, status, stream), "tcb200_selftest_wait")
        rc = L.tcb200_status_check(status, stream, ctypes.byref(code))
        assert rc == ERR_DEVICE_TIMEOUT and code.value == 99
        assert "wait gave up" in cabi.strerror(rc)
        # the word was cleared, and a normal launch that reports into it is correct and leaves it at zero
        I0 = torch.rand((2, 16, 8, 4, 8), generator=torch.Generator().manual_seed(3))
        I1 = torch.rand((2, 8, 2, 4, 8), generator=torch.Generator().manual_seed(4))
        out = torch.full((2, 16, 2, 4, 8), float("nan"), device=cuda)
        plan = cabi.Plan(cabi.tensordot_problem(2, 16, 8, 2, 32))
        d0, d1 = I0.to(cuda), I1.to(cuda)
        plan.launch_ptrs([d0.data_ptr(), d1.data_ptr()], [out.data_ptr()], stream, status.value)
        assert L.tcb200_status_check(status, stream, ctypes.byref(code)) == cabi.OK and code.value == 0
        assert_close(out, orc.loop_tensordot(I0, I1), 8, [I0, I1], STRICT["tensordot"])
    finally:
        L.tcb200_status_destroy(status)


def test_executor_owns_a_status_word(cuda):
    """Every launch of an executor reports into the executor's own word; profile() and check_device_status()
    read it (and would raise): after healthy runs both pass."""
    w = wl.ALL["mlp3"](**wl.SMALL["mlp3"])
    ins = [t.to(cuda) for t in wl.make_inputs(w)]
    exe = tc.compile(w.tc, w.entry, "naive", *ins)
    outs = exe(*ins)
    exe.check_device_status(0)
    assert exe.profile(*ins, outputs=list(outs))["kernel_runtime_us"] > 0


@pytest.mark.parametrize("name", ["batchmatmul", "group_conv"])
def test_profile_times_short_kernels_at_device_pace(cuda, name):
    """profile() replays a short def from a graph until the window holds ~200 us: two calls agree, and the time
    is that of the kernel, not of a host launch (well under the ~20 us one launch through Python costs)."""
    w = wl.ALL[name]()
    ins = [t.to(cuda) for t in wl.make_inputs(w)]
    exe = tc.compile(w.tc, w.entry, "naive", *ins)
    outs = [torch.empty(s, device=cuda) for s in exe.output_shapes()]
    exe.profile(*ins, outputs=outs)
    t = sorted(exe.profile(*ins, outputs=outs)["kernel_runtime_us"] for _ in range(5))
    assert t[0] > 0.5 and t[-1] / t[0] < 1.5, t
    refs = orc.as_list(orc.ATEN[name](*wl.make_inputs(w)))
    assert_close(outs[0], refs[0], w.reduction[0], what=name)  # the replays leave the same output
