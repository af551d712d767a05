"""Shared helpers of the parity tests: run one problem through the C ABI, compare with the checker."""
import numpy as np
import torch

from oracle import oracle as orc
from tensorcomprehensions_b200 import cabi

# Pass criterion: max|out - ref| / max|ref| <= 1e-5 * reduction length (stated by the
# benchmark definition; restates checkRtol, test/test_harness_aten.h:36-54).
RTOL = 1e-5
# Reference-strict machine precisions per benchmark (logged, and asserted for the exact-fp32 kernels):
# tensordot 5e-7 (test/cuda/test_tc_mapper_bugs.cc:105), bmm/tmm/mlp 3e-7, group conv 1e-6.
STRICT = {"tensordot": 5e-7, "batchmatmul": 3e-7, "tmm": 3e-7, "group_conv": 1e-6, "mlp3": 3e-7}


def run_plan(problem, inputs, out_shape, tile=None, out_init=None):
    dev = inputs[0].device
    plan = cabi.Plan(problem, tile, device=dev.index or 0)
    if out_init is not None:
        out = out_init.clone()
    else:
        # NaN canary: a "+=!" kernel must overwrite every element.
        out = torch.full(out_shape, float("nan"), device=dev, dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    plan.launch(inputs, [out], dev_status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "device status %d (%s)" % (int(status.item()), plan.describe())
    return out, plan


def assert_close(out, ref, L, inputs=None, strict=None, what="", strict_is_gate=True):
    """Gate: the benchmark criterion.  `strict` adds the reference's own checkRtol form with the
    machine precision its benchmark uses; it is a gate for the exact-fp32 kernels and (with
    strict_is_gate=False) a logged secondary figure elsewhere."""
    out_np = out.detach().cpu().numpy() if hasattr(out, "detach") else np.asarray(out)
    ref_np = ref.detach().cpu().numpy() if hasattr(ref, "detach") else np.asarray(ref)
    assert out_np.shape == ref_np.shape, (out_np.shape, ref_np.shape)
    assert np.isfinite(out_np).all(), "non-finite output (unwritten canary?) " + what
    ok, e = orc.check_rtol_baseline(out_np, ref_np, L, RTOL)
    assert ok, "%s: rel err %.3e > %.3e" % (what, e, RTOL * L)
    if strict is not None and inputs is not None:
        ok2, d, bound = orc.check_rtol_reference(out_np, ref_np, inputs, L, strict)
        msg = "%s: strict checkRtol: max diff %.3e vs bound %.3e" % (what, d, bound)
        if strict_is_gate:
            assert ok2, msg
        elif not ok2:
            import warnings
            warnings.warn(msg)
    return e
