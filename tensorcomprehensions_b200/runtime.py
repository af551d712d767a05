"""Glue used by the benchmark: compile one benchmark comprehension for a device and run it."""
import torch

from . import cabi


class _Exe:
    def __init__(self, w, dev, steps):
        """steps: list of (problem, input index list, output index) over a value table
        [inputs..., outputs...]."""
        self.w, self.dev, self.steps = w, dev, steps
        self.plans = [cabi.Plan(p, None, dev.index or 0) for p, _, _ in steps]
        self.launches = len(steps)
        tiles = [pl.tile() for pl in self.plans]
        self.split_tf32 = max(t.split_tf32 for t in tiles)
        self.n_in = len(w.shapes)

    def _out_shapes(self):
        return OUT_SHAPES[self.w.name](self.w)

    def prepare_outputs(self):
        return [torch.empty(s, dtype=torch.float32, device=self.dev) for s in self._out_shapes()]

    def run(self, inputs, outputs):
        vals = list(inputs) + list(outputs)
        for pl, (_, ins, out) in zip(self.plans, self.steps):
            pl.launch([vals[i] for i in ins], [vals[out]])

    def describe(self):
        return " ; ".join(pl.describe() for pl in self.plans)


def _td_out(w):
    (N, C1, C2, H, W), (_, _, C3, _, _) = w.shapes
    return [(N, C1, C3, H, W)]


def _bmm_out(w):
    (B, N, M), (_, _, K) = w.shapes
    return [(B, N, K)]


def _tmm_out(w):
    (M, K), (N, _) = w.shapes
    return [(M, N)]


def _gc_out(w):
    (N, G, C, H, W), (_, F, _, KH, KW), _ = w.shapes
    return [(N, G, F, H - KH + 1, W - KW + 1)]


def _mlp_out(w):
    B = w.shapes[0][0]
    return [(B, w.shapes[1][0]), (B, w.shapes[3][0]), (B, w.shapes[5][0])]


OUT_SHAPES = {"tensordot": _td_out, "batchmatmul": _bmm_out, "tmm": _tmm_out, "group_conv": _gc_out,
              "mlp3": _mlp_out}


def compile_workload(w, dev):
    if w.name == "tensordot":
        (N, C1, C2, H, W), (_, _, C3, _, _) = w.shapes
        steps = [(cabi.tensordot_problem(N, C1, C2, C3, H * W), [0, 1], 2)]
    elif w.name == "batchmatmul":
        (B, N, M), (_, _, K) = w.shapes
        steps = [(cabi.contraction_problem(B, N, K, M, True, False), [0, 1], 2)]
    elif w.name == "tmm":
        (M, K), (N, _) = w.shapes
        steps = [(cabi.contraction_problem(1, M, N, K, True, True), [0, 1], 2)]
    elif w.name == "group_conv":
        (N, G, C, H, W), (_, F, _, KH, KW), _ = w.shapes
        steps = [(cabi.group_conv_problem(N, G, C, F, H, W, KH, KW), [0, 1, 2], 3)]
    elif w.name == "mlp3":
        B, n = w.shapes[0]
        o, p, q = w.shapes[1][0], w.shapes[3][0], w.shapes[5][0]
        e = cabi.EPI_BIAS_RELU
        steps = [(cabi.contraction_problem(1, B, o, n, True, True, epilogue=e), [0, 1, 2], 7),
                 (cabi.contraction_problem(1, B, p, o, True, True, epilogue=e), [7, 3, 4], 8),
                 (cabi.contraction_problem(1, B, q, p, True, True, epilogue=e), [8, 5, 6], 9)]
    else:
        raise ValueError(w.name)
    return _Exe(w, dev, steps)
