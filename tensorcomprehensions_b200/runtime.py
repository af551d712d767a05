"""Glue used by the benchmark: compile one benchmark comprehension through the public API
(tc.compile -> tc::aten::compile<CudaBackend>) for a device, optionally with autotuned tiles."""
import torch

from . import api


class CompiledWorkload:
    def __init__(self, w, dev, tune=False):
        self.w, self.dev = w, dev
        # shape-only compile: inputs on the target device decide where the plans live
        probe = [torch.empty(s, dtype=torch.float32, device=dev) for s in w.shapes]
        options = api.autotune(w.tc, w.entry, *probe, starting_options="naive") if tune else "naive"
        self.options = options
        self.exe = api.compile(w.tc, w.entry, options, *probe)
        # kernels per run: one per matched launch, plus the second pass of a launch whose tile splits its reduction
        self.launches = self.exe.num_launches + sum(1 for t in self.exe.tiles() if t[7] > 1)
        self.split_tf32 = min(3, max(t[6] for t in self.exe.tiles()))  # 4 = 3xTF32 with strict accumulation
        self.out_shapes = self.exe.output_shapes()

    def prepare_outputs(self):
        return [torch.empty(s, dtype=torch.float32, device=self.dev) for s in self.out_shapes]

    def run(self, inputs, outputs):
        self.exe.run(inputs, outputs)

    def host_staged(self, depth=2):
        return api.HostStagedExecutor(self.exe, self.dev, depth)

    def describe(self):
        return " ; ".join(l for l in self.exe.compiled_source.strip().split("\n") if not l.startswith("//"))


def compile_workload(w, dev, tune=False):
    return CompiledWorkload(w, dev, tune)
