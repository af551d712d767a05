"""Python face of the backend: the subset of the reference's `tensor_comprehensions` package that
sits on the hot path (tensor_comprehensions/__init__.py:47-71,123-143,145-218,329-403):

    import tensorcomprehensions_b200 as tc
    T = tc.define(TC_TEXT, tc.make_naive_options_factory())
    out = T.tensordot(I0, I1)                       # compiles lazily per input shapes, then runs
    exe = tc.compile(TC_TEXT, "tensordot", "naive", I0, I1); out = exe(I0, I1)
    best = tc.autotune(TC_TEXT, "tensordot", I0, I1, starting_options="naive")
    tc.assert_almost_equal(out, expected, I0, I1, operations=8)

Everything runs through the C++ host (tclib -> tc::aten::compile / run / ATenAutotuner::tune) and
the sm_100a kernel library; there is no eager or CPU fallback: a comprehension that matches no
kernel family raises tclib.ErrorReport from compile.
"""
import time
from typing import Callable, Iterable, List, Optional, Tuple, Union

import torch

from . import tclib  # noqa: F401  (hard import: the native extension is the only path)
from .tclib import MappingOptions

SILENT = True


def assert_almost_equal(actual, expected, *inputs, operations: int = 1, precision: float = 1e-7):
    """max|actual - expected| <= operations * precision * max over inputs of max|input|
    (the reference's Python twin of checkRtol, tensor_comprehensions/__init__.py:47-71)."""
    diff = actual - expected
    max_value = 0.0
    for inp in inputs:
        max_value = max(float(inp.abs().max()), max_value)
    max_diff = float(diff.abs().max())
    assert max_diff <= operations * precision * max_value, (
        "error at relative precision: {}, #operations: {}, max_value: {}, max_diff: {}".format(
            precision, operations, max_value, max_diff))


def _as_options(o) -> MappingOptions:
    if isinstance(o, MappingOptions):
        return o
    if o is None:
        return MappingOptions("naive")
    return MappingOptions(o)


def _stream(inputs):
    for t in inputs:
        if t.is_cuda:
            return torch.cuda.current_stream(t.device).cuda_stream
    return None


class Executor(object):
    """Callable result of compiling one TC def for fixed input sizes."""

    def __init__(self, executor):
        self.executor = executor

    def __call__(self, *inputs, outputs: Optional[Tuple[torch.Tensor]] = None, unchecked: bool = False):
        inputs = list(inputs)
        if outputs is None:
            outs = self.executor.run(inputs, [], _stream(inputs))
        elif unchecked:
            outs = self.executor.unchecked_run(inputs, list(outputs), _stream(inputs))
        else:
            outs = self.executor.run(inputs, list(outputs), _stream(inputs))
        return outs[0] if len(outs) == 1 else tuple(outs)

    def run(self, inputs, outputs):
        """List in, list out, no allocation: the form the benchmark loop uses."""
        return self.executor.unchecked_run(list(inputs), list(outputs), _stream(inputs))

    def profile(self, *inputs, outputs=None):
        return self.executor.profile(list(inputs), list(outputs) if outputs is not None else [])

    @property
    def compiled_source(self):
        return self.executor.compiled_source

    def __getattr__(self, name):
        return getattr(self.executor, name)


class HostStagedExecutor(object):
    """Runs a compiled TC from HOST buffers: pinned inputs are copied in on one stream, the kernels
    run on a second, outputs are copied back on a third, with `depth` sets of device buffers so the
    copies of consecutive calls overlap each other and the compute (PCIe is full duplex).

        staged = tc.HostStagedExecutor(exe, depth=2)
        for batch in batches: staged.submit(batch.inputs, batch.outputs)   # pinned CPU tensors
        staged.synchronize()

    Every call still moves all of its inputs to the device and all of its outputs back."""

    def __init__(self, executor: Executor, device, depth: int = 2):
        self.exe, self.device, self.depth = executor, torch.device(device), depth
        self.out_shapes = executor.output_shapes()
        self.h2d, self.compute, self.d2h = (torch.cuda.Stream(self.device) for _ in range(3))
        self.dev_in = [None] * depth
        self.dev_out = [[torch.empty(s, dtype=torch.float32, device=self.device) for s in self.out_shapes]
                        for _ in range(depth)]
        self.ev_in = [torch.cuda.Event() for _ in range(depth)]
        self.ev_done = [torch.cuda.Event() for _ in range(depth)]
        self.ev_out = [torch.cuda.Event() for _ in range(depth)]
        self.calls = 0

    def submit(self, host_inputs, host_outputs):
        k, slot = self.calls, self.calls % self.depth
        self.calls += 1
        if self.dev_in[slot] is None:
            self.dev_in[slot] = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_inputs]
        with torch.cuda.stream(self.h2d):
            if k >= self.depth:
                self.h2d.wait_event(self.ev_done[slot])  # the kernels that read this input set are done
            for d, h in zip(self.dev_in[slot], host_inputs):
                d.copy_(h, non_blocking=True)
            self.ev_in[slot].record(self.h2d)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(self.ev_in[slot])
            if k >= self.depth:
                self.compute.wait_event(self.ev_out[slot])  # the previous results of this set were copied out
            self.exe.run(self.dev_in[slot], self.dev_out[slot])
            self.ev_done[slot].record(self.compute)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(self.ev_done[slot])
            for h, d in zip(host_outputs, self.dev_out[slot]):
                h.copy_(d, non_blocking=True)
            self.ev_out[slot].record(self.d2h)

    def join(self, stream=None):
        """Makes `stream` (default: the current one) wait for everything submitted so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.h2d, self.compute, self.d2h):
            ev = torch.cuda.Event()
            ev.record(s)
            stream.wait_event(ev)

    def synchronize(self):
        for s in (self.h2d, self.compute, self.d2h):
            s.synchronize()


def compile(tc: str, entry_point: str, mapping_options: Union[str, MappingOptions], *inputs) -> Executor:
    """Compiles `entry_point` of `tc` for the shapes of `inputs` (tensor_comprehensions/__init__.py:123-143)."""
    return Executor(tclib.compile(tc, entry_point, list(inputs), _as_options(mapping_options)))


class TunerConfig(object):
    """Knobs of the tile sweep.  The reference's generations / population / threads settings have no
    meaning for an exhaustive sweep and are accepted and ignored."""

    def __init__(self, profile_iterations: int = 10, **ignored):
        self.profile_iterations = profile_iterations

    def generations(self, n):
        return self

    def pop_size(self, n):
        return self

    def number_elites(self, n):
        return self

    def threads(self, n):
        return self


class MappingOptionsCache(object):
    """Tuned options on disk, keyed by (canonical TC, input and output sizes, backend): the reference's
    MappingOptionsCache (tensor_comprehensions/__init__.py:186-218, pybinds/tclib.cc:395-420).  The file is
    a serialized CudaOptionsCacheProto (tc/proto/compcache.proto), readable by the reference and the other
    way round."""

    def __init__(self, filename: str):
        self.filename = filename

    def load(self, tc: str, entry_point: str, inputs, count: int = 1) -> List[MappingOptions]:
        """Up to `count` options recorded for these sizes, fastest median runtime first."""
        return tclib.cache_load(self.filename, tc, entry_point, list(inputs), count)

    def store(self, tc: str, entry_point: str, inputs, options: MappingOptions, runtime_us: int = 0):
        """Merges one (options, runtime) record into the file (the reference only stores through its
        Tuner; this is the same merge for options that were obtained elsewhere)."""
        tclib.cache_store(self.filename, tc, entry_point, list(inputs), options, int(runtime_us))

    def __len__(self):
        return tclib.cache_size(self.filename)


def autotune(tc: str, entry_point: str, *inputs, starting_options=None, tuner_config: TunerConfig = None,
             cache_filename: Optional[str] = None, load_from_cache: bool = False,
             store_to_cache: bool = False) -> MappingOptions:
    """Times every candidate tile of the matched kernel families on the inputs' device and returns the
    fastest as a MappingOptions (tensor_comprehensions/__init__.py:145-218)."""
    inputs = list(inputs)
    if cache_filename is not None and load_from_cache:
        cached = MappingOptionsCache(cache_filename).load(tc, entry_point, inputs, 1)
        if cached:
            return cached[0]
    base = _as_options(starting_options)
    if tuner_config is not None:
        tclib.set_flag("tuner_profile_iterations", str(tuner_config.profile_iterations))
    if cache_filename is not None and store_to_cache:
        best = tclib.tune_to_cache(tc, entry_point, inputs, base, 1, cache_filename)
    else:
        best = tclib.tune(tc, entry_point, inputs, base, 1)
    return best[0] if best else base


def autotune_and_compile(tc: str, entry_point: str, *inputs, starting_options=None, tuner_config=None,
                         cache_filename=None, load_from_cache=False, store_to_cache=False) -> Executor:
    best = autotune(tc, entry_point, *inputs, starting_options=starting_options, tuner_config=tuner_config,
                    cache_filename=cache_filename, load_from_cache=load_from_cache, store_to_cache=store_to_cache)
    return compile(tc, entry_point, best, *inputs)


class Tuner(object):
    """tc.Tuner(tc_text, cache_file).tune(entry_point, inputs, base_options, config)."""

    def __init__(self, tc: str, cache_filename: Optional[str] = None):
        self.tc, self.cache_filename = tc, cache_filename

    def tune(self, entry_point: str, inputs, base_options: MappingOptions = None, config: TunerConfig = None):
        return autotune(self.tc, entry_point, *inputs, starting_options=base_options, tuner_config=config,
                        cache_filename=self.cache_filename, store_to_cache=self.cache_filename is not None)


def make_naive_options_factory() -> Callable:
    def generate(tc: str, entry_point: str, *inputs) -> MappingOptions:
        return MappingOptions("naive")
    return generate


def make_load_from_cache_options_factory(cache_filename: str) -> Callable:
    def generate(tc: str, entry_point: str, *inputs) -> MappingOptions:
        loaded = MappingOptionsCache(cache_filename).load(tc, entry_point, list(inputs), 1)
        return loaded[0] if loaded else None
    return generate


def make_autotuned_options_factory(starting_options=None, tuner_config=None, cache_filename=None,
                                   load_from_cache=False, store_to_cache=False) -> Callable:
    def generate(tc: str, entry_point: str, *inputs) -> MappingOptions:
        return autotune(tc, entry_point, *inputs, starting_options=starting_options, tuner_config=tuner_config,
                        cache_filename=cache_filename, load_from_cache=load_from_cache,
                        store_to_cache=store_to_cache)
    return generate


class TC(object):
    """Every def of the TC text is a method; calling it compiles lazily for the input sizes (through
    the options factory) and runs (tensor_comprehensions/__init__.py:329-403)."""

    def __init__(self, tc: str, mapping_options_factory: Callable):
        self.tc = tc
        self.mapping_options_factory = mapping_options_factory
        self._executors = {}
        import re
        for name in re.findall(r"\bdef\s+([A-Za-z_][A-Za-z0-9_]*)\s*\(", tc):
            setattr(self, name, self._make_closure(name))

    def _make_closure(self, name):
        def fun(*inputs, outputs=None, unchecked=False):
            return self(name, *inputs, outputs=outputs, unchecked=unchecked)
        return fun

    @staticmethod
    def _key(entry_point, inputs):
        return (entry_point,) + tuple((tuple(t.shape), tuple(t.stride()), t.dtype, str(t.device)) for t in inputs)

    def __call__(self, entry_point: str, *inputs, outputs=None, unchecked=False):
        key = self._key(entry_point, inputs)
        exe = self._executors.get(key)
        if exe is None:
            if not SILENT:
                print('TC "{}" was not explicitly compiled for inputs of sizes:\n  {}\n....Generate implicit '
                      'MappingOptions'.format(entry_point, " ".join(str(tuple(i.size())) for i in inputs)))
            options = self.mapping_options_factory(self.tc, entry_point, *inputs)
            assert options is not None, "No options found for TC {} with inputs of sizes:\n  {}\n".format(
                entry_point, " ".join(str(tuple(i.size())) for i in inputs))
            start = time.perf_counter()
            exe = compile(self.tc, entry_point, options, *inputs)
            self._executors[key] = exe
            if not SILENT:
                print('Done compiling TC "{}" (compile time: {}ms)'.format(
                    entry_point, int((time.perf_counter() - start) * 1e3)))
        return exe(*inputs, outputs=outputs, unchecked=unchecked)


def define(tc: str, mapping_options_factory: Callable) -> TC:
    return TC(tc, mapping_options_factory)


class _AutogradFunction(torch.autograd.Function):
    """Saves the inputs of the forward call; backward hands (inputs..., output gradients...) to the
    user's backward function and returns what it computes, one gradient per input."""

    @staticmethod
    def forward(ctx, forward_fun, backward_fun, *inputs):
        ctx.backward_fun = backward_fun
        ctx.save_for_backward(*inputs)
        return forward_fun(*inputs)

    @staticmethod
    def backward(ctx, *gradients):
        if ctx.backward_fun is None:
            return (None, None) + (None,) * len(ctx.saved_tensors)
        grads = ctx.backward_fun(*ctx.saved_tensors, *(g.contiguous() for g in gradients))
        if isinstance(grads, torch.Tensor):
            grads = (grads,)
        # no gradient for the two callables that travel as the first arguments
        return (None, None) + tuple(grads)


class Autograd(object):
    def __init__(self, forward_fun, backward_fun):
        self.forward_fun, self.backward_fun = forward_fun, backward_fun

    def __call__(self, *inputs):
        return _AutogradFunction.apply(self.forward_fun, self.backward_fun, *inputs)


def make_autograd(forward_fun: Callable, backward_fun: Callable) -> Autograd:
    """A callable with torch.autograd support from a forward and a backward function, both usually entry
    points of a tc.define()d object (tensor_comprehensions/__init__.py:513-601): the backward function
    receives the forward inputs followed by the gradients of the outputs and returns one gradient per
    input.  The backward comprehensions must themselves match a kernel family: the matmul gradients are
    contractions, and so are the convolution gradients of the reference's example for the 1 x 1 filters it uses
    (index differences over 1-wide ranges); convolution gradients of wider filters, which need `where` windows,
    are not matched and raise at first use."""
    return Autograd(forward_fun, backward_fun)


# Debug toggles of the reference's tclib (tensor_comprehensions/__init__.py:25-34).  The stages they
# print from (Halide, the polyhedral mapper, NVRTC, LLVM) do not exist in this backend: the calls are
# accepted and recorded so that scripts written for the reference run unchanged.
_debug_state = {}


def _toggle(name):
    def setter(value=True):
        _debug_state[name] = value
        return value
    setter.__name__ = name
    setter.__doc__ = "Accepted for source compatibility with the reference; nothing is printed by this backend."
    return setter


logtostderr, debug_lang, debug_halide, debug_tc_mapper, debug_tuner, dump_cuda, dump_ptx = (
    _toggle(n) for n in ("logtostderr", "debug_lang", "debug_halide", "debug_tc_mapper", "debug_tuner",
                         "dump_cuda", "dump_ptx"))
cuda_compiler, llvm_flags, nvcc_flags = (_toggle(n) for n in ("cuda_compiler", "llvm_flags", "nvcc_flags"))
