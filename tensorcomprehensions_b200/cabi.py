"""ctypes view of the tcb200 C ABI (include/tcb200.h).

This is the binding a maintainer of the reference would write to reach the kernel
library from Python; the package's own C++ host (libtc_core) calls the same symbols
directly.  The library must be present: there is no CPU or eager fallback, a missing
or unloadable libtcb200.so is a hard error.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libtcb200.so")

FAMILY_CONTRACTION, FAMILY_TENSORDOT, FAMILY_GROUP_CONV, FAMILY_REDUCTION, FAMILY_COPY = 1, 2, 3, 4, 5
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_RELU = 0, 1, 2, 3
VARIANT_AUTO, VARIANT_SIMT, VARIANT_SIMT_SMALL, VARIANT_TCGEN05, VARIANT_TCGEN05_TS, VARIANT_TCGEN05_PAIR = 0, 1, 2, 3, 4, 5
OK = 0

# every symbol include/tcb200.h declares
SYMBOLS = [
    "tcb200_abi_version", "tcb200_strerror", "tcb200_last_cuda_error", "tcb200_device_count",
    "tcb200_query", "tcb200_plan_create", "tcb200_plan_destroy", "tcb200_plan_geometry",
    "tcb200_plan_describe", "tcb200_plan_tile", "tcb200_launch", "tcb200_l2_flush",
    "tcb200_get_device", "tcb200_set_device", "tcb200_device_name", "tcb200_stream_synchronize",
    "tcb200_timer_start", "tcb200_timer_stop", "tcb200_reduce_launch_static", "tcb200_assemble_shards",
    "tcb200_status_create", "tcb200_status_destroy", "tcb200_status_check", "tcb200_selftest_wait",
    "tcb200_replay_begin", "tcb200_replay_end",
]


class Problem(ctypes.Structure):
    _fields_ = [
        ("family", ctypes.c_int32), ("epilogue", ctypes.c_int32), ("accumulate", ctypes.c_int32),
        ("a_k_major", ctypes.c_int32), ("b_k_major", ctypes.c_int32), ("bias_on_m", ctypes.c_int32),
        ("batch", ctypes.c_int64), ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
        ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64), ("stride_c", ctypes.c_int64),
        ("conv", ctypes.c_int64 * 8), ("td", ctypes.c_int64 * 5), ("conv_stride", ctypes.c_int64 * 2), ("red", ctypes.c_int64 * 3),
        ("reduce_op", ctypes.c_int32), ("batch_reduce", ctypes.c_int32),
    ]


class Tile(ctypes.Structure):
    _fields_ = [("variant", ctypes.c_int32), ("bm", ctypes.c_int32), ("bn", ctypes.c_int32),
                ("bk", ctypes.c_int32), ("stages", ctypes.c_int32), ("threads", ctypes.c_int32),
                ("split_tf32", ctypes.c_int32), ("split_k", ctypes.c_int32)]

    def as_tuple(self):
        return (self.variant, self.bm, self.bn, self.bk, self.stages, self.threads, self.split_tf32, self.split_k)

    def __repr__(self):
        return ("Tile(variant=%d, bm=%d, bn=%d, bk=%d, stages=%d, threads=%d, split_tf32=%d, split_k=%d)"
                % self.as_tuple())


class Tcb200Error(RuntimeError):
    def __init__(self, status, what):
        super().__init__("tcb200: %s failed with status %d (%s)" % (what, status, strerror(status)))
        self.status = status


_lib = None


def lib():
    """Loads libtcb200.so (once).  Raises if it is missing: the CUDA path is the only path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "%s is missing: build it with `python -m tensorcomprehensions_b200._build` "
                "(there is no fallback path)" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        L.tcb200_strerror.restype = ctypes.c_char_p
        L.tcb200_strerror.argtypes = [ctypes.c_int]
        L.tcb200_device_count.argtypes = [ctypes.POINTER(ctypes.c_int)]
        L.tcb200_query.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Tile), ctypes.c_int,
                                   ctypes.POINTER(ctypes.c_int)]
        L.tcb200_plan_create.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Tile), ctypes.c_int,
                                         ctypes.POINTER(ctypes.c_void_p)]
        L.tcb200_plan_destroy.argtypes = [ctypes.c_void_p]
        L.tcb200_plan_geometry.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64 * 3),
                                           ctypes.POINTER(ctypes.c_int64 * 3)]
        L.tcb200_plan_describe.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
        L.tcb200_plan_tile.argtypes = [ctypes.c_void_p, ctypes.POINTER(Tile)]
        L.tcb200_launch.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                    ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p,
                                    ctypes.c_void_p]
        L.tcb200_l2_flush.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        L.tcb200_status_create.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        L.tcb200_status_destroy.argtypes = [ctypes.c_void_p]
        L.tcb200_status_check.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
        L.tcb200_selftest_wait.argtypes = [ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
        L.tcb200_replay_begin.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p)]
        L.tcb200_replay_end.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
        L.tcb200_reduce_launch_static.argtypes = [ctypes.c_void_p] * 4
        L.tcb200_assemble_shards.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                             ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
        _lib = L
    return _lib


def strerror(status):
    return lib().tcb200_strerror(status).decode()


def check(status, what):
    if status != OK:
        raise Tcb200Error(status, what)


def tensordot_problem(N, C1, C2, C3, P):
    p = Problem()
    p.family = FAMILY_TENSORDOT
    p.td[:] = [N, C1, C2, C3, P]
    return p


def contraction_problem(batch, M, N, K, a_k_major=True, b_k_major=True, epilogue=EPI_NONE,
                        accumulate=False, lda=None, ldb=None, ldc=None, stride_a=None,
                        stride_b=None, stride_c=None, bias_on_m=False, batch_reduce=False):
    p = Problem()
    p.family = FAMILY_CONTRACTION
    p.epilogue, p.accumulate = epilogue, int(accumulate)
    p.a_k_major, p.b_k_major, p.bias_on_m = int(a_k_major), int(b_k_major), int(bias_on_m)
    p.batch, p.M, p.N, p.K = batch, M, N, K
    p.lda = lda if lda is not None else (K if a_k_major else M)
    p.ldb = ldb if ldb is not None else (K if b_k_major else N)
    p.ldc = ldc if ldc is not None else N
    p.stride_a = stride_a if stride_a is not None else M * K
    p.stride_b = stride_b if stride_b is not None else N * K
    p.stride_c = stride_c if stride_c is not None else M * N
    p.batch_reduce = int(batch_reduce)
    return p


def group_conv_problem(N, G, C, F, H, W, KH, KW, epilogue=EPI_BIAS, accumulate=False, stride=(1, 1)):
    p = Problem()
    p.family = FAMILY_GROUP_CONV
    p.epilogue, p.accumulate = epilogue, int(accumulate)
    p.conv[:] = [N, G, C, F, H, W, KH, KW]
    p.conv_stride[:] = list(stride)
    return p


REDUCE_SUM, REDUCE_MAX, REDUCE_MIN, REDUCE_PROD = 0, 1, 2, 3


def reduction_problem(A, C, B, accumulate=False, op=REDUCE_SUM):
    """O(a, b) = reduce_c I(a, c, b) over the [A][C][B] view of one input (sum, max, min or product);
    accumulate: the output's old value takes part in the reduction (+=, max=, ... without '!')."""
    p = Problem()
    p.family = FAMILY_REDUCTION
    p.epilogue, p.accumulate = EPI_NONE, int(accumulate)
    p.red[:] = [A, C, B]
    p.reduce_op = op
    return p


def query(problem, max_tiles=32):
    tiles = (Tile * max_tiles)()
    n = ctypes.c_int(0)
    check(lib().tcb200_query(ctypes.byref(problem), tiles, max_tiles, ctypes.byref(n)), "tcb200_query")
    out = []
    for i in range(min(n.value, max_tiles)):
        t = Tile()
        ctypes.pointer(t)[0] = tiles[i]
        out.append(t)
    return out


class Plan:
    """Owns one tcb200_plan_t."""

    def __init__(self, problem, tile=None, device=0):
        self._h = ctypes.c_void_p()
        self.problem = problem
        tp = ctypes.byref(tile) if tile is not None else None
        check(lib().tcb200_plan_create(ctypes.byref(problem), tp, device, ctypes.byref(self._h)),
              "tcb200_plan_create")
        self.device = device

    def close(self):
        if self._h and _lib is not None:
            _lib.tcb200_plan_destroy(self._h)
        self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown: module globals may already be gone
            pass

    def geometry(self):
        g, b = (ctypes.c_int64 * 3)(), (ctypes.c_int64 * 3)()
        check(lib().tcb200_plan_geometry(self._h, ctypes.byref(g), ctypes.byref(b)), "tcb200_plan_geometry")
        return tuple(g), tuple(b)

    def describe(self):
        buf = ctypes.create_string_buffer(512)
        check(lib().tcb200_plan_describe(self._h, buf, 512), "tcb200_plan_describe")
        return buf.value.decode()

    def tile(self):
        t = Tile()
        check(lib().tcb200_plan_tile(self._h, ctypes.byref(t)), "tcb200_plan_tile")
        return t

    def launch_ptrs(self, in_ptrs, out_ptrs, stream=0, dev_status=0):
        ins = (ctypes.c_void_p * len(in_ptrs))(*in_ptrs)
        outs = (ctypes.c_void_p * len(out_ptrs))(*out_ptrs)
        check(lib().tcb200_launch(self._h, ins, len(in_ptrs), outs, len(out_ptrs),
                                  ctypes.c_void_p(stream), ctypes.c_void_p(dev_status)), "tcb200_launch")

    def launch_static(self, input, output, stream=None):
        """Reduction plans only: the launch with the library's fixed scratch array (no allocation; calls
        share the array, so calls that can overlap in time race)."""
        import torch
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        check(lib().tcb200_reduce_launch_static(self._h, ctypes.c_void_p(input.data_ptr()),
                                                ctypes.c_void_p(output.data_ptr()), ctypes.c_void_p(stream)),
              "tcb200_reduce_launch_static")

    def launch(self, inputs, outputs, stream=None, dev_status=None):
        """inputs/outputs: CUDA torch tensors (float32, contiguous).  Enqueues on torch's current stream."""
        import torch
        for t in list(inputs) + list(outputs):
            if not (t.is_cuda and t.dtype == torch.float32):
                raise ValueError("tcb200 kernels take float32 CUDA tensors")
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        self.launch_ptrs([t.data_ptr() for t in inputs], [t.data_ptr() for t in outputs], stream,
                         dev_status.data_ptr() if dev_status is not None else 0)


def l2_flush(buf, stream=None):
    import torch
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    check(lib().tcb200_l2_flush(ctypes.c_void_p(buf.data_ptr()), buf.numel() * buf.element_size(),
                                ctypes.c_void_p(stream)), "tcb200_l2_flush")
