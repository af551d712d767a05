"""Data-parallel execution of one comprehension across the GPUs of a box.

Every benchmark comprehension shards along one OUTPUT index that also indexes its large operand
(tensordot/batchmatmul/group conv/MLP3: the batch index; transposed matmul: the rows of B, which
are the columns of C).  No reduction crosses GPUs, so computing needs no collective at all: each
rank compiles the comprehension for its shard shapes and runs it.  Only when the caller asks for
the full output is there an exchange step: an all-gather over NCCL (NVLink/NVSwitch) of equal-size
padded shards, trimmed and concatenated along the shard dimension.

One process per GPU (torch.distributed); the reference has no counterpart (it is single-device;
its autotuner alone uses several GPUs, tc/autotuner/autotuner-inl.h:279-295).
"""
import torch


def shard_bounds(total: int, world: int, rank: int):
    """Contiguous split with the remainder spread over the first ranks: 500 over 8 -> 63,63,63,63,62,...
    Returns (start, count); count may be 0 when world > total."""
    base, rem = divmod(total, world)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, count


def shard_tensor(t, dim, world, rank):
    if dim is None:
        return t
    start, count = shard_bounds(t.shape[dim], world, rank)
    return t.narrow(dim, start, count).contiguous()


def shard_shapes(shapes, shard_dims, world, rank):
    out = []
    for s, d in zip(shapes, shard_dims):
        s = list(s)
        if d is not None:
            s[d] = shard_bounds(s[d], world, rank)[1]
        out.append(tuple(s))
    return out


def _assemble(gathered, out, world, rows, total, inner):
    """[world][rows][max_count * inner] -> [rows][total * inner]: trims the padding of uneven shards and, for a
    shard dimension that is not the outermost one, interleaves the ranks' rows.  CUDA tensors go through the
    kernel library (tcb200_assemble_shards) on the current stream; CPU tensors (the gloo runs that test this
    module's host logic) are sliced with torch."""
    if gathered.is_cuda:
        import ctypes
        from . import cabi
        cabi.check(cabi.lib().tcb200_assemble_shards(
            ctypes.c_void_p(gathered.data_ptr()), ctypes.c_void_p(out.data_ptr()), world, rows, total, inner,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "tcb200_assemble_shards")
        return out
    g = gathered.view(world, rows, -1)
    o = out.view(rows, total * inner)
    for k in range(world):
        start, count = shard_bounds(total, world, k)
        o[:, start * inner:(start + count) * inner] = g[k, :, :count * inner]
    return out


class Gatherer:
    """All-gather of one sharded output, with its buffers allocated once.

    shard_shape: this rank's shard; dim: the sharded dimension; total: its unsharded extent.  gather(shard)
    returns the full tensor on every rank: the shard is padded to the largest shard (only when the extent
    does not divide), one all_gather_into_tensor of equal pieces (NCCL over NVLink on GPUs), then the pieces
    are assembled into the row-major full tensor.  An evenly divided dimension-0 shard is gathered straight
    into the result."""

    def __init__(self, shard_shape, dim, total, device, dtype=torch.float32, group=None):
        import torch.distributed as dist
        self.group, self.dim, self.total = group, dim, total
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        shape = list(shard_shape)
        self.count = shape[dim]
        assert self.count == shard_bounds(total, self.world, self.rank)[1], "shard does not match the split"
        self.max_count = max(shard_bounds(total, self.world, r)[1] for r in range(self.world))
        self.rows = 1
        for s in shape[:dim]:
            self.rows *= s
        self.inner = 1
        for s in shape[dim + 1:]:
            self.inner *= s
        full_shape = shape[:dim] + [total] + shape[dim + 1:]
        self.out = torch.empty(full_shape, dtype=dtype, device=device)
        self.direct = self.rows == 1 and self.max_count * self.world == total
        if not self.direct:
            self.recv = torch.empty((self.world, self.rows, self.max_count * self.inner), dtype=dtype, device=device)
            self.send = None
            if self.count < self.max_count:
                self.send = torch.zeros((self.rows, self.max_count * self.inner), dtype=dtype, device=device)

    def gather(self, shard):
        import torch.distributed as dist
        shard = shard.contiguous()
        if self.direct:
            dist.all_gather_into_tensor(self.out.view(-1), shard.view(-1), group=self.group)
            return self.out
        piece = shard.view(self.rows, self.count * self.inner)
        if self.send is not None:
            self.send[:, :self.count * self.inner].copy_(piece)
            piece = self.send
        dist.all_gather_into_tensor(self.recv.view(-1), piece.reshape(-1), group=self.group)
        return _assemble(self.recv, self.out, self.world, self.rows, self.total, self.inner)


def all_gather_shards(shard, dim, total, group=None):
    """One-off form of Gatherer: all-gather of (possibly unevenly sized) shards along `dim`."""
    return Gatherer(tuple(shard.shape), dim, total, shard.device, shard.dtype, group).gather(shard)


class RankFailure(RuntimeError):
    """Raised on EVERY rank when one or more ranks reported a failure before an exchange."""

    def __init__(self, failed, own_error=None):
        self.failed_ranks = failed
        msg = "rank(s) %s failed before the exchange" % ", ".join(str(r) for r in failed)
        if own_error is not None:
            msg += "; this rank's error: %r" % (own_error,)
        super().__init__(msg)


def agree_all_ranks_ok(ok, group=None, device=None, own_error=None):
    """Every rank says whether its part went well; if any did not, all ranks raise RankFailure naming them, instead
    of the healthy ranks walking into a collective that the failed one never joins.  One tiny all_gather; call it
    between steps, with no kernel's result pending on the answer (it synchronises the host with the flag copy)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device or "cpu")
    flags = torch.empty(world, dtype=torch.int32, device=flag.device)
    dist.all_gather_into_tensor(flags, flag, group=group)
    failed = [r for r, v in enumerate(flags.tolist()) if v == 0]
    if failed:
        raise RankFailure(failed, own_error)


class ShardedProgram:
    """This rank's shard of a workload: compiled for the shard shapes, run on the local GPU.

    compile_fn(tc, entry, options, *inputs) -> executor; executor(*inputs) -> output(s).  The default
    is the package's tc.compile (CUDA only)."""

    def __init__(self, w, world, rank, compile_fn=None, options="naive"):
        self.w, self.world, self.rank = w, world, rank
        self.compile_fn = compile_fn
        self.options = options
        self.exe = None
        self.totals = None

    def shard_inputs(self, full_inputs):
        return [shard_tensor(t, d, self.world, self.rank) for t, d in zip(full_inputs, self.w.shard_inputs)]

    def run(self, shard_inputs):
        if self.exe is None:
            fn = self.compile_fn
            if fn is None:
                from . import api
                fn = api.compile
            self.exe = fn(self.w.tc, self.w.entry, self.options, *shard_inputs)
        outs = self.exe(*shard_inputs)
        return list(outs) if isinstance(outs, (tuple, list)) else [outs]

    def run_and_gather(self, shard_inputs, full_extents, group=None):
        """run() then gather(), with a vote in between: a rank whose compile or launch raised (a shape its kernels
        refuse, a device status that is not clean) makes every rank raise RankFailure before any of them enters
        the all-gather."""
        error, outs = None, None
        try:
            outs = self.run(shard_inputs)
        except Exception as e:  # reported to the other ranks, then re-raised as RankFailure on all of them
            error = e
        device = shard_inputs[0].device if shard_inputs[0].is_cuda else None
        agree_all_ranks_ok(error is None, group, device, error)
        return self.gather(outs, full_extents, group)

    def gather(self, shard_outputs, full_extents, group=None):
        """full_extents[i]: size of output i along its shard dimension before sharding.  The buffers of the
        exchange are allocated at the first call and reused."""
        if getattr(self, "_gatherers", None) is None:
            self._gatherers = [Gatherer(tuple(o.shape), d, n, o.device, o.dtype, group)
                               for o, d, n in zip(shard_outputs, self.w.shard_outputs, full_extents)]
        return [g.gather(o) for g, o in zip(self._gatherers, shard_outputs)]
