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


def all_gather_shards(shard, dim, total, group=None):
    """All-gather of unevenly sized shards: every rank pads its shard to the largest count along
    `dim`, one all_gather of equal buffers, then the padding is trimmed while concatenating."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    max_count = max(shard_bounds(total, world, r)[1] for r in range(world))
    moved = shard.movedim(dim, 0).contiguous()
    if moved.shape[0] < max_count:
        pad = torch.zeros((max_count - moved.shape[0],) + tuple(moved.shape[1:]), dtype=moved.dtype,
                          device=moved.device)
        moved = torch.cat([moved, pad], 0)
    gathered = [torch.empty_like(moved) for _ in range(world)]
    dist.all_gather(gathered, moved, group=group)
    parts = [g[:shard_bounds(total, world, r)[1]] for r, g in enumerate(gathered)]
    return torch.cat(parts, 0).movedim(0, dim).contiguous()


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

    def gather(self, shard_outputs, full_extents, group=None):
        """full_extents[i]: size of output i along its shard dimension before sharding."""
        return [all_gather_shards(o, d, n, group) for o, d, n in
                zip(shard_outputs, self.w.shard_outputs, full_extents)]
