"""Every rank's shard of every configuration, at full size, on one GPU: the shapes a rank of a 2-, 4- or
8-GPU run compiles and launches (other tile choices than the unsharded problem: 2048-row MLP shards, 62-matrix
batches, 4-image convolutions) run through the real kernels, and the outputs, concatenated along the shard
dimension, must equal the unsharded result of ATen."""
import pytest
import torch

from oracle import oracle as orc
from tensorcomprehensions_b200 import sharding
from tensorcomprehensions_b200 import workloads as wl

from helpers import STRICT, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("name", list(wl.ALL))
def test_all_ranks_of_a_sharded_run(cuda, name, world):
    w = wl.ALL[name]()
    full = wl.make_inputs(w)
    refs = orc.as_list(orc.ATEN[name](*full))
    pieces = [[] for _ in refs]
    for rank in range(world):
        prog = sharding.ShardedProgram(w, world, rank)
        shard = [t.to(cuda) for t in prog.shard_inputs(full)]
        outs = prog.run(shard)
        assert len(outs) == len(refs)
        for k, o in enumerate(outs):
            pieces[k].append(o.cpu())
    for k, (ref, dim, L) in enumerate(zip(refs, w.shard_outputs, w.reduction)):
        whole = torch.cat(pieces[k], dim=dim)
        assert_close(whole, ref, L, full, STRICT[name], "%s world=%d output %d" % (name, world, k))


@pytest.mark.parametrize("shape,dim,world", [((500, 26, 26), 0, 8), ((128, 16384), 1, 8), ((128, 2050), 1, 4),
                                             ((7, 3, 5), 0, 2), ((3, 10, 6), 1, 4), ((32, 32, 16, 14, 14), 0, 8)])
def test_assembly_kernel_rebuilds_the_unsharded_tensor(cuda, shape, dim, world):
    """What the all-gather leaves ([rank][rows][padded shard]) -> the row-major full tensor, on one GPU."""
    full = torch.randn(shape, device=cuda)
    total = shape[dim]
    max_count = max(sharding.shard_bounds(total, world, r)[1] for r in range(world))
    rows = 1
    for s in shape[:dim]:
        rows *= s
    inner = 1
    for s in shape[dim + 1:]:
        inner *= s
    gathered = torch.full((world, rows, max_count * inner), float("nan"), device=cuda)
    for r in range(world):
        start, count = sharding.shard_bounds(total, world, r)
        gathered[r, :, :count * inner] = full.narrow(dim, start, count).reshape(rows, count * inner)
    out = torch.full(shape, float("nan"), device=cuda)
    sharding._assemble(gathered, out, world, rows, total, inner)
    torch.cuda.synchronize()
    assert torch.equal(out, full)
    # an output view at a 4-byte offset takes the scalar path
    buf = torch.full((full.numel() + 1,), float("nan"), device=cuda)
    out2 = buf[1:].view(shape)
    sharding._assemble(gathered, out2, world, rows, total, inner)
    torch.cuda.synchronize()
    assert torch.equal(out2, full)
