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
