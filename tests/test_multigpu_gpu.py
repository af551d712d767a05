"""The sharded run on real GPUs with the exchange on NCCL: one process per GPU, every rank compiles and runs
its shard of each benchmark comprehension at full size, the outputs are all-gathered over NCCL (padded to
the largest shard where the split is uneven: 500 matrices over 2 GPUs is even, so a 501-matrix case is run
too; the transposed matmul gathers along the columns of C and goes through the assembly kernel) and every
rank's gathered result must equal the unsharded ATen result.  Needs at least two GPUs: skipped below that."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu

CASES = [("tensordot", {}), ("batchmatmul", {}), ("batchmatmul", dict(B=501)), ("tmm", {}),
         ("tmm", dict(M=128, N=2050, K=512)), ("group_conv", {}), ("group_conv", dict(N=7, G=4)), ("mlp3", {})]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from oracle import oracle as orc
    from tensorcomprehensions_b200 import sharding
    from tensorcomprehensions_b200 import workloads as wl
    from helpers import STRICT, assert_close
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    failures = []
    try:
        for name, kw in CASES:
            w = wl.ALL[name](**kw)
            full = wl.make_inputs(w)  # the same seeded draws on every rank
            prog = sharding.ShardedProgram(w, world, rank)
            shard = [t.to(dev) for t in prog.shard_inputs(full)]
            outs = prog.run(shard)
            refs = orc.as_list(orc.ATEN[name](*full))
            extents = [r.shape[d] for r, d in zip(refs, w.shard_outputs)]
            for _ in range(2):  # the second call reuses the exchange buffers
                gathered = prog.gather(outs, extents)
            torch.cuda.synchronize()
            try:
                for k, (g, r, L) in enumerate(zip(gathered, refs, w.reduction)):
                    assert g.device == dev and tuple(g.shape) == tuple(r.shape)
                    assert_close(g, r, L, full, STRICT[name], "%s %s rank %d output %d" % (name, kw, rank, k))
            except AssertionError as e:
                failures.append(str(e))
        q.put((rank, failures))
    finally:
        dist.destroy_process_group()


def test_nccl_gathered_outputs_match_aten():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, failures in results:
        assert not failures, "rank %d: %s" % (rank, failures)
