"""Host-side logic of the multi-GPU path on CPU: shard arithmetic, and a world_size-2 gloo run in
which each rank computes its shard (with the CPU checker standing in for the kernels) and the
gathered result must equal the unsharded one."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

from tensorcomprehensions_b200 import sharding
from tensorcomprehensions_b200 import workloads as wl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_cover_everything_once():
    for total in (500, 32, 16384, 7, 3):
        for world in (1, 2, 4, 8):
            spans = [sharding.shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    assert [sharding.shard_bounds(500, 8, r)[1] for r in range(8)] == [63, 63, 63, 63, 62, 62, 62, 62]


def test_shard_shapes_follow_the_workload_table():
    w = wl.tmm()
    assert sharding.shard_shapes(w.shapes, w.shard_inputs, 8, 3) == [(128, 4096), (2048, 4096)]
    w = wl.batchmatmul()
    assert sharding.shard_shapes(w.shapes, w.shard_inputs, 8, 7) == [(62, 26, 72), (62, 72, 26)]
    w = wl.mlp3()
    s = sharding.shard_shapes(w.shapes, w.shard_inputs, 8, 0)
    assert s[0] == (2048, 2048) and s[1:] == list(w.shapes[1:])


def _worker(rank, world, port, name, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = wl.ALL[name](**wl.SMALL[name])
        full = wl.make_inputs(w)

        def fake_compile(tc, entry, options, *ins):
            return lambda *xs: orc.ATEN[name](*xs)

        prog = sharding.ShardedProgram(w, world, rank, compile_fn=fake_compile)
        outs = prog.run(prog.shard_inputs(full))
        ref = orc.as_list(orc.ATEN[name](*full))
        extents = [r.shape[d] for r, d in zip(ref, w.shard_outputs)]
        gathered = prog.gather(outs, extents)
        ok = all(torch.allclose(g, r, rtol=1e-5, atol=1e-5) and g.shape == r.shape for g, r in zip(gathered, ref))
        q.put((rank, ok, [tuple(o.shape) for o in outs]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", ["batchmatmul", "tmm", "mlp3", "tensordot", "group_conv"])
def test_two_rank_gloo_shard_run_gather(name):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + hash(name)) % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, name, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results
    # the two shards differ in size when the extent is odd (batchmatmul small: 7 -> 4 + 3)
    if name == "batchmatmul":
        shapes = dict((r, s) for r, _, s in results)
        assert shapes[0][0][0] == 4 and shapes[1][0][0] == 3


def _failing_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        name = "tmm"
        w = wl.ALL[name](**wl.SMALL[name])
        full = wl.make_inputs(w)

        def compile_fn(tc, entry, options, *ins):
            if rank == 1:
                raise ValueError("this rank's kernels refuse the shard")   # the failure is made on the host
            return lambda *xs: orc.ATEN[name](*xs)

        prog = sharding.ShardedProgram(w, world, rank, compile_fn=compile_fn)
        try:
            prog.run_and_gather(prog.shard_inputs(full), [full[1].shape[0]])
            q.put((rank, "no error"))
        except sharding.RankFailure as e:
            q.put((rank, e.failed_ranks, "refuse the shard" in str(e)))
        # the group is still usable: a healthy exchange afterwards goes through on both ranks
        good = sharding.ShardedProgram(w, world, rank, compile_fn=lambda *a: (lambda *xs: orc.ATEN[name](*xs)))
        out = good.run_and_gather(good.shard_inputs(full), [full[1].shape[0]])[0]
        q.put((rank, "recovered", tuple(out.shape)))
    finally:
        dist.destroy_process_group()


def test_a_failing_rank_is_reported_on_every_rank_before_the_exchange():
    """One rank raises on the host while compiling its shard: both ranks get RankFailure naming it, nobody hangs
    in the all-gather, and the next exchange on the same group works."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 977) % 2000
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(4)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    first = sorted(r for r in results if r[1] != "recovered")
    assert first == [(0, [1], False), (1, [1], True)], results   # rank 1 also carries its own error text
    assert sorted(r for r in results if r[1] == "recovered") == [(0, "recovered", (70, 200)), (1, "recovered", (70, 200))]
