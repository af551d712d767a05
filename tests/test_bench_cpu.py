"""bench.py's CPU arm: it honours --steps / --warmup exactly, prints the product arm's `config`, and uses the host
threads the process may use whatever OMP_NUM_THREADS a launcher exported (torchrun sets it to 1)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_line_matches_the_product_arms_contract():
    sys.path.insert(0, ROOT)
    import argparse
    import bench
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "2", "--warmup", "3", "--workload", "batchmatmul"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, "stdout carries the one JSON line"
    d = json.loads(lines[0])
    args = argparse.Namespace(workload="batchmatmul", tune=False)
    assert d["impl"] == "reference" and d["steps"] == 2 and d["warmup"] == 3 and d["n_gpus"] == 2
    assert d["config"] == bench.make_config(args)
    assert d["metric"] == bench.METRIC and d["unit"] == bench.UNIT and d["scaling"] == "strong"
    assert d["cpu_baseline"]["cores"] == bench.host_threads() and d["cpu_baseline"]["kind"] == "port"
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]
    # the other ranks of a torchrun launch print nothing and exit 0
    env["RANK"] = "1"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "2", "--warmup", "3", "--workload", "batchmatmul"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_shards_of_every_workload_add_up():
    sys.path.insert(0, ROOT)
    from tensorcomprehensions_b200 import workloads as wl
    for name in wl.ALL:
        full = wl.ALL[name]()
        for world in (1, 2, 4, 8):
            shards = [wl.shard_of(name, world, r) for r in range(world)]
            assert sum(s.flops for s in shards) == full.flops, (name, world)
            w, ins = wl.make_shard_inputs(name, world, world - 1)
            assert [tuple(t.shape) for t in ins] == [tuple(s) for s in w.shapes]
