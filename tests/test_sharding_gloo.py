"""Host-side logic of the one-process-per-GPU mesh, run as two gloo ranks on CPU:
shard bounds, byte exchange (the path the NCCL id and the mailbox handles take),
max-over-ranks, and that local reduce + all-reduce equals the unsharded oracle."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    import __graft_entry__ as entry
    rx = entry.load_package()
    ref, cpu = entry.load_oracle()
    import torch, torch.distributed as td

    world = int(os.environ["WORLD_SIZE"])
    d = rx.dist.Dist(world, backend="gloo")
    assert d.world == 2 and d.rank in (0, 1)

    # byte exchange: rank 0's blob reaches everyone; the gathered table is in rank order
    blob = d.broadcast_bytes(bytes(range(128)) if d.rank == 0 else None)
    assert blob == bytes(range(128))
    table = d.all_gather_bytes(bytes([d.rank]) * 64)
    assert table == [bytes([0]) * 64, bytes([1]) * 64]

    # max over ranks is what the benchmark reports as its time
    assert d.reduce(10.0 + d.rank, "max") == 11.0 and d.reduce(1.0, "sum") == 2.0

    # sharded sinsum: chunk i of the global vector lives on rank i
    n = 1 << 16
    rng = np.random.default_rng(7)
    x = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
    y = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
    lo, hi = rx.dist.shard_bounds(n, world, d.rank)
    assert (lo, hi) == (d.rank * n // 2, (d.rank + 1) * n // 2)
    local = torch.tensor([cpu.sinsum_add(x[lo:hi], y[lo:hi])], dtype=torch.float32)
    td.all_reduce(local)
    want = float(ref.run_module(rx.programs.sinsum_add(n, num_partitions=world), [x, y])[0])
    terms = np.sin(x.astype(np.float64)) + y
    assert abs(float(local) - want) <= ref.reduction_tolerance(n) * np.linalg.norm(terms)

    # the planner splits the same module the same way
    plan = rx.plan_describe(rx.programs.sinsum_add(n, num_partitions=world))
    assert [s["kind"] for s in plan["steps"]] == ["reduce_full", "all_reduce"] and plan["steps"][0]["dims"] == [hi - lo]
    try:
        rx.dist.shard_bounds(7, 2, 0)
        raise SystemExit("indivisible shard accepted")
    except ValueError:
        pass
    d.close()
    print("rank", d.rank, "ok")
""")


def test_two_rank_host_logic_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29611", WORLD_SIZE="2")
    procs = []
    for rank in range(2):
        e = dict(env, RANK=str(rank), LOCAL_RANK=str(rank))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for rank, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{o}"
        assert f"rank {rank} ok" in o
