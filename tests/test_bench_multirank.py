"""Multi-rank plumbing of bench.py on CPU ranks (gloo, world size 2): the whole-job reduction
(max of the times, sum of the work), the slices the ranks take of the fixed workload, and the
rule that only rank 0 of the reference arm works."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    import bench
    ms, fl = bench.reduce_over_ranks(10.0 + rank, 100.0 * (rank + 1), dist, "cpu")
    q.put((rank, ms, fl))
    dist.barrier()
    dist.destroy_process_group()


def test_reduce_over_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, 11.0, 300.0), (1, 11.0, 300.0)]     # slowest rank's time, work of both


def _shard_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    import bench
    from flashlight_b200.workloads import WORKLOADS, effective_flops, make_inputs, shard
    from oracle.run_config import run_oracle
    # the benchmark's default workload, shortened; every rank builds the same fixed inputs
    w = WORKLOADS["causal_gqa"].scaled(N=3 if world == 3 else 2, S=160)
    t = make_inputs(w, seed=0)
    ws, ts = shard(w, t, rank, world)
    mine = run_oracle(ws, ts)                                 # stands in for the kernel on this rank's GPU
    _, flops_all = bench.reduce_over_ranks(1.0, effective_flops(ws, ts), dist, "cpu")
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    if rank == 0:
        whole = run_oracle(w, t)
        q.put((torch.equal(torch.cat(parts, dim=0), whole), flops_all == effective_flops(w, t),
               [tuple(p.shape) for p in parts]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_take_disjoint_slices_that_cover_the_workload():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_shard_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    same, work_adds_up, shapes = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same and work_adds_up
    assert shapes == [(1, 8, 4, 160, 128)] * 2                # one sequence each, 5-D GQA result


def test_single_process_reduce_is_identity():
    sys.path.insert(0, str(ROOT))
    import bench
    assert bench.reduce_over_ranks(3.5, 7.0, None, "cpu") == (3.5, 7.0)


def test_reference_arm_under_torchrun_prints_one_line():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(ROOT / "bench.py"),
           "--impl", "reference", "--gpus", "2", "--workload", "vanilla", "--steps", "1", "--warmup", "1"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["scaling"] == "strong"
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["value"] > 0
