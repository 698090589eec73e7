"""The multi-process side of bench.py on CPU: two gloo ranks shard the batch, time is the max over
ranks, value is the whole-job aggregate; the reference arm prints one line from rank 0 only."""
import json
import os
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import bench
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ms = bench.max_over_ranks(10.0 + 5.0 * rank, world)          # rank 1 is the slow shard
    seeds = [None] * world
    dist.all_gather_object(seeds, bench.shard_seed(1234, rank))
    if rank == 0:
        out.put((ms, seeds, bench.whole_job_tops(8192, 8192, 8192, world, ms)))
    dist.destroy_process_group()


def test_two_gloo_ranks_take_max_time_and_sum_work():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    ms, seeds, tops = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ms == 15.0                                  # the slowest rank sets the step time
    assert seeds == [1234, 1235]                       # distinct shards
    assert abs(tops - 2 * 2.0 * 8192 ** 3 / 15e-3 / 1e12) < 1e-9   # both ranks' work over that time


def test_single_rank_needs_no_process_group():
    import bench
    assert bench.max_over_ranks(3.5, 1) == 3.5
    assert bench.whole_job_tops(2, 3, 4, 1, 1.0) == 2.0 * 24 / 1e-3 / 1e12


def test_reference_arm_runs_on_rank0_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "int8_gemm_4096",
                        "--steps", "1", "--warmup", "1"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == ""
    env["RANK"] = "0"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "int8_gemm_4096",
                        "--steps", "1", "--warmup", "1"], capture_output=True, text=True, env=env, timeout=300)
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TOPS" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0
