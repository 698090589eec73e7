"""The multi-process side of bench.py on CPU: two gloo ranks shard the batch, time is the max over
ranks, value is the whole-job aggregate; the reference arm prints one line from rank 0 only."""
import json
import os
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import pytest

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


def _layout_worker(rank, world, port, out):
    """Two gloo ranks build the fused all-gather's block layout independently and exchange what they would hand to
    their GEMMs: every (rank -> peer) store target must be the peer's own address of the same slot, slots must not
    overlap each other or the flags, and the flag a rank signals in a peer's block must be the one that peer polls."""
    import importlib
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import load_package
    load_package()
    fp8 = importlib.import_module("itex_b200.fp8")
    shard_bytes = [4096 * (4096 // world) * 2, 4096 * (14336 // world) * 2]
    lay = fp8.peer_gather_layout(world, shard_bytes)
    base = 0x7F0000000000 + rank * (1 << 32)          # pretend device address of this rank's block
    mine = {"base": base, "layout": lay,
            "stores": {(i, peer): fp8.peer_slot_offset(lay, shard_bytes, i, rank) for i in range(2) for peer in range(world) if peer != rank},
            "signals": lay["data_flags"] + 4 * rank}
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    ok = all(e["layout"] == lay for e in everyone)
    spans = []
    for i in range(2):
        for src in range(world):
            off = fp8.peer_slot_offset(lay, shard_bytes, i, src)
            spans.append((off, off + shard_bytes[i]))
    spans.sort()
    ok = ok and all(a[1] <= b[0] for a, b in zip(spans, spans[1:])) and spans[-1][1] <= lay["data_flags"] and spans[0][0] == 0
    ok = ok and lay["data_flags"] + 4 * world <= lay["ack_flags"] and lay["ack_flags"] + 4 * world <= lay["counter"] < lay["status"] < lay["total"]
    # what rank s stores for linear i lands in slot s of the receiver: the receiver reads gathered[i][s] at that same offset
    for e_rank, e in enumerate(everyone):
        for (i, peer), off in e["stores"].items():
            ok = ok and off == lay["linear"][i] + shard_bytes[i] * e_rank
        ok = ok and e["signals"] == lay["data_flags"] + 4 * e_rank
    out[rank] = ok
    dist.destroy_process_group()


def test_peer_gather_layout_agrees_between_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = 29600 + os.getpid() % 2000
    procs = [ctx.Process(target=_layout_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs)
    assert dict(out) == {0: True, 1: True}
    import importlib
    from conftest import load_package
    load_package()
    fp8 = importlib.import_module("itex_b200.fp8")
    with pytest.raises(ValueError):
        fp8.peer_gather_layout(2, [100])
