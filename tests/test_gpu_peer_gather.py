"""The fused all-gather of column-parallel FP8 linears (GEMM epilogue -> peer stores) on two GPUs, one process each:
every rank ends up with the full [world, M, N/world] product, bit-identical to what the Fp8Matmul op computes per shard
and what an NCCL all-gather of those shards assembles.  Needs at least two GPUs of one node; skipped otherwise."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    import importlib
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import load_package
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    load_package()
    fp8 = importlib.import_module("itex_b200.fp8")
    dev = torch.device("cuda", rank)
    m, k = 384, 512
    shards = [(k, 1024), (k, 768)]            # (K, N) per linear; N is split over the ranks
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)                        # activations replicated
    acts = [torch.randn((m, kk), generator=gen, device=dev).to(torch.bfloat16) for kk, _ in shards]
    wgen = torch.Generator(device=dev)
    wgen.manual_seed(100 + rank)              # every rank its own weight shard
    layers, refs = [], []
    for kk, n in shards:
        w = (torch.randn((n // world, kk), generator=wgen, device=dev) * 0.02).to(torch.bfloat16)
        mk = lambda: fp8.Fp8Dense(w, recipe=fp8.DelayedScaling(margin=0, amax_history_len=4), out_dtype="bfloat16", weight_layout="nk")
        layers.append(mk())
        refs.append(mk())

    def exchange(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    pg = fp8.PeerGather([(m, n // world) for _, n in shards], torch.bfloat16, rank, world, dev, exchange)
    ok = True
    for step in range(4):
        scale_up = 1.0 + step
        if step % 2 == 0:                     # the protocol spelled out, everything on one stream
            pg.begin()
            for i, (layer, a) in enumerate(zip(layers, acts)):
                layer(a * scale_up, gather=pg, gather_index=i)
                dist.all_reduce(layer.meta.amax_history[0], op=dist.ReduceOp.MAX)
            pg.publish()
            pg.finish()
            got = [pg.gathered(i).clone() for i in range(len(layers))]
        else:                                 # the same step through the helper, every linear on a stream of its own
            def reduce_amax(rows):
                for row in rows:
                    dist.all_reduce(row, op=dist.ReduceOp.MAX)
            got = [g.clone() for g in pg.linears(layers, [a * scale_up for a in acts], reduce_amax=reduce_amax, streams=True)]
        pg.acknowledge()
        # the reference path: the Fp8Matmul op per shard, shards assembled by NCCL
        for i, (layer, a) in enumerate(zip(refs, acts)):
            y = layer(a * scale_up)
            dist.all_reduce(layer.meta.amax_history[0], op=dist.ReduceOp.MAX)
            want = torch.empty((world,) + tuple(y.shape), dtype=y.dtype, device=dev)
            dist.all_gather_into_tensor(want, y)
            ok = ok and bool((got[i] == want).all()) and bool(torch.isfinite(want.float()).all())
    torch.cuda.synchronize()
    ok = ok and int(pg.status.item()) == 0
    results[rank] = ok
    pg.close(dist.barrier)
    dist.destroy_process_group()


def test_fused_peer_store_gather_equals_nccl_all_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs of one node")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()                     # the exact processes this test started
    assert not alive, "a rank did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: True, 1: True}
