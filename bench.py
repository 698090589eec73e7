"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0).  A step is one pass of the hot path over one batch of
synthetic input: _ITEXQuantizeV2 (fp32 -> quint8, SCALED, HALF_TO_EVEN) followed by
_ITEXQuantizedMatMulWithBiasAndDequantize (u8 x s8 -> fp32, bias and dequantize fused),
both called through the C-ABI op layer of libitexb200.so.  The metric is int8 GEMM
throughput: 2*M*N*K operations per step over the time of the whole step.

Multi-GPU (launched by torch.distributed.run): the batch (rows of the activation matrix)
is sharded, weights are replicated, there is no data-path collective; per-GPU work is
fixed, so scaling is weak and `value` is the sum over ranks.

--impl reference times the CPU path the reference would run (oneDNN int8 inner product,
reached through torch.ops.onednn, plus the oracle's quantize) on the host cores, on a
bounded row sample of the same workload.
"""
import argparse
import ctypes
import importlib
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))

# DRAM bytes (read + write) of one GemmKernel launch, from the ncu captures whose summaries are
# kept under profiles/; null for shapes that were not captured.
GEMM_DRAM_TRAFFIC = {"int8_gemm_8192": 498.8e6, "int8_gemm_4096": 55.4e6}

WORKLOADS = {
    # name: (M per GPU, N, K)
    "int8_gemm_8192": (8192, 8192, 8192),
    "int8_gemm_4096": (4096, 4096, 4096),
    "bert_ffn1": (12288, 4096, 1024),
}


def load_package():
    if "itex_b200" in sys.modules:
        return sys.modules["itex_b200"]
    pkg_dir = os.path.join(ROOT, "intel-extension-for-tensorflow_b200")
    spec = importlib.util.spec_from_file_location("itex_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["itex_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([s.strip() for s in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.1)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": float(self.samples[0][1]), "reasons": reasons,
                "samples": len(self.samples)}


def shard_seed(base_seed, rank):
    """Every rank owns its own batch shard (rows of the activation matrix): same distribution, its own seed."""
    return base_seed + rank


def max_over_ranks(ms, world, device=None):
    """Slowest rank's time in ms (all-reduce MAX); the job is as fast as its slowest shard."""
    if world <= 1:
        return float(ms)
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def pipelined_e2e(steps, dev, h2d, compute, d2h, barrier):
    """End-to-end steps the way a serving loop overlaps them: the host->device copy of step i+1, the compute of
    step i and the device->host copy of step i-1 run on three streams over two buffer slots (PCIe is full duplex).
    h2d(slot), compute(slot), d2h(slot) enqueue on the current stream.  Every step's copies are inside the timed
    region; returns milliseconds for all steps."""
    import torch
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record(main)
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    for i in range(steps):
        b = i & 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_done[b])      # the compute that read this input slot two steps ago has finished
            h2d(b)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        if i >= 2:
            main.wait_event(ev_out[b])           # the copy-out that read this output slot two steps ago has finished
        compute(b)
        ev_done[b].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            d2h(b)
            ev_out[b].record(s_out)
    main.wait_stream(s_in)
    main.wait_stream(s_out)
    t1.record(main)
    barrier()
    return t0.elapsed_time(t1)


def whole_job_tops(m, n, k, world, ms_step):
    """Weak scaling: every rank does 2*m*n*k operations per step; value is the sum over ranks per unit time."""
    return 2.0 * m * n * k * world / (ms_step * 1e-3) / 1e12


def synth_weights(n, k, seed):
    """int8 weights [K,N] from N(0, 0.02), symmetric per-tensor (the named op honours one weight range)."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02))
    amax = float(np.abs(w).max())
    q = np.clip(np.rint(w * (127.0 / amax)), -127, 127).astype(np.int8)
    bias = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.1))
    return q, -amax, amax, bias


def cpu_reference_step(x_rows, qw_kn, wmin, wmax, bias, state):
    """One CPU step on a row sample: quantize + int8 matmul + bias + dequantize.
    Returns (fp32 output, label of what ran)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import itex_oracle as o
    import oracle_c as oc
    import torch
    mn, mx = float(x_rows.min()), float(x_rows.max())
    amin, amax = o.adjust_input_min_max(mn, mx)
    scale, absr = o.scaled_scale(amin, amax, "quint8", True)
    qa = oc.quantize_scaled(x_rows, scale, False)
    out_scale = o.matmul_output_scale(0.0, absr, wmin, wmax, "float")
    if "bias_s" not in state:
        state["bias_s"] = o.matmul_scaled_bias(bias, qw_kn[:1], 0.0, absr, wmin, wmax, "SCALED", "float", out_scale)
        state["w_nk"] = np.ascontiguousarray(qw_kn.T)
        try:
            state["pw"] = torch.ops.onednn.qlinear_prepack(torch.from_numpy(state["w_nk"]), None)
            state["ws"] = torch.full((qw_kn.shape[1],), float(out_scale))
            state["wz"] = torch.zeros(qw_kn.shape[1], dtype=torch.int64)
            state["label"] = "oneDNN int8 inner product via torch.ops.onednn.qlinear_pointwise + C oracle quantize"
        except Exception:
            state["pw"] = None
            state["label"] = "C/OpenMP oracle port (oracle/itex_oracle_c.c)"
    if state["pw"] is not None:
        y = torch.ops.onednn.qlinear_pointwise(torch.from_numpy(qa), 1.0, 0, state["pw"], state["ws"], state["wz"],
                                               torch.from_numpy(state["bias_s"]), 1.0, 0, torch.float32, "none", [], "")
        return y.numpy(), state["label"]
    return oc.gemm_fused(qa, state["w_nk"], out_scale, state["bias_s"], False, "float"), state["label"]


def run_reference(args, m, n, k):
    """The reference arm: CPU only, rank 0 only."""
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m_s = min(m, 512)
    rng = np.random.default_rng(1234)
    x = rng.uniform(-1, 1, (m_s, k)).astype(np.float32)
    qw, wmin, wmax, bias = synth_weights(n, k, 1235)
    state = {}
    for _ in range(max(args.warmup, 1)):
        _, label = cpu_reference_step(x, qw, wmin, wmax, bias, state)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(x, qw, wmin, wmax, bias, state)
    dt = (time.perf_counter() - t0) / args.steps
    tops = 2.0 * m_s * n * k / dt / 1e12
    sample = "%d of %d rows per step (%s), %d host threads" % (m_s, m, label, cores)
    line = {"impl": "reference", "metric": "int8_quantized_gemm_tops", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "s8xu8->s32", "data": "synthetic",
            "config": {"workload": args.workload, "m_per_gpu": m, "n": n, "k": k, "cpu_sample_rows": m_s},
            "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_resnet50(args, rank, world, local, dev, K):
    """INT8 ResNet-50 v1.5 inference, batch 128 per GPU (batch-sharded replicas, no collective): images/s.
    A step is one forward pass of the captured graph over one batch of synthetic uint8 images."""
    import torch
    rn = importlib.import_module("itex_b200.resnet50")
    batch = args.batch
    net = rn.ResNet50Int8(device=dev, seed=1237)           # same weights on every rank
    gen = torch.Generator(device=dev)
    gen.manual_seed(shard_seed(1236, rank))
    x = torch.randint(0, 256, (batch, 224, 224, 3), dtype=torch.uint8, device=dev, generator=gen)
    calib = torch.randint(0, 256, (16, 224, 224, 3), dtype=torch.uint8, device=dev, generator=torch.Generator(device=dev).manual_seed(99))
    net.forward(calib, calibrate=True)                     # ranges frozen from one seeded batch, identical on all ranks
    graph, logits = net.capture(x)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    t_warm, n_warm = time.perf_counter(), 0
    while n_warm < args.warmup or time.perf_counter() - t_warm < args.min_warmup_seconds:
        graph.replay()
        n_warm += 1
        if n_warm % 20 == 0:
            torch.cuda.synchronize()
    barrier()
    launches0 = K.launch_count()
    net.forward(x)                                         # eager pass: counts this library's launches per step
    torch.cuda.synchronize()
    launches_per_step = K.launch_count() - launches0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    sampler.stop_flag.set()
    sampler.join()
    ms_step = max_over_ranks(e0.elapsed_time(e1), world, dev) / args.steps
    value = batch * world / (ms_step * 1e-3)
    # end to end: pinned host images in, logits out, every step; the copies run on their own streams into
    # staging slots, and the captured graph's fixed input / output buffers are filled / drained on the compute stream
    x_host = torch.empty((batch, 224, 224, 3), dtype=torch.uint8, pin_memory=True)
    x_host.copy_(x.cpu())
    out_host = torch.empty(tuple(logits.shape), dtype=torch.float32, pin_memory=True)
    x_slot = [torch.empty_like(x) for _ in range(2)]
    o_slot = [torch.empty_like(logits) for _ in range(2)]

    def e2e_h2d(b):
        x_slot[b].copy_(x_host, non_blocking=True)

    def e2e_compute(b):
        x.copy_(x_slot[b], non_blocking=True)
        graph.replay()
        o_slot[b].copy_(logits, non_blocking=True)

    def e2e_d2h(b):
        out_host.copy_(o_slot[b], non_blocking=True)

    pipelined_e2e(2, dev, e2e_h2d, e2e_compute, e2e_d2h, barrier)
    e2e_ms = max_over_ranks(pipelined_e2e(args.e2e_steps, dev, e2e_h2d, e2e_compute, e2e_d2h, barrier), world, dev) / args.e2e_steps
    if rank == 0:
        peaks = measured_peaks()
        macs = net.macs_per_image(224)
        tops = 2.0 * macs * batch / (ms_step * 1e-3) / 1e12
        line = {
            "metric": "resnet50_int8_images_per_s", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8xs8->s32", "data": "synthetic",
            "config": {"workload": "resnet50_int8", "batch_per_gpu": batch, "image": 224, "graph": "53 fused quantized convs + maxpool + avgpool + fc, CUDA graph",
                       "gmacs_per_image": macs / 1e9, "l2": "activations larger than L2 (batch %d)" % batch,
                       "parallelism": "batch-sharded x%d, no collective" % world},
            "roofline": {"bound": "tensor", "kernel": "whole graph (GemmKernel int8 dominates)", "achieved": tops, "peak": 2.0 * peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": tops / (2.0 * peaks["bf16_tflops"]), "traffic": None,
                         "peak_source": "2 x bf16_tflops (burst) of MEASURED_PEAKS.json (%s)" % peaks["source"]},
            "e2e": {"value": batch * world / (e2e_ms * 1e-3), "unit": "images/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": batch * 224 * 224 * 3 * world, "d2h_bytes_per_step": int(logits.numel()) * 4 * world,
                    "checksum": float(out_host.double().sum())},
            "gpu_launches": int(launches_per_step * args.steps), "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)


def run_bert(args, rank, world, local, dev, K):
    """INT8 BERT-large-shaped encoder forward (24 layers, hidden 1024, 16 heads, FFN 4096) on 32 x 384 = 12288
    tokens per GPU (batch-sharded replicas, no collective): tokens/s.  A step is one forward pass replayed as a
    CUDA graph.  The int8 nodes (dynamic-range quantize + fused int8 matmul) are also timed alone."""
    import torch
    bert = importlib.import_module("itex_b200.bert_int8")
    batch, seq = 32, 384
    tokens = batch * seq
    enc = bert.BertInt8Encoder(device=dev, seed=1238)      # same weights on every rank
    gen = torch.Generator(device=dev)
    gen.manual_seed(shard_seed(1238, rank))
    x = torch.randn((tokens, enc.hidden), generator=gen, device=dev).to(torch.bfloat16)
    ctx = torch.randn((tokens, enc.hidden), generator=gen, device=dev).to(torch.bfloat16)
    mid = torch.randn((tokens, enc.ffn), generator=gen, device=dev).to(torch.bfloat16)
    graph, y = enc.capture(enc.forward, x, batch, seq)
    graph8, _ = enc.capture(enc.forward_int8_only, x, ctx, mid)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    t_warm, n_warm = time.perf_counter(), 0
    while n_warm < args.warmup or time.perf_counter() - t_warm < args.min_warmup_seconds:
        graph.replay()
        n_warm += 1
        if n_warm % 5 == 0:
            torch.cuda.synchronize()
    barrier()
    launches0 = K.launch_count()
    enc.forward(x, batch, seq)                             # eager pass: counts this library's launches per step
    torch.cuda.synchronize()
    launches_per_step = K.launch_count() - launches0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1), world, dev) / args.steps
    i0, i1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(2):
        graph8.replay()
    barrier()
    i0.record()
    for _ in range(args.steps):
        graph8.replay()
    i1.record()
    barrier()
    sampler.stop_flag.set()
    sampler.join()
    int8_ms = max_over_ranks(i0.elapsed_time(i1), world, dev) / args.steps
    # end to end: pinned host embeddings in, hidden states out, every step (copies on their own streams)
    x_host = torch.empty((tokens, enc.hidden), dtype=torch.bfloat16, pin_memory=True)
    x_host.copy_(x.cpu())
    out_host = torch.empty((tokens, enc.hidden), dtype=torch.bfloat16, pin_memory=True)
    x_slot = [torch.empty_like(x) for _ in range(2)]
    o_slot = [torch.empty_like(y) for _ in range(2)]

    def e2e_h2d(b):
        x_slot[b].copy_(x_host, non_blocking=True)

    def e2e_compute(b):
        x.copy_(x_slot[b], non_blocking=True)
        graph.replay()
        o_slot[b].copy_(y, non_blocking=True)

    def e2e_d2h(b):
        out_host.copy_(o_slot[b], non_blocking=True)

    pipelined_e2e(2, dev, e2e_h2d, e2e_compute, e2e_d2h, barrier)
    e2e_ms = max_over_ranks(pipelined_e2e(args.e2e_steps, dev, e2e_h2d, e2e_compute, e2e_d2h, barrier), world, dev) / args.e2e_steps
    if rank == 0:
        peaks = measured_peaks()
        ops_step = enc.int8_ops_per_token() * tokens
        tops = ops_step / (int8_ms * 1e-3) / 1e12
        line = {
            "metric": "bert_large_int8_tokens_per_s", "value": tokens * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "s8xs8->s32", "data": "synthetic",
            "config": {"workload": "bert_large_int8", "tokens_per_gpu": tokens, "batch": batch, "seq_len": seq, "layers": enc.layers,
                       "hidden": enc.hidden, "heads": enc.heads, "ffn": enc.ffn,
                       "graph": "per layer 4 x (min/max, quantize, scale, int8 matmul) + bf16 attention, LayerNorm, residuals in PyTorch; CUDA graph",
                       "int8_path_ms": int8_ms, "int8_tops_per_forward": ops_step / 1e12, "l2": "activations larger than L2",
                       "parallelism": "batch-sharded x%d, no collective" % world},
            "roofline": {"bound": "tensor", "kernel": "int8 nodes of the forward pass (GemmKernel int8 + quantize passes)", "achieved": tops,
                         "peak": 2.0 * peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tops / (2.0 * peaks["bf16_tflops"]), "traffic": None,
                         "peak_source": "2 x bf16_tflops (burst) of MEASURED_PEAKS.json (%s)" % peaks["source"]},
            "e2e": {"value": tokens * world / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": tokens * enc.hidden * 2 * world, "d2h_bytes_per_step": tokens * enc.hidden * 2 * world,
                    "checksum": float(out_host.double().sum())},
            "gpu_launches": int(launches_per_step * args.steps), "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)


FP8_LINEARS = ((4096, 4096), (4096, 14336), (14336, 4096))  # (K, N) of the Llama-3-8B-shaped linears, M = 4096 tokens


def run_fp8_linears(args, rank, world, local, dev, K):
    """FP8 e4m3 linears with delayed scaling, column-parallel: rank r holds rows [r*N/g, (r+1)*N/g) of each
    [N,K] weight, activations are replicated, each rank computes [M, N/g] in bf16 and an NCCL all-gather
    assembles [g, M, N/g] (shard-major; the consumer reads that layout).  A step is the three linears:
    scale update, Fp8Quantize(activations), Fp8Quantize(weight shard), Fp8Matmul, all-gather.  Per-shard
    weight amax values are combined with an all-reduce(max) so every rank keeps the same scaling state."""
    import torch
    import torch.distributed as dist
    fp8 = importlib.import_module("itex_b200.fp8")
    m = 4096
    gen = torch.Generator(device=dev)
    gen.manual_seed(1238)                                   # activations are replicated: same seed on every rank
    layers = []
    for (k, n) in FP8_LINEARS:
        assert n % world == 0
        wgen = torch.Generator(device=dev)
        wgen.manual_seed(shard_seed(1239 + k + n, rank))
        w = (torch.randn((n // world, k), generator=wgen, device=dev) * 0.02).to(torch.bfloat16)
        a = torch.randn((m, k), generator=gen, device=dev).to(torch.bfloat16)
        layer = fp8.Fp8Dense(w, recipe=fp8.DelayedScaling(margin=0, amax_history_len=16, amax_compute_algo="max"),
                             out_dtype="bfloat16", weight_layout="nk")
        gathered = torch.empty((world, m, n // world), dtype=torch.bfloat16, device=dev)
        layers.append((layer, a, gathered, k, n))

    comm = torch.cuda.Stream(device=dev)

    def step():
        # The all-gather of linear i runs on a second stream under the quantize + GEMM of linear i+1.
        main = torch.cuda.current_stream(dev)
        comm.wait_stream(main)
        keep = []
        for layer, a, gathered, k, n in layers:
            y = layer(a)
            keep.append(y)
            if world > 1:
                comm.wait_stream(main)
                with torch.cuda.stream(comm):
                    # 12 bytes; the state only has to agree before the next step's scale update
                    dist.all_reduce(layer.meta.amax_history[0], op=dist.ReduceOp.MAX)
                    dist.all_gather_into_tensor(gathered, y)
                    y.record_stream(comm)
            else:
                gathered[0].copy_(y)
        main.wait_stream(comm)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    # A fixed number of warm-up steps: every step holds collectives, so all ranks must run the same count
    # (a time-based loop would let ranks disagree and dead-lock).  >= 17 steps fill the 16-deep amax history.
    n_warm = max(args.warmup, 17, int(args.min_warmup_seconds * 600))
    for _ in range(n_warm):
        step()
    barrier()
    # One CUDA graph per step (kernels and NCCL collectives): removes ~20 host-side op calls per step,
    # which otherwise bound the step once the per-GPU GEMMs shrink with the shard count.
    eager_step = step
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        eager_step()
    torch.cuda.current_stream(dev).wait_stream(side)
    barrier()
    with torch.cuda.graph(graph):
        eager_step()
    step = graph.replay
    for _ in range(3):
        step()
    barrier()
    launches0 = K.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.stop_flag.set()
    sampler.join()
    eager_step()                                            # graph replays do not pass through the library's launch counter
    torch.cuda.synchronize()
    launches = (K.launch_count() - launches0) * args.steps
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1), world, dev) / args.steps
    flops = sum(2.0 * m * k * n for k, n in FP8_LINEARS)
    # end to end: activations from pinned host memory, gathered outputs back to the host
    hosts = [(torch.empty_like(a, device="cpu").pin_memory().copy_(a), torch.empty(tuple(g_.shape), dtype=torch.bfloat16, pin_memory=True))
             for _, a, g_, _, _ in layers]

    def e2e_step():
        for (layer, a, gathered, k, n), (ah, oh) in zip(layers, hosts):
            a.copy_(ah, non_blocking=True)
        step()
        for (layer, a, gathered, k, n), (ah, oh) in zip(layers, hosts):
            oh.copy_(gathered, non_blocking=True)

    e2e_step()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.e2e_steps):
        e2e_step()
    t1.record()
    barrier()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1), world, dev) / args.e2e_steps
    if rank == 0:
        peaks = measured_peaks()
        tflops = flops / (ms_step * 1e-3) / 1e12
        line = {
            "metric": "fp8_llama_linears_tokens_per_s", "value": m / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": n_warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "e4m3xe4m3->f32", "data": "synthetic",
            "config": {"workload": "fp8_llama_linears", "tokens": m, "linears_k_n": FP8_LINEARS, "delayed_scaling": "margin 0, history 16, max",
                       "output": "bfloat16 [g, M, N/g] after all-gather", "l2": "weights + activations larger than L2",
                       "parallelism": "column-parallel x%d, NCCL all-gather of outputs" % world, "tflops": tflops},
            "roofline": {"bound": "tensor", "kernel": "GemmKernel<256,fp8> (tcgen05.mma kind::f8f6f4)", "achieved": tflops,
                         "peak": 2.0 * peaks["bf16_tflops"] * world, "unit": "TFLOP/s", "frac": tflops / (2.0 * peaks["bf16_tflops"] * world),
                         "traffic": None, "peak_source": "2 x bf16_tflops (burst) x GPUs, whole step incl. quantize passes and all-gather"},
            "e2e": {"value": m / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": sum(m * k * 2 for k, _ in FP8_LINEARS), "d2h_bytes_per_step": sum(m * n * 2 for _, n in FP8_LINEARS)},
            "gpu_launches": int(launches), "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="int8_gemm_8192", choices=sorted(WORKLOADS) + ["resnet50_int8", "fp8_llama_linears", "bert_large_int8"])
    ap.add_argument("--batch", type=int, default=128, help="images per GPU for --workload resnet50_int8")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--min-warmup-seconds", type=float, default=1.0,
                    help="keep warming up at least this long so the clock sampler sees the load (0 for profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    m, n, k = WORKLOADS.get(args.workload, WORKLOADS["int8_gemm_8192"])
    if args.impl == "reference":
        run_reference(args, m, n, k)
        return

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        if "ITEXB_NCCL_DEBUG" in os.environ:
            os.environ["NCCL_DEBUG"] = os.environ["ITEXB_NCCL_DEBUG"]
        else:
            os.environ["NCCL_DEBUG_FILE"] = os.devnull              # keep stdout to the one JSON line
        import datetime
        # a short timeout turns any mismatch between ranks into a quick error instead of a long hang
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    itex = load_package()
    ops = importlib.import_module("itex_b200.ops")
    K = importlib.import_module("itex_b200.kernels")
    dev = torch.device("cuda", local)
    if args.workload == "fp8_llama_linears":
        run_fp8_linears(args, rank, world, local, dev, K)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "bert_large_int8":
        run_bert(args, rank, world, local, dev, K)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "resnet50_int8":
        run_resnet50(args, rank, world, local, dev, K)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- synthetic inputs, resident in HBM (seed depends on the rank: each GPU has its own batch shard)
    gen = torch.Generator(device=dev)
    gen.manual_seed(shard_seed(1234, rank))
    x = torch.rand((m, k), device=dev, generator=gen) * 2 - 1
    qw, wmin, wmax, bias_h = synth_weights(n, k, 1235)
    w = torch.from_numpy(qw).to(dev)
    bias = torch.from_numpy(bias_h).to(dev)
    xmin, xmax = float(x.min()), float(x.max())  # the graph's frozen activation range
    q_op = ops.Op("_ITEXQuantizeV2", T="quint8", mode="SCALED", round_mode="HALF_TO_EVEN", narrow_range=False, axis=-1,
                  ensure_minimum_range=0.01, dtype="float")
    mm_op = ops.Op("_ITEXQuantizedMatMulWithBiasAndDequantize", T1="quint8", T2="qint8", Tbias="float", Toutput="float",
                   transpose_a=False, transpose_b=False, input_quant_mode="SCALED", is_weight_const=True)

    def step(x_dev):
        q, qmin, qmax = q_op(x_dev, xmin, xmax)
        return mm_op(q, w, bias, qmin, qmax, wmin, wmax, 0.0, 0.0), q, qmin, qmax

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # clocks are sampled from the warm-up on (one nvidia-smi query takes longer than a step),
    # so the record covers the device under this load, the timed region included
    sampler = ClockSampler(local)
    sampler.start()
    t_warm = time.perf_counter()
    n_warm = 0
    while n_warm < args.warmup or time.perf_counter() - t_warm < args.min_warmup_seconds:
        out, q, qmin, qmax = step(x)
        n_warm += 1
        if n_warm % 50 == 0:
            torch.cuda.synchronize()
    barrier()

    # ---- timed region: K steps, CUDA events on the launching stream.  The K steps are recorded once in a
    #      CUDA graph (the way a serving loop would run a fixed step) so that the host's launch pace, which
    #      varies with how many ranks share the host's cores, is not what is measured; timing events around
    #      every matmul are part of the graph.  Without external-event support the steps run eagerly.
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph = None
    try:
        g0 = [torch.cuda.Event(enable_timing=True, external=True) for _ in range(args.steps)]
        g1 = [torch.cuda.Event(enable_timing=True, external=True) for _ in range(args.steps)]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        launches0 = K.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(args.steps):
                q, qmin, qmax = q_op(x, xmin, xmax)
                g0[i].record()
                out = mm_op(q, w, bias, qmin, qmax, wmin, wmax, 0.0, 0.0)
                g1[i].record()
        launches = K.launch_count() - launches0
        graph.replay()                      # one untimed replay: graph upload, and it proves the capture ran
        torch.cuda.synchronize()
    except Exception as exc:                # noqa: BLE001 - any capture problem means: measure eagerly
        if rank == 0:
            print("bench.py: CUDA-graph timing unavailable (%s); timing eager launches" % type(exc).__name__, file=sys.stderr)
        graph = None
        torch.cuda.synchronize()
        g0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        g1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    if graph is not None:
        e0.record()
        graph.replay()
        e1.record()
    else:
        launches0 = K.launch_count()
        e0.record()
        for i in range(args.steps):
            q, qmin, qmax = q_op(x, xmin, xmax)
            g0[i].record()
            out = mm_op(q, w, bias, qmin, qmax, wmin, wmax, 0.0, 0.0)
            g1[i].record()
        e1.record()
        launches = K.launch_count() - launches0
    barrier()
    sampler.stop_flag.set()
    sampler.join()
    ms_total = e0.elapsed_time(e1)
    gemm_ms = sum(a.elapsed_time(b) for a, b in zip(g0, g1)) / args.steps
    ms_step = max_over_ranks(ms_total, world, dev) / args.steps
    value = whole_job_tops(m, n, k, world, ms_step)

    # ---- end to end through the public op API with host buffers (pinned), every step H2D in, D2H out
    x_host = torch.empty((m, k), dtype=torch.float32, pin_memory=True)
    x_host.copy_(x.cpu())
    out_host = [torch.empty((m, n), dtype=torch.float32, pin_memory=True) for _ in range(2)]
    x_stage = [torch.empty_like(x) for _ in range(2)]
    outs = [None, None]

    def e2e_h2d(b):
        x_stage[b].copy_(x_host, non_blocking=True)

    def e2e_compute(b):
        outs[b] = step(x_stage[b])[0]

    def e2e_d2h(b):
        out_host[b].copy_(outs[b], non_blocking=True)

    pipelined_e2e(2, dev, e2e_h2d, e2e_compute, e2e_d2h, barrier)          # untimed: allocations, first touch
    e2e_ms = max_over_ranks(pipelined_e2e(args.e2e_steps, dev, e2e_h2d, e2e_compute, e2e_d2h, barrier), world, dev) / args.e2e_steps
    out_host = out_host[(args.e2e_steps - 1) & 1]
    e2e_value = whole_job_tops(m, n, k, world, e2e_ms)
    checksum = float(out_host[::997, ::991].double().sum())

    # cuBLAS int8 -> int32 on the same shape (no epilogue): a library ceiling to read the fraction against
    lib_tops = None
    if rank == 0:
        try:
            a8 = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
            b8 = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev).t()
            best = float("inf")
            for i in range(13):
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record()
                torch._int_mm(a8, b8)
                c1.record()
                torch.cuda.synchronize()
                if i >= 3:
                    best = min(best, c0.elapsed_time(c1))
            lib_tops = 2.0 * m * n * k / (best * 1e-3) / 1e12
            del a8, b8
        except Exception:  # noqa: BLE001 - the figure is informative only
            lib_tops = None
    if rank == 0:
        peaks = measured_peaks()
        gemm_tops = 2.0 * m * n * k / (gemm_ms * 1e-3) / 1e12
        int8_peak = 2.0 * peaks["bf16_tflops"]
        line = {
            "metric": "int8_quantized_gemm_tops", "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8xu8->s32", "data": "synthetic",
            "config": {"workload": args.workload, "m_per_gpu": m, "n": n, "k": k, "ops": ["_ITEXQuantizeV2", "_ITEXQuantizedMatMulWithBiasAndDequantize"],
                       "output": "float32", "l2": "inputs larger than L2 (%.0f MB touched per step)" % ((m * k * 5 + n * k + m * n * 4) / 1e6),
                       "launch": "K steps in one CUDA graph" if graph is not None else "eager",
                       "parallelism": "batch-sharded x%d, no collective" % world},
            "roofline": {"bound": "tensor", "kernel": "GemmKernel<256,int8> (tcgen05.mma kind::i8)", "achieved": gemm_tops,
                         "peak": int8_peak, "unit": "TFLOP/s", "frac": gemm_tops / int8_peak,
                         "peak_source": "2 x bf16_tflops (burst) of MEASURED_PEAKS.json (%s); int8 MMA rate is twice bf16" % peaks["source"],
                         "gemm_ms": gemm_ms, "traffic": GEMM_DRAM_TRAFFIC.get(args.workload),
                         "algorithmic_bytes": m * k + n * k + m * n * 4,
                         "library_int_mm_tops": lib_tops, "frac_of_library": None if not lib_tops else gemm_tops / lib_tops},
            "e2e": {"value": e2e_value, "unit": "TOPS", "ms_per_step": e2e_ms, "h2d_bytes_per_step": m * k * 4 * world,
                    "d2h_bytes_per_step": m * n * 4 * world, "checksum": checksum},
            "gpu_launches": int(launches), "clocks": sampler.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            m_s = min(m, 512)
            xs = x[:m_s].cpu().numpy()
            state = {}
            ref, label = cpu_reference_step(xs, qw, wmin, wmax, bias_h, state)
            reps, t_cpu = 0, time.perf_counter()
            while reps < 3 or (time.perf_counter() - t_cpu < 5.0 and reps < 50):
                cpu_reference_step(xs, qw, wmin, wmax, bias_h, state)
                reps += 1
            dt = (time.perf_counter() - t_cpu) / reps
            # the CPU sample also checks the GPU result of the same rows (range = that of the full batch)
            line["cpu_baseline"] = {"value": 2.0 * m_s * n * k / dt / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
                                    "sample": "%d of %d rows per step (%s), %d host threads, %d reps" % (m_s, m, label, cores, reps)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
