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

The default run also measures the other pieces of the path and puts them under "secondary" in
the same line, each with its own value, ms_per_step, roofline, e2e and (one GPU) cpu_baseline:
quantize_f32_u8 / dequantize_u8_f32 at the reference benchmark's sizes (102 760 448 and 3 211 264
elements), conv_cfg2 (the fused int8 3x3 convolution at [32,56,56,64]), resnet50_int8 (images/s,
batch 128 per GPU, weak scaling) and fp8_llama_linears (tokens/s, column-parallel with an all-gather,
strong scaling).  --no-secondary skips them; --workload NAME runs one of them as the headline.

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
GEMM_DRAM_TRAFFIC = {"int8_gemm_8192": 539.4e6, "int8_gemm_4096": 59.1e6}

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


def cpu_reference_step(x_rows, qw_kn, wmin, wmax, bias, state, x_range=None):
    """One CPU step on a row sample: quantize + int8 matmul + bias + dequantize.  x_range: the activation range
    the graph froze (that of the whole batch); by default the sample's own.
    Returns (fp32 output, label of what ran)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import itex_oracle as o
    import oracle_c as oc
    import torch
    mn, mx = (float(x_rows.min()), float(x_rows.max())) if x_range is None else x_range
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


def run_reference(args, m, n, k, emit):
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
    emit(line)


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
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_resnet50(net, calib, args)
        return line
    return None


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
        return line
    return None


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
    # auto: both ways are warmed up and timed on this node, the faster one runs the timed region (which way wins depends
    # on the shard count: the copies of a fused launch cannot overlap a main loop that is a single wave of tiles)
    mode = args.fp8_gather if world > 1 else "nccl"
    pg = None
    layers_nccl = layers
    layers_fused = layers
    if mode != "nccl":
        def exchange(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out
        pg = fp8.PeerGather([(m, n // world) for _, _, _, _, n in layers], torch.bfloat16, rank, world, dev, exchange)
        layers_fused = [(layer, a, pg.gathered(i), k, n) for i, (layer, a, _, k, n) in enumerate(layers)]

    def step_nccl():
        # The all-gather of linear i runs on a second stream under the quantize + GEMM of linear i+1.
        main = torch.cuda.current_stream(dev)
        comm.wait_stream(main)
        keep = []
        for layer, a, gathered, k, n in layers_nccl:
            y = layer(a, out=gathered[rank])            # the shard is computed in its place of the gather buffer
            keep.append(y)
            if world > 1:
                comm.wait_stream(main)
                with torch.cuda.stream(comm):
                    # 12 bytes; the state only has to agree before the next step's scale update
                    dist.all_reduce(layer.meta.amax_history[0], op=dist.ReduceOp.MAX)
                    dist.all_gather_into_tensor(gathered, y)    # in place: y is this rank's slice of `gathered`
        main.wait_stream(comm)

    def reduce_amax(rows):
        # one NCCL launch for the three 12-byte rows; the state only has to agree before the next step's scale update
        with dist._coalescing_manager(device=dev):
            for row in rows:
                dist.all_reduce(row, op=dist.ReduceOp.MAX)

    def step_fused(overlap=False):
        # Every GEMM's copying warps store its shard into all ranks' gather buffers while the next tiles are computed; one
        # publish / finish pair covers the three linears; the amax all-reduce stays on NCCL, on a second stream.
        # overlap: the three linears are independent, so each runs on a stream of its own (PeerGather.linears).
        pg.linears([l[0] for l in layers_fused], [l[1] for l in layers_fused], reduce_amax=reduce_amax, streams=overlap)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    # A fixed number of warm-up steps: every step holds collectives, so all ranks must run the same count
    # (a time-based loop would let ranks disagree and dead-lock).  >= 17 steps fill the 16-deep amax history.
    n_warm = max(args.warmup, 17, int(args.min_warmup_seconds * 600))

    def prepare(way):
        """Warm-up, then one CUDA graph per step (kernels and NCCL collectives): removes ~20 host-side op calls per step,
        which otherwise bound the step once the per-GPU GEMMs shrink with the shard count."""
        fused_way = way != "nccl"
        eager = {"nccl": step_nccl, "fused": step_fused, "fused_streams": lambda: step_fused(True)}[way]
        # after finish() the gathered buffers are complete and may be read; acknowledge() tells the peers that this rank
        # is done reading, which is what lets them store the next step's shards
        ack = pg.acknowledge if fused_way else (lambda: None)
        for _ in range(n_warm):
            eager()
            ack()
        barrier()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            eager()
            ack()
        torch.cuda.current_stream(dev).wait_stream(side)
        barrier()
        with torch.cuda.graph(graph):
            eager()
            ack()           # the timed loop has no consumer: the step is acknowledged inside the graph
        for _ in range(3):
            graph.replay()
        barrier()
        return eager, ack, graph

    def trial_ms(graph, reps=10):
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        c0.record()
        for _ in range(reps):
            graph.replay()
        c1.record()
        barrier()
        return max_over_ranks(c0.elapsed_time(c1), world, dev) / reps

    trials = None
    if mode == "auto":
        ways = {w: prepare(w) for w in ("nccl", "fused", "fused_streams")}
        trials = {w + "_ms": trial_ms(ways[w][2]) for w in ways}                   # the same on every rank
        # a bounded wait that ran out anywhere (a peer that never signalled) disqualifies the fused ways
        trials["fused_status"] = int(max_over_ranks(float(pg.status.item()), world, dev))
        # same inputs and, once the amax history is full, the same scales in every step: what the last fused trial left in
        # the peer-mapped buffers must be what the NCCL trial left in its own, bit for bit, on every rank
        differs = any(not torch.equal(layers_fused[i][2], layers_nccl[i][2]) for i in range(len(layers)))
        trials["fused_equals_nccl"] = max_over_ranks(1.0 if differs else 0.0, world, dev) == 0.0
        ok = trials["fused_status"] == 0 and trials["fused_equals_nccl"]
        mode = min(ways, key=lambda w: trials[w + "_ms"]) if ok else "nccl"
        eager_step, consumed, graph = ways[mode]
    else:
        eager_step, consumed, graph = prepare(mode)
    fused = mode != "nccl"
    layers = layers_fused if fused else layers_nccl
    step = graph.replay
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
    consumed()
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
                       "parallelism": ("column-parallel x%d, all-gather fused into the GEMM kernel (copies to peer memory over NVLink)" if fused
                                       else "column-parallel x%d, NCCL all-gather of outputs") % world,
                       "gather": mode if world > 1 else "none", "gather_trials": trials, "tflops": tflops,
                       "nvlink_bytes_sent_per_gpu_per_step": sum(m * (n // world) * 2 * (world - 1) for _, n in FP8_LINEARS) if world > 1 else 0,
                       "peer_status": int(pg.status.item()) if fused else None},
            "roofline": {"bound": "tensor", "kernel": "GemmKernel<256,fp8> (tcgen05.mma kind::f8f6f4)", "achieved": tflops,
                         "peak": 2.0 * peaks["bf16_tflops"] * world, "unit": "TFLOP/s", "frac": tflops / (2.0 * peaks["bf16_tflops"] * world),
                         "traffic": None, "peak_source": "2 x bf16_tflops (burst) x GPUs, whole step incl. quantize passes and all-gather"},
            "e2e": {"value": m / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": sum(m * k * 2 for k, _ in FP8_LINEARS), "d2h_bytes_per_step": sum(m * n * 2 for _, n in FP8_LINEARS)},
            "gpu_launches": int(launches), "clocks": sampler.summary(),
        }
        if world == 1:
            # cuBLASLt FP8 on the same three shapes (no quantize passes, no scale update): a library ceiling for the GEMMs alone
            try:
                one = torch.ones((), device=dev)
                best_total = 0.0
                for k, n in FP8_LINEARS:
                    a8 = torch.randn((m, k), device=dev).to(torch.float8_e4m3fn)
                    b8 = torch.randn((n, k), device=dev).to(torch.float8_e4m3fn)
                    best = float("inf")
                    for i in range(8):
                        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        c0.record()
                        torch._scaled_mm(a8, b8.t(), one, one, out_dtype=torch.bfloat16)
                        c1.record()
                        torch.cuda.synchronize()
                        if i >= 3:
                            best = min(best, c0.elapsed_time(c1))
                    best_total += best
                line["roofline"]["library_scaled_mm_tflops"] = flops / (best_total * 1e-3) / 1e12
                line["roofline"]["library_scaled_mm_ms"] = best_total
            except Exception:  # noqa: BLE001 - informative only
                line["roofline"]["library_scaled_mm_tflops"] = None
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_fp8_linears(layers, m)
    if pg is not None:
        status = int(pg.status.item())
        del graph
        pg.close(dist.barrier)
        if status != 0:
            raise SystemExit("bench.py: rank %d: the fused all-gather reported status %d (a bounded wait on a peer ran out)" % (rank, status))
    return line if rank == 0 else None


def timed_us(calls, reps):
    """Mean device time per call in microseconds.  `calls` is a list of zero-argument functions that do the same work on
    DIFFERENT input buffers; together the buffers are larger than L2 (126 MB), so cycling through them gives every
    launch cold data without a flush kernel in between.  `reps` rounds over the list are recorded back to back in one
    CUDA graph between a single pair of timing events: what is measured is the kernels on the device at the rate a
    serving loop would issue them, not the host's launch path (a few microseconds of Python and driver per call, more
    than the kernels of the small cases take).  Falls back to eager launches if the capture fails."""
    import torch
    dev = torch.cuda.current_device()
    n = reps * len(calls)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    try:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                for fn in calls:
                    fn()
        graph.replay()
        torch.cuda.synchronize()
        t0.record()
        graph.replay()
        t1.record()
        torch.cuda.synchronize()
        return 1e3 * t0.elapsed_time(t1) / n
    except Exception as exc:                # noqa: BLE001
        print("bench.py: graph timing unavailable (%s); timing eager launches" % type(exc).__name__, file=sys.stderr)
        torch.cuda.synchronize()
    t0.record()
    for _ in range(reps):
        for fn in calls:
            fn()
    t1.record()
    torch.cuda.synchronize()
    return 1e3 * t0.elapsed_time(t1) / n


def rotating_inputs(x, bytes_per_call):
    """Copies of x, enough of them that one round over all touches more than twice the L2 capacity."""
    import torch
    copies = max(1, min(64, -(-(256 << 20) // max(1, bytes_per_call))))
    return [x] + [x.clone() for _ in range(copies - 1)]


def run_pointwise(args, rank, world, local, dev, K, ops, which, count, real=None):
    """_ITEXQuantizeV2 (fp32 -> quint8, SCALED, HALF_TO_EVEN) or _ITEXDequantize (quint8 -> fp32, SCALED) over `count`
    elements through the op layer: achieved GB/s of the 5 algorithmic bytes per element.  The sizes are the reference
    benchmark's (test/benchmark/test_quantize.py:55-56).  The smaller one fits in L2, so the timed launches cycle over
    enough copies of the input to exceed it; the larger one is 4x L2 by itself."""
    import torch
    gen = torch.Generator(device=dev)
    gen.manual_seed(shard_seed(1240, rank))
    shape = (count // 1024, 1024)
    real = real or getattr(args, "real_dtype", "float")      # the real-valued side: float (the reference benchmark's) or bfloat16
    tdt, rb = (torch.bfloat16, 2) if real == "bfloat16" else (torch.float32, 4)
    kernel = {"quantize": "QuantizeKernel", "dequantize": "DequantizeKernel", "fp8_quantize": "Fp8QuantizeKernel",
              "fp8_dequantize": "Fp8DequantizeKernel"}[which]
    if which == "quantize":
        x = (torch.rand(shape, device=dev, generator=gen) * 2 - 1).to(tdt)
        op = ops.Op("_ITEXQuantizeV2", T="quint8", mode="SCALED", round_mode="HALF_TO_EVEN", narrow_range=False, axis=-1,
                    ensure_minimum_range=0.01, dtype=real)
        call = lambda t: op(t, -1.0, 1.0)[0]
        in_b, out_b = rb, 1
    elif which == "dequantize":
        x = torch.randint(0, 256, shape, dtype=torch.uint8, device=dev, generator=gen)
        op = ops.Op("_ITEXDequantize", T="quint8", mode="SCALED", narrow_range=False, axis=-1, dtype=real)
        call = lambda t: op(t, 0.0, 6.0)
        in_b, out_b = 1, rb
    elif which == "fp8_quantize":
        x = torch.randn(shape, device=dev, generator=gen).to(tdt)
        amax, scale = torch.zeros(1, device=dev), torch.full((1,), 64.0, device=dev)
        op = ops.Op("Fp8Quantize", in_dtype=real, fp8_meta_index=0, fp8_dtype="E4M3")
        call = lambda t: op(t, amax, scale)
        in_b, out_b = rb, 1
    else:
        x = torch.randint(0, 120, shape, dtype=torch.int8, device=dev, generator=gen)
        sinv = torch.full((1,), 1.0 / 64.0, device=dev)
        op = ops.Op("Fp8Dequantize", out_dtype=real, fp8_meta_index=0, fp8_dtype="E4M3")
        call = lambda t: op(t, sinv, dtypes={0: ops.L.DT_INT8})     # FP8 bytes travel as plain int8, not as a quantized type
        in_b, out_b = 1, rb
    per_elem = in_b + out_b
    xs = rotating_inputs(x, count * per_elem)
    for _ in range(max(args.warmup, 3)):
        y = call(x)
    torch.cuda.synchronize()
    n0 = K.launch_count()
    us = timed_us([(lambda t=t: call(t)) for t in xs], max(3, 40 // len(xs)))
    launches = K.launch_count() - n0
    del xs
    us = max_over_ranks(us, world, dev)
    # end to end: pinned host tensor in, result back to pinned host memory, every step
    xh = torch.empty(shape, dtype=x.dtype, pin_memory=True)
    xh.copy_(x.cpu())
    yh = torch.empty(shape, dtype=y.dtype, pin_memory=True)
    xd = torch.empty_like(x)

    def e2e_step():
        xd.copy_(xh, non_blocking=True)
        yh.copy_(call(xd), non_blocking=True)

    e2e_step()
    torch.cuda.synchronize()
    e2e_reps = 3
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(e2e_reps):
        e2e_step()
    t1.record()
    torch.cuda.synchronize()
    e2e_us = max_over_ranks(1e3 * t0.elapsed_time(t1) / e2e_reps, world, dev)
    if rank != 0:
        return None
    peaks = measured_peaks()
    gbs = count * per_elem / (us * 1e-6) / 1e9
    tname = {"float": "f32", "bfloat16": "bf16"}[real]
    io = {"quantize": "%s->u8" % tname, "dequantize": "u8->%s" % tname, "fp8_quantize": "%s->e4m3" % tname, "fp8_dequantize": "e4m3->%s" % tname}[which]
    line = {"metric": "%s_gb_per_s" % which, "value": gbs * world, "unit": "GB/s", "ms_per_step": us * 1e-3, "n_gpus": world, "scaling": "weak",
            "dtype": io,
            "config": {"workload": "%s_%s_%d" % (which, io.replace("->", "_"), count), "elements_per_gpu": count,
                       "op": {"quantize": "_ITEXQuantizeV2", "dequantize": "_ITEXDequantize", "fp8_quantize": "Fp8Quantize", "fp8_dequantize": "Fp8Dequantize"}[which],
                       "l2": "launches cycle over input copies that together exceed L2; back-to-back launches in one CUDA graph"},
            "roofline": {"bound": "hbm", "kernel": kernel, "achieved": gbs,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                         "algorithmic_bytes": count * per_elem, "bytes_per_element": per_elem,
                         "peak_source": "hbm_gbs of MEASURED_PEAKS.json (%s)" % peaks["source"]},
            "e2e": {"value": count * per_elem * world / (e2e_us * 1e-6) / 1e9, "unit": "GB/s", "ms_per_step": e2e_us * 1e-3,
                    "h2d_bytes_per_step": count * in_b * world, "d2h_bytes_per_step": count * out_b * world},
            "gpu_launches": int(launches)}
    if world == 1 and not args.no_cpu_baseline and which in ("quantize", "dequantize") and real == "float":
        line["cpu_baseline"] = cpu_pointwise(which, x[: min(x.shape[0], 3136)].cpu().numpy())
    return line


def cpu_pointwise(which, sample):
    """The C/OpenMP oracle's quantize / dequantize on a 3 211 264-element sample, all host threads."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_c as oc
    fn = (lambda: oc.quantize_scaled(sample, np.float32(255.0), False)) if which == "quantize" else (lambda: oc.dequantize(sample, np.float32(6.0 / 255.0)))
    fn()
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 2.0 and reps < 200):
        fn()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": sample.size * 5 / dt / 1e9, "unit": "GB/s", "cores": oc.num_threads(), "kind": "port",
            "sample": "%d elements, C/OpenMP oracle (oracle/itex_oracle_c.c), %d reps" % (sample.size, reps)}


CONV_CFG2 = dict(n=32, h=56, w=56, c=64, k=3, co=64)


def run_conv_cfg2(args, rank, world, local, dev, K, ops):
    """_ITEXQuantizedConv2DWithBiasAndReluAndRequantize at [32,56,56,64] x 3x3x64x64, stride 1, SAME, u8 -> u8: the
    fused int8 convolution of the reference's conv configuration.  Input + output + filter (12.9 MB) fit in L2, so the timed
    launches cycle over enough copies of the input to exceed it.  Both roofline fractions are given: tensor (2 x measured
    bf16) and HBM."""
    import torch
    c = CONV_CFG2
    gen = torch.Generator(device=dev)
    gen.manual_seed(shard_seed(1236, rank))
    x = torch.randint(0, 256, (c["n"], c["h"], c["w"], c["c"]), dtype=torch.uint8, device=dev, generator=gen)
    rng = np.random.default_rng(1236)
    f = (rng.standard_normal((c["k"], c["k"], c["c"], c["co"])) * 0.05).astype(np.float32)
    amax = np.abs(f).reshape(-1, c["co"]).max(axis=0).astype(np.float32)
    qf_h = np.clip(np.rint(f * (127.0 / amax)), -127, 127).astype(np.int8)
    bias_h = (rng.standard_normal(c["co"]) * 0.1).astype(np.float32)
    qf, bias = torch.from_numpy(qf_h).to(dev), torch.from_numpy(bias_h).to(dev)
    rng_in, rng_out = (0.0, 12.75), (0.0, 20.0)
    op = ops.Op("_ITEXQuantizedConv2DWithBiasAndReluAndRequantize", Tinput="quint8", Tfilter="qint8", Tbias="float", out_type="quint8",
                strides=[1, 1, 1, 1], padding="SAME", dilations=[1, 1, 1, 1], data_format="NHWC", is_filter_const=True, is_bias_const=True)
    call = lambda t: op(t, qf, bias, rng_in[0], rng_in[1], -amax, amax, rng_out[0], rng_out[1])[0]
    xs = rotating_inputs(x, 2 * int(x.numel()))
    for _ in range(max(args.warmup, 3)):
        y = call(x)
    torch.cuda.synchronize()
    n0 = K.launch_count()
    us = timed_us([(lambda t=t: call(t)) for t in xs], 3)
    launches = K.launch_count() - n0
    del xs
    us = max_over_ranks(us, world, dev)
    xh = torch.empty(tuple(x.shape), dtype=torch.uint8, pin_memory=True)
    xh.copy_(x.cpu())
    yh = torch.empty(tuple(y.shape), dtype=torch.uint8, pin_memory=True)
    xd = torch.empty_like(x)

    def e2e_step():
        xd.copy_(xh, non_blocking=True)
        yh.copy_(call(xd), non_blocking=True)

    e2e_step()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(10):
        e2e_step()
    t1.record()
    torch.cuda.synchronize()
    e2e_us = max_over_ranks(1e3 * t0.elapsed_time(t1) / 10, world, dev)
    if rank != 0:
        return None
    peaks = measured_peaks()
    ops_n = 2.0 * c["n"] * c["h"] * c["w"] * c["co"] * c["k"] * c["k"] * c["c"]
    bytes_n = 2 * c["n"] * c["h"] * c["w"] * c["c"] + c["k"] * c["k"] * c["c"] * c["co"] + 8 * c["co"]
    tops = ops_n / (us * 1e-6) / 1e12
    gbs = bytes_n / (us * 1e-6) / 1e9
    line = {"metric": "conv_cfg2_tops", "value": tops * world, "unit": "TOPS", "ms_per_step": us * 1e-3, "n_gpus": world, "scaling": "weak",
            "dtype": "u8xs8->s32",
            "config": {"workload": "conv_cfg2", "input": [c["n"], c["h"], c["w"], c["c"]], "filter": [c["k"], c["k"], c["c"], c["co"]],
                       "op": "_ITEXQuantizedConv2DWithBiasAndReluAndRequantize", "stride": 1, "padding": "SAME", "output": "quint8",
                       "l2": "launches cycle over input copies that together exceed L2; back-to-back launches in one CUDA graph"},
            "roofline": {"bound": "hbm", "kernel": "GemmKernel<64,int8,im2col> (tcgen05.mma kind::i8, TMA im2col A operand)", "achieved": gbs,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": None, "algorithmic_bytes": bytes_n,
                         "tensor": {"achieved": tops, "peak": 2.0 * peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tops / (2.0 * peaks["bf16_tflops"])},
                         "note": "574 op/B: the HBM floor (%.2f us) and the tensor floor (%.2f us) of this layer are within 15 %% of each other"
                                 % (bytes_n / peaks["hbm_gbs"] / 1e3, ops_n / (2.0 * peaks["bf16_tflops"]) / 1e6),
                         "peak_source": "hbm_gbs and 2 x bf16_tflops (burst) of MEASURED_PEAKS.json (%s)" % peaks["source"]},
            "e2e": {"value": ops_n * world / (e2e_us * 1e-6) / 1e12, "unit": "TOPS", "ms_per_step": e2e_us * 1e-3,
                    "h2d_bytes_per_step": int(x.numel()) * world, "d2h_bytes_per_step": int(y.numel()) * world},
            "gpu_launches": int(launches)}
    if world == 1 and not args.no_cpu_baseline:
        import torch
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import itex_oracle as o
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        node = CpuConv(qf_h, bias_h, rng_in, (-amax, amax), rng_out, 1, True, "quint8", o)
        xc = x.cpu().permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)
        ref = node(xc)
        same = bool((ref.permute(0, 2, 3, 1) == y.cpu()).all())
        if not same:
            raise SystemExit("bench.py: conv_cfg2: the GPU output differs from the oneDNN CPU result on the same input")
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t0 < 3.0 and reps < 100):
            node(xc)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": ops_n / dt / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
                                "sample": "the whole layer, oneDNN int8 convolution via torch.ops.onednn.qconv2d_pointwise, %d host threads, %d reps" % (cores, reps)}
        line["parity_checked"] = "whole output bit-identical to the CPU result"
    return line


class CpuConv:
    """One fused quantized convolution on the CPU through real oneDNN (torch.ops.onednn.qconv2d_pointwise), driven the way
    the reference drives dnnl::convolution_forward: combined per-channel scale on the weights argument, pre-scaled bias,
    ReLU and the u8 summand as post-ops (quantized_conv_ops.h:329-446).  NCHW channels_last tensors in and out."""

    def __init__(self, qf_hwio, bias, rng_in, rng_filter, rng_out, stride, relu, out_type, o, in_type="quint8"):
        import torch
        self.torch = torch
        kh = qf_hwio.shape[0]
        co = qf_hwio.shape[3]
        self.stride, self.relu, self.out_type, self.kh = stride, relu, out_type, kh
        self.scales = o.conv_output_scale(rng_in[0], rng_in[1], rng_filter[0], rng_filter[1], in_type, out_type, rng_out[0], rng_out[1])
        self.bias = torch.from_numpy(o.conv_scaled_bias(bias, rng_in[0], rng_in[1], rng_filter[0], rng_filter[1], in_type, out_type, self.scales))
        self.ws = torch.from_numpy(self.scales.copy())
        self.wz = torch.zeros(co, dtype=torch.int64)
        qw = torch.from_numpy(np.ascontiguousarray(qf_hwio.transpose(3, 2, 0, 1)))
        self.rng_out = rng_out
        self.o = o
        self._packed = {}
        self.qw = qw

    def _pads(self, h, w):
        oh, pt, pb = self.o.same_padding(h, self.kh, self.stride)
        ow, pl, pr = self.o.same_padding(w, self.kh, self.stride)
        return pt, pb, pl, pr

    def __call__(self, x, summand=None, sum_range=None):
        torch = self.torch
        pt, pb, pl, pr = self._pads(x.shape[2], x.shape[3])
        if pt != pb or pl != pr:      # the binding takes symmetric padding only
            x = torch.nn.functional.pad(x, (pl, pr, pt, pb)).contiguous(memory_format=torch.channels_last)
            pad = [0, 0]
        else:
            pad = [pt, pl]
        key = tuple(pad)
        if key not in self._packed:
            self._packed[key] = torch.ops.onednn.qconv_prepack(self.qw, self.ws, 1.0, 0, [self.stride] * 2, pad, [1, 1], 1, None)
        pw = self._packed[key]
        odt = torch.uint8 if self.out_type == "quint8" else torch.int8
        st = [self.stride] * 2
        if summand is None:
            return torch.ops.onednn.qconv2d_pointwise(x, 1.0, 0, pw, self.ws, self.wz, self.bias, st, pad, [1, 1], 1, 1.0, 0, odt,
                                                      "relu" if self.relu else "none", [], "")
        so = np.float32(max(abs(np.float32(self.rng_out[0])), abs(np.float32(self.rng_out[1]))))
        ss = np.float32(max(abs(np.float32(sum_range[0])), abs(np.float32(sum_range[1]))))
        if summand.dtype == torch.uint8:
            return torch.ops.onednn.qconv2d_pointwise.binary(x, 1.0, 0, pw, self.ws, self.wz, summand.clone(), self.bias, st, pad, [1, 1], 1, 1.0, 0,
                                                             odt, float(np.float32(ss / so)), 0, "sum", 1.0, "relu", [], "")
        # signed summand into an unsigned output: this binding's sum post-op wants one data type, so this node (4 of 53)
        # takes the convolution in fp32 and does the post-op here: one fused multiply-add like the post-op itself
        # (formed in float64, where the product of a float and a byte is exact, and rounded once)
        sum_scale = np.float32(np.float32(np.float32(255.0) * ss) / np.float32(so * np.float32(127.0)))
        v = torch.ops.onednn.qconv2d_pointwise(x, 1.0, 0, pw, self.ws, self.wz, self.bias, st, pad, [1, 1], 1, 1.0, 0, torch.float32, "none", [], "")
        v = torch.relu((v.double() + summand.double() * float(sum_scale)).float())
        return torch.clamp(torch.round(v), 0, 255).to(torch.uint8)


def cpu_resnet50(net, calib, args):
    """INT8 ResNet-50 forward on the host cores through real oneDNN (qconv2d_pointwise per node, pooling and the final
    int8 matmul in torch), batch 16, with the GPU graph's weights and frozen ranges; its logits must equal the GPU's."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import itex_oracle as o
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x_dev = calib[:16]
    gpu_logits = net.forward(x_dev).cpu()

    # ranges of each node's input are only known along the graph: build the CPU nodes while walking it once
    cpu_nodes = {}

    def run(node, q, rng, sm=None, srng=None):
        key = node.name
        if key not in cpu_nodes:
            cpu_nodes[key] = CpuConv(node.filter.cpu().numpy(), node.bias.cpu().numpy(), rng, (node.min_filter, node.max_filter),
                                     (node.min_out, node.max_out), node.stride, node.relu, node.out_type, o,
                                     in_type="quint8" if q.dtype == torch.uint8 else "qint8")
        return cpu_nodes[key](q, sm, srng), (node.min_out, node.max_out)

    fc_w = net.fc_w.cpu().numpy()
    fc_b = net.fc_b.cpu().numpy()

    def forward(xc):
        q, r = run(net.stem, xc, net.input_range)
        # SAME 3x3/2 on 112 rows: one pixel of padding after (zeros never win against uint8 values); torch's CPU max pooling
        # has no uint8 kernel for this size, so the values pass through fp32 (exact)
        q = torch.nn.functional.max_pool2d(torch.nn.functional.pad(q, (0, 1, 0, 1)).float(), 3, 2).to(torch.uint8)
        q = q.contiguous(memory_format=torch.channels_last)
        for proj, c1, c2, c3 in net.blocks:
            if proj is not None:
                s, sr = run(proj, q, r)
            else:
                s, sr = q, r
            a, ar = run(c1, q, r)
            b, br = run(c2, a, ar)
            q, r = run(c3, b, br, s, sr)
        # _ITEXQuantizedAvgPool: integer mean, rounded half away from zero on the fp32 quotient like the op
        hw = q.shape[2] * q.shape[3]
        pooled = o.quantized_pool2d(q.permute(0, 2, 3, 1).numpy(), (1, q.shape[2], q.shape[3], 1), (1, q.shape[2], q.shape[3], 1), "VALID", avg=True)
        feat = pooled.reshape(pooled.shape[0], -1)
        out, _, _ = o.quantized_matmul_with_bias(feat, fc_w, fc_b, r[0], r[1], net.fc_range[0], net.fc_range[1], 0.0, 0.0, toutput="float",
                                                 input_quant_mode="SCALED", scaled_bias_mode="intended")
        return torch.from_numpy(out)

    xc = x_dev.cpu().permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)
    logits = forward(xc)
    same = bool((logits == gpu_logits).all())
    diff = float((logits - gpu_logits).abs().max())
    if not same and diff > 0.05 * float(gpu_logits.abs().max()):
        raise SystemExit("bench.py: resnet50_int8: GPU logits differ from the oneDNN CPU forward on the same 16 images by %g" % diff)
    reps, t0 = 0, time.perf_counter()
    while reps < 2 or (time.perf_counter() - t0 < 8.0 and reps < 50):
        forward(xc)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": 16 / dt, "unit": "images/s", "cores": cores, "kind": "port",
            "parity": "logits of the 16 images bit-identical to the GPU graph's" if same else
                      "logits differ from the GPU graph's by at most %g (%.2f %% of the largest logit)" % (diff, 100 * diff / float(gpu_logits.abs().max())),
            "sample": "batch 16 forward, 53 oneDNN int8 convolutions via torch.ops.onednn.qconv2d_pointwise (+ pooling and the "
                      "final matmul in torch / NumPy), %d host threads, %d reps" % (cores, reps)}


def cpu_fp8_linears(layers, m):
    """The reference registers Fp8Matmul for its GPU only (fp8_matmul_op.cc:100-110), so there is no reference CPU
    kernel to time: the baseline is the NumPy restatement (dequantize both operands, float64 matmul) on a 64-token sample
    of the three linears."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import itex_oracle as o
    rows = 64
    work = []
    for layer, a, gathered, k, n in layers:
        amax = np.zeros(3, np.float32)
        scale = layer.meta.scale.cpu().numpy()
        qa = o.fp8_quantize(a[:rows].float().cpu().numpy(), amax, scale, 0)
        qw = o.fp8_quantize(layer.kernel.float().cpu().numpy(), amax, scale, 1)
        work.append((qa, qw, (1.0 / scale).astype(np.float32), k, n))
    t0 = time.perf_counter()
    for qa, qw, sinv, k, n in work:
        o.fp8_matmul(qa, qw, None, None, sinv, sinv, None, None, transpose_b=True, sum_dtype="bfloat16", out_dtype="bfloat16")
    dt = time.perf_counter() - t0
    return {"value": rows / dt, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": "%d of %d tokens through the three linears, NumPy restatement (oracle/itex_oracle.py fp8_matmul), 1 rep" % (rows, m)}


def run_gemm(args, rank, world, local, dev, K, ops, m, n, k):
    """The headline: _ITEXQuantizeV2 + _ITEXQuantizedMatMulWithBiasAndDequantize at [m,k] x [k,n]."""
    import torch
    import torch.distributed as dist
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
    gemm_each = sorted(a.elapsed_time(b) for a, b in zip(g0, g1))
    gemm_ms = sum(gemm_each) / args.steps
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
    if rank != 0:
        return None
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
                     "gemm_ms": gemm_ms, "gemm_ms_min_median_max": [gemm_each[0], gemm_each[len(gemm_each) // 2], gemm_each[-1]], "traffic": GEMM_DRAM_TRAFFIC.get(args.workload),
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, ncu capture summarised in profiles/int8_gemm_quantize_matmul.md",
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
        # the CPU sample also checks the GPU result of the same rows: quantized with the full batch's range, as the GPU step was
        ref, label = cpu_reference_step(xs, qw, wmin, wmax, bias_h, state, (xmin, xmax))
        got = step(x)[0][:m_s].cpu().numpy()
        bad = int((got != ref).sum())
        if bad:
            raise SystemExit("bench.py: %d of %d outputs of the first %d rows differ from the CPU result (%s)" % (bad, ref.size, m_s, label))
        line["parity_rows_checked"] = m_s
        reps, t_cpu = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t_cpu < 5.0 and reps < 50):
            cpu_reference_step(xs, qw, wmin, wmax, bias_h, state, (xmin, xmax))
            reps += 1
        dt = (time.perf_counter() - t_cpu) / reps
        line["cpu_baseline"] = {"value": 2.0 * m_s * n * k / dt / 1e12, "unit": "TOPS", "cores": cores, "kind": "port",
                                "sample": "%d of %d rows per step (%s), %d host threads, %d reps" % (m_s, m, label, cores, reps)}
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="int8_gemm_8192",
                    choices=sorted(WORKLOADS) + ["resnet50_int8", "fp8_llama_linears", "bert_large_int8", "conv_cfg2", "quantize", "dequantize",
                                                 "fp8_quantize", "fp8_dequantize"])
    ap.add_argument("--batch", type=int, default=128, help="images per GPU for --workload resnet50_int8")
    ap.add_argument("--elements", type=int, default=102760448, help="elements per GPU for --workload [fp8_]quantize / [fp8_]dequantize")
    ap.add_argument("--real-dtype", default="float", choices=["float", "bfloat16"],
                    help="type of the real-valued side for --workload [fp8_]quantize / [fp8_]dequantize")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--fp8-gather", default="auto", choices=["auto", "fused", "fused_streams", "nccl"],
                    help="fp8_llama_linears on several GPUs: all-gather fused into the GEMM kernel (copies to peer memory), the same "
                         "with each linear on a stream of its own, NCCL's, or whichever is fastest in a trial during warm-up")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="headline workload only (profiler runs, quick checks)")
    ap.add_argument("--min-warmup-seconds", type=float, default=1.0,
                    help="keep warming up at least this long so the clock sampler sees the load (0 for profiler runs)")
    args = ap.parse_args()
    # stdout carries exactly one line, the JSON record: everything else any library writes to file descriptor 1 (NCCL's
    # version banner ignores NCCL_DEBUG_FILE) is sent to stderr, and the record goes to the saved descriptor at the end
    sys.stdout.flush()
    record_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        sys.stdout.flush()
        os.write(record_fd, (json.dumps(line) + "\n").encode())

    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    m, n, k = WORKLOADS.get(args.workload, WORKLOADS["int8_gemm_8192"])
    if args.impl == "reference":
        run_reference(args, m, n, k, emit)
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
        # NCCL's own log (communicator and ring/tree set-up, "nranks N") is written to file descriptor 1, which by now is
        # stderr; stdout stays the one JSON line.  (NCCL_DEBUG_FILE=/dev/stderr would reopen - and truncate - a stderr
        # that is redirected to a file, once per rank.)
        if os.environ.get("NCCL_DEBUG", "").upper() not in ("INFO", "TRACE"):
            os.environ["NCCL_DEBUG"] = "INFO"       # an inherited VERSION / WARN would hide the communicator lines
            os.environ.setdefault("NCCL_DEBUG_SUBSYS", "INIT")
        import datetime
        # a short timeout turns any mismatch between ranks into a quick error instead of a long hang
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    load_package()
    ops = importlib.import_module("itex_b200.ops")
    K = importlib.import_module("itex_b200.kernels")
    dev = torch.device("cuda", local)
    common = (args, rank, world, local, dev, K)

    def release():
        import gc
        gc.collect()
        torch.cuda.empty_cache()

    if args.workload == "fp8_llama_linears":
        line = run_fp8_linears(*common)
    elif args.workload == "bert_large_int8":
        line = run_bert(*common)
    elif args.workload == "resnet50_int8":
        line = run_resnet50(*common)
    elif args.workload == "conv_cfg2":
        line = run_conv_cfg2(*common, ops)
    elif args.workload in ("quantize", "dequantize", "fp8_quantize", "fp8_dequantize"):
        line = run_pointwise(*common, ops, args.workload, args.elements)
    else:
        line = run_gemm(*common, ops, m, n, k)
        if args.workload == "int8_gemm_8192" and not args.no_secondary:
            secondary = {}
            for name, fn in (
                    ("quantize_f32_u8_102760448", lambda: run_pointwise(*common, ops, "quantize", 102760448)),
                    ("quantize_f32_u8_3211264", lambda: run_pointwise(*common, ops, "quantize", 3211264)),
                    ("dequantize_u8_f32_102760448", lambda: run_pointwise(*common, ops, "dequantize", 102760448)),
                    ("dequantize_u8_f32_3211264", lambda: run_pointwise(*common, ops, "dequantize", 3211264)),
                    ("fp8_quantize_bf16_e4m3_58720256", lambda: run_pointwise(*common, ops, "fp8_quantize", 58720256, "bfloat16")),
                    ("conv_cfg2", lambda: run_conv_cfg2(*common, ops)),
                    ("resnet50_int8", lambda: run_resnet50(*common)),
                    ("fp8_llama_linears", lambda: run_fp8_linears(*common))):
                release()
                t0 = time.perf_counter()
                sub = fn()
                if rank == 0:
                    sub["bench_seconds"] = round(time.perf_counter() - t0, 1)
                    secondary[name] = sub
            if rank == 0:
                line["secondary"] = secondary
    if rank == 0:
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
