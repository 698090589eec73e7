"""INT8 BERT-large-shaped encoder assembled from the quantized matmul path of this library.

What an INC-quantized, ITEX-rewritten BERT contains per layer is four fused int8 matmuls with dynamic
per-tensor activation ranges (QKV, attention output, FFN up with GELU, FFN down): in the reference each is
a Min/Max reduction, a copy of the two scalars to the host (the ranges are HostMemory inputs), `_ITEXQuantizeV2`
and `_ITEXQuantizedMatMul` (fused_ops BiasAdd [+ GeluApproximate] + Dequantize, per-channel int8 weights,
int8 activations).  Here the range stays on the device: `itexb_minmax`, `itexb_quantize_dynamic_scales` (which
also derives the matmul's per-channel scales) and the GEMM are stream-ordered launches with no host round trip,
so a whole forward pass can be replayed as one CUDA graph.  The arithmetic is the reference's
(QuantizeV2 SCALED, per-channel scale range_input*range_weight/(127*127), bias added after scaling in real
units); the per-node tests compare every int8 node with the oracle.

Softmax attention, LayerNorm and the residual additions are not on the quantized path; they are plain
PyTorch (bf16) and are timed separately by the benchmark.  Weights are synthetic (N(0, 0.02), seeded).
"""
import torch

from . import _lib as L
from . import kernels as K


class Int8Linear:
    """One int8 matmul node: per-output-channel symmetric int8 weight, fp32 bias, optional fused GELU."""

    def __init__(self, name, k, n, gen, device, gelu=False, out_dtype=L.DT_BFLOAT16):
        self.name, self.k, self.n, self.gelu, self.out_dtype = name, k, n, gelu, out_dtype
        w = torch.randn((k, n), generator=gen, device=device) * 0.02
        amax = w.abs().amax(dim=0).clamp_min(1e-12)
        self.w_kn = torch.clamp(torch.round(w * (127.0 / amax)), -127, 127).to(torch.int8).contiguous()   # TF layout [K, N]
        self.w_nk = K.pack_weights_kn(self.w_kn)                                                          # K-major, packed once
        self.weight_range = amax.float().contiguous()       # max(|min_b|, |max_b|) per output channel
        self.bias = (torch.randn(n, generator=gen, device=device) * 0.1).contiguous()
        self.scales = torch.empty(n, dtype=torch.float32, device=device)
        self.minmax = torch.empty(2, dtype=torch.float32, device=device)

    def __call__(self, x, trace=None):
        """x: [tokens, k] float32 or bfloat16 on the device -> [tokens, n] in out_dtype."""
        mm = K.minmax(x, out=self.minmax)
        q, range3, sc = K.quantize_dynamic(x, L.DT_QINT8, mm, weight_range=self.weight_range, scales=self.scales)
        ep = K.make_epilogue(scale=sc, bias=self.bias, activation=L.ACT_GELU_TANH if self.gelu else L.ACT_NONE)
        y = K.gemm(q, self.w_nk, self.out_dtype, ep=ep, k=self.k)
        if trace is not None:
            trace.append((self, x, q, range3.clone(), y))
        return y


class BertInt8Encoder:
    def __init__(self, layers=24, hidden=1024, heads=16, ffn=4096, device="cuda", seed=1238):
        self.layers, self.hidden, self.heads, self.ffn = layers, hidden, heads, ffn
        self.device = torch.device(device)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        self.blocks = []
        for i in range(layers):
            p = "layer%d_" % i
            self.blocks.append(dict(
                qkv=Int8Linear(p + "qkv", hidden, 3 * hidden, gen, self.device),
                out=Int8Linear(p + "attn_out", hidden, hidden, gen, self.device),
                up=Int8Linear(p + "ffn_up", hidden, ffn, gen, self.device, gelu=True),
                down=Int8Linear(p + "ffn_down", ffn, hidden, gen, self.device),
                ln1=(torch.ones(hidden, device=self.device, dtype=torch.bfloat16), torch.zeros(hidden, device=self.device, dtype=torch.bfloat16)),
                ln2=(torch.ones(hidden, device=self.device, dtype=torch.bfloat16), torch.zeros(hidden, device=self.device, dtype=torch.bfloat16))))

    def linears(self):
        for b in self.blocks:
            for key in ("qkv", "out", "up", "down"):
                yield b[key]

    def int8_ops_per_token(self):
        """Multiply-accumulate operations x 2 of the int8 matmuls per token, from the layer table."""
        return 2 * sum(l.k * l.n for l in self.linears())

    def _attention(self, qkv, batch, seq):
        h, d = self.heads, self.hidden // self.heads
        q, k, v = qkv.view(batch, seq, 3, h, d).permute(2, 0, 3, 1, 4)   # each [batch, heads, seq, d]
        ctx = torch.nn.functional.scaled_dot_product_attention(q, k, v)
        return ctx.permute(0, 2, 1, 3).reshape(batch * seq, self.hidden)

    def forward(self, x, batch, seq, trace=None):
        """x: [batch*seq, hidden] bfloat16 embeddings -> [batch*seq, hidden] bfloat16."""
        ln = torch.nn.functional.layer_norm
        for b in self.blocks:
            qkv = b["qkv"](x, trace)
            ctx = self._attention(qkv, batch, seq)
            x = ln(x + b["out"](ctx, trace), (self.hidden,), *b["ln1"])
            x = ln(x + b["down"](b["up"](x, trace), trace), (self.hidden,), *b["ln2"])
        return x

    def forward_int8_only(self, x, ctx, mid):
        """The int8 nodes of forward() on fixed inputs (x, ctx: [tokens, hidden], mid: [tokens, ffn]): what the
        quantized path alone costs, without attention, LayerNorm and residuals."""
        y = None
        for b in self.blocks:
            b["qkv"](x)
            b["out"](ctx)
            b["up"](x)
            y = b["down"](mid)
        return y

    def capture(self, fn, *args):
        """Records fn(*args) in a CUDA graph after two warm-up runs; returns (graph, static output)."""
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(2):
                fn(*args)
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = fn(*args)
        return g, out
