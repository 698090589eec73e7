"""INT8 ResNet-50 v1.5 inference graph assembled from the quantized ops of this library.

This is the graph an INC-quantized, ITEX-rewritten ResNet-50 contains: every convolution is one
fused `_ITEXQuantizedConv2DWithBias[Sum][AndRelu]AndRequantize` node (uint8 activations with a frozen
per-tensor range, int8 per-output-channel weights, fp32 folded-batch-norm bias), plus
`_ITEXQuantizedMaxPool`, `_ITEXQuantizedAvgPool` and a final `_ITEXQuantizedMatMulWithBiasAndDequantize`.
Weights are synthetic (He-normal, seeded) because no checkpoint is available; activation ranges are
calibrated once on a seeded batch with an fp32 reference and then frozen, as a calibration tool would.

v1.5: the stride-2 convolution of each down-sampling bottleneck is the 3x3 one.
"""
import math

import torch

from . import ops

STAGES = ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2))  # (width, blocks, stride of the first block)


def _quantize_filter_per_channel(w):
    """fp32 HWIO -> (int8 HWIO, min[co], max[co]) symmetric per output channel (axis 3)."""
    amax = w.abs().amax(dim=(0, 1, 2)).clamp_min(1e-12)
    q = torch.clamp(torch.round(w * (127.0 / amax)), -127, 127).to(torch.int8)
    return q.contiguous(), (-amax).cpu().numpy(), amax.cpu().numpy()


class ConvNode:
    """One fused quantized convolution node with its constants."""

    def __init__(self, name, cin, cout, k, stride, relu, gen, device, summand=None):
        self.name, self.cin, self.cout, self.k, self.stride, self.relu, self.summand = name, cin, cout, k, stride, relu, summand
        w = torch.randn((k, k, cin, cout), generator=gen, device=device) * math.sqrt(2.0 / (k * k * cin))
        self.w_f32 = w
        self.filter, self.min_filter, self.max_filter = _quantize_filter_per_channel(w)
        self.bias = (torch.randn(cout, generator=gen, device=device) * 0.1).contiguous()
        self.out_type = "quint8" if relu else "qint8"
        self.min_out, self.max_out = 0.0, 1.0          # frozen by calibrate()
        if summand is None:
            op_name = "_ITEXQuantizedConv2DWithBiasAndReluAndRequantize" if relu else "_ITEXQuantizedConv2DWithBiasAndRequantize"
        else:
            op_name = None                             # chosen at run time from the summand's type (u8: Sum, s8: SignedSum)
        self.op_name = op_name
        self._ops = {}

    def _op(self, op_name, in_dtype):
        key = (op_name, in_dtype)
        if key not in self._ops:
            self._ops[key] = ops.Op(op_name, Tinput=in_dtype, Tfilter="qint8", Tbias="float", out_type=self.out_type,
                                    strides=[1, self.stride, self.stride, 1], padding="SAME", dilations=[1, 1, 1, 1],
                                    data_format="NHWC", is_filter_const=True, is_bias_const=True)
        return self._ops[key]

    def __call__(self, x, min_x, max_x, summand=None, min_s=None, max_s=None):
        args = [x, self.filter, self.bias, min_x, max_x, self.min_filter, self.max_filter, self.min_out, self.max_out]
        if summand is None:
            return self._op(self.op_name, x.dtype)(*args)
        name = ("_ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize" if summand.dtype == torch.uint8
                else "_ITEXQuantizedConv2DWithBiasSignedSumAndReluAndRequantize")
        return self._op(name, x.dtype)(*args, summand, min_s, max_s)


def _deq(q, mn, mx):
    """SCALED dequantize in torch (calibration helper only)."""
    lim = 255.0 if q.dtype == torch.uint8 else 127.0
    return q.float() * (max(abs(mn), abs(mx)) / lim)


class ResNet50Int8:
    def __init__(self, device="cuda", seed=1237, num_classes=1000):
        self.device = torch.device(device)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        self.stem = ConvNode("conv1", 3, 64, 7, 2, True, gen, self.device)
        self.blocks = []
        cin = 64
        for si, (width, nblocks, stride) in enumerate(STAGES):
            for bi in range(nblocks):
                s = stride if bi == 0 else 1
                pre = "res%d_%d" % (si + 2, bi)
                proj = ConvNode(pre + "_proj", cin, 4 * width, 1, s, False, gen, self.device) if bi == 0 else None
                c1 = ConvNode(pre + "_a", cin, width, 1, 1, True, gen, self.device)
                c2 = ConvNode(pre + "_b", width, width, 3, s, True, gen, self.device)
                c3 = ConvNode(pre + "_c", width, 4 * width, 1, 1, True, gen, self.device, summand=True)
                self.blocks.append((proj, c1, c2, c3))
                cin = 4 * width
        self.maxpool = ops.Op("_ITEXQuantizedMaxPool", T="quint8", ksize=[1, 3, 3, 1], strides=[1, 2, 2, 1], padding="SAME")
        self._avgpools = {}
        fc = torch.randn((2048, num_classes), generator=gen, device=self.device) * math.sqrt(1.0 / 2048)
        amax = float(fc.abs().max())
        self.fc_w = torch.clamp(torch.round(fc * (127.0 / amax)), -127, 127).to(torch.int8).contiguous()
        self.fc_range = (-amax, amax)
        self.fc_b = (torch.randn(num_classes, generator=gen, device=self.device) * 0.1).contiguous()
        self.fc = ops.Op("_ITEXQuantizedMatMulWithBiasAndDequantize", T1="quint8", T2="qint8", Tbias="float", Toutput="float",
                         input_quant_mode="SCALED", is_weight_const=True, _scaled_bias_mode="intended")
        self.input_range = (0.0, 255.0)   # the uint8 image is its own quantized form
        self.calibrated = False

    def conv_nodes(self):
        yield self.stem
        for proj, c1, c2, c3 in self.blocks:
            for n in (proj, c1, c2, c3):
                if n is not None:
                    yield n

    def macs_per_image(self, image=224):
        """Multiply-accumulates of one forward pass (convolutions + the final matmul), from the layer table."""
        total, h = 0, image
        h = (h + 1) // 2
        total += h * h * 7 * 7 * 3 * 64
        h = (h + 1) // 2
        cin = 64
        for width, nblocks, stride in STAGES:
            for bi in range(nblocks):
                s = stride if bi == 0 else 1
                ho = (h + s - 1) // s
                if bi == 0:
                    total += ho * ho * cin * 4 * width
                total += h * h * cin * width + ho * ho * 9 * width * width + ho * ho * width * 4 * width
                h, cin = ho, 4 * width
        return total + 2048 * self.fc_w.shape[1]

    def _avgpool(self, hw):
        if hw not in self._avgpools:
            self._avgpools[hw] = ops.Op("_ITEXQuantizedAvgPool", T="quint8", ksize=[1, hw, hw, 1], strides=[1, hw, hw, 1], padding="VALID")
        return self._avgpools[hw]

    def _ref_conv(self, node, xf, summand_f=None):
        """fp32 reference of one node on dequantized operands (calibration only)."""
        scale = torch.from_numpy(node.max_filter).to(self.device) / 127.0
        wf = node.filter.float() * scale
        k, s = node.k, node.stride
        h, w = xf.shape[1], xf.shape[2]
        oh, ow = (h + s - 1) // s, (w + s - 1) // s
        ph, pw = max(0, (oh - 1) * s + k - h), max(0, (ow - 1) * s + k - w)
        xp = torch.nn.functional.pad(xf.permute(0, 3, 1, 2), (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2))
        y = torch.nn.functional.conv2d(xp, wf.permute(3, 2, 0, 1), node.bias, stride=s).permute(0, 2, 3, 1)
        if summand_f is not None:
            y = y + summand_f
        return torch.relu(y) if node.relu else y

    def forward(self, x, calibrate=False, trace=None):
        """x: uint8 NHWC images on the device -> fp32 logits.  With calibrate=True each node's output range
        is set from the 99.9th percentile of its fp32 reference before the node runs, then frozen."""
        def run(node, q, mn, mx, sm=None, smn=None, smx=None):
            if calibrate:
                ref = self._ref_conv(node, _deq(q, mn, mx), None if sm is None else _deq(sm, smn, smx))
                flat = ref.abs().flatten()
                if flat.numel() > 4_000_000:
                    flat = flat[:: flat.numel() // 4_000_000 + 1]
                hi = max(float(torch.quantile(flat, 0.999)), 1e-3)
                node.min_out, node.max_out = (0.0, hi) if node.relu else (-hi, hi)
            out = node(q, mn, mx, sm, smn, smx)
            if trace is not None:
                trace.append((node, (q, mn, mx, sm, smn, smx), out))
            return out
        q, mn, mx = run(self.stem, x, *self.input_range)
        q, mn, mx = self.maxpool(q, mn, mx)
        if trace is not None:
            trace.append(("maxpool", None, (q, mn, mx)))
        for proj, c1, c2, c3 in self.blocks:
            if proj is not None:
                s, smn, smx = run(proj, q, mn, mx)
            else:
                s, smn, smx = q, mn, mx
            a, amn, amx = run(c1, q, mn, mx)
            b, bmn, bmx = run(c2, a, amn, amx)
            q, mn, mx = run(c3, b, bmn, bmx, s, smn, smx)
        pooled, pmn, pmx = self._avgpool(q.shape[1])(q, mn, mx)
        if trace is not None:
            trace.append(("avgpool", (q, mn, mx), (pooled, pmn, pmx)))
        feat = pooled.reshape(pooled.shape[0], -1)
        logits = self.fc(feat, self.fc_w, self.fc_b, pmn, pmx, self.fc_range[0], self.fc_range[1], 0.0, 0.0)
        if trace is not None:
            trace.append(("fc", (feat, pmn, pmx), logits))
        if calibrate:
            self.calibrated = True
        return logits

    def capture(self, x_static):
        """Records forward(x_static) in a CUDA graph after a warm-up run; returns (graph, static logits).
        Replaying the graph removes the per-node host work (about sixty launches per batch)."""
        assert self.calibrated, "calibrate first: ranges are host scalars baked into the captured launches"
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(2):
                self.forward(x_static)
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self.forward(x_static)
        return g, out
