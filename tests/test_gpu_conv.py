"""GPU parity of _ITEXQuantizedConv2DWithBias[AndRelu]AndRequantize (+ Sum variants)."""
import os

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import dev, host, modules

pytestmark = pytest.mark.gpu


def _filter(rng, kh, kw, c, co, std=0.05):
    f = (rng.standard_normal((kh, kw, c, co)) * std).astype(np.float32)
    amax = np.abs(f).reshape(-1, co).max(axis=0).astype(np.float32)
    q = np.clip(np.rint(f * (127.0 / amax)), -127, 127).astype(np.int8)
    return f, q, -amax, amax


def test_against_onednn_fixtures(golden_dir):
    itex, K, ops = modules()
    g = np.load(os.path.join(golden_dir, "onednn_conv.npz"))
    for name in ("c3s1", "c3s2", "c1s1"):
        s = int(g[name + "_stride"])
        out, mn, mx = ops._ITEXQuantizedConv2DWithBiasAndReluAndRequantize(
            dev(g[name + "_x"]), dev(g[name + "_f"]), dev(g[name + "_bias"]), float(g["min_input"]), float(g["max_input"]),
            g[name + "_min_f"], g[name + "_max_f"], float(g["min_out"]), float(g["max_out"]), strides=(1, s, s, 1), padding="SAME")
        np.testing.assert_array_equal(host(out), g[name + "_y_quint8"])
        assert (mn, mx) == (float(g["min_out"]), float(g["max_out"]))


def test_config2_full_size():
    """uint8 NHWC [32,56,56,64] ~U{0..255}, scale 0.05; int8 3x3x64x64 filter N(0,0.05) per-channel; stride 1, SAME;
    fp32 bias; uint8 output with a fixed range.  Bit-exact against the oracle at full size; run twice."""
    itex, K, ops = modules()
    rng = np.random.default_rng(1236)
    x = rng.integers(0, 256, (32, 56, 56, 64), dtype=np.uint8)
    f32, qf, mnf, mxf = _filter(rng, 3, 3, 64, 64)
    bias = (rng.standard_normal(64) * 0.1).astype(np.float32)
    mni, mxi = 0.0, 0.05 * 255
    mno, mxo = 0.0, 28.5  # 99.9th percentile of the fp32 conv+bias+relu output for this seed, fixed
    ref, _, _ = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf, mxf, mno, mxo, out_type="quint8", relu=True)
    assert 0.0002 < (ref == 255).mean() < 0.005 and (ref > 0).mean() > 0.3  # the range is neither slack nor saturated
    X, F, B = dev(x), dev(qf), dev(bias)
    for _ in range(2):
        out, mn, mx = ops._ITEXQuantizedConv2DWithBiasAndReluAndRequantize(X, F, B, mni, mxi, mnf, mxf, mno, mxo)
        np.testing.assert_array_equal(host(out), ref)
        assert (mn, mx) == (mno, mxo)


@pytest.mark.parametrize("case", [
    # n, h, w, c, kh, kw, co, stride, padding
    (1, 6, 6, 4, 3, 3, 4, 1, "SAME"),        # the reference's native_quantized_conv_test shape
    (2, 13, 9, 16, 3, 3, 40, 2, "SAME"),
    (2, 14, 14, 32, 1, 1, 64, 1, "VALID"),   # pointwise: no staging
    (2, 14, 14, 32, 1, 1, 24, 2, "SAME"),    # strided projection shortcut
    (1, 23, 23, 3, 7, 7, 64, 2, "SAME"),     # ResNet stem: 3 channels padded to 16
    (3, 8, 8, 128, 3, 3, 136, 1, "VALID"),
    (1, 5, 5, 48, 5, 5, 16, 1, "SAME"),
])
@pytest.mark.parametrize("tin", ["quint8", "qint8"])
def test_shapes_strides_paddings(case, tin):
    itex, K, ops = modules()
    n, h, w, c, kh, kw, co, s, padding = case
    rng = np.random.default_rng(sum(case[:8]))
    x = rng.integers(0, 256, (n, h, w, c)).astype(np.uint8) if tin == "quint8" else rng.integers(-128, 128, (n, h, w, c)).astype(np.int8)
    f32, qf, mnf, mxf = _filter(rng, kh, kw, c, co)
    bias = (rng.standard_normal(co) * 0.1).astype(np.float32)
    bias32 = rng.integers(-3000, 3000, co).astype(np.int32)
    mni, mxi, mno, mxo = (0.0, 12.75, 0.0, 6.0) if tin == "quint8" else (-6.4, 6.35, 0.0, 6.0)
    for bvec, tbias in ((bias, "float"), (bias32, "qint32")):
        out, mn, mx = ops._ITEXQuantizedConv2DWithBiasAndReluAndRequantize(
            dev(x), dev(qf), dev(bvec), mni, mxi, mnf, mxf, mno, mxo, strides=(1, s, s, 1), padding=padding)
        ref, _, _ = o.quantized_conv2d(x, qf, bvec, mni, mxi, mnf, mxf, mno, mxo, strides=(1, s, s, 1), padding=padding,
                                       out_type="quint8", relu=True, tbias=tbias)
        assert tuple(out.shape) == ref.shape
        np.testing.assert_array_equal(host(out), ref)
    # no ReLU, signed output, per-tensor filter range
    out, _, _ = ops._ITEXQuantizedConv2DWithBiasAndReluAndRequantize(
        dev(x), dev(qf), dev(bias), mni, mxi, float(mnf.min()), float(mxf.max()), -6.0, 6.0, strides=(1, s, s, 1), padding=padding,
        out_type="qint8", op_name="_ITEXQuantizedConv2DWithBiasAndRequantize")
    ref, _, _ = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf.min(), mxf.max(), -6.0, 6.0, strides=(1, s, s, 1), padding=padding,
                                   out_type="qint8", relu=False)
    np.testing.assert_array_equal(host(out), ref)


def test_sum_fused_variants():
    """conv + bias + sum + relu + requantize with u8 and s8 summands (sum scale rule, quantized_conv_ops.h:398-434)."""
    itex, K, ops = modules()
    rng = np.random.default_rng(77)
    x = rng.integers(0, 256, (2, 10, 10, 32), dtype=np.uint8)
    f32, qf, mnf, mxf = _filter(rng, 3, 3, 32, 48)
    bias = (rng.standard_normal(48) * 0.1).astype(np.float32)
    for sdt, name in ((np.uint8, "_ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize"),
                      (np.int8, "_ITEXQuantizedConv2DWithBiasSignedSumAndReluAndRequantize")):
        summ = rng.integers(0, 200, (2, 10, 10, 48)).astype(sdt) if sdt == np.uint8 else rng.integers(-100, 100, (2, 10, 10, 48)).astype(sdt)
        out, mn, mx = ops._ITEXQuantizedConv2DWithBiasAndReluAndRequantize(
            dev(x), dev(qf), dev(bias), 0.0, 12.75, mnf, mxf, 0.0, 8.0, summand=dev(summ), min_summand=0.0 if sdt == np.uint8 else -5.0,
            max_summand=5.0, op_name=name)
        ref, _, _ = o.quantized_conv2d(x, qf, bias, 0.0, 12.75, mnf, mxf, 0.0, 8.0, out_type="quint8", relu=True, summand=summ,
                                       min_summand=0.0 if sdt == np.uint8 else -5.0, max_summand=5.0)
        np.testing.assert_array_equal(host(out), ref)


def test_reference_style_vs_fp32():
    """native_quantized_conv_test.py:33-198 pattern: compare the dequantized result with the fp32 conv at 0.3."""
    itex, K, ops = modules()
    rng = np.random.default_rng(7)
    x = rng.uniform(0, 1, (1, 6, 6, 4)).astype(np.float32)
    w = rng.uniform(-1, 1, (3, 3, 4, 4)).astype(np.float32)
    b = rng.uniform(-1, 1, 4).astype(np.float32)
    qx, xmin, xmax = ops._ITEXQuantizeV2(dev(x), float(x.min()), float(x.max()), T="quint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    qw, wmin, wmax = ops._ITEXQuantizeV2(dev(w), float(w.min()), float(w.max()), T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    xt = torch.from_numpy(x).permute(0, 3, 1, 2)
    wt = torch.from_numpy(w).permute(3, 2, 0, 1)
    f = torch.relu(torch.nn.functional.conv2d(xt, wt, torch.from_numpy(b), padding=1)).permute(0, 2, 3, 1).numpy()
    out, mn, mx = ops._ITEXQuantizedConv2DWithBiasAndReluAndRequantize(qx, qw, dev(b), xmin, xmax, wmin, wmax, float(f.min()), float(f.max()))
    deq = ops._ITEXDequantize(out, mn, mx, mode="SCALED")
    np.testing.assert_allclose(host(deq), f, rtol=0.3, atol=0.3)


def test_conv_argument_errors():
    itex, K, ops = modules()
    x = torch.zeros((1, 4, 4, 8), dtype=torch.uint8, device="cuda")
    f = torch.zeros((3, 3, 16, 8), dtype=torch.int8, device="cuda")
    b = torch.zeros(8, device="cuda")
    with pytest.raises(itex.ItexError) as e:
        ops._ITEXQuantizedConv2DWithBiasAndReluAndRequantize(x, f, b, 0.0, 1.0, -1.0, 1.0, 0.0, 1.0)
    assert "input and filter must have the same depth" in str(e.value)


def _abi_conv(itex, x, f, scale, bias, stride, dil, pad, oh, ow, c_pad, out_dtype=None):
    """One convolution through the C-ABI with the packed filter's tap pitch chosen by the caller."""
    import ctypes as C
    lib, L = itex.load(), itex._lib
    n, h, w, c = x.shape
    kh, kw, _, co = f.shape
    p = L.ConvParams()
    p.n, p.h, p.w, p.c, p.kh, p.kw, p.co = n, h, w, c, kh, kw, co
    p.stride_h = p.stride_w = stride
    p.dil_h = p.dil_w = dil
    p.pad_top = p.pad_left = pad
    p.oh, p.ow = oh, ow
    if c_pad == "preferred":
        c_pad = lib.itexb_conv2d_filter_c_pad(C.byref(p))
    p.c_pad = c_pad
    p.x_dtype, p.out_dtype = L.DT_QUINT8, L.DT_QUINT8
    fpk = torch.empty((co, (kh * kw * c_pad + 15) // 16 * 16), dtype=torch.int8, device="cuda")
    out = torch.full((n, oh, ow, co), 99, dtype=torch.uint8, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    L.check(lib.itexb_pack_filter_hwio(C.c_void_p(f.data_ptr()), C.c_void_p(fpk.data_ptr()), kh, kw, c, co, c_pad, stream))
    p.x, p.filter_packed, p.out = x.data_ptr(), fpk.data_ptr(), out.data_ptr()
    p.ep.scale, p.ep.scale_count, p.ep.bias, p.ep.relu = scale.data_ptr(), co, bias.data_ptr(), 1
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p.status_word = status.data_ptr()
    ws_bytes = lib.itexb_conv2d_workspace_bytes(C.byref(p))
    ws = torch.empty(max(1, ws_bytes), dtype=torch.uint8, device="cuda")
    p.workspace = ws.data_ptr()
    L.check(lib.itexb_conv2d(C.byref(p), stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return host(out), c_pad, ws_bytes


@pytest.mark.parametrize("case", [
    # n, h, w, c, k, co, stride, dilation
    (2, 14, 14, 64, 3, 64, 1, 1),      # c = 64: the TMA im2col path runs 64-byte k-blocks (one tap each, 64-byte swizzle)
    (3, 9, 11, 32, 3, 40, 2, 1),       # ragged: 3*5*6 = 90 pixels in one tile, stride 2, odd sizes; 32-byte k-blocks
    (2, 10, 13, 48, 3, 72, 1, 1),      # c = 48: taps padded to 64 channels, each box a quarter outside the tensor
    (2, 17, 17, 128, 3, 96, 1, 2),     # dilation 2
    (2, 12, 12, 192, 3, 272, 2, 1),    # c = 128 + 64: second k-block of a tap is half outside the tensor
    (1, 7, 7, 256, 1, 64, 2, 1),       # strided 1x1 (projection shortcut)
    (5, 20, 20, 16, 5, 24, 1, 1),      # 5x5, smallest channel run, several tiles per image row group
])
def test_lowerings_agree(case):
    """The three ways the A operand is produced (patch matrix in scratch, cp.async gather inside the GEMM,
    TMA im2col loads) give identical bytes, and those equal the oracle's.  (With c_pad = c the dense-filter run
    takes the cp.async gather unless c is itself a k-block width the im2col path accepts: 32, 64 or a multiple of 128.)"""
    itex, K, ops = modules()
    n, h, w, c, k, co, stride, dil = case
    rng = np.random.default_rng(sum(case))
    eff = (k - 1) * dil + 1
    oh, ow = (h + stride - 1) // stride, (w + stride - 1) // stride
    pad_h = max(0, (oh - 1) * stride + eff - h) // 2
    x = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
    f = rng.integers(-127, 128, (k, k, c, co)).astype(np.int8)
    scale = rng.uniform(2e-5, 6e-5, co).astype(np.float32)
    bias = rng.standard_normal(co).astype(np.float32)
    xd, fd, sd, bd = dev(x), dev(f), dev(scale), dev(bias)
    im2col, c_pad, ws0 = _abi_conv(itex, xd, fd, sd, bd, stride, dil, pad_h, oh, ow, "preferred")
    assert c_pad == (32 if c <= 32 else (64 if c <= 64 else (c + 127) // 128 * 128)) and ws0 == 0
    dense, _, ws1 = _abi_conv(itex, xd, fd, sd, bd, stride, dil, pad_h, oh, ow, c)
    if c % 128 != 0:
        assert ws1 == 0                      # cp.async gather: no scratch either
    # explicit lowering: shift the problem to a channel count that is not a multiple of 16 by appending a zero channel
    x1 = np.concatenate([x, np.zeros((n, h, w, 1), np.uint8)], axis=3)
    f1 = np.concatenate([f, np.zeros((k, k, 1, co), np.int8)], axis=2)
    explicit, _, ws2 = _abi_conv(itex, dev(x1), dev(f1), sd, bd, stride, dil, pad_h, oh, ow, c + 1)
    assert ws2 > 0
    # oracle: int32 accumulation, then scale, bias, relu, saturating round to uint8
    xp = np.pad(x.astype(np.int32), ((0, 0), (pad_h, eff), (pad_h, eff), (0, 0)))
    acc = np.zeros((n, oh, ow, co), np.int64)
    for ky in range(k):
        for kx in range(k):
            patch = xp[:, ky * dil: ky * dil + (oh - 1) * stride + 1: stride, kx * dil: kx * dil + (ow - 1) * stride + 1: stride, :]
            acc += np.tensordot(patch, f[ky, kx].astype(np.int64), axes=([3], [0]))
    v = acc.astype(np.float32) * scale + bias
    want = np.clip(np.rint(np.maximum(v, 0)), 0, 255).astype(np.uint8)
    np.testing.assert_array_equal(im2col, want)
    np.testing.assert_array_equal(dense, want)
    np.testing.assert_array_equal(explicit, want)


@pytest.mark.parametrize("tin", ["quint8", "qint8"])
def test_legacy_family_qint32_and_no_bias(tin):
    """QuantizedConv2D / PerChannel (exact accumulators), WithBias[AndRelu] (qint32 with the bias brought to
    accumulator units), AndRequantize / AndReluAndRequantize (no bias): bit-exact against the oracle, output
    ranges included."""
    itex, K, ops = modules()
    rng = np.random.default_rng(31)
    n, h, w, c, co = 3, 13, 15, 32, 48
    x = rng.integers(0, 256, (n, h, w, c)).astype(np.uint8) if tin == "quint8" else rng.integers(-127, 128, (n, h, w, c)).astype(np.int8)
    f32, qf, mnf, mxf = _filter(rng, 3, 3, c, co)
    bias = (rng.standard_normal(co) * 0.5).astype(np.float32)
    mni, mxi = (0.0, 6.0) if tin == "quint8" else (-3.0, 3.0)
    X, F, B = dev(x), dev(qf), dev(bias)
    kw = dict(strides=(1, 2, 2, 1), padding="SAME")
    # accumulators, per-channel and per-tensor filter ranges
    for name, mn, mx in (("_ITEXQuantizedConv2DPerChannel", mnf, mxf), ("QuantizedConv2D", float(mnf.min()), float(mxf.max()))):
        ref, rmn, rmx = o.quantized_conv2d(x, qf, None, mni, mxi, mn, mx, out_type="qint32", relu=False, strides=(1, 2, 2, 1))
        got, gmn, gmx = ops.QuantizedConv2D(name, X, F, None, mni, mxi, mn, mx, **kw)
        np.testing.assert_array_equal(host(got), ref)
        np.testing.assert_array_equal(np.asarray(gmn), np.asarray(rmn))
        np.testing.assert_array_equal(np.asarray(gmx), np.asarray(rmx))
    for name, relu in (("_ITEXQuantizedConv2DWithBias", False), ("QuantizedConv2DWithBiasAndRelu", True)):
        ref, rmn, rmx = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf, mxf, out_type="qint32", relu=relu, strides=(1, 2, 2, 1))
        got, gmn, gmx = ops.QuantizedConv2D(name, X, F, B, mni, mxi, mnf, mxf, **kw)
        np.testing.assert_array_equal(host(got), ref)
        np.testing.assert_array_equal(gmx, rmx)
    acc, _, _ = o.quantized_conv2d(x, qf, None, mni, mxi, mnf, mxf, out_type="qint32", relu=False, strides=(1, 2, 2, 1))
    real = acc.astype(np.float64) * (max(abs(mni), abs(mxi)) / (255.0 if tin == "quint8" else 127.0)) * (mxf / 127.0)
    hi = float(np.abs(real).max())
    ref, _, _ = o.quantized_conv2d(x, qf, None, mni, mxi, mnf, mxf, -hi, hi, out_type="qint8", relu=False, strides=(1, 2, 2, 1))
    got, gmn, gmx = ops.QuantizedConv2D("_ITEXQuantizedConv2DAndRequantize", X, F, None, mni, mxi, mnf, mxf, -hi, hi, out_type="qint8", **kw)
    np.testing.assert_array_equal(host(got), ref)
    assert (gmn, gmx) == (np.float32(-hi), np.float32(hi))
    ref, _, _ = o.quantized_conv2d(x, qf, None, mni, mxi, mnf, mxf, 0.0, hi, out_type="quint8", relu=True, strides=(1, 2, 2, 1))
    got, _, _ = ops.QuantizedConv2D("QuantizedConv2DAndReluAndRequantize", X, F, None, mni, mxi, mnf, mxf, 0.0, hi, out_type="quint8", **kw)
    np.testing.assert_array_equal(host(got), ref)


def test_remapper_fusions_around_the_requantizing_conv():
    """_ITEXQuantizedConv2DWithDequantize / ...WithCast (a ...WithBiasAndRequantize with its Dequantize or Cast consumer
    folded in: real-valued output, the frozen range inputs kept but unused) and _ITEXQuantizeV2WithQuantizedConv2D
    (a QuantizeV2 folded into the ...WithBiasAndReluAndRequantize it feeds): bit-exact against the oracle, and the
    quantize fusion identical to running the two ops one after the other."""
    itex, K, ops = modules()
    rng = np.random.default_rng(43)
    n, h, w, c, co = 2, 12, 12, 32, 48
    f32, qf, mnf, mxf = _filter(rng, 3, 3, c, co)
    bias = (rng.standard_normal(co) * 0.5).astype(np.float32)
    F, B = dev(qf), dev(bias)
    for tin, (mni, mxi) in (("quint8", (0.0, 6.0)), ("qint8", (-3.0, 3.0))):
        x = rng.integers(0, 256, (n, h, w, c)).astype(np.uint8) if tin == "quint8" else rng.integers(-127, 128, (n, h, w, c)).astype(np.int8)
        for name, tout in (("_ITEXQuantizedConv2DWithDequantize", "float"), ("_ITEXQuantizedConv2DWithDequantize", "bfloat16"),
                           ("_ITEXQuantizedConv2DWithCast", "half")):
            ref, _, _ = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf, mxf, out_type=tout, relu=False, strides=(1, 1, 1, 1))
            got = ops.QuantizedConv2D(name, dev(x), F, B, mni, mxi, mnf, mxf, -7.0, 7.0, out_type=tout, strides=(1, 1, 1, 1))
            assert isinstance(got, torch.Tensor) and got.dtype == {"float": torch.float32, "bfloat16": torch.bfloat16, "half": torch.float16}[tout]
            np.testing.assert_array_equal(host(got), np.asarray(ref, np.float32))
    # quantize + conv
    xf = (rng.standard_normal((n, h, w, c)) * 1.5 + 1.0).astype(np.float32)
    lo, hi = float(xf.min()), float(xf.max())
    ref, rmn, rmx = o.quantize_v2_with_quantized_conv2d(xf, qf, bias, lo, hi, mnf, mxf, 0.0, 9.0, strides=(1, 2, 2, 1))
    got, gmn, gmx = ops.QuantizedConv2D("_ITEXQuantizeV2WithQuantizedConv2D", dev(xf), F, B, lo, hi, mnf, mxf, 0.0, 9.0, out_type="quint8",
                                        strides=(1, 2, 2, 1), mode="SCALED", round_mode="HALF_TO_EVEN")
    np.testing.assert_array_equal(host(got), ref)
    assert (gmn, gmx) == (np.float32(0.0), np.float32(9.0))
    q, qmn, qmx = ops._ITEXQuantizeV2(dev(xf), lo, hi, T="quint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    two, _, _ = ops._ITEXQuantizedConv2DWithBiasAndReluAndRequantize(q, F, B, qmn, qmx, mnf, mxf, 0.0, 9.0, strides=(1, 2, 2, 1))
    assert torch.equal(got, two)
    with pytest.raises(itex.ItexError, match="only mode SCALED"):
        ops.QuantizedConv2D("_ITEXQuantizeV2WithQuantizedConv2D", dev(xf), F, B, lo, hi, mnf, mxf, 0.0, 9.0, out_type="quint8", mode="MIN_FIRST")


def test_new_api_fused_ops():
    """_QuantizedConv2D / _ITEXQuantizedConv2DV2: fusion given by the fused_ops attr, list-typed arguments in the new order
    (summand before the ranges, frozen output range last).  Bit-exact for integer outputs and algebraic post-ops."""
    itex, K, ops = modules()
    rng = np.random.default_rng(41)
    n, h, w, c, co = 2, 14, 14, 64, 64
    x = rng.integers(0, 256, (n, h, w, c)).astype(np.uint8)
    f32, qf, mnf, mxf = _filter(rng, 3, 3, c, co)
    bias = (rng.standard_normal(co) * 0.5).astype(np.float32)
    mni, mxi = 0.0, 5.1
    X, F, B = dev(x), dev(qf), dev(bias)
    rng4 = [mni, mxi, mnf, mxf]
    # Dequantize: real-valued output, no ranges
    for tout in ("float", "bfloat16"):
        ref, _, _ = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf, mxf, out_type=tout, relu=False)
        got = ops._QuantizedConv2D([X, F, B], rng4, fused_ops=["BiasAdd", "Dequantize"], out_type=tout)
        np.testing.assert_array_equal(host(got), ref.astype(np.float32))
    real, _, _ = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf, mxf, out_type="float", relu=False)
    hi = float(np.abs(real).max())
    # Relu + Requantize = the legacy op
    ref, _, _ = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf, mxf, 0.0, hi, out_type="quint8", relu=True)
    got, gmn, gmx = ops._QuantizedConv2D([X, F, B], rng4 + [0.0, hi], fused_ops=["BiasAdd", "Relu", "Requantize"], out_type="quint8",
                                         op_name="_ITEXQuantizedConv2DV2")
    np.testing.assert_array_equal(host(got), ref)
    assert (gmn, gmx) == (np.float32(0.0), np.float32(hi))
    # LeakyRelu + Requantize to qint8
    ref, _, _ = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf, mxf, -hi, hi, out_type="qint8", relu=False, activation_name="LeakyRelu", alpha=0.25)
    got, _, _ = ops._QuantizedConv2D([X, F, B], rng4 + [-hi, hi], fused_ops=["BiasAdd", "LeakyRelu", "Requantize"], out_type="qint8", alpha=0.25)
    np.testing.assert_array_equal(host(got), ref)
    # Sum + Relu + Requantize: summand right after the bias, its range before the frozen output range
    sq = rng.integers(0, 256, ref.shape).astype(np.uint8)
    ref, _, _ = o.quantized_conv2d(x, qf, bias, mni, mxi, mnf, mxf, 0.0, hi, out_type="quint8", relu=True, summand=sq, min_summand=0.0,
                                   max_summand=hi * 0.5)
    got, _, _ = ops._QuantizedConv2D([X, F, B, dev(sq)], rng4 + [0.0, hi * 0.5, 0.0, hi], fused_ops=["BiasAdd", "Sum", "Relu", "Requantize"],
                                     out_type="quint8", Tsummand="quint8")
    np.testing.assert_array_equal(host(got), ref)
    # nothing fused: accumulators and their per-channel ranges
    ref, rmn, rmx = o.quantized_conv2d(x, qf, None, mni, mxi, mnf, mxf, out_type="qint32", relu=False)
    got, gmn, gmx = ops._QuantizedConv2D([X, F], rng4, fused_ops=[], out_type="qint32")
    np.testing.assert_array_equal(host(got), ref)
    np.testing.assert_array_equal(gmx, rmx)
    with pytest.raises(itex._lib.ItexError) as e:
        ops._QuantizedConv2D([X, F, B], rng4, fused_ops=["BiasAdd", "Mish"], out_type="qint32")
    assert "unsupported fusion" in str(e.value)


def test_sum_post_op_matches_real_onednn_on_rounding_ties(golden_dir):
    """_ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize on the real-oneDNN fixture whose pixels sit on rounding ties of
    the sum post-op: the device epilogue (one fused multiply-add for the summand) gives oneDNN's bytes."""
    import os
    itex, K, ops = modules()
    d = np.load(os.path.join(golden_dir, "onednn_conv_sum.npz"))
    op = ops.Op("_ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize", Tinput="quint8", Tfilter="qint8", Tbias="float", out_type="quint8",
                strides=[1, 1, 1, 1], padding="SAME", dilations=[1, 1, 1, 1], data_format="NHWC")
    out, mn, mx = op(dev(d["x"]), dev(d["f"]), dev(d["bias"]), float(d["min_input"]), float(d["max_input"]), d["min_f"], d["max_f"],
                     float(d["min_out"]), float(d["max_out"]), dev(d["summand"]), float(d["min_summand"]), float(d["max_summand"]))
    np.testing.assert_array_equal(host(out), d["y"])
