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
