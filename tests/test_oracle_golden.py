"""Pins the CPU oracle: the reference's own known-answer tests (transcribed into
tests/golden/reference_kat.json) and real-oneDNN outputs (tests/golden/onednn_*.npz)."""
import json
import os

import numpy as np
import pytest

import itex_oracle as o


@pytest.fixture(scope="module")
def kat(golden_dir):
    with open(os.path.join(golden_dir, "reference_kat.json")) as f:
        return json.load(f)


def scale_per_slice(shape, axis, values):
    out = np.take(values, np.remainder(np.arange(np.prod(shape)), len(values))).reshape(shape)
    if axis is not None:
        ss = [1] * len(shape)
        ss[axis] = shape[axis]
        out = out * np.arange(1, shape[axis] + 1).reshape(ss)
    return out


def test_quantize_axis_exact(kat):
    k = kat["quantize_axis"]
    shape = np.array(k["shape"])
    values = np.array(k["values"], np.float32)
    expected = scale_per_slice(shape, None, np.array(k["quant_values"], np.int32))
    for axis in k["axes"]:
        x = scale_per_slice(shape, axis, values).astype(np.float32)
        if axis is None:
            mn, mx = k["min_per_slice"], k["max_per_slice"]
            axes = [-1]
        else:
            mn = [k["min_per_slice"] * (i + 1) for i in range(shape[axis])]
            mx = [k["max_per_slice"] * (i + 1) for i in range(shape[axis])]
            axes = [axis]
        for ax in axes:
            q, omin, omax = o.quantize_v2(x, mn, mx, T=k["T"], mode=k["mode"], round_mode=k["round_mode"],
                                          narrow_range=k["narrow_range"], axis=ax)
            assert q.dtype == np.int8
            np.testing.assert_array_equal(q.astype(np.int32), expected)
            np.testing.assert_allclose(np.asarray(omax), np.abs(mn))  # |min| = 1.0*(i+1) dominates


def test_quantize_min_first_variants(kat):
    for name, kwargs in (("quantize_min_first", {}), ("quantize_asymmetric_legacy", {}),
                         ("quantize_asymmetric_classic", {"classic_asymmetric_algorithm": True})):
        k = kat[name]
        q, _, _ = o.quantize_v2(np.array(k["x"], np.float32), k["min"], k["max"], T=k["T"], mode="MIN_FIRST",
                                round_mode="HALF_AWAY_FROM_ZERO", **kwargs)
        np.testing.assert_allclose(q.astype(np.float32), k["expected"], atol=k["atol"])
    # bf16 input takes the same path (quantized_ops_test.py:70-90)
    k = kat["quantize_min_first"]
    q, _, _ = o.quantize_v2(o.to_bf16_rne(np.array(k["x"], np.float32)), k["min"], k["max"], T=k["T"],
                            mode="MIN_FIRST", round_mode="HALF_AWAY_FROM_ZERO")
    np.testing.assert_allclose(q.astype(np.float32), k["expected"], atol=k["atol"])


def test_dequantize_axis(kat):
    k = kat["dequantize_axis"]
    shape = np.array(k["shape"])
    q = scale_per_slice(shape, None, np.array(k["values"], np.int32)).astype(np.int8)
    for axis in k["axes"]:
        expected = scale_per_slice(shape, axis, np.array(k["dequant_values"], np.float32))
        if axis is None:
            mn, mx, ax = k["min_per_slice"], k["max_per_slice"], -1
        else:
            mn = [k["min_per_slice"] * (i + 1) for i in range(shape[axis])]
            mx = [k["max_per_slice"] * (i + 1) for i in range(shape[axis])]
            ax = axis
        y = o.dequantize(q, mn, mx, T=k["T"], mode=k["mode"], narrow_range=True, axis=ax)
        np.testing.assert_allclose(y, expected, rtol=k["rtol"], atol=k["atol"])


def test_dequantize_scaled_closed_form(kat):
    k = kat["dequantize_scaled"]
    for c in k["cases"]:
        for narrow in (False, True):
            q = np.array(c["q"], np.int8)
            vmin = -127 if narrow else -128
            sf = max(c["min"] / vmin, c["max"] / 127)
            y = o.dequantize(q, c["min"], c["max"], T=k["T"], narrow_range=narrow)
            np.testing.assert_allclose(y, q.astype(np.float32) * sf, rtol=k["rtol"], atol=k["atol"])
    k = kat["dequantize_min_first"]
    y = o.dequantize(np.array(k["q"], np.uint8), k["min"], k["max"], T=k["T"], mode="MIN_FIRST")
    np.testing.assert_allclose(y, k["expected"], atol=k["atol"])


def _matmul_case(kat):
    k = kat["matmul_min_first"]
    x = np.array(k["x_f32"], np.float32)
    y = np.array(k["y_f32"], np.float32)
    b = np.array(k["bias_f32"], np.float32)
    qx, xmin, xmax = o.quantize_v2(x, x.min(), x.max(), T="quint8", mode="MIN_FIRST",
                                   round_mode="HALF_AWAY_FROM_ZERO")
    qy, ymin, ymax = o.quantize_v2(y, y.min(), y.max(), T="qint8", mode="SCALED", narrow_range=True)
    return k, x, y, b, qx, xmin, xmax, qy, ymin, ymax


def test_matmul_reference_sanity_cases(kat):
    """quantized_matmul_op_test.py: the four QuantizedMatMulWithBias* ops vs fp32 math at 0.2."""
    k, x, y, b, qx, xmin, xmax, qy, ymin, ymax = _matmul_case(kat)
    tol = dict(rtol=k["rtol"], atol=k["atol"])
    f = x @ y + b
    # ...AndReluAndRequantize
    fr = np.maximum(f, 0)
    out, mn, mx = o.quantized_matmul_with_bias(qx, qy, b, xmin, xmax, ymin, ymax, fr.min(), fr.max(),
                                               toutput="quint8", relu=True)
    np.testing.assert_allclose(o.dequantize(out, mn, mx, T="quint8", narrow_range=True), fr, **tol)
    # ...AndDequantize
    out, _, _ = o.quantized_matmul_with_bias(qx, qy, b, xmin, xmax, ymin, ymax, f.min(), f.max(), toutput="float")
    np.testing.assert_allclose(out, f, **tol)
    # WithBias / WithBiasAndRelu -> qint32; dequantize linearly over [min_out, max_out]
    for relu in (False, True):
        out, mn, mx = o.quantized_matmul_with_bias(qx, qy, b, xmin, xmax, ymin, ymax, toutput="qint32", relu=relu)
        deq = out.astype(np.float64) * (float(mx) / (2 ** 31 - 1))
        np.testing.assert_allclose(deq, np.maximum(f, 0) if relu else f, **tol)


def test_matmul_against_onednn(golden_dir):
    g = np.load(os.path.join(golden_dir, "onednn_matmul.npz"))
    n_exact = 0
    for tout in ("float", "quint8", "bfloat16"):
        for mode in ("SCALED", "MIN_FIRST"):
            for sbm in ("literal", "intended"):
                for relu in (0, 1):
                    ref = g["y_%s_%s_%s_%d" % (tout, mode, sbm, relu)]
                    out, _, _ = o.quantized_matmul_with_bias(
                        g["a"], g["b"], g["bias"], g["min_a"], g["max_a"], g["min_b"], g["max_b"],
                        g["min_freezed"], g["max_freezed"], toutput=tout, relu=bool(relu),
                        input_quant_mode=mode, scaled_bias_mode=sbm)
                    if tout == "quint8":
                        np.testing.assert_array_equal(out, ref)
                    else:
                        np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-6)
                    n_exact += int(np.array_equal(out, ref))
    assert n_exact >= 16  # the restated epilogue order reproduces oneDNN bit for bit on most cases


def test_conv_against_onednn(golden_dir):
    g = np.load(os.path.join(golden_dir, "onednn_conv.npz"))
    for name in ("c3s1", "c3s2", "c1s1"):
        s = int(g[name + "_stride"])
        for tout in ("quint8", "float"):
            out, mn, mx = o.quantized_conv2d(
                g[name + "_x"], g[name + "_f"], g[name + "_bias"], g["min_input"], g["max_input"],
                g[name + "_min_f"], g[name + "_max_f"], g["min_out"], g["max_out"],
                strides=(1, s, s, 1), padding="SAME", out_type=tout, relu=True)
            ref = g["%s_y_%s" % (name, tout)]
            assert out.shape == ref.shape
            if tout == "quint8":
                np.testing.assert_array_equal(out, ref)
                assert mn == g["min_out"] and mx == g["max_out"]
            else:
                np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-6)


def test_conv_sum_post_op_against_onednn(golden_dir):
    """The residual-sum convolution against real oneDNN on pixels chosen to sit on rounding ties: the restated tail
    (scale and bias as separate roundings, the sum post-op as ONE fused multiply-add) reproduces oneDNN on all of them;
    the model with a separately rounded product does not, which is what the fixture is for."""
    d = np.load(os.path.join(golden_dir, "onednn_conv_sum.npz"))
    kw = dict(out_type="quint8", relu=True, summand=d["summand"], min_summand=d["min_summand"], max_summand=d["max_summand"])
    out, _, _ = o.quantized_conv2d(d["x"], d["f"], d["bias"], d["min_input"], d["max_input"], d["min_f"], d["max_f"], d["min_out"], d["max_out"], **kw)
    np.testing.assert_array_equal(out, d["y"])
    # the two-rounding model, spelled out: it must differ on every tie pixel
    acc = o.int_conv2d_nhwc(d["x"], d["f"])
    sc = o.conv_output_scale(d["min_input"], d["max_input"], d["min_f"], d["max_f"], "quint8", "quint8", d["min_out"], d["max_out"])
    b = o.conv_scaled_bias(d["bias"], d["min_input"], d["max_input"], d["min_f"], d["max_f"], "quint8", "quint8", sc)
    f = (acc.astype(np.float32) * sc + b).astype(np.float32)
    ss = np.float32(d["max_summand"] / d["max_out"])
    two = o.sat_rne(np.maximum((f + (ss * d["summand"].astype(np.float32)).astype(np.float32)).astype(np.float32), 0), "quint8")
    ties = int(d["n_tie_pixels"])
    assert ((two != d["y"]).any(axis=3)[0, 0, :ties]).all() and not (two != d["y"])[0, 0, ties:].any()


def test_conv_reference_style_vs_fp32():
    """native_quantized_conv_test.py:33-198 pattern: random 1x6x6x4 . 3x3x4x4, SAME, SCALED
    inputs, compared with the fp32 convolution at rtol=atol=0.3."""
    rng = np.random.default_rng(7)
    x = rng.uniform(0, 1, (1, 6, 6, 4)).astype(np.float32)
    w = rng.uniform(-1, 1, (3, 3, 4, 4)).astype(np.float32)
    b = rng.uniform(-1, 1, 4).astype(np.float32)
    qx, xmin, xmax = o.quantize_v2(x, x.min(), x.max(), T="quint8")
    qw, wmin, wmax = o.quantize_v2(w, w.min(), w.max(), T="qint8")
    xp = np.zeros((1, 8, 8, 4), np.float32)
    xp[:, 1:7, 1:7] = x
    f = np.zeros((1, 6, 6, 4), np.float32)
    for i in range(3):
        for j in range(3):
            f += np.tensordot(xp[:, i:i + 6, j:j + 6], w[i, j], axes=([3], [0]))
    f = np.maximum(f + b, 0)
    out, mn, mx = o.quantized_conv2d(qx, qw, b, xmin, xmax, wmin, wmax, f.min(), f.max(), out_type="quint8")
    np.testing.assert_allclose(o.dequantize(out, mn, mx, T="quint8"), f, rtol=0.3, atol=0.3)


def test_fp8_cast_and_delayed_scaling():
    # saturation and RNE on e4m3 (float8.h kSaturate=true): 448 is max, 464 is the tie to 448|480(sat)
    v = np.array([0.0, 1.0, 447.0, 448.0, 460.0, 1e9, -1e9, 0.0625 + 0.0078125 / 2], np.float32)
    back = o.fp8_to_f32(o.fp8_cast_sat(v))
    assert back[3] == 448 and back[4] == 448 and back[5] == 448 and back[6] == -448
    hist = np.zeros((16, 3), np.float32)
    scale = np.ones(3, np.float32)
    hist[0] = [3.7, 0.0, 1000.0]
    nh, sf, sfi = o.fp8_amax_and_scale_update(hist, scale)
    # 448/3.7=121.08 -> 2^6; amax 0 keeps the old scale; 448/1000 -> exp=-2 -> 1/4
    np.testing.assert_array_equal(sf, [64.0, 1.0, 0.25])
    np.testing.assert_array_equal(sfi, [1 / 64.0, 1.0, 4.0])
    assert (nh[0] == 0).all() and (nh[15] == hist[0]).all()


def test_fused_matmul_reference_cases(kat):
    """native_quantized_fused_matmul_test.py: _QuantizedFusedMatMulAndDequantize / _QuantizedMatMul with
    BiasAdd + GeluApproximate (per-tensor and per-channel weights) and BiasAdd + Add, vs fp32 math at 0.2."""
    k = kat["fused_matmul_min_first"]
    x = np.array(k["x_f32"], np.float32)
    y = np.array(k["y_f32"], np.float32)
    b = np.array(k["bias_f32"], np.float32)
    z = np.array(k["z_f32"], np.float32) * 2
    qx, xmin, xmax = o.quantize_v2(x, x.min(), x.max(), T="quint8", mode="MIN_FIRST", round_mode="HALF_AWAY_FROM_ZERO")
    tol = dict(rtol=k["rtol"], atol=k["atol"])
    for case in k["cases"]:
        if case["per_channel"]:
            qy, ymin, ymax = o.quantize_v2(y, y.min(axis=0), y.max(axis=0), T="qint8", mode="SCALED", narrow_range=True, axis=1)
        else:
            qy, ymin, ymax = o.quantize_v2(y, y.min(), y.max(), T="qint8", mode="SCALED", narrow_range=True)
        f = x @ y + b
        if "Add" in case["fused_ops"]:
            want = f + z
        else:
            want = o.activation(f, "GeluApproximate")
        out, _, _ = o.quantized_fused_matmul(qx, qy, b, xmin, xmax, ymin, ymax, fused_ops=case["fused_ops"], t1="quint8",
                                             toutput="float", input_quant_mode="MIN_FIRST", addend=z)
        np.testing.assert_allclose(out, want, **tol)
        # V2 spelling of the same fusion
        out2, _, _ = o.quantized_fused_matmul(qx, qy, b, xmin, xmax, ymin, ymax, fused_ops=case["fused_ops"] + ["Dequantize"],
                                              t1="quint8", toutput="float", input_quant_mode="MIN_FIRST", addend=z)
        np.testing.assert_array_equal(out, out2)


def test_batch_matmul_reference_cases(kat):
    """test/sanity/array/quantized_batch_matmul_test.py: BMM, BMM + Mul, BMM + Mul + Add on qint8 operands quantized
    SCALED / HALF_TO_EVEN / narrow_range, vs fp32 math at rtol = atol = 0.5; V1 and V2 spellings agree."""
    k = kat["batch_matmul"]
    x = np.array(k["x_f32"], np.float32)
    y = np.array(k["y_f32"], np.float32)
    mul = np.float32(k["mul"])
    add = np.array(k["add_f32"], np.float32)
    q = dict(T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN", narrow_range=True)
    qx, xmin, xmax = o.quantize_v2(x, x.min(), x.max(), **q)
    qy, ymin, ymax = o.quantize_v2(y, y.min(), y.max(), **q)
    for fused in k["cases"]:
        want = np.matmul(x, y)
        if "Mul" in fused:
            want = want * mul
        if "Add" in fused:
            want = want + add
        out = o.quantized_batch_matmul(qx, qy, xmin, xmax, ymin, ymax, fused_ops=fused, mul=mul, addend=add)
        assert out.shape == (2, 2, 2) and out.dtype == np.float32
        np.testing.assert_allclose(out, want, rtol=k["rtol"], atol=k["atol"])
        np.testing.assert_allclose(out, want, rtol=0, atol=0.03)  # what int8 operands of range 1.84 x 1.82 actually give
        out2 = o.quantized_batch_matmul(qx, qy, xmin, xmax, ymin, ymax, fused_ops=list(fused) + ["Dequantize"], mul=mul, addend=add)
        np.testing.assert_array_equal(out, out2)
    # adjoint flags and broadcast batch dims (MatMulBCast)
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, (2, 3, 5, 16)).astype(np.int8)
    b = rng.integers(-127, 128, (3, 7, 16)).astype(np.int8)
    out = o.quantized_batch_matmul(a, b, -1.0, 1.0, -2.0, 2.0, adj_y=True)
    want = np.einsum("bhmk,hnk->bhmn", a.astype(np.int64), b.astype(np.int64)).astype(np.float32) * np.float32(np.float32(2.0) / np.float32(127 * 127))
    np.testing.assert_array_equal(out, want)
    out_t = o.quantized_batch_matmul(np.swapaxes(a, -1, -2), b, -1.0, 1.0, -2.0, 2.0, adj_x=True, adj_y=True)
    np.testing.assert_array_equal(out, out_t)


def test_fused_matmul_scale_rules():
    """Requantize folds 255|127 / range into the per-channel scale when no activation follows, and into the
    activation's post scale otherwise (quantized_matmul_common.h:1651-1700); s8 activations use 127 (H3)."""
    rng = np.random.default_rng(7)
    a = rng.integers(-127, 128, (5, 32)).astype(np.int8)
    w = rng.integers(-127, 128, (32, 6)).astype(np.int8)
    bias = rng.standard_normal(6).astype(np.float32)
    mnb, mxb = -np.linspace(0.5, 1.5, 6).astype(np.float32), np.linspace(0.5, 1.5, 6).astype(np.float32)
    sc = o.fused_matmul_output_scale(-2.0, 2.0, mnb, mxb, "qint8", 6)
    np.testing.assert_allclose(sc, 2.0 * mxb / (127.0 * 127.0), rtol=1e-6)
    deq, _, _ = o.quantized_fused_matmul(a, w, bias, -2.0, 2.0, mnb, mxb, fused_ops=["BiasAdd"], t1="qint8", toutput="float",
                                         scaled_bias_mode="intended")
    np.testing.assert_allclose(deq, (a.astype(np.int64) @ w.astype(np.int64)) * sc + bias, rtol=1e-5, atol=1e-5)
    q, mn, mx = o.quantized_fused_matmul(a, w, bias, -2.0, 2.0, mnb, mxb, -40.0, 40.0, fused_ops=["BiasAdd"], t1="qint8",
                                         toutput="qint8", scaled_bias_mode="intended")
    np.testing.assert_allclose(q, np.clip(np.rint(deq * (127.0 / 40.0)), -128, 127), atol=1)
    qr, _, _ = o.quantized_fused_matmul(a, w, bias, -2.0, 2.0, mnb, mxb, 0.0, 40.0, fused_ops=["BiasAdd", "Relu"], t1="qint8",
                                        toutput="quint8", scaled_bias_mode="intended")
    np.testing.assert_allclose(qr, np.clip(np.rint(np.maximum(deq, 0) * (255.0 / 40.0)), 0, 255), atol=1)
    lit, _, _ = o.quantized_fused_matmul(a, w, bias, -2.0, 2.0, mnb, mxb, 0.0, 40.0, fused_ops=["BiasAdd", "Relu"], t1="qint8",
                                         toutput="quint8", scaled_bias_mode="intended", postop_scale_mode="literal")
    np.testing.assert_array_equal(lit, np.clip(np.rint(np.maximum(deq, 0)), 0, 255).astype(np.uint8))


@pytest.mark.parametrize("fmt", ["E4M3", "E5M2"])
def test_fp8_cast_pinned_to_the_format_definition(fmt):
    """The oracle's FP8 cast and decode against the bit layout written out in tests/fp8_format.py (no ml_dtypes): all 256
    codes decoded; every finite value, every tie between neighbours and its float32 neighbours, overflow, infinities and
    NaN encoded - round to nearest even, saturation of finite overflow, infinity -> NaN (e4m3fn) / infinity (e5m2), the
    behaviour itex/core/utils/float8.h:651-766 states."""
    import fp8_format as F
    t = F.table(fmt)
    got = o.fp8_to_f32(np.arange(256, dtype=np.uint8), fmt).astype(np.float64)
    assert np.array_equal(np.isnan(got), np.isnan(t)) and np.array_equal(got[~np.isnan(t)], t[~np.isnan(t)])
    assert np.nanmax(np.where(np.isfinite(t), t, np.nan)) == o.FP8_MAX[fmt]
    xs = F.probe_inputs(fmt)
    want = F.encode_many(xs, fmt)
    assert F.same_codes(o.fp8_cast_sat(xs, fmt), want, fmt)
    # a few decisions spelled out by hand (e4m3: neighbours 1.0 | 1.125, 384 | 416 | 448, subnormal step 2^-9)
    if fmt == "E4M3":
        hand = [(1.0625, 0x38), (1.0625 + 2 ** -20, 0x39), (1.1875, 0x3A), (400.0, 0x7C), (432.0, 0x7E), (464.0, 0x7E), (1e9, 0x7E),
                (-1e9, 0xFE), (2 ** -10, 0x00), (2 ** -10 + 2 ** -30, 0x01), (3 * 2 ** -10, 0x02), (0.0, 0x00), (-0.0, 0x80)]
        for x, code in hand:
            assert int(o.fp8_cast_sat(np.array([x], np.float32), fmt)[0]) == code, x
        assert np.isnan(o.fp8_to_f32(o.fp8_cast_sat(np.array([np.inf, -np.inf], np.float32), fmt), fmt)).all()
    else:
        assert list(o.fp8_cast_sat(np.array([np.inf, -np.inf, 57344.0, 61440.0, 1e30], np.float32), fmt)) == [0x7C, 0xFC, 0x7B, 0x7B, 0x7B]


def fp8_scale_hand_vectors():
    """(amax, old scale, fp8_max, margin) -> new scale, worked by hand from _default_sf_compute,
    itex/python/fp8/autocast.py:44-51: exp = floor(log2(fp8_max / amax)) - margin; sf = round(2^|exp|);
    amax <= 0 or not finite keeps the old scale; exp < 0 takes the reciprocal (of whatever sf is by then)."""
    inf, nan = float("inf"), float("nan")
    return [
        ((1.0, 7.0, 448.0, 0), 256.0),         # log2(448) = 8.8 -> 8
        ((1.0, 7.0, 448.0, 2), 64.0),          # margin 2 -> exp 6
        ((448.0, 7.0, 448.0, 0), 1.0),         # exp 0
        ((449.0, 7.0, 448.0, 0), 0.5),         # log2(0.9978) -> floor -1 -> 1 / 2
        ((1000.0, 7.0, 448.0, 0), 0.25),       # log2(0.448) = -1.16 -> -2 -> 1 / 4
        ((1000.0, 7.0, 448.0, 3), 1.0 / 32),   # exp -2 - 3 = -5
        ((3.7, 7.0, 448.0, 0), 64.0),          # 121.08 -> 6
        ((0.0, 7.0, 448.0, 0), 7.0),           # amax 0: old scale (exp = +inf is not < 0)
        ((-1.0, 7.0, 448.0, 0), 7.0),          # negative amax: log2 of a negative is NaN; old scale
        ((nan, 7.0, 448.0, 0), 7.0),           # NaN: old scale, exp < 0 is false
        ((inf, 8.0, 448.0, 0), 0.125),         # inf: old scale is selected, then exp = -inf < 0 takes its reciprocal
        ((1e-38, 7.0, 448.0, 0), inf),         # 448 / 1e-38 overflows fp32: exp = +inf, 2^inf = inf, kept because amax is finite and > 0
        ((1.0, 7.0, 57344.0, 0), 32768.0),     # e5m2 range: log2(57344) = 15.8
        ((2.0 ** -20, 7.0, 448.0, 0), 2.0 ** 28),
    ]


def test_fp8_scale_update_hand_vectors():
    for (amax, old, fmax, margin), want in fp8_scale_hand_vectors():
        got = o.fp8_default_sf_compute(np.array([amax], np.float32), np.array([old], np.float32), fmax, margin)
        assert got.dtype == np.float32 and got.shape == (1,)
        assert float(got[0]) == want, (amax, old, fmax, margin, float(got[0]), want)
    # history roll: row 0 zeroed, the other rows move up by one, the old row 0 lands in the last row (autocast.py:53-58)
    h = np.arange(12, dtype=np.float32).reshape(4, 3) + 1
    nh, sf, sfi = o.fp8_amax_and_scale_update(h, np.ones(3, np.float32), 448.0, 0, "most_recent")
    np.testing.assert_array_equal(nh, [[0, 0, 0], [7, 8, 9], [10, 11, 12], [1, 2, 3]])
    np.testing.assert_array_equal(sf, [256.0, 128.0, 128.0])      # amax = row 0 = 1, 2, 3
    nh, sf, sfi = o.fp8_amax_and_scale_update(h, np.ones(3, np.float32), 448.0, 0, "max")
    np.testing.assert_array_equal(sf, [32.0, 32.0, 32.0])         # amax = 10, 11, 12 -> 448/12 = 37.3 -> 5
    np.testing.assert_array_equal(sfi, [1 / 32.0] * 3)


def test_layout_ops_move_elements_and_pass_the_range_through():
    """QuantizedReshape / _QuantizedTranspose / QuantizedConcatV2 (common/quantized_reshape_op.h:33-200, gpu/transpose_op.cc,
    common/quantized_concat_op.cc:34-247): element moves only; the range is an output equal to the input's (input 0's for
    the concat, which refuses unequal ranges)."""
    rng = np.random.default_rng(11)
    x = rng.integers(-128, 128, (2, 3, 4, 5)).astype(np.int8)
    y, mn, mx = o.quantized_transpose(x, [0, 3, 1, 2], -1.5, 2.5)
    assert np.array_equal(y, np.transpose(x, (0, 3, 1, 2))) and (float(mn), float(mx)) == (-1.5, 2.5)
    with pytest.raises(ValueError):
        o.quantized_transpose(x, [0, 1, 1, 2], 0.0, 1.0)          # not a permutation
    with pytest.raises(ValueError):
        o.quantized_transpose(x, [0, 1, 2], 0.0, 1.0)             # wrong length
    y, mn, mx = o.quantized_reshape(x, [-1, 20], 0.0, 6.0)
    assert y.shape == (6, 20) and np.array_equal(y.reshape(-1), x.reshape(-1)) and (float(mn), float(mx)) == (0.0, 6.0)
    assert o.quantized_reshape(np.zeros((0, 4), np.uint8), [0, -1], 0.0, 1.0)[0].shape == (0, 4)
    for bad in ([-1, -1], [7, -1], [-2, 60], [5, 5]):
        with pytest.raises(ValueError):
            o.quantized_reshape(x, bad, 0.0, 1.0)
    a, b = x[:, :, :, :2], x[:, :, :, 2:]
    y, mn, mx = o.quantized_concat_v2([a, b], -1, [-1.0, -1.0], [1.0, 1.0 + 5e-7])
    assert np.array_equal(y, x) and (float(mn), float(mx)) == (-1.0, 1.0)
    with pytest.raises(NotImplementedError):
        o.quantized_concat_v2([a, b], 3, [-1.0, -1.0], [1.0, 1.5])
    with pytest.raises(ValueError):
        o.quantized_concat_v2([a, b], 0, [-1.0, -1.0], [1.0, 1.0])  # sizes differ off the axis
    with pytest.raises(ValueError):
        o.quantized_concat_v2([a, b], 4, [-1.0, -1.0], [1.0, 1.0])
