"""GPU parity of _QuantizedFusedMatMul[AndRequantize|AndDequantize] and _QuantizedMatMul (V2) through the op layer.

Integer outputs and float outputs of the algebraic post-ops (none, Relu, LeakyRelu, Relu6, Add) are bit-exact against
the oracle.  Transcendental post-ops (Gelu, Sigmoid, Tanh, Elu, Swish) are compared at rtol 1e-5 + atol 1e-6 for float
outputs; after requantization they may differ by one level where the activation lands within an ulp of a rounding tie.
"""
import json
import os

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import dev, host, modules

pytestmark = pytest.mark.gpu

EXACT_ACTS = (None, "Relu", "LeakyRelu", "Relu6")
SMOOTH_ACTS = ("GeluExact", "GeluApproximate", "Sigmoid", "Tanh", "Elu", "_ITEXSwish")


def _case(m, k, n, t1, per_channel, seed):
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.3).astype(np.float32)
    qa, mna, mxa = o.quantize_v2(x, x.min(), x.max(), T=t1)
    if per_channel:
        qb, mnb, mxb = o.quantize_v2(w, w.min(axis=0), w.max(axis=0), T="qint8", axis=1, narrow_range=True)
    else:
        qb, mnb, mxb = o.quantize_v2(w, w.min(), w.max(), T="qint8", narrow_range=True)
    return x, w, bias, qa, mna, mxa, qb, mnb, mxb


def _ranges(mn, mx):
    return (float(mn), float(mx)) if np.ndim(mn) == 0 else (np.asarray(mn, np.float32), np.asarray(mx, np.float32))


def test_reference_fused_matmul_cases(golden_dir):
    """kernel_tests/native_quantized_fused_matmul_test.py: BiasAdd + GeluApproximate (per-tensor and per-channel weights)
    and BiasAdd + Add, V1 and V2 spellings, MIN_FIRST input, against fp32 math at rtol=atol=0.2 - and against the oracle."""
    itex, K, ops = modules()
    k = json.load(open(os.path.join(golden_dir, "reference_kat.json")))["fused_matmul_min_first"]
    x = np.array(k["x_f32"], np.float32)
    y = np.array(k["y_f32"], np.float32)
    b = np.array(k["bias_f32"], np.float32)
    z = np.array(k["z_f32"], np.float32) * 2
    qx, xmin, xmax = ops._ITEXQuantizeV2(dev(x), float(x.min()), float(x.max()), T="quint8", mode="MIN_FIRST")
    for case in k["cases"]:
        if case["per_channel"]:
            qy, ymin, ymax = ops._ITEXQuantizeV2(dev(y), y.min(axis=0), y.max(axis=0), T="qint8", mode="SCALED",
                                                 round_mode="HALF_TO_EVEN", narrow_range=True, axis=1)
        else:
            qy, ymin, ymax = ops._ITEXQuantizeV2(dev(y), float(y.min()), float(y.max()), T="qint8", mode="SCALED",
                                                 round_mode="HALF_TO_EVEN", narrow_range=True)
        has_add = "Add" in case["fused_ops"]
        f = x @ y + b
        want = f + z if has_add else o.activation(f, "GeluApproximate")
        args = [dev(b), dev(z)] if has_add else [dev(b)]
        ref, _, _ = o.quantized_fused_matmul(host(qx), host(qy), b, xmin, xmax, ymin, ymax, fused_ops=case["fused_ops"], t1="quint8",
                                             toutput="float", input_quant_mode="MIN_FIRST", addend=z)
        for _ in range(2):  # the reference runs twice to exercise its object cache
            v1 = ops._QuantizedFusedMatMul(qx, qy, args, xmin, xmax, ymin, ymax, Toutput="float", fused_ops=case["fused_ops"],
                                           input_quant_mode="MIN_FIRST")
            v2 = ops._QuantizedMatMul(args[:0] + [qx, qy] + args, [xmin, xmax, ymin, ymax], T1="quint8", T2="qint8",
                                      Tdevice_outputs=["float"], fused_ops=case["fused_ops"] + ["Dequantize"],
                                      input_quant_mode="MIN_FIRST")
            np.testing.assert_allclose(host(v1), want, rtol=k["rtol"], atol=k["atol"])
            np.testing.assert_array_equal(host(v1), host(v2))
            if has_add:
                np.testing.assert_array_equal(host(v1), ref)
            else:
                np.testing.assert_allclose(host(v1), ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("t1", ["quint8", "qint8"])
@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("act", EXACT_ACTS)
def test_config1b_dequantize_exact(t1, per_channel, act):
    """cfg 1b: int8 (or uint8) activations, per-output-channel int8 weights, fp32 bias, dequantized fp32/bf16 output."""
    itex, K, ops = modules()
    x, w, bias, qa, mna, mxa, qb, mnb, mxb = _case(64, 1024, 1024, t1, per_channel, 1235)
    fused = ["BiasAdd"] + ([act] if act else [])
    mnb_a, mxb_a = _ranges(mnb, mxb)
    for tout in ("float", "bfloat16"):
        ref, _, _ = o.quantized_fused_matmul(qa, qb, bias, mna, mxa, mnb, mxb, fused_ops=fused, t1=t1, toutput=tout,
                                             scaled_bias_mode="intended", leakyrelu_alpha=0.1)
        got = ops._QuantizedFusedMatMul(dev(qa), dev(qb), [dev(bias)], float(mna), float(mxa), mnb_a, mxb_a, Toutput=tout,
                                        fused_ops=fused, scaled_bias_mode="intended", leakyrelu_alpha=0.1)
        np.testing.assert_array_equal(host(got), ref.astype(np.float32))
        got2 = ops._QuantizedMatMul([dev(qa), dev(qb), dev(bias)], [float(mna), float(mxa), mnb_a, mxb_a], Tout=tout,
                                    fused_ops=fused + ["Dequantize"], scaled_bias_mode="intended", leakyrelu_alpha=0.1,
                                    op_name="_ITEXQuantizedMatMul")
        np.testing.assert_array_equal(host(got2), ref.astype(np.float32))
    if act is None and t1 == "qint8":  # the quantized product approximates the fp32 one
        f = x @ w + bias
        assert np.abs(host(got).astype(np.float32) - f).max() < 0.08


@pytest.mark.parametrize("act", SMOOTH_ACTS)
def test_smooth_activations(act):
    itex, K, ops = modules()
    x, w, bias, qa, mna, mxa, qb, mnb, mxb = _case(200, 256, 136, "qint8", True, 77)
    fused = ["BiasAdd", act]
    ref, _, _ = o.quantized_fused_matmul(qa, qb, bias, mna, mxa, mnb, mxb, fused_ops=fused, t1="qint8", toutput="float",
                                         scaled_bias_mode="intended")
    got = ops._QuantizedFusedMatMul(dev(qa), dev(qb), [dev(bias)], float(mna), float(mxa), mnb, mxb, Toutput="float",
                                    fused_ops=fused, scaled_bias_mode="intended")
    np.testing.assert_allclose(host(got), ref, rtol=1e-5, atol=1e-6)
    # requantized after the activation: the post-op scale is applied ("intended") or dropped ("literal")
    lo, hi = float(ref.min()), float(ref.max())
    tq = "qint8" if lo < 0 else "quint8"
    for mode in ("intended", "literal"):
        refq, rmn, rmx = o.quantized_fused_matmul(qa, qb, bias, mna, mxa, mnb, mxb, lo, hi, fused_ops=fused, t1="qint8",
                                                  toutput=tq, scaled_bias_mode="intended", postop_scale_mode=mode)
        gq, gmn, gmx = ops._QuantizedFusedMatMul(dev(qa), dev(qb), [dev(bias)], float(mna), float(mxa), mnb, mxb, lo, hi,
                                                 Toutput=tq, fused_ops=fused, scaled_bias_mode="intended", postop_scale_mode=mode)
        diff = np.abs(host(gq).astype(np.int32) - refq.astype(np.int32))
        assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
        assert (gmn, gmx) == (np.float32(lo), np.float32(hi))


@pytest.mark.parametrize("tout", ["quint8", "qint8"])
@pytest.mark.parametrize("mode", ["SCALED", "MIN_FIRST"])
def test_requantize_and_qint32(tout, mode):
    """Requantize with and without an activation (bit-exact), ragged sizes, both input modes, and the qint32 variant
    with per-channel output ranges."""
    itex, K, ops = modules()
    t1 = "quint8" if mode == "MIN_FIRST" else "qint8"
    rng = np.random.default_rng(5)
    m, k, n = 77, 200, 90
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.3).astype(np.float32)
    qa, mna, mxa = o.quantize_v2(x, x.min(), x.max(), T=t1, mode=mode,
                                 round_mode="HALF_TO_EVEN" if mode == "SCALED" else "HALF_AWAY_FROM_ZERO")
    qb, mnb, mxb = o.quantize_v2(w, w.min(axis=0), w.max(axis=0), T="qint8", axis=1, narrow_range=True)
    f = x @ w + bias
    for fused in (["BiasAdd"], ["BiasAdd", "Relu"]):
        fr = np.maximum(f, 0) if len(fused) > 1 else f
        lo, hi = (float(fr.min()), float(fr.max()))
        if tout == "quint8":
            lo = 0.0
        ref, rmn, rmx = o.quantized_fused_matmul(qa, qb, bias, mna, mxa, mnb, mxb, lo, hi, fused_ops=fused, t1=t1, toutput=tout,
                                                 input_quant_mode=mode, scaled_bias_mode="intended")
        got, gmn, gmx = ops._QuantizedFusedMatMul(dev(qa), dev(qb), [dev(bias)], float(mna), float(mxa), mnb, mxb, lo, hi,
                                                  Toutput=tout, fused_ops=fused, input_quant_mode=mode, scaled_bias_mode="intended")
        np.testing.assert_array_equal(host(got), ref)
        v2 = ops._QuantizedMatMul([dev(qa), dev(qb), dev(bias)], [float(mna), float(mxa), mnb, mxb, lo, hi], Tout=tout,
                                  fused_ops=fused + ["Requantize"], input_quant_mode=mode, scaled_bias_mode="intended")
        np.testing.assert_array_equal(host(v2[0]), ref)
        assert (v2[1], v2[2]) == (np.float32(lo), np.float32(hi)) == (gmn, gmx)
        if len(fused) == 1 and tout == "qint8":  # dequantized, it approximates the fp32 product
            deq = ref.astype(np.float32) * (max(abs(lo), abs(hi)) / 127.0)
            assert np.abs(deq - f).max() < 0.1
    ref, rmn, rmx = o.quantized_fused_matmul(qa, qb, bias, mna, mxa, mnb, mxb, fused_ops=["BiasAdd"], t1=t1, toutput="qint32",
                                             input_quant_mode=mode, scaled_bias_mode="intended")
    got, gmn, gmx = ops._QuantizedFusedMatMul(dev(qa), dev(qb), [dev(bias)], float(mna), float(mxa), mnb, mxb, Toutput="qint32",
                                              fused_ops=["BiasAdd"], input_quant_mode=mode, scaled_bias_mode="intended")
    np.testing.assert_array_equal(host(got), ref)
    np.testing.assert_array_equal(gmn, rmn)
    np.testing.assert_array_equal(gmx, rmx)


def test_add_then_activation_and_errors():
    itex, K, ops = modules()
    x, w, bias, qa, mna, mxa, qb, mnb, mxb = _case(96, 128, 64, "qint8", True, 3)
    z = np.random.default_rng(4).standard_normal((96, 64)).astype(np.float32)
    fused = ["BiasAdd", "Add", "Relu", "Dequantize"]
    ref, _, _ = o.quantized_fused_matmul(qa, qb, bias, mna, mxa, mnb, mxb, fused_ops=fused, t1="qint8", toutput="float",
                                         addend=z, scaled_bias_mode="intended")
    got = ops._QuantizedMatMul([dev(qa), dev(qb), dev(bias), dev(z)], [float(mna), float(mxa), mnb, mxb], Tout="float",
                               fused_ops=fused, scaled_bias_mode="intended")
    np.testing.assert_array_equal(host(got), ref)
    # no bias at all (fused_ops = []): the raw scaled product
    ref0, _, _ = o.quantized_fused_matmul(qa, qb, None, mna, mxa, mnb, mxb, fused_ops=[], t1="qint8", toutput="float")
    got0 = ops._QuantizedFusedMatMul(dev(qa), dev(qb), [], float(mna), float(mxa), mnb, mxb, Toutput="float", fused_ops=[])
    np.testing.assert_array_equal(host(got0), ref0)
    L = itex._lib
    with pytest.raises(L.ItexError) as e:
        ops._QuantizedFusedMatMul(dev(qa), dev(qb), [dev(bias)], 0.0, 1.0, mnb, mxb, Toutput="float", fused_ops=["Relu"])
    assert "first post op must be BiasAdd" in str(e.value)
    with pytest.raises(L.ItexError) as e:
        ops._QuantizedFusedMatMul(dev(qa), dev(qb), [dev(bias)], 0.0, 1.0, mnb, mxb, Toutput="float", fused_ops=["BiasAdd", "Softmax"])
    assert "unsupported fusion" in str(e.value)
    with pytest.raises(L.ItexError) as e:
        ops._QuantizedMatMul([dev(qa), dev(qb), dev(bias), dev(z)], [float(mna), float(mxa), mnb, mxb, 0.0, 1.0], Tout="quint8",
                             fused_ops=["BiasAdd", "Add", "Requantize"])
    assert "Quantized addend tensor is not implemented yet" in str(e.value)
