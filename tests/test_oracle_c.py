"""The C twin of the oracle agrees bit for bit with the NumPy oracle (which is pinned to the
reference's known-answer tests and to real oneDNN)."""
import numpy as np

import itex_oracle as o
import oracle_c as oc


def test_c_quantize_dequantize():
    rng = np.random.default_rng(0)
    x = rng.uniform(-1.5, 1.5, (3, 5, 16)).astype(np.float32)
    x.flat[:4] = [0.5 / 63.5, 1.5 / 63.5, np.nan, 1e9]
    for T in ("qint8", "quint8"):
        np.testing.assert_array_equal(oc.quantize_scaled(x, 63.5, T == "qint8"), o.sat_rne(x * np.float32(63.5), T))
    sc = np.array([1.0, 2.0, 3.0, 4.0, 5.0], np.float32)
    q, _, _ = o.quantize_v2(x, -1 / sc, 1 / sc, T="qint8", axis=1)
    np.testing.assert_array_equal(oc.quantize_scaled(x, np.float32(127) / (1 / sc), True, inner=16), q)
    np.testing.assert_array_equal(oc.dequantize(q, (1 / sc) / np.float32(127), inner=16), o.dequantize(q, -1 / sc, 1 / sc, axis=1))


def test_c_gemm_and_epilogue():
    rng = np.random.default_rng(1)
    a = rng.integers(0, 256, (37, 200), dtype=np.uint8)
    b = rng.integers(-127, 128, (200, 53)).astype(np.int8)
    acc = o.int_matmul(a, b)
    np.testing.assert_array_equal(oc.gemm_acc(a, b.T), acc)
    np.testing.assert_array_equal(oc.gemm_acc(a.view(np.int8), b.T), o.int_matmul(a.view(np.int8), b))
    scale = rng.uniform(1e-4, 1e-3, 53).astype(np.float32)
    bias = rng.standard_normal(53).astype(np.float32)
    for tout in ("float", "quint8", "qint8", "qint32"):
        for relu in (False, True):
            sc = scale * (100 if tout in ("quint8", "qint8") else 1)
            np.testing.assert_array_equal(oc.gemm_fused(a, b.T, sc, bias, relu, tout), o.epilogue(acc, sc.astype(np.float32), bias, relu, tout))


def test_c_conv():
    rng = np.random.default_rng(2)
    x = rng.integers(0, 256, (2, 9, 7, 5), dtype=np.uint8)
    f = rng.integers(-127, 128, (3, 3, 5, 6)).astype(np.int8)
    for s in (1, 2):
        oh, pt, _ = o.same_padding(9, 3, s)
        ow, pl, _ = o.same_padding(7, 3, s)
        np.testing.assert_array_equal(oc.conv_acc(x, f, (s, s), (pt, pl), (oh, ow)), o.int_conv2d_nhwc(x, f, (s, s), "SAME"))
