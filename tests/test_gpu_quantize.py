"""GPU parity of _ITEXQuantizeV2 / _ITEXDequantize through the C-ABI op layer.
Bit-exact against the reference's known-answer tests and the CPU oracle."""
import json
import os

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import Canary, dev, host, modules, scale_per_slice

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kat(golden_dir):
    with open(os.path.join(golden_dir, "reference_kat.json")) as f:
        return json.load(f)


def test_quantize_axis_known_answers(kat):
    """quantized_ops_test.py:_testAxis - SCALED, HALF_TO_EVEN, qint8, per tensor and per axis, assertAllEqual."""
    itex, K, ops = modules()
    k = kat["quantize_axis"]
    shape = np.array(k["shape"])
    values = np.array(k["values"], np.float32)
    expected = scale_per_slice(shape, None, np.array(k["quant_values"], np.int32))
    for axis in k["axes"]:
        x = scale_per_slice(shape, axis, values).astype(np.float32)
        if axis is None:
            mn, mx = k["min_per_slice"], k["max_per_slice"]
        else:
            mn = [k["min_per_slice"] * (i + 1) for i in range(shape[axis])]
            mx = [k["max_per_slice"] * (i + 1) for i in range(shape[axis])]
        q, omin, omax = ops._ITEXQuantizeV2(dev(x), mn, mx, T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN",
                                            narrow_range=True, axis=axis)
        np.testing.assert_array_equal(host(q).astype(np.int32), expected)
        q_ref, rmin, rmax = o.quantize_v2(x, mn, mx, T="qint8", axis=-1 if axis is None else axis)
        np.testing.assert_array_equal(np.asarray(omin), np.asarray(rmin))
        np.testing.assert_array_equal(np.asarray(omax), np.asarray(rmax))
        # the stock op name dispatches to the same kernel
        q2, _, _ = ops._ITEXQuantizeV2(dev(x), mn, mx, T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN",
                                       narrow_range=True, axis=axis, op_name="QuantizeV2")
        np.testing.assert_array_equal(host(q2), host(q))


def test_quantize_min_first_known_answers(kat):
    itex, K, ops = modules()
    for name, kw in (("quantize_min_first", {}), ("quantize_asymmetric_legacy", {}),
                     ("quantize_asymmetric_classic", {"classic_asymmetric_algorithm": True})):
        k = kat[name]
        for dt in (torch.float32, torch.bfloat16):
            x = torch.tensor(k["x"], dtype=dt, device="cuda")
            q, mn, mx = ops._ITEXQuantizeV2(x, k["min"], k["max"], T=k["T"], mode="MIN_FIRST", **kw)
            np.testing.assert_allclose(host(q).astype(np.float32), k["expected"], atol=k["atol"])
            ref, rmn, rmx = o.quantize_v2(host(x), k["min"], k["max"], T=k["T"], mode="MIN_FIRST",
                                          round_mode="HALF_AWAY_FROM_ZERO", **kw)
            if dt == torch.float32:
                np.testing.assert_array_equal(host(q), ref)
            assert mn == rmn and mx == rmx


@pytest.mark.parametrize("T", ["qint8", "quint8"])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_quantize_matches_oracle_on_odd_sizes(T, dt):
    itex, K, ops = modules()
    rng = np.random.default_rng(11)
    for shape in ((1,), (15,), (17,), (64, 1024), (3, 5, 7, 11), (4099,)):
        x = torch.from_numpy(rng.uniform(-1.5, 1.5, shape).astype(np.float32)).to(dt).cuda()
        q, mn, mx = ops._ITEXQuantizeV2(x, -1.0, 0.8, T=T, mode="SCALED", round_mode="HALF_TO_EVEN")
        ref, rmn, rmx = o.quantize_v2(host(x), -1.0, 0.8, T=T)
        np.testing.assert_array_equal(host(q), ref)
        assert (mn, mx) == (rmn, rmx)


def test_quantize_config1_activations_and_rerun():
    """fp32 [64,1024] ~U[-1,1) -> quint8/qint8 with the tensor's own range; second run identical."""
    itex, K, ops = modules()
    x = np.random.default_rng(1235).uniform(-1, 1, (64, 1024)).astype(np.float32)
    for T in ("quint8", "qint8"):
        a = ops._ITEXQuantizeV2(dev(x), float(x.min()), float(x.max()), T=T, mode="SCALED", round_mode="HALF_TO_EVEN")
        b = ops._ITEXQuantizeV2(dev(x), float(x.min()), float(x.max()), T=T, mode="SCALED", round_mode="HALF_TO_EVEN")
        ref, rmn, rmx = o.quantize_v2(x, x.min(), x.max(), T=T)
        np.testing.assert_array_equal(host(a[0]), ref)
        np.testing.assert_array_equal(host(b[0]), ref)
        assert a[1:] == (rmn, rmx)


def test_quantize_ties_saturation_nan_and_unaligned_pointers():
    itex, K, ops = modules()
    L = itex._lib
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.5, 300.0, -127.5, -128.5, -300.0, np.nan, np.inf, -np.inf, 0.0, 3.3],
                 np.float32)
    for T, dt in (("qint8", L.DT_QINT8), ("quint8", L.DT_QUINT8)):
        ref = o.sat_rne(x, T)
        got = K.quantize(dev(x), dt, 1.0)
        np.testing.assert_array_equal(host(got), ref)
    # unaligned input/output pointers take the element-wise kernel and must not touch neighbours
    big = dev(np.random.default_rng(2).uniform(-2, 2, 1003).astype(np.float32))
    c = Canary(1003 + 16)
    out = c.payload[3:3 + 1000].view(torch.int8)
    src = big[1:1001]
    K.quantize(src, L.DT_QINT8, 63.5, out=out)
    torch.cuda.synchronize()
    c.check()
    np.testing.assert_array_equal(host(out), o.sat_rne(host(src) * np.float32(63.5), "qint8"))


def test_quantize_rejects_bad_ranges_like_the_reference():
    itex, K, ops = modules()
    x = torch.zeros(8, device="cuda")
    with pytest.raises(itex.ItexError) as e:
        ops._ITEXQuantizeV2(x, 1.0, -1.0, T="qint8")
    assert e.value.code == itex._lib.INVALID_ARGUMENT and "input_max_range must be larger than input_min_range" in str(e.value)
    with pytest.raises(itex.ItexError) as e:  # HostMemory argument passed on the device
        ops.Op("_ITEXQuantizeV2", T="qint8")(x, torch.zeros(1, device="cuda"), torch.ones(1, device="cuda"))
    assert "HostMemory" in str(e.value)
    q, mn, mx = ops._ITEXQuantizeV2(torch.zeros((0, 4), device="cuda"), -1.0, 1.0, T="qint8")  # empty input
    assert tuple(q.shape) == (0, 4) and (mn, mx) == (-1.0, 1.0)
    # ensure_minimum_range nudges a degenerate range (quantize_op.h:137-151)
    q, mn, mx = ops._ITEXQuantizeV2(torch.full((4,), 0.001, device="cuda"), 0.0, 0.0, T="quint8")
    ref, rmn, rmx = o.quantize_v2(np.full(4, 0.001, np.float32), 0.0, 0.0, T="quint8")
    np.testing.assert_array_equal(host(q), ref)
    assert (mn, mx) == (rmn, rmx)


def test_dequantize_known_answers(kat):
    itex, K, ops = modules()
    k = kat["dequantize_axis"]
    shape = np.array(k["shape"])
    q = scale_per_slice(shape, None, np.array(k["values"], np.int32)).astype(np.int8)
    for axis in k["axes"]:
        expected = scale_per_slice(shape, axis, np.array(k["dequant_values"], np.float32))
        if axis is None:
            mn, mx = k["min_per_slice"], k["max_per_slice"]
        else:
            mn = [k["min_per_slice"] * (i + 1) for i in range(shape[axis])]
            mx = [k["max_per_slice"] * (i + 1) for i in range(shape[axis])]
        y = ops._ITEXDequantize(dev(q), mn, mx, mode="SCALED", narrow_range=True, axis=axis)
        np.testing.assert_allclose(host(y), expected, rtol=k["rtol"], atol=k["atol"])
        np.testing.assert_array_equal(host(y), o.dequantize(q, mn, mx, axis=-1 if axis is None else axis))
    for c in kat["dequantize_scaled"]["cases"]:
        qq = np.array(c["q"], np.int8)
        y = ops._ITEXDequantize(dev(qq), c["min"], c["max"], mode="SCALED")
        sf = max(c["min"] / -127, c["max"] / 127)
        np.testing.assert_allclose(host(y), qq.astype(np.float32) * sf, rtol=1e-2, atol=1e-2)
    k = kat["dequantize_min_first"]
    y = ops._ITEXDequantize(dev(np.array(k["q"], np.uint8)), k["min"], k["max"], mode="MIN_FIRST")
    np.testing.assert_allclose(host(y), k["expected"], atol=k["atol"])


@pytest.mark.parametrize("out", ["float", "bfloat16", "half"])
def test_dequantize_matches_oracle(out):
    itex, K, ops = modules()
    rng = np.random.default_rng(5)
    for shape, qdt in (((128, 7, 7, 32), np.uint8), ((33, 17), np.int8), ((5,), np.uint8)):
        q = rng.integers(0, 256, shape).astype(qdt) if qdt == np.uint8 else rng.integers(-128, 128, shape).astype(qdt)
        y = ops._ITEXDequantize(dev(q), -3.0, 5.5, mode="SCALED", dtype=out)
        ref = o.dequantize(q, -3.0, 5.5, dtype=out)
        np.testing.assert_array_equal(host(y), ref.astype(np.float32))


def test_quantize_dequantize_round_trip_at_benchmark_size():
    """3 211 264 elements (test/benchmark/test_quantize.py): |dequant(quant(x)) - x| <= half a step,
    and quantize is idempotent on its own output grid."""
    itex, K, ops = modules()
    n = 3211264
    x = torch.empty(n, device="cuda").uniform_(-5, 5)
    q, mn, mx = ops._ITEXQuantizeV2(x, -5.0, 5.0, T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    y = ops._ITEXDequantize(q, mn, mx, mode="SCALED")
    step = 5.0 / 127
    assert float((y - x).abs().max()) <= step / 2 * 1.0001
    q2, _, _ = ops._ITEXQuantizeV2(y, -5.0, 5.0, T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    assert bool((q2 == q).all())


def test_dynamic_range_path_matches_host_path():
    """Range reduced on the device (no host sync) gives the bytes the host-range op gives."""
    itex, K, ops = modules()
    L = itex._lib
    x = torch.from_numpy(np.random.default_rng(9).standard_normal((12288, 64)).astype(np.float32)).cuda()
    mm = K.minmax(x)
    q, out3 = K.quantize_dynamic(x, L.DT_QINT8, mm)
    mmh = host(mm)
    ref, rmn, rmx = ops._ITEXQuantizeV2(x, float(mmh[0]), float(mmh[1]), T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    assert float(mmh[0]) == float(x.min()) and float(mmh[1]) == float(x.max())
    assert bool((q == ref).all())
    o3 = host(out3)
    assert (o3[1], o3[2]) == (rmn, rmx)
