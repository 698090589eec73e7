"""GPU parity of the batched int8 matmul ops (_QuantizedBatchMatMulV2AndDequantize, the fused and the V2 forms)
through the op layer, against the oracle.

The unfused product and the Add fusion are bit-exact (one multiply by the dequantize scale, one add).  With a
fused Mul the kernel multiplies the accumulator by fl(scale * mul) where the post-op chain of the reference rounds
acc * scale first: outputs are compared at rtol 2.5e-7 (two fp32 roundings) for float, and within one ulp of the
16-bit output type.
"""
import json
import os

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import dev, host, modules

pytestmark = pytest.mark.gpu

TORCH_OF = {"float": torch.float32, "bfloat16": torch.bfloat16, "half": torch.float16}


def _quant(x):
    return o.quantize_v2(x, x.min(), x.max(), T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN", narrow_range=True)


def _check(got, want, toutput, fused_mul):
    got = host(got)
    want = np.asarray(want, np.float32)
    assert got.shape == want.shape
    if not fused_mul:
        np.testing.assert_array_equal(got, want)
    elif toutput == "float":
        np.testing.assert_allclose(got, want, rtol=2.5e-7, atol=1e-30)
    else:
        eps = 2.0 ** -8 if toutput == "bfloat16" else 2.0 ** -11
        np.testing.assert_allclose(got, want, rtol=eps, atol=1e-30)


def test_reference_batch_matmul_cases(golden_dir):
    """test/sanity/array/quantized_batch_matmul_test.py: BMM, BMM + Mul, BMM + Mul + Add, V1 and V2 spellings,
    against fp32 math at rtol = atol = 0.5 - and against the oracle."""
    itex, K, ops = modules()
    k = json.load(open(os.path.join(golden_dir, "reference_kat.json")))["batch_matmul"]
    x = np.array(k["x_f32"], np.float32)
    y = np.array(k["y_f32"], np.float32)
    mul = np.float32(k["mul"])
    add = np.array(k["add_f32"], np.float32)
    q = dict(T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN", narrow_range=True)
    qx, xmin, xmax = ops._ITEXQuantizeV2(dev(x), float(x.min()), float(x.max()), **q)
    qy, ymin, ymax = ops._ITEXQuantizeV2(dev(y), float(y.min()), float(y.max()), **q)
    np.testing.assert_array_equal(host(qx), _quant(x)[0])
    for fused in k["cases"]:
        want = np.matmul(x, y)
        args = []
        if "Mul" in fused:
            want = want * mul
            args.append(dev(np.array(mul, np.float32)))
        if "Add" in fused:
            want = want + add
            args.append(dev(add))
        if not fused:
            v1 = ops._QuantizedBatchMatMulV2AndDequantize(qx, qy, xmin, xmax, ymin, ymax)
        else:
            v1 = ops._QuantizedFusedBatchMatMulV2AndDequantize(qx, qy, args, xmin, xmax, ymin, ymax, fused_ops=fused)
        v2 = ops._QuantizedBatchMatMul([qx, qy] + args, [xmin, xmax, ymin, ymax], fused_ops=list(fused) + ["Dequantize"],
                                       Tdevice_outputs=["float"])
        np.testing.assert_allclose(host(v1), want, rtol=k["rtol"], atol=k["atol"])
        np.testing.assert_array_equal(host(v1), host(v2))
        ref = o.quantized_batch_matmul(host(qx), host(qy), xmin, xmax, ymin, ymax, fused_ops=fused, mul=mul, addend=add)
        _check(v1, ref, "float", "Mul" in fused)


# (batch dims of x, batch dims of y, m, k, n, adj_x, adj_y)
SHAPES = [
    ((4, 16), (4, 16), 128, 64, 128, False, True),     # attention scores: Q x K^T
    ((4, 16), (4, 16), 128, 128, 64, False, False),    # attention context: P x V (V arrives [k, n])
    ((3,), (3,), 200, 80, 72, True, False),            # both operands transposed per batch
    ((2, 3), (2, 3), 33, 40, 20, False, True),         # ragged tile edges, k not a multiple of 16
    ((5,), (), 70, 48, 96, False, True),               # right operand shared by every batch
    ((), (4,), 64, 32, 48, False, False),              # left operand shared
    ((), (), 50, 64, 40, False, False),                # rank 2
    ((2,), (1,), 17, 16, 9, False, False),             # odd n: the output pitch is not 16-byte aligned
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("toutput", ["float", "bfloat16"])
def test_batch_matmul_shapes(shape, toutput):
    itex, K, ops = modules()
    bx, by, m, k, n, adj_x, adj_y = shape
    rng = np.random.default_rng(hash((bx, by, m, k, n)) % (2 ** 31))
    x = rng.integers(-127, 128, bx + ((k, m) if adj_x else (m, k))).astype(np.int8)
    y = rng.integers(-127, 128, by + ((n, k) if adj_y else (k, n))).astype(np.int8)
    xmin, xmax, ymin, ymax = -3.5, 2.25, -0.75, 1.5
    got = ops._QuantizedBatchMatMulV2AndDequantize(dev(x), dev(y), xmin, xmax, ymin, ymax, Toutput=toutput, adj_x=adj_x, adj_y=adj_y)
    assert got.dtype == TORCH_OF[toutput]
    want = o.quantized_batch_matmul(x, y, xmin, xmax, ymin, ymax, adj_x=adj_x, adj_y=adj_y, toutput=toutput)
    _check(got, want, toutput, False)


@pytest.mark.parametrize("toutput", ["float", "bfloat16", "half"])
@pytest.mark.parametrize("fused", [["Mul"], ["Add"], ["Mul", "Add"]])
@pytest.mark.parametrize("add_shape", ["full", "mask", "scalar"])
def test_fused_mul_add(toutput, fused, add_shape):
    """The attention-score fusion of a quantized BERT: Q x K^T * 1/sqrt(d) + mask, the mask broadcast over heads and rows."""
    itex, K, ops = modules()
    b, h, s, d = 2, 4, 96, 64
    rng = np.random.default_rng(11)
    qf = rng.standard_normal((b, h, s, d)).astype(np.float32)
    kf = rng.standard_normal((b, h, s, d)).astype(np.float32)
    qx, xmin, xmax = _quant(qf)
    qy, ymin, ymax = _quant(kf)
    tt = TORCH_OF[toutput]
    mul_t = torch.tensor(1.0 / np.sqrt(d), dtype=tt, device="cuda")
    if add_shape == "full":
        add_t = torch.from_numpy(rng.standard_normal((b, h, s, s)).astype(np.float32)).to(tt).cuda()
    elif add_shape == "mask":
        add_t = torch.from_numpy(np.where(rng.random((b, 1, 1, s)) < 0.2, -10000.0, 0.0).astype(np.float32)).to(tt).cuda()
    else:
        add_t = torch.tensor(0.375, dtype=tt, device="cuda")
    args = ([mul_t] if "Mul" in fused else []) + ([add_t] if "Add" in fused else [])
    got = ops._QuantizedFusedBatchMatMulV2AndDequantize(dev(qx), dev(qy), args, xmin, xmax, ymin, ymax, fused_ops=fused,
                                                        Toutput=toutput, adj_y=True)
    want = o.quantized_batch_matmul(qx, qy, xmin, xmax, ymin, ymax, fused_ops=fused, mul=host(mul_t), addend=host(add_t),
                                    adj_y=True, toutput=toutput)
    if "Mul" in fused and "Add" in fused:
        # the sum's rounding can amplify the scale product's rounding where the terms cancel
        got_h = host(got)
        eps = {"float": 2.0 ** -23, "bfloat16": 2.0 ** -8, "half": 2.0 ** -11}[toutput]
        mag = np.abs(host(add_t)).max() + np.abs(want).max()
        np.testing.assert_allclose(got_h, np.asarray(want, np.float32), rtol=eps, atol=float(mag) * 2.0 ** -22)
    else:
        _check(got, want, toutput, "Mul" in fused)
    v2 = ops._QuantizedBatchMatMul([dev(qx), dev(qy)] + args, [xmin, xmax, ymin, ymax], fused_ops=fused + ["Dequantize"],
                                   Tout=toutput, adj_y=True)
    assert torch.equal(got, v2)


def test_errors():
    itex, K, ops = modules()
    x = dev(np.zeros((2, 8, 16), np.int8))
    y = dev(np.zeros((2, 16, 8), np.int8))
    with pytest.raises(itex.ItexError, match="mismatch"):
        ops._QuantizedBatchMatMulV2AndDequantize(x, x, -1.0, 1.0, -1.0, 1.0)
    with pytest.raises(itex.ItexError, match="compatible batch"):
        ops._QuantizedBatchMatMulV2AndDequantize(x, dev(np.zeros((3, 16, 8), np.int8)), -1.0, 1.0, -1.0, 1.0)
    with pytest.raises(itex.ItexError, match="not implemented"):
        ops._QuantizedFusedBatchMatMulV2AndDequantize(x, y, [dev(np.zeros((), np.float32))], -1.0, 1.0, -1.0, 1.0, fused_ops=["Relu"])
    with pytest.raises(itex.ItexError, match="same number"):
        ops._QuantizedFusedBatchMatMulV2AndDequantize(x, y, [], -1.0, 1.0, -1.0, 1.0, fused_ops=["Mul"])
    with pytest.raises(itex.ItexError, match="scalar or have 3 dims"):
        ops._QuantizedFusedBatchMatMulV2AndDequantize(x, y, [dev(np.zeros((8,), np.float32))], -1.0, 1.0, -1.0, 1.0, fused_ops=["Add"])
    with pytest.raises(itex.ItexError, match="only qint8 x qint8"):
        ops._QuantizedBatchMatMulV2AndDequantize(dev(np.zeros((2, 8, 16), np.uint8)), y, 0.0, 1.0, -1.0, 1.0)
    # empty batch: an empty output, no launch
    out = ops._QuantizedBatchMatMulV2AndDequantize(dev(np.zeros((0, 8, 16), np.int8)), dev(np.zeros((0, 16, 8), np.int8)), -1.0, 1.0, -1.0, 1.0)
    assert tuple(out.shape) == (0, 8, 8)
