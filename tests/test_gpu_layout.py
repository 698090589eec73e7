"""GPU parity of the data-movement ops between the quantized matmuls and convolutions: [_ITEX]QuantizedReshape,
_QuantizedTranspose / _ITEXQuantizedTranspose, QuantizedConcatV2 / _ITEXQuantizedConcatV2.  Byte work: bit-exact."""
import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import dev, host, modules

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,perm", [
    ((4, 128, 16, 64), (0, 2, 1, 3)),      # [B,S,H,D] -> [B,H,S,D]: rows of 64 bytes move whole
    ((4, 16, 128, 64), (0, 1, 3, 2)),      # K^T: the two innermost dimensions swap, batched
    ((3, 5, 77, 130), (0, 1, 3, 2)),       # the same with ragged 64 x 64 tiles and unaligned rows
    ((33, 65), (1, 0)),
    ((2, 3, 4, 5, 6), (4, 2, 0, 3, 1)),    # nothing stays in place
    ((7, 1, 48), (1, 0, 2)),               # only an extent-1 dimension moves: a plain copy
    ((6, 9, 32), (2, 0, 1)),
    ((5, 0, 3), (2, 1, 0)),                # empty
    ((11,), (0,)),
])
@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
def test_quantized_transpose(shape, perm, dtype):
    itex, K, ops = modules()
    rng = np.random.default_rng(sum(shape) + len(perm))
    x = rng.integers(0 if dtype == np.uint8 else -128, 256 if dtype == np.uint8 else 128, shape).astype(dtype)
    want, wmn, wmx = o.quantized_transpose(x, perm, -1.5, 2.5)
    for name, tperm in (("_ITEXQuantizedTranspose", "int32"), ("_QuantizedTranspose", "int64")):
        y, mn, mx = ops._ITEXQuantizedTranspose(dev(x), perm, -1.5, 2.5, Tperm=tperm, op_name=name)
        assert tuple(y.shape) == want.shape
        np.testing.assert_array_equal(host(y), want)
        assert (mn, mx) == (float(wmn), float(wmx))


def test_quantized_transpose_qint32_and_errors():
    itex, K, ops = modules()
    rng = np.random.default_rng(5)
    x = rng.integers(-2 ** 31, 2 ** 31 - 1, (6, 10, 12), dtype=np.int64).astype(np.int32)
    for perm in ((1, 0, 2), (2, 1, 0)):
        y, _, _ = ops._ITEXQuantizedTranspose(dev(x), perm, 0.0, 1.0)
        np.testing.assert_array_equal(host(y), np.transpose(x, perm))
    q = dev(np.zeros((2, 3, 4), np.uint8))
    for perm, msg in (((0, 1), "vector of size 3"), ((0, 1, 3), "out of range"), ((0, 1, 1), "is missing from")):
        with pytest.raises(itex.ItexError) as e:
            ops._ITEXQuantizedTranspose(q, perm, 0.0, 1.0)
        assert e.value.code == itex._lib.INVALID_ARGUMENT and msg in str(e.value)
        with pytest.raises(ValueError):
            o.quantized_transpose(host(q), perm, 0.0, 1.0)
    with pytest.raises(itex.ItexError) as e:
        ops._ITEXQuantizedTranspose(q, (0, 1, 2), [0.0, 1.0], 1.0)
    assert "min_x must be a scalar or a vector of 1 element" in str(e.value)


@pytest.mark.parametrize("shape,new_shape", [((4, 128, 1024), (512, 1024)), ((4, 128, 1024), (4, 128, 16, -1)), ((6, 0, 5), (0, -1)),
                                             ((3, 7), (-1,)), ((2, 3, 4), (4, 3, 2))])
def test_quantized_reshape(shape, new_shape):
    itex, K, ops = modules()
    rng = np.random.default_rng(len(shape))
    x = rng.integers(0, 256, shape).astype(np.uint8)
    want, wmn, wmx = o.quantized_reshape(x, new_shape, 0.0, 6.0)
    for name, tshape in (("_ITEXQuantizedReshape", "int32"), ("QuantizedReshape", "int64")):
        y, mn, mx = ops._ITEXQuantizedReshape(dev(x), new_shape, 0.0, 6.0, Tshape=tshape, op_name=name)
        assert tuple(y.shape) == want.shape
        np.testing.assert_array_equal(host(y), want)
        assert (mn, mx) == (0.0, 6.0)


def test_quantized_reshape_errors():
    itex, K, ops = modules()
    q = dev(np.zeros((4, 6), np.int8))
    for new_shape, msg in (((-1, -1), "Only one input size may be -1"), ((5, -1), "requires a multiple of 5"), ((4, 5), "the requested shape has 20"),
                           ((-2, 12), "must be non-negative")):
        with pytest.raises(itex.ItexError) as e:
            ops._ITEXQuantizedReshape(q, new_shape, -1.0, 1.0)
        assert e.value.code == itex._lib.INVALID_ARGUMENT and msg in str(e.value)
        with pytest.raises(ValueError):
            o.quantized_reshape(host(q), new_shape, -1.0, 1.0)


@pytest.mark.parametrize("shapes,axis", [(((8, 28, 28, 64), (8, 28, 28, 96), (8, 28, 28, 32)), 3), (((8, 28, 28, 64), (8, 28, 28, 96)), -1),
                                         (((5, 7), (3, 7), (9, 7)), 0), (((2, 3, 5), (2, 4, 5)), 1), (((4, 0, 3), (4, 2, 3)), 1)])
def test_quantized_concat(shapes, axis):
    itex, K, ops = modules()
    rng = np.random.default_rng(len(shapes) + axis)
    vals = [rng.integers(0, 256, s).astype(np.uint8) for s in shapes]
    mins, maxes = [0.0] * len(vals), [5.5] * len(vals)
    want, wmn, wmx = o.quantized_concat_v2(vals, axis, mins, maxes)
    for name, tidx in (("_ITEXQuantizedConcatV2", "int32"), ("QuantizedConcatV2", "int64")):
        y, mn, mx = ops._ITEXQuantizedConcatV2([dev(v) for v in vals], axis, mins, maxes, Tidx=tidx, op_name=name)
        assert tuple(y.shape) == want.shape
        np.testing.assert_array_equal(host(y), want)
        assert (mn, mx) == (0.0, 5.5)


def test_quantized_concat_errors():
    itex, K, ops = modules()
    L = itex._lib
    a, b = dev(np.zeros((2, 3), np.int8)), dev(np.zeros((2, 4), np.int8))
    with pytest.raises(itex.ItexError) as e:           # the reference's kernel does not requantize either
        ops._ITEXQuantizedConcatV2([a, b], 1, [-1.0, -2.0], [1.0, 2.0])
    assert e.value.code == L.ABORTED and "unequal input_mins / input_maxes" in str(e.value)
    with pytest.raises(NotImplementedError):
        o.quantized_concat_v2([host(a), host(b)], 1, [-1.0, -2.0], [1.0, 2.0])
    for vals, axis, msg in (([a, b], 0, "Dimensions of inputs should match"), ([a, b], 2, "Expected concatenating dimensions"),
                            ([a, dev(np.zeros((2, 3, 1), np.int8))], 1, "Ranks of all input tensors should match")):
        with pytest.raises(itex.ItexError) as e:
            ops._ITEXQuantizedConcatV2(vals, axis, [-1.0, -1.0], [1.0, 1.0])
        assert e.value.code == L.INVALID_ARGUMENT and msg in str(e.value)
        with pytest.raises(ValueError):
            o.quantized_concat_v2([host(v) for v in vals], axis, [-1.0, -1.0], [1.0, 1.0])
