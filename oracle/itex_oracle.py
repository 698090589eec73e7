"""CPU restatement (NumPy) of the ITEX quantized-inference arithmetic.

TEST INFRASTRUCTURE ONLY.  This module is the checker the parity tests, the
smoke test and the CPU-baseline leg of the benchmark compare against.  The
product (the CUDA library) never imports or calls it.

Every function follows one reference function; citations are paths inside
intel/intel-extension-for-tensorflow.  All scalar host math is done in fp32
with the operator order of the cited lines, because re-associating changes
the last bit of a scale and therefore integer outputs at rounding ties.

Parity pins (see tests/test_oracle_golden.py):
  * quantize / dequantize: pinned bit-exact / 1e-5 against the reference's own
    known-answer tests (block_layout/quantized_ops_test.py,
    block_layout/dequantize_op_test.py).
  * int8 matmul / conv: pinned against real oneDNN (through
    torch.ops.onednn.q*_pointwise) by committed fixtures and against the
    reference's loose fp32-math tests.
  * FP8 ops and SCALED-mode input on the QuantizedMatMulWithBias* ops:
    PARITY UNPINNED - the reference has no test that exercises them.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np

f32 = np.float32

QINT8 = "qint8"
QUINT8 = "quint8"
QINT32 = "qint32"

_INT_LIMITS = {QINT8: (-128, 127), QUINT8: (0, 255), QINT32: (-(2 ** 31), 2 ** 31 - 1)}
_NP_OF = {QINT8: np.int8, QUINT8: np.uint8, QINT32: np.int32}


def _as_f32(x) -> np.ndarray:
    """bf16/f16/f32 -> f32 (exact widening)."""
    a = np.asarray(x)
    if a.dtype == np.float32:
        return a
    return a.astype(np.float32)


def to_bf16_rne(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 round-to-nearest-even, returned as f32 holding the bf16 value."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = np.isnan(x)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32).copy()
    out[nan] = np.float32(np.nan)
    return out


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 holding bf16-representable values (or any f32, RNE) -> uint16 bit pattern."""
    return (to_bf16_rne(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def sat_rne(f: np.ndarray, T: str) -> np.ndarray:
    """Saturate to T's full range then round to nearest even (oneDNN's f32->int
    conversion: clamp, then nearbyint under the default rounding mode)."""
    lo, hi = _INT_LIMITS[T]
    f = np.asarray(f, dtype=np.float32)
    # qint32: float(2^31-1) rounds to 2^31; clamp in f64 so the cast is defined.
    c = np.clip(f.astype(np.float64), lo, hi)
    c = np.where(np.isnan(c), 0.0, c)
    return np.rint(c).astype(np.int64).astype(_NP_OF[T])


# --------------------------------------------------------------------------
# QuantizeV2 / Dequantize
# --------------------------------------------------------------------------
def adjust_input_min_max(min_in: float, max_in: float, ensure_minimum_range: float = 0.01
                         ) -> Tuple[np.float32, np.float32]:
    """QuantizeV2Op::AdjustInputMinMaxRange, itex/core/kernels/common/quantize_op.h:130-152."""
    min_in, max_in, emr = f32(min_in), f32(max_in), f32(ensure_minimum_range)
    if not (max_in >= min_in):
        raise ValueError("input_max_range must be larger than input_min_range.")
    adj_min = min(f32(0.0), min_in)
    eps = f32(max(f32(1.0), max(abs(min_in), abs(max_in))) * emr)
    adj_max = max(f32(0.0), max(max_in, f32(adj_min + eps)))
    return f32(adj_min), f32(adj_max)


def scaled_scale(min_v: float, max_v: float, T: str, quantize: bool
                 ) -> Tuple[np.float32, np.float32]:
    """GetScaleAndZeropointAndAlignMinMax<T>, SCALED branch,
    itex/core/utils/quantization_util.h:61-71.  Returns (scale, abs_range)."""
    max_int = f32(_INT_LIMITS[T][1])  # int64 -> float in the division
    abs_range = f32(max(abs(f32(min_v)), abs(f32(max_v))))
    with np.errstate(divide="ignore", invalid="ignore"):
        scale = f32(max_int / abs_range) if quantize else f32(abs_range / max_int)
    return scale, abs_range


def min_first_scale_zp(min_v: float, max_v: float, T: str, quantize: bool):
    """GetScaleAndZeropointAndAlignMinMax<T>, MIN_FIRST branch,
    itex/core/utils/quantization_util.h:72-83."""
    lo, hi = _INT_LIMITS[T]
    min_v, max_v = f32(min_v), f32(max_v)
    if quantize:
        scale = f32(f32(hi - lo) / f32(max_v - min_v))
        zp = int(np.round(f32(f32(hi) - f32(max_v * scale))))
    else:
        scale = f32(f32(max_v - min_v) / f32(hi - lo))
        zp = int(np.round(f32(f32(hi) - f32(max_v / scale))))
    return scale, zp


def _per_slice(values: Sequence[float], shape, axis: int) -> np.ndarray:
    v = np.asarray(values, dtype=np.float32)
    if v.size == 1:
        return v.reshape([1] * len(shape))
    bs = [1] * len(shape)
    bs[axis] = shape[axis]
    return v.reshape(bs)


def quantize_v2(x, min_range, max_range, T: str = QINT8, mode: str = "SCALED",
                round_mode: str = "HALF_TO_EVEN", narrow_range: bool = False, axis: int = -1,
                ensure_minimum_range: float = 0.01, classic_asymmetric_algorithm: bool = False):
    """_ITEXQuantizeV2, QuantizeV2Op::Compute, itex/core/kernels/common/quantize_op.h:154-417.

    narrow_range is read and ignored (quantize_op.h:58-60); round_mode is validated
    in the constructor (:95-117) and otherwise unused - the oneDNN reorder always
    rounds to nearest even.  A negative axis means per-tensor (`axis_ > -1` test, :167).
    Returns (q, output_min, output_max) with output_min/max scalars or [num_slices].
    """
    if mode not in ("MIN_COMBINED", "MIN_FIRST", "SCALED"):
        raise ValueError("Mode string must be 'MIN_COMBINED', 'MIN_FIRST', or 'SCALED', is '%s'" % mode)
    if mode == "MIN_COMBINED":
        raise ValueError("_ITEXQuantizeV2 only supports SCALED and MIN_FIRST MODE")
    if round_mode not in ("HALF_AWAY_FROM_ZERO", "HALF_TO_EVEN"):
        raise ValueError("Round mode string must be 'HALF_AWAY_FROM_ZERO' or 'HALF_TO_EVEN', is '%s'" % round_mode)
    if round_mode == "HALF_TO_EVEN" and mode != "SCALED":
        raise ValueError("Round mode 'HALF_TO_EVEN' only supported for mode 'SCALED', but mode is '%s'." % mode)
    xf = _as_f32(x)
    mins = np.atleast_1d(np.asarray(min_range, dtype=np.float32))
    maxs = np.atleast_1d(np.asarray(max_range, dtype=np.float32))
    num_slices = mins.size if axis > -1 else 1
    adj = [adjust_input_min_max(mins[i], maxs[i], ensure_minimum_range) for i in range(num_slices)]
    mn = np.array([a[0] for a in adj], dtype=np.float32)
    mx = np.array([a[1] for a in adj], dtype=np.float32)
    if mode == "SCALED":
        sc = np.empty(num_slices, np.float32)
        for i in range(num_slices):
            sc[i], ab = scaled_scale(mn[i], mx[i], T, True)
            mn[i], mx[i] = -ab, ab
        scale = _per_slice(sc, xf.shape, axis)
        q = sat_rne(xf * scale, T)
        out_min = np.zeros_like(mn) if T == QUINT8 else mn
        out_max = mx
    elif classic_asymmetric_algorithm:
        sc = np.empty(num_slices, np.float32)
        zp = np.empty(num_slices, np.float32)
        for i in range(num_slices):
            sc[i], z = min_first_scale_zp(mn[i], mx[i], T, True)
            zp[i] = z
        f = xf * _per_slice(sc, xf.shape, axis) + _per_slice(zp, xf.shape, axis)
        q = sat_rne(f, T)
        out_min, out_max = mn, mx
    else:
        # legacy MIN_FIRST: binary_add(src, shift) with the same scale on both
        # sources (quantize_op.h:185-195, 292-314): (x*s) + ((-min)*s).
        steps = f32((1 << (8 * np.dtype(_NP_OF[T]).itemsize)) - 1.0)
        sc = (steps / (mx - mn)).astype(np.float32)
        s = _per_slice(sc, xf.shape, axis)
        shift = _per_slice(-mn, xf.shape, axis)
        q = sat_rne(xf * s + shift * s, T)
        out_min, out_max = mn, mx
    if num_slices == 1:
        return q, f32(out_min[0]), f32(out_max[0])
    return q, out_min, out_max


def dequantize(q, min_range, max_range, T: Optional[str] = None, mode: str = "SCALED",
               narrow_range: bool = False, axis: int = -1, dtype: str = "float"):
    """_ITEXDequantize, DequantizeOp::Compute, itex/core/kernels/common/dequantize_op.h:67-178.
    y = dtype((float(q) - zp) * scale); zp = 0 in SCALED mode."""
    q = np.asarray(q)
    if T is None:
        T = QINT8 if q.dtype == np.int8 else QUINT8
    if mode not in ("MIN_FIRST", "SCALED"):
        raise ValueError("_ITEXDequantize only supports SCALED and MIN_FIRST MODE")
    mins = np.atleast_1d(np.asarray(min_range, dtype=np.float32))
    maxs = np.atleast_1d(np.asarray(max_range, dtype=np.float32))
    num_slices = mins.size if axis > -1 else 1
    sc = np.empty(num_slices, np.float32)
    zp = np.zeros(num_slices, np.float32)
    for i in range(num_slices):
        if mode == "SCALED":
            sc[i], _ = scaled_scale(mins[i], maxs[i], T, False)
        else:
            sc[i], z = min_first_scale_zp(mins[i], maxs[i], T, False)
            zp[i] = z
    qf = q.astype(np.float32)
    y = (qf - _per_slice(zp, q.shape, axis)) * _per_slice(sc, q.shape, axis)
    y = y.astype(np.float32)
    if dtype in ("bfloat16", "bf16"):
        return to_bf16_rne(y)
    if dtype in ("half", "float16", "f16"):
        return y.astype(np.float16)
    return y


# --------------------------------------------------------------------------
# int8 matmul family
# --------------------------------------------------------------------------
def int_matmul(a: np.ndarray, b_kn: np.ndarray) -> np.ndarray:
    """Exact Σ_k a[m,k]·b[k,n] as int32 (f64 BLAS is exact below 2^53)."""
    acc = a.astype(np.float64) @ b_kn.astype(np.float64)
    return acc.astype(np.int64).astype(np.int32)


def float_for_one_quantized_level(range_min, range_max, T: str) -> np.float32:
    """OneDnnFloatForOneQuantizedLevel<T>, itex/core/kernels/onednn/block/quantized_ops.h:24-36."""
    lo, hi = _INT_LIMITS[T]
    if lo < -hi:
        lo += 1
    return f32(f32(f32(range_max) - f32(range_min)) / f32(hi - lo))


def quantization_range_for_multiplication(min_a, max_a, min_b, max_b, T1=QUINT8, T2=QINT8
                                          ) -> Tuple[np.float32, np.float32]:
    """OneDnnQuantizationRangeForMultiplication<T1,T2,qint32>, quantized_ops.h:38-54."""
    c = f32(float_for_one_quantized_level(min_a, max_a, T1) * float_for_one_quantized_level(min_b, max_b, T2))
    return f32(c * f32(-(2 ** 31))), f32(c * f32(2 ** 31 - 1))


def matmul_output_scale(min_a, max_a, min_b0, max_b0, toutput: str,
                        min_freezed=None, max_freezed=None) -> Optional[np.float32]:
    """QuantizedMatMulOp::ExtendInt8PostOps, quantized_matmul_common.h:1472-1508.
    Returns None for Toutput=qint32 (no output scale is set)."""
    if toutput == QINT32:
        return None
    mn, mx = quantization_range_for_multiplication(min_a, max_a, min_b0, max_b0)
    scale_int32 = f32(max(abs(mn), abs(mx)))
    if toutput in ("float", "bfloat16", "half"):
        return f32(scale_int32 / f32(2.0 ** 31))
    scale_eightbit = f32(max(abs(f32(min_freezed)), abs(f32(max_freezed))))
    if toutput == QUINT8:
        return f32(f32(scale_int32 / scale_eightbit) / f32(1 << 23))
    return f32(f32(scale_int32 / scale_eightbit) / f32(1 << 24))


def matmul_scaled_bias(bias, b_kn, min_a, max_a, min_b, max_b, mode: str, toutput: str,
                       out_scale, tbias: str = "float", scaled_bias_mode: str = "literal",
                       t1: str = QUINT8) -> np.ndarray:
    """GetScaledBias: float bias quantized_matmul_common.h:466-660; qint32 bias :1153-1334.

    scaled_bias_mode selects how the SCALED-mode float bias is treated:
      "literal"  - bias * 255*127/(ri*rw)  (what the cited lines compute)
      "intended" - the bias expressed in the units of the value it is added to (what the primitive's
                   y = scale*acc + b needs): unchanged for float outputs, times the requantize factor for 8-bit
                   outputs, times 255*127/(ri*rw) for qint32 outputs
    """
    n = b_kn.shape[1]
    lim = f32(255.0) if t1 == QUINT8 else f32(127.0)   # max_int8_input, :509-510
    min_a, max_a = f32(min_a), f32(max_a)
    min_b = np.atleast_1d(np.asarray(min_b, np.float32))
    max_b = np.atleast_1d(np.asarray(max_b, np.float32))
    ri = f32(max_a - min_a) if mode == "MIN_FIRST" else f32(max(abs(min_a), abs(max_a)))
    rw = np.maximum(np.abs(min_b), np.abs(max_b)).astype(np.float32)
    os_ = None if out_scale is None else np.broadcast_to(np.atleast_1d(np.asarray(out_scale, np.float32)), (n,)) \
        if np.size(out_scale) in (1, n) else None
    if tbias == QINT32:
        bf = np.asarray(bias).astype(np.int32).astype(np.float32)
        s = (f32(ri) * rw / f32(lim * f32(127.0))).astype(np.float32)
        s = np.broadcast_to(s, (n,)) if s.size == 1 else s
        if mode == "MIN_FIRST":
            if toutput in ("float", "bfloat16", "half"):
                return (bf * s).astype(np.float32)
            if toutput in (QUINT8, QINT8):
                return (bf * os_).astype(np.float32)
            return bf
        return (bf * s).astype(np.float32)
    bias = _as_f32(bias)
    s = (f32(lim * f32(127.0)) / (f32(ri) * rw)).astype(np.float32)
    s = np.broadcast_to(s, (n,)) if s.size == 1 else s
    if mode == "MIN_FIRST":
        colsum = b_kn.astype(np.int32).sum(axis=0, dtype=np.int32)
        qmin = f32(lim * min_a / ri)
        cs = colsum.astype(np.float32)  # `sum * q_min_input` promotes the int to float
        if toutput in ("float", "bfloat16", "half"):
            return (bias + (cs * qmin / s)).astype(np.float32)
        if toutput in (QUINT8, QINT8):
            return (bias * s * os_ + (cs * qmin * os_)).astype(np.float32)
        return (bias * s + (cs * qmin)).astype(np.float32)
    if scaled_bias_mode == "intended":
        # the bias in the units of the value it is added to, i.e. the MIN_FIRST formulas without compensation
        if toutput in ("float", "bfloat16", "half"):
            return bias.astype(np.float32).copy()
        if toutput in (QUINT8, QINT8):
            return (bias * s * os_).astype(np.float32)
        return (bias * s).astype(np.float32)
    return (bias * s).astype(np.float32)


def epilogue(acc: np.ndarray, scale, bias, relu: bool, toutput: str,
             summand=None, sum_scale: float = 1.0) -> np.ndarray:
    """oneDNN int8 primitive tail: f=(float)acc; f*=scale[n]; f+=bias[n]; [f=fma(sum_scale, summand, f)];
    [relu]; convert (ints: saturate + RNE; floats: cast).  The scale multiply and the bias add are separate fp32
    roundings; the sum post-op is ONE fused multiply-add, which is what oneDNN's kernels execute: with real oneDNN
    (tests/golden/onednn_conv_sum.npz) the separate-rounding model is off by one on rounding ties, the fused one is
    exact.  The fused multiply-add is formed in float64 (the product of a float and an 8- or 16-bit summand is exact
    there, and so is the sum for all but astronomically distant exponents) and rounded once to float32."""
    f = acc.astype(np.float32)
    if scale is not None:
        f = (f * np.asarray(scale, np.float32)).astype(np.float32)
    if bias is not None:
        f = (f + np.asarray(bias, np.float32)).astype(np.float32)
    if summand is not None:
        f = (np.float64(f32(sum_scale)) * np.asarray(summand).astype(np.float32).astype(np.float64) + f.astype(np.float64)).astype(np.float32)
    if relu:
        f = np.maximum(f, f32(0.0))
    if toutput == "float":
        return f
    if toutput == "bfloat16":
        return to_bf16_rne(f)
    if toutput == "half":
        return f.astype(np.float16)
    return sat_rne(f, toutput)


def quantized_matmul_with_bias(a, b, bias, min_a, max_a, min_b, max_b,
                               min_freezed_output=None, max_freezed_output=None, *,
                               toutput: str = QINT32, relu: bool = False, tbias: str = "float",
                               transpose_a: bool = False, transpose_b: bool = False,
                               input_quant_mode: str = "MIN_FIRST", scaled_bias_mode: str = "literal"):
    """_ITEXQuantizedMatMulWithBias[AndRelu][AndRequantize|AndDequantize]
    (QuantizedMatMulOp / QuantizedMatMulReluOp over LegacyQuantizedMatMulOpBase,
    itex/core/kernels/common/quantized_matmul_common.h:61-336, 1414-1531).

    Returns (out, min_out, max_out); min/max are None for float outputs
    (AllocateNativeOutputMinMax, onednn/block/quantized_ops.h:142-203)."""
    if input_quant_mode not in ("MIN_FIRST", "SCALED"):
        raise ValueError("Quantization mode must be either MIN_FIRST or SCALED, but received " + input_quant_mode)
    a = np.asarray(a)
    b = np.asarray(b)
    a_mk = a.T if transpose_a else a
    b_kn = b.T if transpose_b else b
    acc = int_matmul(a_mk, b_kn)
    mb0 = np.atleast_1d(np.asarray(min_b, np.float32))[0]
    xb0 = np.atleast_1d(np.asarray(max_b, np.float32))[0]
    scale = matmul_output_scale(min_a, max_a, mb0, xb0, toutput, min_freezed_output, max_freezed_output)
    bias_s = matmul_scaled_bias(bias, b_kn, min_a, max_a, min_b, max_b, input_quant_mode, toutput,
                                scale, tbias, scaled_bias_mode)
    out = epilogue(acc, scale, bias_s, relu, toutput)
    if toutput in (QUINT8, QINT8):
        return out, f32(min_freezed_output), f32(max_freezed_output)
    if toutput == QINT32:
        mbv = np.atleast_1d(np.asarray(min_b, np.float32))
        xbv = np.atleast_1d(np.asarray(max_b, np.float32))
        if np.ndim(min_b) == 0:
            mn, mx = quantization_range_for_multiplication(min_a, max_a, mbv[0], xbv[0])
            return out, mn, mx
        r = [quantization_range_for_multiplication(min_a, max_a, mbv[i], xbv[i]) for i in range(mbv.size)]
        return out, np.array([x[0] for x in r], np.float32), np.array([x[1] for x in r], np.float32)
    return out, None, None


def fused_matmul_output_scale(min_a, max_a, min_b, max_b, t1: str, n: int, mode: str = "SCALED") -> np.ndarray:
    """Per-channel dequantize scale of QuantizedFusedMatMulOp / V2,
    quantized_matmul_common.h:1610-1650, 1817-1842: ri*rw[j]/(max_int8_in*127)."""
    min_a, max_a = f32(min_a), f32(max_a)
    lim = f32(255.0) if t1 == QUINT8 else f32(127.0)
    ri = f32(max_a - min_a) if mode == "MIN_FIRST" else f32(max(abs(min_a), abs(max_a)))
    rw = np.maximum(np.abs(np.atleast_1d(np.asarray(min_b, np.float32))),
                    np.abs(np.atleast_1d(np.asarray(max_b, np.float32)))).astype(np.float32)
    sc = ((ri * rw).astype(np.float32) / f32(lim * f32(127.0))).astype(np.float32)
    return np.broadcast_to(sc, (n,)).copy() if sc.size == 1 else sc


ACTIVATIONS = ("Relu", "LeakyRelu", "Relu6", "GeluExact", "GeluApproximate", "Sigmoid", "Tanh", "Elu", "_ITEXSwish")


def activation(f: np.ndarray, name: str, leakyrelu_alpha: float = 0.2) -> np.ndarray:
    """Element-wise post-ops by their fused_ops names, with the oneDNN algorithms and alpha/beta of
    PostOpUtil::GetAllPostOpInfo (itex/core/utils/onednn/onednn_post_op_util.cc:22-71).  Evaluated in
    float64 and rounded once to fp32 (oneDNN's own kernels use polynomial approximations; the GPU
    tests compare at 1e-5)."""
    x = f.astype(np.float64)
    if name == "Relu":
        y = np.maximum(x, 0.0)
    elif name == "LeakyRelu":
        y = np.where(x > 0, x, x * np.float64(f32(leakyrelu_alpha)))
    elif name == "Relu6":
        y = np.clip(x, 0.0, 6.0)
    elif name == "GeluExact":
        from math import erf
        y = 0.5 * x * (1.0 + np.vectorize(erf)(x / np.sqrt(2.0)))
    elif name == "GeluApproximate":
        y = 0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x ** 3)))
    elif name == "Sigmoid":
        y = 1.0 / (1.0 + np.exp(-x))
    elif name == "Tanh":
        y = np.tanh(x)
    elif name == "Elu":
        y = np.where(x > 0, x, np.expm1(x))
    elif name == "_ITEXSwish":
        y = x / (1.0 + np.exp(-x))
    else:
        raise ValueError("Found unsupported fusion: " + name)
    return y.astype(np.float32)


def quantized_fused_matmul(a, b, bias, min_a, max_a, min_b, max_b, min_freezed_output=None, max_freezed_output=None, *,
                           fused_ops=("BiasAdd",), t1: str = QUINT8, toutput: str = "float", tbias: str = "float",
                           input_quant_mode: str = "SCALED", addend=None, transpose_a: bool = False,
                           transpose_b: bool = False, leakyrelu_alpha: float = 0.2,
                           scaled_bias_mode: str = "literal", postop_scale_mode: str = "intended"):
    """_[ITEX]QuantizedFusedMatMul[AndRequantize|AndDequantize] and _[ITEX]QuantizedMatMul (V2):
    QuantizedFusedMatMulOp / QuantizedFusedMatMulV2Op, quantized_matmul_common.h:1534-1908, over the
    same base class as the WithBias ops (bias scaling :466-660, output ranges quantized_ops.h:142-203).

    fused_ops: BiasAdd, then optionally "Add" (sum post-op, scale 1, float outputs only) and/or one
    activation; "Dequantize"/"Requantize" entries (V2 spelling) are accepted and ignored - the output kind
    is given by `toutput`.  postop_scale_mode: "intended" multiplies the activation's result by
    max_int8_output/range_output when requantizing after an activation (what :1669-1700, 1866-1884 compute);
    "literal" drops it, as oneDNN 3 eltwise post-ops take no scale (onednn_post_op_util.cc:255).
    Returns (out, min_out, max_out) like quantized_matmul_with_bias."""
    a = np.asarray(a)
    b = np.asarray(b)
    a_mk = a.T if transpose_a else a
    b_kn = b.T if transpose_b else b
    n = b_kn.shape[1]
    acts = [f for f in fused_ops if f in ACTIVATIONS]
    if len(acts) > 1:
        raise ValueError("more than one activation in fused_ops")
    act = acts[0] if acts else None
    has_bias = "BiasAdd" in fused_ops
    has_add = "Add" in fused_ops
    if has_add and toutput not in ("float", "bfloat16", "half"):
        raise NotImplementedError("Quantized addend tensor is not implemented yet.")
    acc = int_matmul(a_mk, b_kn)
    scale, post = None, f32(1.0)
    if toutput != QINT32:
        scale = fused_matmul_output_scale(min_a, max_a, min_b, max_b, t1, np.size(min_b), input_quant_mode)
        if toutput in (QUINT8, QINT8):
            ro = f32(max(abs(f32(min_freezed_output)), abs(f32(max_freezed_output))))
            factor = f32((f32(255.0) if toutput == QUINT8 else f32(127.0)) / ro)
            if act is None:
                scale = (scale * factor).astype(np.float32)
            elif postop_scale_mode == "intended":
                post = factor
    bias_s = None
    if has_bias:
        bias_s = matmul_scaled_bias(bias, b_kn, min_a, max_a, min_b, max_b, input_quant_mode, toutput, scale, tbias,
                                    scaled_bias_mode, t1)
    f = acc.astype(np.float32)
    if scale is not None:
        f = (f * (scale if scale.size > 1 else scale[0])).astype(np.float32)
    if bias_s is not None:
        f = (f + bias_s).astype(np.float32)
    if has_add:
        f = (f + np.asarray(addend).astype(np.float32)).astype(np.float32)
    if act is not None:
        f = (activation(f, act, leakyrelu_alpha) * post).astype(np.float32)
    if toutput == "float":
        out = f
    elif toutput == "bfloat16":
        out = to_bf16_rne(f)
    elif toutput == "half":
        out = f.astype(np.float16)
    else:
        out = sat_rne(f, toutput)
    if toutput in (QUINT8, QINT8):
        return out, f32(min_freezed_output), f32(max_freezed_output)
    if toutput == QINT32:
        mbv = np.atleast_1d(np.asarray(min_b, np.float32))
        xbv = np.atleast_1d(np.asarray(max_b, np.float32))
        r = [quantization_range_for_multiplication(min_a, max_a, mbv[i], xbv[i], t1) for i in range(mbv.size)]
        if np.ndim(min_b) == 0:
            return out, r[0][0], r[0][1]
        return out, np.array([x[0] for x in r], np.float32), np.array([x[1] for x in r], np.float32)
    return out, None, None


# --------------------------------------------------------------------------
# int8 conv
# --------------------------------------------------------------------------
def quantized_batch_matmul(x, y, min_x, max_x, min_y, max_y, *, fused_ops=(), mul=None, addend=None, adj_x: bool = False,
                           adj_y: bool = False, toutput: str = "float") -> np.ndarray:
    """_[ITEX]QuantizedBatchMatMulV2AndDequantize, _[ITEX]QuantizedFusedBatchMatMulV2AndDequantize and
    _[ITEX]QuantizedBatchMatMul: QuantizedBatchMatMulV2Op, itex/core/kernels/common/batch_matmul_op.h:441-522.
    qint8 x qint8 (the types registered for the GPU, itex/core/kernels/gpu/matmul_op.cc:612-654), batch dims
    broadcast (MatMulBCast, :104-128); output = acc * range_x*range_y/(127*127) (AccumulateMulAndInt8Scale
    :497-514), then the binary post-ops in fused_ops order: "Mul" by `mul` and "Add" of `addend`, both broadcast
    to the output (:350-377).  "Dequantize" entries (V2 spelling) are ignored."""
    x = np.asarray(x).astype(np.int64)
    y = np.asarray(y).astype(np.int64)
    if adj_x:
        x = np.swapaxes(x, -1, -2)
    if adj_y:
        y = np.swapaxes(y, -1, -2)
    acc = np.matmul(x, y)
    assert np.abs(acc).max(initial=0) < 2 ** 31
    range_lhs = f32(max(abs(f32(min_x)), abs(f32(max_x))))
    range_rhs = f32(max(abs(f32(min_y)), abs(f32(max_y))))
    scale_output = f32(f32(range_lhs * range_rhs) / f32(f32(127.0) * f32(127.0)))
    f = (acc.astype(np.float32) * scale_output).astype(np.float32)
    for op in fused_ops:
        if op == "Mul":
            f = (f * _as_f32(mul)).astype(np.float32)
        elif op == "Add":
            f = (f + _as_f32(addend)).astype(np.float32)
        elif op != "Dequantize":
            raise NotImplementedError("Fusion is not implemented for QuantizedBatchMatMul: [%s]" % op)
    if toutput == "bfloat16":
        return to_bf16_rne(f)
    if toutput == "half":
        return f.astype(np.float16)
    return f


def same_padding(in_size: int, k: int, stride: int, dilation: int = 1) -> Tuple[int, int, int]:
    """GetWindowedOutputSizeVerboseV2, SAME branch, itex/core/utils/common_shape_fns.cc:42-81.
    Returns (out_size, pad_before, pad_after); the extra pixel goes after."""
    eff = (k - 1) * dilation + 1
    out = (in_size + stride - 1) // stride
    need = max(0, (out - 1) * stride + eff - in_size)
    return out, need // 2, need - need // 2


def valid_padding(in_size: int, k: int, stride: int, dilation: int = 1) -> Tuple[int, int, int]:
    eff = (k - 1) * dilation + 1
    return (in_size - eff + stride) // stride, 0, 0


def int_conv2d_nhwc(x: np.ndarray, f_hwio: np.ndarray, strides=(1, 1), padding="SAME",
                    dilations=(1, 1), explicit_pads=None) -> np.ndarray:
    """Exact int32 NHWC x HWIO convolution with zero padding."""
    n, h, w, c = x.shape
    kh, kw, ci, co = f_hwio.shape
    assert ci == c
    sh, sw = strides
    dh, dw = dilations
    if padding == "SAME":
        oh, pt, pb = same_padding(h, kh, sh, dh)
        ow, pl, pr = same_padding(w, kw, sw, dw)
    elif padding == "VALID":
        oh, pt, pb = valid_padding(h, kh, sh, dh)
        ow, pl, pr = valid_padding(w, kw, sw, dw)
    else:
        pt, pb, pl, pr = explicit_pads
        oh = (h + pt + pb - ((kh - 1) * dh + 1)) // sh + 1
        ow = (w + pl + pr - ((kw - 1) * dw + 1)) // sw + 1
    xp = np.zeros((n, h + pt + pb + kh * dh, w + pl + pr + kw * dw, c), dtype=np.float64)
    xp[:, pt:pt + h, pl:pl + w, :] = x
    acc = np.zeros((n, oh, ow, co), dtype=np.float64)
    ff = f_hwio.astype(np.float64)
    for i in range(kh):
        for j in range(kw):
            patch = xp[:, i * dh:i * dh + (oh - 1) * sh + 1:sh, j * dw:j * dw + (ow - 1) * sw + 1:sw, :]
            acc += np.tensordot(patch, ff[i, j], axes=([3], [0]))
    return acc.astype(np.int64).astype(np.int32)


def conv_output_scale(min_input, max_input, min_filter, max_filter, tinput: str, toutput: str,
                      min_freezed=None, max_freezed=None) -> np.ndarray:
    """LegacyQuantizedConvOpBase::ExtendInt8PostOps, quantized_conv_ops.h:329-395."""
    mf = np.atleast_1d(np.asarray(min_filter, np.float32))
    xf = np.atleast_1d(np.asarray(max_filter, np.float32))
    depth = mf.size
    scales = np.ones(depth, np.float32)
    if toutput == QINT32:
        return scales
    min_input, max_input = f32(min_input), f32(max_input)
    if toutput in ("float", "bfloat16", "half"):
        lim_in = f32(255.0) if tinput == QUINT8 else f32(127.0)
        src_q = f32(max(abs(min_input), abs(max_input)) / lim_in)
        for i in range(depth):
            wei_q = f32(max(abs(mf[i]), abs(xf[i])) / f32(127.0))
            scales[i] = f32(src_q * wei_q)
        return scales
    lim_out = f32(255.0) if toutput == QUINT8 else f32(127.0)
    ri = f32(max(abs(min_input), abs(max_input)))
    ro = f32(max(abs(f32(min_freezed)), abs(f32(max_freezed))))
    lim = f32(255.0 * 127.0) if tinput == QUINT8 else f32(127.0 * 127.0)
    for i in range(depth):
        rf = f32(max(abs(mf[i]), abs(xf[i])))
        scales[i] = f32(f32(f32(lim_out * ri) * rf) / f32(lim * ro))
    return scales


def conv_scaled_bias(bias, min_input, max_input, min_filter, max_filter, tinput: str, toutput: str,
                     scales: np.ndarray, tbias: str = "float") -> np.ndarray:
    """LegacyQuantizedConvOpBase::GetBiasHandle, quantized_conv_ops.h:448-597."""
    mf = np.atleast_1d(np.asarray(min_filter, np.float32))
    xf = np.atleast_1d(np.asarray(max_filter, np.float32))
    depth = mf.size
    min_input, max_input = f32(min_input), f32(max_input)
    lim = f32(255.0 * 127.0) if tinput == QUINT8 else f32(127.0 * 127.0)
    ri = f32(max(abs(max_input), abs(min_input)))
    if tbias == QINT32:
        bf = np.asarray(bias).astype(np.int32).astype(np.float32)
        if toutput == QINT32:
            return bf
        if toutput in ("float", "bfloat16", "half"):
            s = np.array([f32(f32(ri * f32(max(abs(xf[i]), abs(mf[i])))) / lim) for i in range(depth)], np.float32)
        else:
            s = scales
        return (bf * s).astype(np.float32)
    bias = _as_f32(bias)
    s = np.empty(depth, np.float32)
    for i in range(depth):
        tmp = f32(lim / f32(ri * f32(max(abs(xf[i]), abs(mf[i])))))
        s[i] = f32(tmp * scales[i])
    return (bias * s).astype(np.float32)


def quantized_conv2d(x, filt, bias, min_input, max_input, min_filter, max_filter,
                     min_freezed_output=None, max_freezed_output=None, *, strides=(1, 1, 1, 1),
                     padding="SAME", dilations=(1, 1, 1, 1), explicit_pads=None, out_type: str = QUINT8,
                     relu: bool = True, tbias: str = "float", summand=None, min_summand=None,
                     max_summand=None, activation_name: Optional[str] = None, alpha: float = 0.0):
    """_ITEXQuantizedConv2DWithBias[AndRelu]AndRequantize (+ Sum variants, + Dequantize-fused
    variant when out_type is a float type).  LegacyQuantizedConvOpBase,
    itex/core/kernels/common/quantized_conv_ops.h:71-729 over ConvOpBase
    (itex/core/kernels/common/conv_ops.h:718-1133).  NHWC input, HWIO filter."""
    x = np.asarray(x)
    tinput = QUINT8 if x.dtype == np.uint8 else QINT8
    acc = int_conv2d_nhwc(x, np.asarray(filt), (strides[1], strides[2]), padding,
                          (dilations[1], dilations[2]), explicit_pads)
    scales = conv_output_scale(min_input, max_input, min_filter, max_filter, tinput, out_type,
                               min_freezed_output, max_freezed_output)
    b = None if bias is None else conv_scaled_bias(bias, min_input, max_input, min_filter, max_filter,
                                                    tinput, out_type, scales, tbias)
    sum_scale = 1.0
    if summand is not None and out_type != QINT32:
        so = f32(max(abs(f32(min_freezed_output)), abs(f32(max_freezed_output))))
        ss = f32(max(abs(f32(min_summand)), abs(f32(max_summand))))
        if out_type == QUINT8 and np.asarray(summand).dtype == np.int8:
            sum_scale = f32(f32(f32(255.0) * ss) / f32(so * f32(127.0)))
        else:
            sum_scale = f32(ss / so)
    if out_type == QINT32 and b is None and not relu and summand is None and activation_name is None:
        out = acc.astype(np.int32)   # no post-op at all: the accumulators themselves
    elif activation_name is None:
        out = epilogue(acc, scales if out_type != QINT32 else None, b, relu, out_type, summand, sum_scale)
    else:
        # new-API element-wise post-ops run on the scaled value with post-op scale 1 (quantized_conv_ops.h:437-445)
        f = epilogue(acc, scales if out_type != QINT32 else None, b, relu, "float", summand, sum_scale)
        f = activation(f, activation_name, alpha)
        out = f if out_type == "float" else (to_bf16_rne(f) if out_type == "bfloat16" else sat_rne(f, out_type))
    if out_type in (QUINT8, QINT8):
        return out, f32(min_freezed_output), f32(max_freezed_output)
    if out_type == QINT32:
        # AllocateNativeOutputMinMax, onednn/block/quantized_ops.h:166-195: per filter range
        mf = np.atleast_1d(np.asarray(min_filter, np.float32))
        xf = np.atleast_1d(np.asarray(max_filter, np.float32))
        r = [quantization_range_for_multiplication(min_input, max_input, mf[i], xf[i], tinput) for i in range(mf.size)]
        if np.ndim(min_filter) == 0:
            return out, r[0][0], r[0][1]
        return out, np.array([v[0] for v in r], np.float32), np.array([v[1] for v in r], np.float32)
    return out, None, None


def quantize_v2_with_quantized_conv2d(x, filt, bias, min_input, max_input, min_filter, max_filter, min_freezed_output,
                                      max_freezed_output, *, ensure_minimum_range: float = 0.01, **conv_kwargs):
    """_ITEXQuantizeV2WithQuantizedConv2D: the QuantizeV2 (SCALED, to quint8) the remapper folds into the
    _ITEXQuantizedConv2DWithBiasAndReluAndRequantize it feeds (itex/core/graph/remapper/remapper.cc:2099-2123; kernel
    OneDnnQuantizeV2WithQuantizedConv2DOp, itex/core/kernels/onednn/block/conv_ops_impl.h:1238-1420).  min_input /
    max_input are the QuantizeV2's range inputs; the convolution sees the range the quantize step outputs."""
    q, qmin, qmax = quantize_v2(x, min_input, max_input, T=QUINT8, mode="SCALED", ensure_minimum_range=ensure_minimum_range)
    return quantized_conv2d(q, filt, bias, qmin, qmax, min_filter, max_filter, min_freezed_output, max_freezed_output,
                            out_type=QUINT8, relu=True, **conv_kwargs)


# --------------------------------------------------------------------------
# FP8 (parity unpinned: the reference has no FP8 test)
# --------------------------------------------------------------------------
FP8_MAX = {"E4M3": 448.0, "E5M2": 57344.0}  # itex/python/fp8/recipe.py:27


def _fp8_np(fp8_dtype: str):
    import ml_dtypes
    return ml_dtypes.float8_e4m3fn if fp8_dtype == "E4M3" else ml_dtypes.float8_e5m2


def fp8_cast_sat(f: np.ndarray, fp8_dtype: str = "E4M3") -> np.ndarray:
    """float -> fp8 bits (uint8): RNE; finite values beyond the largest finite code saturate to it; NaN stays NaN;
    an infinite input gives the target's numeric_limits::infinity(), i.e. NaN for e4m3fn and +-inf for e5m2
    (itex/core/utils/float8.h:72-74 kSaturate=true; ConvertImpl::run :651-766: the infinity test at :665-668
    comes before the saturating overflow branch at :713-718; infinity() at :313-315 and :400)."""
    f = np.asarray(f, np.float32)
    m = f32(FP8_MAX[fp8_dtype])
    c = np.where(np.isinf(f), f, np.clip(f, -m, m))  # clip keeps NaN; the cast below maps inf to NaN (e4m3fn) or inf (e5m2)
    return c.astype(_fp8_np(fp8_dtype)).view(np.uint8)


def fp8_to_f32(bits: np.ndarray, fp8_dtype: str = "E4M3") -> np.ndarray:
    return np.asarray(bits).view(np.uint8).view(_fp8_np(fp8_dtype)).astype(np.float32)


def fp8_quantize(x, amax_row0: np.ndarray, scale: np.ndarray, fp8_meta_index: int,
                 fp8_dtype: str = "E4M3") -> np.ndarray:
    """Fp8Quantize (itex/core/kernels/gpu/fp8/fp8_quantize_op.cc:24-49; kernel
    vectorized_pointwise.h:43-77): y = fp8(float(x)*scale[i]); amax[i] = max(amax[i], max|x|).
    amax_row0 is mutated in place like the op mutates row 0 of amax_history."""
    t = _as_f32(x)
    amax = f32(np.max(np.abs(t))) if t.size else f32(0)
    amax_row0[fp8_meta_index] = max(f32(amax_row0[fp8_meta_index]), amax)
    return fp8_cast_sat((t * f32(scale[fp8_meta_index])).astype(np.float32), fp8_dtype)


def fp8_gelu(x, amax_row0: np.ndarray, scale: np.ndarray, fp8_meta_index: int, fp8_dtype: str = "E4M3") -> np.ndarray:
    """Fp8Gelu: functor::Fp8Gelu over PointWiseKernel (itex/core/kernels/gpu/fp8/fp8_gelu_gpu.h:29-58,
    vectorized_pointwise.h:43-77): g = gelu(x) in fp32, amax raised to max|g|, y = fp8(g * scale).  Parity unpinned."""
    v = _as_f32(x).astype(np.float64)
    g = (v * (0.5 + 0.5 * np.tanh(v * (0.79788456 + 0.03567741 * v * v)))).astype(np.float32)
    amax_row0[fp8_meta_index] = max(f32(amax_row0[fp8_meta_index]), f32(np.abs(g).max())) if g.size else amax_row0[fp8_meta_index]
    return fp8_cast_sat((g * f32(scale[fp8_meta_index])).astype(np.float32), fp8_dtype)


def fp8_dgelu(x) -> np.ndarray:
    """dgelu(), itex/core/kernels/gpu/fp8/fp8_quantize_fusion_gpu.h:33-43 (float64 here, rounded to fp32)."""
    v = _as_f32(x).astype(np.float64)
    th = np.tanh(0.79788456 * v * (1.0 + 0.044715 * v * v))
    return (0.5 * v * ((1.0 - th * th) * (0.79788456 + 0.1070322243 * v * v)) + 0.5 * (1.0 + th)).astype(np.float32)


def fp8_quantize_dbias(grad, amax_row0: np.ndarray, scale: np.ndarray, fp8_meta_index: int, fp8_dtype: str = "E5M2", gelu_inp=None,
                       out_dtype: str = "float"):
    """Fp8QuantizeDbias / Fp8QuantizeDbiasDgelu (itex/core/kernels/gpu/fp8/fp8_quantize_fusion_op.cc:24-104; kernels
    fp8_quantize_fusion_gpu.h:45-300): t = grad, or dgelu(gelu_inp) * grad; out = fp8(scale * t); dbias = column sums of
    t (fp32 in the reference, in its own block order; float64 here); amax raised to max|t|.  Returns (out bits, dbias).
    Parity unpinned (the reference has no test for these ops)."""
    t = _as_f32(grad)
    if gelu_inp is not None:
        t = (fp8_dgelu(gelu_inp) * t).astype(np.float32)
    if t.size:
        amax_row0[fp8_meta_index] = max(f32(amax_row0[fp8_meta_index]), f32(np.abs(t).max()))
    out = fp8_cast_sat((f32(scale[fp8_meta_index]) * t).astype(np.float32), fp8_dtype)
    dbias = t.astype(np.float64).sum(axis=0).astype(np.float32)
    if out_dtype in ("bfloat16", "bf16"):
        dbias = to_bf16_rne(dbias)
    elif out_dtype == "half":
        dbias = dbias.astype(np.float16).astype(np.float32)
    return out, dbias


def fp8_layernorm(x, gamma, beta, amax_row0: Optional[np.ndarray], scale: Optional[np.ndarray], fp8_meta_index: int, *,
                  epsilon: float = 1e-4, fp8_dtype: str = "E4M3", out_dtype: str = "int8"):
    """Fp8LayerNorm forward (itex/core/kernels/gpu/fp8/fp8_layernorm_gpu.h:108-257): per row mu = mean(x),
    rsigma = rsqrt(mean((x - mu)^2) + epsilon), v = gamma * (rsigma * (x - mu)) + beta; FP8 output: amax raised to
    max|v|, z = fp8(v * scale); real output: z = v.  Sums in float64 then rounded (the device sums fp32 in tree order).
    Returns (z, mu, rsigma).  Parity unpinned."""
    xf = _as_f32(x).astype(np.float64)
    mu = xf.mean(axis=1)
    var = ((xf - mu[:, None]) ** 2).mean(axis=1)
    rs = 1.0 / np.sqrt(var + np.float64(f32(epsilon)))
    v = (_as_f32(gamma).astype(np.float64) * (rs[:, None] * (xf - mu[:, None])) + _as_f32(beta).astype(np.float64)).astype(np.float32)
    if out_dtype == "int8":
        amax_row0[fp8_meta_index] = max(f32(amax_row0[fp8_meta_index]), f32(np.abs(v).max()))
        z = fp8_cast_sat((v * f32(scale[fp8_meta_index])).astype(np.float32), fp8_dtype)
    elif out_dtype == "bfloat16":
        z = to_bf16_rne(v)
    elif out_dtype == "half":
        z = v.astype(np.float16)
    else:
        z = v
    return z, mu.astype(np.float32), rs.astype(np.float32)


def fp8_dequantize(q, scale_inv: np.ndarray, fp8_meta_index: int, fp8_dtype: str = "E4M3",
                   out_dtype: str = "float") -> np.ndarray:
    """Fp8Dequantize (fp8_quantize_op.cc:53-83): y = out_dtype(float(q)*scale_inv[i])."""
    y = (fp8_to_f32(q, fp8_dtype) * f32(scale_inv[fp8_meta_index])).astype(np.float32)
    return to_bf16_rne(y) if out_dtype in ("bfloat16", "bf16") else y


def fp8_matmul(src, weight, bias, post_add, a_scale_inv, b_scale_inv, c_amax, c_scale, *,
               fp8_meta_index_a=0, fp8_meta_index_b=1, fp8_meta_index_c=-1, transpose_a=False,
               transpose_b=False, use_bias=False, has_post_add=False, sum_dtype="bfloat16",
               out_dtype="bfloat16", fp8_dtype_a="E4M3", fp8_dtype_b="E4M3", fp8_dtype_c="E4M3"):
    """Fp8Matmul (fp8_matmul_op.cc:44-90; functor fp8_matmul_gpu.h:34-162):
    dequantize both operands to sum_dtype, matmul with f32 accumulation, + bias, + post_add,
    result rounded to sum_dtype, optionally re-quantized to fp8 with amax update."""
    rnd = to_bf16_rne if sum_dtype in ("bfloat16", "bf16") else (lambda v: np.asarray(v, np.float32))
    A = rnd(fp8_to_f32(src, fp8_dtype_a) * f32(a_scale_inv[fp8_meta_index_a]))
    B = rnd(fp8_to_f32(weight, fp8_dtype_b) * f32(b_scale_inv[fp8_meta_index_b]))
    if transpose_a:
        A = A.T
    if transpose_b:
        B = B.T
    D = (A.astype(np.float64) @ B.astype(np.float64))
    if use_bias:
        D = D + _as_f32(bias).astype(np.float64)[None, :]
    if has_post_add:
        D = D + _as_f32(post_add).astype(np.float64)
    D = rnd(D.astype(np.float32))
    if out_dtype == "int8":
        return fp8_quantize(D, c_amax, c_scale, fp8_meta_index_c, fp8_dtype_c)
    return D


def fp8_default_sf_compute(amax, scale, fp8_max: float, margin: int) -> np.ndarray:
    """_default_sf_compute, itex/python/fp8/autocast.py:44-51."""
    amax = np.asarray(amax, np.float32)
    scale = np.asarray(scale, np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        exp = np.floor(np.log2(f32(fp8_max) / amax)).astype(np.float32) - f32(margin)
        sf = np.round(np.power(f32(2.0), np.abs(exp))).astype(np.float32)
        sf = np.where(amax > 0.0, sf, scale)
        sf = np.where(np.isfinite(amax), sf, scale)
        sf = np.where(exp < 0.0, f32(1.0) / sf, sf)
    return sf.astype(np.float32)


def fp8_amax_and_scale_update(amax_history, scale, fp8_max: float = 448.0, margin: int = 0,
                              amax_compute_algo: str = "max"):
    """amax_and_scale_update / fused_amax_and_scale_update, itex/python/fp8/autocast.py:53-121.
    Returns (new_history, new_scale, new_scale_inv)."""
    h = np.asarray(amax_history, np.float32)
    if amax_compute_algo == "max":
        amax = h.max(axis=0)
    elif amax_compute_algo == "most_recent":
        amax = h[0]
    else:
        raise ValueError("We only support the fp8 recipe with 'max' or 'most_recent' amax_compute_algo")
    sf = fp8_default_sf_compute(amax, scale, fp8_max, margin)
    nh = np.roll(h, -1, axis=0)
    nh[0] = 0
    return nh, sf, (f32(1.0) / sf).astype(np.float32)


# --------------------------------------------------------------------------
# quantized pooling (row (f)-1: what an un-decomposed int8 ResNet graph also needs)
# --------------------------------------------------------------------------
def quantized_pool2d(x, ksize, strides, padding="SAME", avg=False):
    """[_ITEX]QuantizedMaxPool / QuantizedAvgPool on NHWC u8|s8 (itex/core/kernels/cpu/maxpooling_op.cc:43-52,
    cpu/avgpooling_op.cc:50-58): max, or rne(float(sum)/float(count)) over the window cells inside the
    image (padding excluded); the min/max range passes through unchanged."""
    x = np.asarray(x)
    n, h, w, c = x.shape
    kh, kw = ksize[1], ksize[2]
    sh, sw = strides[1], strides[2]
    if padding == "SAME":
        oh, pt, _ = same_padding(h, kh, sh)
        ow, pl, _ = same_padding(w, kw, sw)
    else:
        oh, pt, _ = valid_padding(h, kh, sh)
        ow, pl, _ = valid_padding(w, kw, sw)
    T = QUINT8 if x.dtype == np.uint8 else QINT8
    out = np.empty((n, oh, ow, c), x.dtype)
    xi = x.astype(np.int32)
    for oy in range(oh):
        y0, y1 = max(0, oy * sh - pt), min(h, oy * sh - pt + kh)
        for ox in range(ow):
            x0, x1 = max(0, ox * sw - pl), min(w, ox * sw - pl + kw)
            win = xi[:, y0:y1, x0:x1, :].reshape(n, -1, c)
            if avg:
                out[:, oy, ox, :] = sat_rne((win.sum(axis=1).astype(np.float32) / f32(win.shape[1])).astype(np.float32), T)
            else:
                out[:, oy, ox, :] = win.max(axis=1).astype(x.dtype)
    return out


# --------------------------------------------------------------------------
# data movement between the quantized ops: reshape, transpose, concat
# --------------------------------------------------------------------------
def quantized_reshape(tensor, shape, input_min, input_max):
    """[_ITEX]QuantizedReshape (itex/core/kernels/common/quantized_reshape_op.h:33-200): the element order is kept, one
    entry of `shape` may be -1 (zero-sized entries stay out of the product it is inferred from), the range passes
    through.  -> (output, output_min, output_max); ValueError where the reference raises InvalidArgument."""
    tensor = np.asarray(tensor)
    sizes = [int(s) for s in np.asarray(shape).reshape(-1)]
    if sum(1 for s in sizes if s == -1) > 1:
        raise ValueError("Only one input size may be -1")
    if any(s < -1 for s in sizes):
        raise ValueError("Size must be non-negative")
    product, has_zero = 1, False
    for s in sizes:
        if s == 0:
            has_zero = True
        elif s > 0:
            product *= s
    dims = [1 if s == -1 else s for s in sizes]
    if -1 in sizes:
        elems, input_has_zero = 1, False
        for d in tensor.shape:
            if d > 0 or not has_zero:
                elems *= d
            else:
                input_has_zero = True
        missing = elems // product
        if not input_has_zero and product * missing != elems:
            raise ValueError("the requested shape requires a multiple of %d" % product)
        dims[sizes.index(-1)] = missing
    if int(np.prod(dims, dtype=np.int64)) != tensor.size:
        raise ValueError("Input to reshape is a tensor with %d values, but the requested shape has %d" % (tensor.size, int(np.prod(dims, dtype=np.int64))))
    return tensor.reshape(dims).copy(), f32(input_min), f32(input_max)


def quantized_transpose(x, perm, min_x, max_x):
    """_QuantizedTranspose / _ITEXQuantizedTranspose (itex/core/kernels/common/transpose_op.h:92-236): y.shape[d] =
    x.shape[perm[d]]; the range passes through."""
    x = np.asarray(x)
    perm = [int(p) for p in np.asarray(perm).reshape(-1)]
    if len(perm) != x.ndim:
        raise ValueError("transpose expects a vector of size %d" % x.ndim)
    for p in perm:
        if not 0 <= p < x.ndim:
            raise ValueError("%d is out of range [0 .. %d)" % (p, x.ndim))
    for d in range(x.ndim):
        if d not in perm:
            raise ValueError("%d is missing from {%s}." % (d, ",".join(str(p) for p in perm)))
    return np.ascontiguousarray(np.transpose(x, perm)), f32(min_x), f32(max_x)


def quantized_concat_v2(values, axis, input_mins, input_maxes):
    """QuantizedConcatV2 / _ITEXQuantizedConcatV2 (itex/core/kernels/common/quantized_concat_op.cc:34-247): the bytes are
    concatenated as they are; the kernel only serves inputs whose ranges agree within 1e-6 (anything else is the
    reference's Aborted "Not implemented the case unequal input_mins / input_maxes") and hands out input 0's range."""
    values = [np.asarray(v) for v in values]
    mins = [f32(m) for m in input_mins]
    maxes = [f32(m) for m in input_maxes]
    rank = values[0].ndim
    ax = int(axis) + rank if int(axis) < 0 else int(axis)
    if not 0 <= ax < rank:
        raise ValueError("ConcatOp : Expected concatenating dimensions in the range [%d, %d)" % (-rank, rank))
    for v in values:
        if v.ndim != rank:
            raise ValueError("ConcatOp : Ranks of all input tensors should match")
        if any(d != ax and v.shape[d] != values[0].shape[d] for d in range(rank)):
            raise ValueError("ConcatOp : Dimensions of inputs should match")
    for mn, mx in zip(mins[1:], maxes[1:]):
        if abs(float(mins[0]) - float(mn)) > 1.0e-6 or abs(float(maxes[0]) - float(mx)) > 1.0e-6:
            raise NotImplementedError("unequal input_mins / input_maxes")
    return np.concatenate(values, axis=ax), mins[0], maxes[0]
