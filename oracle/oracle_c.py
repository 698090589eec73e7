"""ctypes face of oracle/_build/libitex_oracle.so (the C twin of itex_oracle.py).
Test infrastructure only."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def load():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "_build", "libitex_oracle.so")
        if not os.path.exists(path):
            import build_oracle
            build_oracle.build()
        _lib = C.CDLL(path)
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def num_threads():
    return load().oracle_num_threads()


def quantize_scaled(x, scale, signed, inner=1):
    x = np.ascontiguousarray(x, np.float32)
    scale = np.ascontiguousarray(np.atleast_1d(scale), np.float32)
    q = np.empty(x.shape, np.int8 if signed else np.uint8)
    load().oracle_quantize_scaled(_p(x), C.c_int64(x.size), C.c_int64(inner), C.c_int64(scale.size), _p(scale), int(signed), _p(q))
    return q


def dequantize(q, scale, zp=None, inner=1):
    q = np.ascontiguousarray(q)
    scale = np.ascontiguousarray(np.atleast_1d(scale), np.float32)
    zpa = None if zp is None else np.ascontiguousarray(np.atleast_1d(zp), np.float32)
    y = np.empty(q.shape, np.float32)
    load().oracle_dequantize(_p(q), C.c_int64(q.size), C.c_int64(inner), C.c_int64(scale.size), _p(scale),
                             None if zpa is None else _p(zpa), int(q.dtype == np.int8), _p(y))
    return y


def gemm_acc(a, b_nk):
    a = np.ascontiguousarray(a)
    b_nk = np.ascontiguousarray(b_nk, np.int8)
    m, k = a.shape
    n = b_nk.shape[0]
    acc = np.empty((m, n), np.int32)
    load().oracle_gemm_acc(_p(a), int(a.dtype == np.int8), _p(b_nk), C.c_int64(m), C.c_int64(n), C.c_int64(k), _p(acc))
    return acc


_KIND = {"float": (0, np.float32), "quint8": (1, np.uint8), "qint8": (2, np.int8), "qint32": (3, np.int32)}


def gemm_fused(a, b_nk, scale, bias, relu, toutput):
    a = np.ascontiguousarray(a)
    b_nk = np.ascontiguousarray(b_nk, np.int8)
    m, k = a.shape
    n = b_nk.shape[0]
    kind, dt = _KIND[toutput]
    out = np.empty((m, n), dt)
    sc = None if scale is None else np.ascontiguousarray(np.atleast_1d(scale), np.float32)
    bi = None if bias is None else np.ascontiguousarray(bias, np.float32)
    load().oracle_gemm_fused(_p(a), int(a.dtype == np.int8), _p(b_nk), C.c_int64(m), C.c_int64(n), C.c_int64(k),
                             None if sc is None else _p(sc), C.c_int64(0 if sc is None else sc.size),
                             None if bi is None else _p(bi), int(relu), kind, _p(out))
    return out


def epilogue(acc, scale, bias, relu, toutput):
    acc = np.ascontiguousarray(acc, np.int32)
    m, n = acc.reshape(-1, acc.shape[-1]).shape
    kind, dt = _KIND[toutput]
    out = np.empty(acc.shape, dt)
    sc = None if scale is None else np.ascontiguousarray(np.atleast_1d(scale), np.float32)
    bi = None if bias is None else np.ascontiguousarray(bias, np.float32)
    load().oracle_epilogue(_p(acc), C.c_int64(m), C.c_int64(n), None if sc is None else _p(sc),
                           C.c_int64(0 if sc is None else sc.size), None if bi is None else _p(bi), int(relu), kind, _p(out))
    return out


def conv_acc(x, f_hwio, strides=(1, 1), pads=(0, 0), out_hw=None, dilations=(1, 1)):
    x = np.ascontiguousarray(x)
    nb, h, w, c = x.shape
    kh, kw, _, co = f_hwio.shape
    f = np.ascontiguousarray(np.transpose(f_hwio, (3, 0, 1, 2)), np.int8)
    oh, ow = out_hw
    acc = np.empty((nb, oh, ow, co), np.int32)
    load().oracle_conv_acc(_p(x), int(x.dtype == np.int8), _p(f), *[C.c_int64(v) for v in (
        nb, h, w, c, kh, kw, co, strides[0], strides[1], dilations[0], dilations[1], pads[0], pads[1], oh, ow)], _p(acc))
    return acc
