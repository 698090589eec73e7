"""Kernel-level Python face of libitexb200 for torch tensors that live on a CUDA device.

torch supplies device memory and streams only; every function here is one call into the
C-ABI (layer 2 of include/itexb200.h) on torch's current stream.
"""
import ctypes as C

import torch

from . import _lib as L

_TORCH_TO_DT = {torch.float32: L.DT_FLOAT, torch.bfloat16: L.DT_BFLOAT16, torch.float16: L.DT_HALF,
                torch.int8: L.DT_QINT8, torch.uint8: L.DT_QUINT8, torch.int32: L.DT_QINT32}
_DT_TO_TORCH = {L.DT_FLOAT: torch.float32, L.DT_BFLOAT16: torch.bfloat16, L.DT_HALF: torch.float16,
                L.DT_QINT8: torch.int8, L.DT_QUINT8: torch.uint8, L.DT_QINT32: torch.int32,
                L.DT_INT8: torch.int8, L.DT_UINT8: torch.uint8, L.DT_INT32: torch.int32,
                L.DT_FP8_E4M3: torch.uint8, L.DT_FP8_E5M2: torch.uint8}


def dt_of(t: torch.Tensor) -> int:
    return _TORCH_TO_DT[t.dtype]


def torch_dtype(dt: int):
    return _DT_TO_TORCH[dt]


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("itex_b200 kernels take CUDA tensors; got a %s tensor" % t.device)


def quantize(x, q_dtype, scale, *, shift=None, kind=0, inner=1, nslice=1, out=None):
    """q = sat(rne(affine(x))).  `scale`/`shift` are floats (per-tensor) or device fp32 vectors."""
    _require_cuda(x, out)
    x = x.contiguous()
    q = out if out is not None else torch.empty(x.shape, dtype=torch_dtype(q_dtype), device=x.device)
    sd = scale if isinstance(scale, torch.Tensor) else None
    hd = shift if isinstance(shift, torch.Tensor) else None
    L.check(L.load().itexb_quantize(_ptr(x), dt_of(x), _ptr(q), q_dtype, C.c_int64(x.numel()), C.c_int64(inner),
                                    C.c_int64(nslice), kind, _ptr(sd), _ptr(hd),
                                    C.c_float(0.0 if sd is not None else float(scale)),
                                    C.c_float(0.0 if (hd is not None or shift is None) else float(shift)), stream_ptr()))
    return q


def dequantize(q, y_dtype, scale, *, zp=None, inner=1, nslice=1, q_dtype=None, out=None):
    _require_cuda(q, out)
    q = q.contiguous()
    y = out if out is not None else torch.empty(q.shape, dtype=torch_dtype(y_dtype), device=q.device)
    sd = scale if isinstance(scale, torch.Tensor) else None
    zd = zp if isinstance(zp, torch.Tensor) else None
    L.check(L.load().itexb_dequantize(_ptr(q), q_dtype or dt_of(q), _ptr(y), y_dtype, C.c_int64(q.numel()),
                                      C.c_int64(inner), C.c_int64(nslice), _ptr(sd), _ptr(zd),
                                      C.c_float(0.0 if sd is not None else float(scale)),
                                      C.c_float(0.0 if (zd is not None or zp is None) else float(zp)), stream_ptr()))
    return y


def pack_weights_kn(b_kn, k_pad=None):
    """[k,n] 8-bit weights -> packed [n,k_pad] (k padded with zeros to a multiple of 16)."""
    _require_cuda(b_kn)
    k, n = b_kn.shape
    k_pad = k_pad or (k + 15) // 16 * 16
    out = torch.empty((n, k_pad), dtype=b_kn.dtype, device=b_kn.device)
    L.check(L.load().itexb_pack_weights_kn(_ptr(b_kn.contiguous()), _ptr(out), C.c_int64(k), C.c_int64(n),
                                           C.c_int64(k_pad), stream_ptr()))
    return out


def make_epilogue(scale=None, bias=None, relu=False, raw_acc=False, summand=None, sum_scale=1.0,
                  alpha_a=None, alpha_b=None, out_scale=None, amax=None, summand_dtype=None,
                  activation=0, act_alpha=0.0, act_beta=0.0, post_scale=0.0):
    ep = L.Epilogue()
    keep = [scale, bias, summand, alpha_a, alpha_b, out_scale, amax]
    if scale is not None:
        ep.scale = scale.data_ptr()
        ep.scale_count = scale.numel()
    if bias is not None:
        ep.bias = bias.data_ptr()
    if summand is not None:
        ep.summand = summand.data_ptr()
        ep.summand_dtype = summand_dtype or dt_of(summand)
        ep.ld_summand = summand.shape[-1]
    ep.sum_scale = float(sum_scale)
    ep.relu = int(bool(relu))
    ep.raw_acc = int(bool(raw_acc))
    ep.activation, ep.act_alpha, ep.act_beta, ep.post_scale = int(activation), float(act_alpha), float(act_beta), float(post_scale)
    for name, t in (("alpha_a", alpha_a), ("alpha_b", alpha_b), ("out_scale", out_scale), ("amax", amax)):
        if t is not None:
            setattr(ep, name, t.data_ptr())
    ep._keep = keep
    return ep


def gemm(a, b_nk, out_dtype, *, a_dtype=None, b_dtype=None, ep=None, out=None, status_word=None, n=None, k=None, peer_out=None):
    """out[m,n] = epilogue(sum_k a[m,k] * b_nk[n,k]); a and b_nk are 8-bit CUDA tensors.  Three-dimensional a [batch,m,k]
    and b_nk [batch,n,k] give a batched product out [batch,m,n].  peer_out: device addresses (ints) of buffers on other
    GPUs laid out like `out`; every output block is stored there too (the fused all-gather of itexb_gemm)."""
    _require_cuda(a, b_nk, out)
    batched = a.dim() == 3
    m = a.shape[-2]
    k = k or a.shape[-1]
    n = n or b_nk.shape[-2]
    ep = ep or make_epilogue()
    tdt = torch.int32 if ep.raw_acc else torch_dtype(out_dtype)
    shape = (a.shape[0], m, n) if batched else (m, n)
    o = out if out is not None else torch.empty(shape, dtype=tdt, device=a.device)
    p = L.GemmParams()
    p.m, p.n, p.k = m, n, k
    p.a_dtype = a_dtype or dt_of(a)
    p.b_dtype = b_dtype or dt_of(b_nk)
    p.out_dtype = out_dtype
    p.a, p.lda = a.data_ptr(), a.stride(-2)
    p.b, p.ldb = b_nk.data_ptr(), b_nk.stride(-2)
    p.out, p.ldo = o.data_ptr(), o.stride(-2)
    if batched:
        p.batch, p.stride_a, p.stride_b, p.stride_out = a.shape[0], a.stride(0), b_nk.stride(0), o.stride(0)
    p.ep = ep
    p.status_word = 0 if status_word is None else status_word.data_ptr()
    if peer_out:
        arr = (C.c_void_p * len(peer_out))(*[int(v) for v in peer_out])
        p.num_peers, p.peer_out = len(peer_out), arr
    L.check(L.load().itexb_gemm(C.byref(p), stream_ptr()))
    return o


def fp8_quantize(x, scale, amax=None, fp8_dtype=L.DT_FP8_E4M3, out=None):
    """y = fp8(float(x)*scale[0]) (uint8 bit patterns); amax[0] raised to max|x|."""
    _require_cuda(x, scale, amax, out)
    x = x.contiguous()
    y = out if out is not None else torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    L.check(L.load().itexb_fp8_quantize(_ptr(x), dt_of(x), _ptr(y), fp8_dtype, C.c_int64(x.numel()), _ptr(scale),
                                        _ptr(amax), stream_ptr()))
    return y


def fp8_dequantize(x, scale_inv, y_dtype=L.DT_FLOAT, fp8_dtype=L.DT_FP8_E4M3, out=None):
    _require_cuda(x, scale_inv, out)
    x = x.contiguous()
    y = out if out is not None else torch.empty(x.shape, dtype=torch_dtype(y_dtype), device=x.device)
    L.check(L.load().itexb_fp8_dequantize(_ptr(x), fp8_dtype, _ptr(y), y_dtype, C.c_int64(x.numel()), _ptr(scale_inv),
                                          stream_ptr()))
    return y


def fp8_amax_and_scale_update(amax_history, scale, scale_inv, fp8_max=448.0, margin=0.0, algo="max"):
    """In-place delayed-scaling update of [H,n] history and [n] scale / scale_inv on the device."""
    _require_cuda(amax_history, scale, scale_inv)
    h, n = amax_history.shape
    L.check(L.load().itexb_fp8_amax_and_scale_update(_ptr(amax_history), _ptr(scale), _ptr(scale_inv), h, n,
                                                     C.c_float(fp8_max), C.c_float(margin),
                                                     {"max": 0, "most_recent": 1}[algo], stream_ptr()))


def minmax(x, out=None):
    _require_cuda(x)
    mm = out if out is not None else torch.empty(2, dtype=torch.float32, device=x.device)
    lib = L.load()
    L.check(lib.itexb_minmax_init(_ptr(mm), stream_ptr()))
    L.check(lib.itexb_minmax(_ptr(x.contiguous()), dt_of(x), C.c_int64(x.numel()), _ptr(mm), stream_ptr()))
    return mm


def quantize_dynamic(x, q_dtype, mm, ensure_minimum_range=0.01, weight_range=None, scales=None):
    """QuantizeV2 SCALED with the range read from the device tensor mm; -> (q, {scale, out_min, out_max}).  With
    weight_range (and optionally a preallocated scales) the consuming matmul's per-channel scales are written too."""
    _require_cuda(x, mm, weight_range, scales)
    x = x.contiguous()
    q = torch.empty(x.shape, dtype=torch_dtype(q_dtype), device=x.device)
    out3 = torch.empty(3, dtype=torch.float32, device=x.device)
    if weight_range is not None and scales is None:
        scales = torch.empty(weight_range.numel(), dtype=torch.float32, device=x.device)
    L.check(L.load().itexb_quantize_dynamic_scales(_ptr(x), dt_of(x), _ptr(q), q_dtype, C.c_int64(x.numel()), _ptr(mm),
                                                   C.c_float(ensure_minimum_range), _ptr(out3), _ptr(weight_range),
                                                   0 if weight_range is None else weight_range.numel(), _ptr(scales), stream_ptr()))
    return (q, out3) if weight_range is None else (q, out3, scales)


def matmul_scales_dynamic(range3, weight_range, a_dtype, out=None):
    """Per-channel output scales from a device-resident activation range (see itexb_matmul_scales_dynamic)."""
    _require_cuda(range3, weight_range, out)
    n = weight_range.numel()
    sc = out if out is not None else torch.empty(n, dtype=torch.float32, device=weight_range.device)
    L.check(L.load().itexb_matmul_scales_dynamic(_ptr(range3), _ptr(weight_range), n, a_dtype, _ptr(sc), stream_ptr()))
    return sc


def launch_count() -> int:
    return int(L.load().itexb_launch_count())
