"""Op-level Python face of libitexb200: ITEX's op names, attrs and argument order.

An `Op` is one graph node: created once from the op name and attrs (like the reference's
kernel constructor), computed many times.  Device arguments are torch CUDA tensors;
HostMemory arguments (every min_*/max_* range) are Python floats, sequences or NumPy
arrays and HostMemory outputs come back as NumPy.  Outputs and temporaries are allocated
through callbacks, the way a TensorFlow shim would answer TF_AllocateOutput /
TF_AllocateTemp - here with torch's allocator, so results are ordinary torch tensors.

The module-level functions mirror the generated Python wrappers the reference's tests
call (`load_ops_library._ITEXQuantizeV2(input=..., min_range=..., T=...)`, see
itex/python/ops/load_ops_library.py:29-72).
"""
import ctypes as C
import weakref

import numpy as np
import torch

from . import _lib as L
from .kernels import torch_dtype

_NAME_TO_DT = {
    "float": L.DT_FLOAT, "float32": L.DT_FLOAT, "bfloat16": L.DT_BFLOAT16, "half": L.DT_HALF, "float16": L.DT_HALF,
    "qint8": L.DT_QINT8, "quint8": L.DT_QUINT8, "qint32": L.DT_QINT32, "int8": L.DT_INT8, "int32": L.DT_INT32, "int64": L.DT_INT64,
}
_TORCH_TO_DT = {torch.float32: L.DT_FLOAT, torch.bfloat16: L.DT_BFLOAT16, torch.float16: L.DT_HALF,
                torch.int8: L.DT_QINT8, torch.uint8: L.DT_QUINT8, torch.int32: L.DT_QINT32}
_TYPE_ATTRS = {"T", "T1", "T2", "Tshape", "Tperm", "Tidx", "Tbias", "Toutput", "Tinput", "Tfilter", "out_type", "dtype", "sum_dtype", "out_dtype", "grad_dtype",
               "in_dtype", "Tsummand", "Targs", "Tout", "U", "weight_dtype"}


def as_dtype(v):
    """Accepts an itexb_dtype_t number, a TF-style name ('qint8') or a torch dtype."""
    if isinstance(v, int):
        return v
    if isinstance(v, torch.dtype):
        return _TORCH_TO_DT[v]
    return _NAME_TO_DT[str(v)]


def _setup(lib):
    if getattr(lib, "_ops_ready", False):
        return
    lib.itexb_op_list.restype = C.POINTER(C.c_char_p)
    lib.itexb_op_delete.restype = None
    lib.itexb_op_create.argtypes = [C.c_char_p, C.POINTER(L.Attr), C.c_int, C.POINTER(C.c_void_p)]
    lib.itexb_op_compute.argtypes = [C.c_void_p, C.POINTER(L.OpContext)]
    lib.itexb_op_delete.argtypes = [C.c_void_p]
    lib.itexb_op_check.argtypes = [C.c_void_p, C.c_int]
    lib._ops_ready = True


def op_list():
    lib = L.load()
    _setup(lib)
    names, p, i = [], lib.itexb_op_list(), 0
    while p[i]:
        names.append(p[i].decode())
        i += 1
    return names


def op_signature(name):
    lib = L.load()
    nin, nout, hin, hout = C.c_int(), C.c_int(), C.c_uint32(), C.c_uint32()
    L.check(lib.itexb_op_signature(name.encode(), C.byref(nin), C.byref(nout), C.byref(hin), C.byref(hout)))
    return nin.value, nout.value, hin.value, hout.value


def make_attrs(attrs):
    """dict -> (itexb_attr_t array, keep-alive list): the marshalling the Op class uses, for other C-ABI calls that take attrs."""
    arr, _, keep = _make_attrs(attrs)
    return arr, keep


def _make_attrs(attrs):
    arr = (L.Attr * max(1, len(attrs)))()
    keep = []
    for i, (k, v) in enumerate(attrs.items()):
        a = arr[i]
        kb = k.encode()
        keep.append(kb)
        a.name = kb
        if k in _TYPE_ATTRS:
            a.type, a.i = 4, as_dtype(v)
        elif isinstance(v, bool):
            a.type, a.i = 2, int(v)
        elif isinstance(v, int):
            a.type, a.i = 0, v
        elif isinstance(v, float):
            a.type, a.f = 1, v
        elif isinstance(v, str):
            sb = v.encode()
            keep.append(sb)
            a.type, a.s = 3, sb
        elif isinstance(v, (list, tuple)) and all(isinstance(e, str) for e in v) and len(v) > 0:
            bs = [e.encode() for e in v]
            sl = (C.c_char_p * len(bs))(*bs)
            keep += [bs, sl]
            a.type, a.list_s, a.list_len = 6, sl, len(bs)
        elif isinstance(v, (list, tuple)):
            il = (C.c_int64 * max(1, len(v)))(*[int(e) for e in v])
            keep.append(il)
            a.type, a.list_i, a.list_len = 5, il, len(v)
        else:
            raise TypeError("attr %s: unsupported value %r" % (k, v))
    return arr, len(attrs), keep


class Op:
    """One kernel instance (itexb_op_t)."""

    def __init__(self, op_name, **attrs):
        self.lib = L.load()
        _setup(self.lib)
        self.name = op_name
        self.nin, self.nout, self.host_in, self.host_out = op_signature(op_name)
        arr, n, keep = _make_attrs(attrs)
        h = C.c_void_p()
        L.check(self.lib.itexb_op_create(op_name.encode(), arr, n, C.byref(h)))
        self._h = h
        self._outputs = {}
        self._temps = []
        # The callbacks reach the instance through a weak reference: a bound method kept on the instance would be a
        # reference cycle, and the kernel instance would then live until some later garbage collection instead of
        # being deleted with its last user.
        ref = weakref.ref(self)
        self._alloc_out_cb = L.ALLOC_OUTPUT_FN(lambda user, index, tp: ref()._allocate_output(user, index, tp))
        self._alloc_tmp_cb = L.ALLOC_TEMP_FN(lambda user, nbytes, on_host, pp: ref()._allocate_temp(user, nbytes, on_host, pp))
        self._device = None
        self._given = None

    def check(self, wait=True):
        """Raises ItexError (ABORTED) if a kernel launched by this instance gave up on a bounded wait (itexb_op_check)."""
        L.check(self.lib.itexb_op_check(self._h, 1 if wait else 0))

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self.lib.itexb_op_delete(self._h)
                self._h = None
        except Exception:
            pass

    # -- callbacks (the role of TF_AllocateOutput / TF_AllocateTemp) --------------------
    def _allocate_output(self, user, index, tp):
        try:
            t = tp.contents
            shape = [t.dims[i] for i in range(t.rank)]
            if t.on_host:
                arr = np.empty(shape, dtype=np.float32 if t.dtype == L.DT_FLOAT else np.uint8)
                t.data = arr.ctypes.data
                self._outputs[index] = arr
            else:
                ten = self._given.get(index) if self._given else None
                if ten is not None:
                    # the caller's buffer (TensorFlow forwards an input buffer to an output the same way): it has to be what
                    # the kernel asked for
                    if list(ten.shape) != shape or ten.dtype != torch_dtype(t.dtype) or not ten.is_contiguous() or ten.device != self._device:
                        return L.INVALID_ARGUMENT
                else:
                    ten = torch.empty(shape, dtype=torch_dtype(t.dtype), device=self._device)
                t.data = ten.data_ptr()
                self._outputs[index] = ten
            return L.OK
        except Exception:  # allocation failure surfaces as a status, never as an exception in C
            return L.RESOURCE_EXHAUSTED

    def _allocate_temp(self, user, nbytes, on_host, pp):
        try:
            if on_host:
                buf = np.empty(max(1, nbytes), dtype=np.uint8)
                pp[0] = buf.ctypes.data
            else:
                buf = torch.empty(max(1, nbytes), dtype=torch.uint8, device=self._device)
                pp[0] = buf.data_ptr()
            self._temps.append(buf)
            return L.OK
        except Exception:
            return L.RESOURCE_EXHAUSTED

    def __call__(self, *inputs, device=None, dtypes=None, out=None):
        """Runs Compute.  `dtypes` optionally overrides the itexb dtype of tensor inputs
        (e.g. DT_INT8 for FP8 bytes held in a torch.int8/uint8 tensor).  `out` = {output index: tensor} makes the kernel
        write those device outputs into the caller's tensors (shape, type and device must be what the kernel produces)."""
        self._given = out
        keep = []
        tens = (L.Tensor * max(1, len(inputs)))()
        dev = device
        for i, x in enumerate(inputs):
            t = tens[i]
            if isinstance(x, torch.Tensor) and x.is_cuda:
                x = x.contiguous()
                dev = dev or x.device
                t.dtype = (dtypes or {}).get(i, _TORCH_TO_DT[x.dtype])
                t.rank = x.dim()
                for d in range(x.dim()):
                    t.dims[d] = x.shape[d]
                t.data = x.data_ptr()
                t.on_host = 0
                keep.append(x)
            else:
                if isinstance(x, torch.Tensor):
                    x = x.numpy()
                if isinstance(x, np.ndarray) and x.dtype in (np.int32, np.int64):   # shape / perm / axis arguments
                    arr = np.ascontiguousarray(x)
                    t.dtype = L.DT_INT32 if x.dtype == np.int32 else L.DT_INT64
                else:
                    arr = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
                    t.dtype = L.DT_FLOAT
                t.rank = arr.ndim
                for d in range(arr.ndim):
                    t.dims[d] = arr.shape[d]
                t.data = arr.ctypes.data
                t.on_host = 1
                keep.append(arr)
        self._device = dev or torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
        self._outputs = {}
        ctx = L.OpContext()
        ctx.user = None
        ctx.num_inputs = len(inputs)
        ctx.inputs = tens
        ctx.device_ordinal = self._device.index or 0
        ctx.stream = torch.cuda.current_stream(self._device).cuda_stream if torch.cuda.is_available() else None
        ctx.allocate_output = self._alloc_out_cb
        ctx.allocate_temp = self._alloc_tmp_cb
        try:
            L.check(self.lib.itexb_op_compute(self._h, C.byref(ctx)))
        finally:
            self._temps = []  # torch's allocator is stream-ordered: safe to release after enqueue
            self._given = None
        nout = self.nout if self.nout >= 0 else (max(self._outputs) + 1 if self._outputs else 0)  # -1: decided per call
        outs = [self._outputs.get(i) for i in range(nout)]
        outs = [o.reshape(()).item() if isinstance(o, np.ndarray) and o.ndim == 0 else o for o in outs]
        return outs[0] if nout == 1 else tuple(outs)


def _cached(op_name, attrs):
    """The functional wrappers below run one node once: every call builds its own kernel instance, as every node of a
    graph has its own (the per-instance caches - packed constant weight, scaled bias, scale vectors - belong to one node;
    sharing an instance between call sites with equal attrs would serve one site's constants to the other).  Code that
    runs the same node repeatedly keeps an `Op` and calls it, which is where those caches pay."""
    return Op(op_name, **attrs)


def _ITEXQuantizeV2(input, min_range, max_range, T="qint8", mode="SCALED", round_mode="HALF_AWAY_FROM_ZERO",
                    narrow_range=False, axis=-1, ensure_minimum_range=0.01, dtype="float",
                    classic_asymmetric_algorithm=False, op_name="_ITEXQuantizeV2"):
    """-> (output, output_min, output_max)"""
    attrs = dict(T=T, mode=mode, round_mode=round_mode, narrow_range=bool(narrow_range), axis=-1 if axis is None else int(axis),
                 ensure_minimum_range=float(ensure_minimum_range), dtype=dtype,
                 classic_asymmetric_algorithm=bool(classic_asymmetric_algorithm))
    return _cached(op_name, attrs)(input, min_range, max_range)


def _ITEXDequantize(input, min_range, max_range, mode="SCALED", narrow_range=False, axis=-1, dtype="float",
                    op_name="_ITEXDequantize"):
    attrs = dict(T=_TORCH_TO_DT[input.dtype], mode=mode, narrow_range=bool(narrow_range),
                 axis=-1 if axis is None else int(axis), dtype=dtype)
    return _cached(op_name, attrs)(input, min_range, max_range)


def _quantized_matmul(op_name, a, b, bias, min_a, max_a, min_b, max_b, freezed, attrs):
    args = [a, b, bias, min_a, max_a, min_b, max_b] + list(freezed)
    dtypes = {2: L.DT_QINT32} if bias.dtype == torch.int32 else None
    return _cached(op_name, attrs)(*args, dtypes=dtypes)


def _mm_attrs(bias, Toutput, transpose_a, transpose_b, input_quant_mode, is_weight_const, scaled_bias_mode, with_tbias=True):
    attrs = dict(T1="quint8", T2="qint8", Toutput=Toutput, transpose_a=bool(transpose_a), transpose_b=bool(transpose_b),
                 input_quant_mode=input_quant_mode, is_weight_const=bool(is_weight_const))
    if with_tbias:
        attrs["Tbias"] = "qint32" if bias.dtype == torch.int32 else _TORCH_TO_DT[bias.dtype]
    if scaled_bias_mode is not None:
        attrs["_scaled_bias_mode"] = scaled_bias_mode
    return attrs


def _ITEXQuantizedMatMulWithBias(a, b, bias, min_a, max_a, min_b, max_b, Toutput="qint32", transpose_a=False,
                                 transpose_b=False, input_quant_mode="MIN_FIRST", is_weight_const=True,
                                 scaled_bias_mode=None, op_name="_ITEXQuantizedMatMulWithBias"):
    """-> (out, min_out, max_out)"""
    return _quantized_matmul(op_name, a, b, bias, min_a, max_a, min_b, max_b, (),
                             _mm_attrs(bias, Toutput, transpose_a, transpose_b, input_quant_mode, is_weight_const, scaled_bias_mode))


def _ITEXQuantizedMatMulWithBiasAndRelu(a, b, bias, min_a, max_a, min_b, max_b, Toutput="qint32", transpose_a=False,
                                        transpose_b=False, input_quant_mode="MIN_FIRST", is_weight_const=True,
                                        scaled_bias_mode=None, op_name="_ITEXQuantizedMatMulWithBiasAndRelu"):
    return _quantized_matmul(op_name, a, b, bias, min_a, max_a, min_b, max_b, (),
                             _mm_attrs(bias, Toutput, transpose_a, transpose_b, input_quant_mode, is_weight_const,
                                       scaled_bias_mode, with_tbias=False))


def _ITEXQuantizedMatMulWithBiasAndRequantize(a, b, bias, min_a, max_a, min_b, max_b, min_freezed_output, max_freezed_output,
                                              Toutput="quint8", transpose_a=False, transpose_b=False,
                                              input_quant_mode="MIN_FIRST", is_weight_const=True, scaled_bias_mode=None,
                                              op_name="_ITEXQuantizedMatMulWithBiasAndRequantize"):
    return _quantized_matmul(op_name, a, b, bias, min_a, max_a, min_b, max_b, (min_freezed_output, max_freezed_output),
                             _mm_attrs(bias, Toutput, transpose_a, transpose_b, input_quant_mode, is_weight_const, scaled_bias_mode))


def _ITEXQuantizedMatMulWithBiasAndReluAndRequantize(a, b, bias, min_a, max_a, min_b, max_b, min_freezed_output,
                                                     max_freezed_output, Toutput="quint8", transpose_a=False, transpose_b=False,
                                                     input_quant_mode="MIN_FIRST", is_weight_const=True, scaled_bias_mode=None,
                                                     op_name="_ITEXQuantizedMatMulWithBiasAndReluAndRequantize"):
    return _quantized_matmul(op_name, a, b, bias, min_a, max_a, min_b, max_b, (min_freezed_output, max_freezed_output),
                             _mm_attrs(bias, Toutput, transpose_a, transpose_b, input_quant_mode, is_weight_const, scaled_bias_mode))


def _ITEXQuantizedMatMulWithBiasAndDequantize(a, b, bias, min_a, max_a, min_b, max_b, min_freezed_output, max_freezed_output,
                                              Toutput="float", transpose_a=False, transpose_b=False,
                                              input_quant_mode="MIN_FIRST", is_weight_const=True, scaled_bias_mode=None,
                                              op_name="_ITEXQuantizedMatMulWithBiasAndDequantize"):
    """-> out"""
    return _quantized_matmul(op_name, a, b, bias, min_a, max_a, min_b, max_b, (min_freezed_output, max_freezed_output),
                             _mm_attrs(bias, Toutput, transpose_a, transpose_b, input_quant_mode, is_weight_const, scaled_bias_mode))


def _bias_attr(t):
    return "qint32" if t.dtype == torch.int32 else _TORCH_TO_DT[t.dtype]


def _QuantizedFusedMatMul(a, b, args, min_a, max_a, min_b, max_b, min_freezed_output=None, max_freezed_output=None,
                          Toutput="qint32", fused_ops=(), transpose_a=False, transpose_b=False, input_quant_mode="SCALED",
                          is_filter_const=True, is_bias_const=True, leakyrelu_alpha=0.2, scaled_bias_mode=None,
                          postop_scale_mode=None, op_name=None):
    """_[ITEX]QuantizedFusedMatMul / ...AndRequantize / ...AndDequantize (the op name follows from Toutput unless
    given).  `args` = [bias] or [bias, addend] as fused_ops says.  -> (product, min_product, max_product) or product."""
    tout = Toutput if isinstance(Toutput, str) else {L.DT_FLOAT: "float", L.DT_BFLOAT16: "bfloat16", L.DT_HALF: "half",
                                                     L.DT_QINT8: "qint8", L.DT_QUINT8: "quint8", L.DT_QINT32: "qint32"}[as_dtype(Toutput)]
    if op_name is None:
        op_name = "_QuantizedFusedMatMul" + ("" if tout == "qint32" else ("AndRequantize" if tout in ("qint8", "quint8") else "AndDequantize"))
    attrs = dict(T1=_TORCH_TO_DT[a.dtype], T2="qint8", Toutput=tout, num_args=len(args), transpose_a=bool(transpose_a),
                 transpose_b=bool(transpose_b), input_quant_mode=input_quant_mode, is_filter_const=bool(is_filter_const),
                 is_bias_const=bool(is_bias_const), leakyrelu_alpha=float(leakyrelu_alpha))
    if len(args) > 0:
        attrs["Targs"] = _bias_attr(args[0])
    if len(fused_ops) > 0:
        attrs["fused_ops"] = list(fused_ops)
    if scaled_bias_mode is not None:
        attrs["_scaled_bias_mode"] = scaled_bias_mode
    if postop_scale_mode is not None:
        attrs["_postop_scale_mode"] = postop_scale_mode
    inputs = [a, b] + list(args) + [min_a, max_a, min_b, max_b]
    if tout in ("qint8", "quint8"):
        inputs += [min_freezed_output, max_freezed_output]
    dtypes = {2: L.DT_QINT32} if len(args) > 0 and args[0].dtype == torch.int32 else None
    return _cached(op_name, attrs)(*inputs, dtypes=dtypes)


def _QuantizedMatMul(device_inputs, host_inputs, T1=None, T2="qint8", Tbias=None, Tout=None, Tdevice_outputs=None,
                     fused_ops=(), transpose_a=False, transpose_b=False, input_quant_mode="SCALED", output_quant_mode="SCALED",
                     is_weight_const=True, is_bias_const=True, leakyrelu_alpha=0.2, scaled_bias_mode=None,
                     postop_scale_mode=None, op_name="_QuantizedMatMul"):
    """_[ITEX]QuantizedMatMul (V2): device_inputs = [a, b, bias(, addend)], host_inputs = [min_a, max_a, min_b, max_b
    (, min_out, max_out)].  -> tuple of the device outputs followed by the host outputs (one element for float outputs)."""
    if Tout is None:
        Tout = Tdevice_outputs[0] if Tdevice_outputs else "float"
    attrs = dict(T1=T1 if T1 is not None else _TORCH_TO_DT[device_inputs[0].dtype], T2=T2, Tout=Tout,
                 transpose_a=bool(transpose_a), transpose_b=bool(transpose_b), input_quant_mode=input_quant_mode,
                 output_quant_mode=output_quant_mode, is_weight_const=bool(is_weight_const), is_bias_const=bool(is_bias_const),
                 leakyrelu_alpha=float(leakyrelu_alpha), fused_ops=list(fused_ops))
    if len(device_inputs) > 2:
        attrs["Tbias"] = Tbias if Tbias is not None else _bias_attr(device_inputs[2])
    if scaled_bias_mode is not None:
        attrs["_scaled_bias_mode"] = scaled_bias_mode
    if postop_scale_mode is not None:
        attrs["_postop_scale_mode"] = postop_scale_mode
    dtypes = {2: L.DT_QINT32} if len(device_inputs) > 2 and device_inputs[2].dtype == torch.int32 else None
    return _cached(op_name, attrs)(*(list(device_inputs) + list(host_inputs)), dtypes=dtypes)


def _QuantizedBatchMatMulV2AndDequantize(x, y, min_x, max_x, min_y, max_y, Toutput="float", adj_x=False, adj_y=False,
                                         is_filter_const=False, op_name="_QuantizedBatchMatMulV2AndDequantize"):
    """-> output [..., m, n] (batch dims broadcast)."""
    attrs = dict(T1=_TORCH_TO_DT[x.dtype], T2=_TORCH_TO_DT[y.dtype], Toutput=Toutput, adj_x=bool(adj_x), adj_y=bool(adj_y),
                 is_filter_const=bool(is_filter_const))
    return _cached(op_name, attrs)(x, y, min_x, max_x, min_y, max_y)


def _QuantizedFusedBatchMatMulV2AndDequantize(x, y, args, min_x, max_x, min_y, max_y, fused_ops=(), Toutput="float", T=None,
                                              adj_x=False, adj_y=False, is_filter_const=False,
                                              op_name="_QuantizedFusedBatchMatMulV2AndDequantize"):
    """`args` = one device tensor per fused op ("Mul": a scalar tensor, "Add": broadcasts to the output)."""
    attrs = dict(T1=_TORCH_TO_DT[x.dtype], T2=_TORCH_TO_DT[y.dtype], Toutput=Toutput, adj_x=bool(adj_x), adj_y=bool(adj_y),
                 is_filter_const=bool(is_filter_const), num_args=len(args), fused_ops=list(fused_ops))
    if T is not None or len(args) > 0:
        attrs["T"] = T if T is not None else _TORCH_TO_DT[args[0].dtype]
    return _cached(op_name, attrs)(*([x, y] + list(args) + [min_x, max_x, min_y, max_y]))


def _QuantizedBatchMatMul(device_inputs, host_inputs, T1="qint8", T2="qint8", U=None, Tout=None, Tdevice_outputs=None,
                          fused_ops=("Dequantize",), adj_x=False, adj_y=False, input_quant_mode="SCALED",
                          output_quant_mode="SCALED", op_name="_QuantizedBatchMatMul"):
    """V2: device_inputs = [x, y, args...], host_inputs = [min_x, max_x, min_y, max_y]; fused_ops ends in "Dequantize"."""
    if Tout is None:
        Tout = Tdevice_outputs[0] if Tdevice_outputs else "float"
    attrs = dict(T1=T1, T2=T2, Tout=Tout, adj_x=bool(adj_x), adj_y=bool(adj_y), fused_ops=list(fused_ops),
                 input_quant_mode=input_quant_mode, output_quant_mode=output_quant_mode)
    if U is not None:
        attrs["U"] = U
    return _cached(op_name, attrs)(*(list(device_inputs) + list(host_inputs)))


def _ITEXQuantizedConv2DWithBiasAndReluAndRequantize(input, filter, bias, min_input, max_input, min_filter, max_filter,
                                                     min_freezed_output, max_freezed_output, strides=(1, 1, 1, 1),
                                                     padding="SAME", dilations=(1, 1, 1, 1), out_type="quint8",
                                                     padding_list=(), is_filter_const=True, is_bias_const=True,
                                                     summand=None, min_summand=None, max_summand=None,
                                                     op_name="_ITEXQuantizedConv2DWithBiasAndReluAndRequantize"):
    """-> (output, min_output, max_output).  With `summand` the Sum-fused op names apply."""
    attrs = dict(Tinput=_TORCH_TO_DT[input.dtype], Tfilter="qint8",
                 Tbias="qint32" if bias.dtype == torch.int32 else _TORCH_TO_DT[bias.dtype], out_type=out_type,
                 strides=list(strides), padding=padding, dilations=list(dilations), data_format="NHWC",
                 is_filter_const=bool(is_filter_const), is_bias_const=bool(is_bias_const))
    if padding_list:
        attrs["padding_list"] = list(padding_list)
    args = [input, filter, bias, min_input, max_input, min_filter, max_filter, min_freezed_output, max_freezed_output]
    if summand is not None:
        args += [summand, min_summand, max_summand]
    dtypes = {2: L.DT_QINT32} if bias.dtype == torch.int32 else None
    return _cached(op_name, attrs)(*args, dtypes=dtypes)


def QuantizedConv2D(op_name, input, filter, bias, min_input, max_input, min_filter, max_filter, min_freezed_output=None,
                    max_freezed_output=None, strides=(1, 1, 1, 1), padding="SAME", dilations=(1, 1, 1, 1), out_type="qint32",
                    is_filter_const=True, is_bias_const=True, **extra_attrs):
    """The other members of the legacy conv family by name: QuantizedConv2D, ...PerChannel, ...AndRelu, ...WithBias,
    ...WithBiasAndRelu (qint32 outputs; `bias` None for the first three), ...AndRequantize, ...AndReluAndRequantize
    (no bias, frozen output range), _ITEXQuantizedConv2DWithDequantize / ...WithCast (real-valued output) and
    _ITEXQuantizeV2WithQuantizedConv2D (real-valued input; extra_attrs carry the QuantizeV2 attrs mode, round_mode,
    ensure_minimum_range).  -> (output, min_output, max_output), or output for a real-valued output."""
    attrs = dict(Tinput=_TORCH_TO_DT[input.dtype], Tfilter="qint8", out_type=out_type, strides=list(strides), padding=padding,
                 dilations=list(dilations), data_format="NHWC", is_filter_const=bool(is_filter_const),
                 is_bias_const=bool(is_bias_const))
    attrs.update(extra_attrs)
    args = [input, filter]
    dtypes = None
    if bias is not None:
        attrs["Tbias"] = _bias_attr(bias)
        args.append(bias)
        dtypes = {2: L.DT_QINT32} if bias.dtype == torch.int32 else None
    args += [min_input, max_input, min_filter, max_filter]
    if min_freezed_output is not None:
        args += [min_freezed_output, max_freezed_output]
    return _cached(op_name, attrs)(*args, dtypes=dtypes)


def _QuantizedConv2D(device_inputs, host_inputs, fused_ops=(), out_type="qint32", Tbias=None, Tsummand=None, strides=(1, 1, 1, 1),
                     padding="SAME", dilations=(1, 1, 1, 1), alpha=0.0, is_filter_const=True, is_bias_const=True,
                     op_name="_QuantizedConv2D"):
    """New-API quantized conv (_QuantizedConv2D / _ITEXQuantizedConv2DV2): device_inputs = [input, filter(, bias)(, summand)],
    host_inputs = [min_input, max_input, min_filter, max_filter(, min_summand, max_summand)(, min_freezed_output,
    max_freezed_output)].  -> the device output followed by the host outputs (one element for a float output)."""
    attrs = dict(Tinput=_TORCH_TO_DT[device_inputs[0].dtype], Tfilter="qint8", out_type=out_type, strides=list(strides), padding=padding,
                 dilations=list(dilations), data_format="NHWC", is_filter_const=bool(is_filter_const),
                 is_bias_const=bool(is_bias_const), alpha=float(alpha))
    if len(fused_ops) > 0:
        attrs["fused_ops"] = list(fused_ops)
    dtypes = None
    if "BiasAdd" in fused_ops:
        attrs["Tbias"] = Tbias if Tbias is not None else _bias_attr(device_inputs[2])
        dtypes = {2: L.DT_QINT32} if device_inputs[2].dtype == torch.int32 else None
    if Tsummand is not None:
        attrs["Tsummand"] = Tsummand
    return _cached(op_name, attrs)(*(list(device_inputs) + list(host_inputs)), dtypes=dtypes)


def _ITEXQuantizedReshape(tensor, shape, input_min, input_max, Tshape="int32", op_name="_ITEXQuantizedReshape"):
    """-> (output, output_min, output_max); one entry of `shape` may be -1."""
    idt = np.int64 if Tshape == "int64" else np.int32
    return _cached(op_name, dict(T=_TORCH_TO_DT[tensor.dtype], Tshape=Tshape))(tensor, np.asarray(shape, dtype=idt).reshape(-1), input_min, input_max)


def _ITEXQuantizedTranspose(x, perm, min_x, max_x, Tperm="int32", op_name="_ITEXQuantizedTranspose"):
    """-> (y, min_y, max_y)"""
    idt = np.int64 if Tperm == "int64" else np.int32
    return _cached(op_name, dict(T=_TORCH_TO_DT[x.dtype], Tperm=Tperm))(x, np.asarray(perm, dtype=idt).reshape(-1), min_x, max_x)


def _ITEXQuantizedConcatV2(values, axis, input_mins, input_maxes, Tidx="int32", op_name="_ITEXQuantizedConcatV2"):
    """-> (output, output_min, output_max); the reference's GPU kernel (and this one) serves equal input ranges only."""
    idt = np.int64 if Tidx == "int64" else np.int32
    args = list(values) + [np.asarray(axis, dtype=idt).reshape(())] + list(input_mins) + list(input_maxes)
    return _cached(op_name, dict(N=len(values), T=_TORCH_TO_DT[values[0].dtype], Tidx=Tidx))(*args)


def Fp8Quantize(x, x_amax, x_scale, fp8_meta_index, fp8_dtype="E4M3"):
    """-> y (int8 tensor holding fp8 bytes); x_amax[fp8_meta_index] is raised in place."""
    op = _cached("Fp8Quantize", dict(in_dtype=_TORCH_TO_DT[x.dtype], fp8_meta_index=int(fp8_meta_index), fp8_dtype=fp8_dtype))
    return op(x, x_amax, x_scale)


def Fp8QuantizeDbias(grad, amax, scale, fp8_meta_index, fp8_dtype="E5M2"):
    """-> (quantize_out int8 [rows, cols], dbias [cols])"""
    op = _cached("Fp8QuantizeDbias", dict(grad_dtype=_TORCH_TO_DT[grad.dtype], fp8_meta_index=int(fp8_meta_index), fp8_dtype=fp8_dtype))
    return op(grad, amax, scale)


def Fp8QuantizeDbiasDgelu(grad, gelu_inp, amax, scale, fp8_meta_index, fp8_dtype="E5M2"):
    """-> (dgelu int8 [rows, cols], dbias [cols])"""
    op = _cached("Fp8QuantizeDbiasDgelu", dict(grad_dtype=_TORCH_TO_DT[grad.dtype], in_dtype=_TORCH_TO_DT[gelu_inp.dtype],
                                               fp8_meta_index=int(fp8_meta_index), fp8_dtype=fp8_dtype))
    return op(grad, gelu_inp, amax, scale)


def Fp8Gelu(inp, amax, scale, fp8_meta_index, fp8_dtype="E4M3"):
    """-> gelu_out (int8 tensor holding fp8 bytes of gelu(inp) * scale); amax[fp8_meta_index] is raised in place."""
    op = _cached("Fp8Gelu", dict(in_dtype=_TORCH_TO_DT[inp.dtype], fp8_meta_index=int(fp8_meta_index), fp8_dtype=fp8_dtype))
    return op(inp, amax, scale)


def Fp8LayerNorm(x, gamma, beta, z_amax, z_scale, fp8_meta_index, epsilon=1e-4, fp8_dtype="E4M3", out_dtype="int8"):
    """-> (z, mu, rsigma); z is FP8 bytes (out_dtype int8) or a real tensor."""
    op = _cached("Fp8LayerNorm", dict(in_dtype=_TORCH_TO_DT[x.dtype], weight_dtype=_TORCH_TO_DT[gamma.dtype], out_dtype=out_dtype,
                                      fp8_meta_index=int(fp8_meta_index), epsilon=float(epsilon), fp8_dtype=fp8_dtype))
    return op(x, gamma, beta, z_amax, z_scale)


def Fp8Dequantize(x, x_scale_inv, fp8_meta_index, fp8_dtype="E4M3", out_dtype="float"):
    op = _cached("Fp8Dequantize", dict(out_dtype=out_dtype, fp8_meta_index=int(fp8_meta_index), fp8_dtype=fp8_dtype))
    return op(x, x_scale_inv, dtypes={0: L.DT_INT8})


def Fp8Matmul(src, weight, bias, post_add, a_scale_inv, b_scale_inv, c_amax, c_scale, fp8_meta_index_a, fp8_meta_index_b,
              fp8_meta_index_c=-1, transpose_a=False, transpose_b=False, use_bias=False, has_post_add=False,
              sum_dtype="float", out_dtype="float", fp8_dtype_a="E4M3", fp8_dtype_b="E4M3", fp8_dtype_c=""):
    op = _cached("Fp8Matmul", dict(fp8_meta_index_a=int(fp8_meta_index_a), fp8_meta_index_b=int(fp8_meta_index_b),
                                   fp8_meta_index_c=int(fp8_meta_index_c), transpose_a=bool(transpose_a),
                                   transpose_b=bool(transpose_b), use_bias=bool(use_bias), has_post_add=bool(has_post_add),
                                   sum_dtype=sum_dtype, out_dtype=out_dtype, fp8_dtype_a=fp8_dtype_a, fp8_dtype_b=fp8_dtype_b,
                                   fp8_dtype_c=fp8_dtype_c))
    return op(src, weight, bias, post_add, a_scale_inv, b_scale_inv, c_amax, c_scale, dtypes={0: L.DT_INT8, 1: L.DT_INT8})
