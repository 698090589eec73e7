"""ctypes binding of libitexb200.so (the C-ABI declared in include/itexb200.h).

The library is the product; there is no Python or CPU fallback.  If the shared
object has not been built the import fails with the build command to run.
"""
import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libitexb200.so")

MAX_DIMS = 8

# itexb_dtype_t
DT_FLOAT, DT_INT32, DT_UINT8, DT_INT8, DT_INT64 = 1, 3, 4, 6, 9
DT_QINT8, DT_QUINT8, DT_QINT32, DT_BFLOAT16, DT_HALF = 11, 12, 13, 14, 19
DT_FP8_E4M3, DT_FP8_E5M2 = 101, 102
# itexb_activation_t
(ACT_NONE, ACT_RELU, ACT_CLIP, ACT_GELU_ERF, ACT_GELU_TANH, ACT_SIGMOID, ACT_TANH, ACT_ELU, ACT_SWISH,
 ACT_LINEAR) = range(10)

# itexb_status_t
OK, INVALID_ARGUMENT, NOT_FOUND, RESOURCE_EXHAUSTED = 0, 3, 5, 8
FAILED_PRECONDITION, ABORTED, UNIMPLEMENTED, INTERNAL = 9, 10, 12, 13

STATUS_NAMES = {0: "OK", 3: "INVALID_ARGUMENT", 5: "NOT_FOUND", 8: "RESOURCE_EXHAUSTED",
                9: "FAILED_PRECONDITION", 10: "ABORTED", 12: "UNIMPLEMENTED", 13: "INTERNAL"}


class ItexError(RuntimeError):
    """A non-OK itexb_status_t; `.code` is the status, the text is itexb_last_error()."""

    def __init__(self, code, message):
        super().__init__("%s: %s" % (STATUS_NAMES.get(code, str(code)), message))
        self.code = code


class Epilogue(C.Structure):
    _fields_ = [("scale", C.c_void_p), ("scale_count", C.c_int32), ("alpha_a", C.c_void_p),
                ("alpha_b", C.c_void_p), ("bias", C.c_void_p), ("summand", C.c_void_p),
                ("summand_dtype", C.c_int32), ("ld_summand", C.c_int64), ("sum_scale", C.c_float),
                ("relu", C.c_int32), ("raw_acc", C.c_int32), ("out_scale", C.c_void_p),
                ("amax", C.c_void_p), ("mid_dtype", C.c_int32), ("activation", C.c_int32),
                ("act_alpha", C.c_float), ("act_beta", C.c_float), ("post_scale", C.c_float)]


class GemmParams(C.Structure):
    _fields_ = [("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("a_dtype", C.c_int32),
                ("b_dtype", C.c_int32), ("out_dtype", C.c_int32), ("a", C.c_void_p), ("lda", C.c_int64),
                ("b", C.c_void_p), ("ldb", C.c_int64), ("out", C.c_void_p), ("ldo", C.c_int64),
                ("ep", Epilogue), ("status_word", C.c_void_p), ("batch", C.c_int32), ("stride_a", C.c_int64),
                ("stride_b", C.c_int64), ("stride_out", C.c_int64), ("num_peers", C.c_int32), ("peer_out", C.POINTER(C.c_void_p))]


class ConvParams(C.Structure):
    _fields_ = [("n", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("c", C.c_int32),
                ("kh", C.c_int32), ("kw", C.c_int32), ("co", C.c_int32),
                ("stride_h", C.c_int32), ("stride_w", C.c_int32), ("dil_h", C.c_int32), ("dil_w", C.c_int32),
                ("pad_top", C.c_int32), ("pad_left", C.c_int32), ("oh", C.c_int32), ("ow", C.c_int32),
                ("c_pad", C.c_int32), ("x_dtype", C.c_int32), ("out_dtype", C.c_int32),
                ("x", C.c_void_p), ("filter_packed", C.c_void_p), ("out", C.c_void_p), ("ep", Epilogue),
                ("status_word", C.c_void_p), ("workspace", C.c_void_p)]


class PoolParams(C.Structure):
    _fields_ = [("n", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("c", C.c_int32), ("kh", C.c_int32), ("kw", C.c_int32),
                ("stride_h", C.c_int32), ("stride_w", C.c_int32), ("pad_top", C.c_int32), ("pad_left", C.c_int32),
                ("oh", C.c_int32), ("ow", C.c_int32), ("dtype", C.c_int32), ("is_avg", C.c_int32), ("x", C.c_void_p),
                ("out", C.c_void_p)]


class Tensor(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rank", C.c_int32), ("dims", C.c_int64 * MAX_DIMS),
                ("data", C.c_void_p), ("on_host", C.c_int32), ("reserved", C.c_int32)]


class Attr(C.Structure):
    _fields_ = [("name", C.c_char_p), ("type", C.c_int32), ("i", C.c_int64), ("f", C.c_float),
                ("s", C.c_char_p), ("list_i", C.POINTER(C.c_int64)), ("list_s", C.POINTER(C.c_char_p)),
                ("list_len", C.c_int32)]


class AllocatorStats(C.Structure):
    _fields_ = [("num_allocs", C.c_int64), ("bytes_in_use", C.c_int64), ("peak_bytes_in_use", C.c_int64),
                ("bytes_reserved", C.c_int64), ("largest_alloc_size", C.c_int64), ("bytes_limit", C.c_int64)]


class OpDef(C.Structure):
    _fields_ = [("name", C.c_char_p), ("defined_by_plugin", C.c_int32), ("num_inputs", C.c_int32), ("inputs", C.POINTER(C.c_char_p)),
                ("num_outputs", C.c_int32), ("outputs", C.POINTER(C.c_char_p)), ("num_attrs", C.c_int32), ("attrs", C.POINTER(C.c_char_p))]


class RewriteQuery(C.Structure):
    _fields_ = [("op", C.c_char_p), ("attrs", C.POINTER(Attr)), ("num_attrs", C.c_int32), ("on_gpu", C.c_int32),
                ("all_consumers_are_dequantize", C.c_int32)]


class RewriteResult(C.Structure):
    _fields_ = [("new_op", C.c_char_p), ("num_added", C.c_int32), ("added", Attr * 4)]


ALLOC_OUTPUT_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.POINTER(Tensor))
ALLOC_TEMP_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.POINTER(C.c_void_p))


class OpContext(C.Structure):
    _fields_ = [("user", C.c_void_p), ("num_inputs", C.c_int32), ("inputs", C.POINTER(Tensor)),
                ("device_ordinal", C.c_int32), ("stream", C.c_void_p), ("allocate_output", ALLOC_OUTPUT_FN),
                ("allocate_temp", ALLOC_TEMP_FN)]


_lib = None


def load():
    """Loads libitexb200.so; raises ImportError with the build command when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libitexb200.so is not built (%s). Build it with: python %s" % (LIB_PATH, os.path.join(PKG, "build.py")))
    lib = C.CDLL(LIB_PATH)
    lib.itexb_last_error.restype = C.c_char_p
    lib.itexb_version.restype = C.c_char_p
    lib.itexb_launch_count.restype = C.c_uint64
    lib.itexb_conv2d_workspace_bytes.restype = C.c_size_t
    lib.itexb_conv2d_filter_c_pad.restype = C.c_int32
    lib.itexb_op_check.argtypes = [C.c_void_p, C.c_int]
    lib.itexb_op_def.argtypes = [C.c_char_p, C.POINTER(OpDef)]
    lib.itexb_debug_set.argtypes = [C.c_char_p, C.c_int64]
    lib.itexb_rewrite_node.argtypes = [C.POINTER(RewriteQuery), C.POINTER(RewriteResult)]
    lib.itexb_rewrite_rule.argtypes = [C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p)]
    lib.itexb_rt_allocate.argtypes = [C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]
    lib.itexb_rt_deallocate.argtypes = [C.c_int, C.c_void_p]
    lib.itexb_rt_ipc_export.argtypes = [C.c_void_p, C.c_char_p]
    lib.itexb_rt_ipc_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.itexb_rt_ipc_close.argtypes = [C.c_void_p]
    lib.itexb_peer_signal.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.itexb_peer_wait.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.itexb_peer_advance.argtypes = [C.c_void_p, C.c_void_p]
    _lib = lib
    return lib


def check(status):
    if status != OK:
        raise ItexError(status, load().itexb_last_error().decode("utf-8", "replace"))
