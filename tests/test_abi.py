"""CPU checks of the C-ABI boundary: the library loads without a GPU, exports every
function include/itexb200.h declares, and the op layer reproduces the reference's
construction-time errors (OP_REQUIRES in the kernel constructors)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "itexb200.h")).read()
    return sorted(set(re.findall(r"ITEXB_API\s+[^;(]*?\b(itexb_\w+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol(itex):
    lib = itex.load()
    names = declared_symbols()
    assert len(names) >= 55
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert b"sm_100a" in lib.itexb_version()


def test_no_device_is_reported_not_hidden(itex):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = itex.load()
    n = ctypes.c_int(-1)
    st = lib.itexb_rt_device_count(ctypes.byref(n))
    assert st == itex._lib.FAILED_PRECONDITION and n.value == 0
    assert b"CUDA" in lib.itexb_last_error()


def test_op_registry_names_and_host_memory_masks(itex):
    import importlib
    ops = importlib.import_module("itex_b200.ops")
    names = set(ops.op_list())
    for base in ("QuantizeV2", "Dequantize", "QuantizedMatMulWithBias", "QuantizedMatMulWithBiasAndRelu",
                 "QuantizedMatMulWithBiasAndRequantize", "QuantizedMatMulWithBiasAndReluAndRequantize",
                 "QuantizedMatMulWithBiasAndDequantize", "QuantizedConv2DWithBiasAndReluAndRequantize"):
        assert base in names and "_ITEX" + base in names  # stock and _ITEX names, like the reference GPU build
    for n in ("Fp8Quantize", "Fp8Dequantize", "Fp8Matmul"):
        assert n in names
    # min_range/max_range and output_min/output_max are HostMemory (gpu/quantize_op.cc:25-31)
    assert ops.op_signature("_ITEXQuantizeV2") == (3, 3, 0b110, 0b110)
    assert ops.op_signature("_ITEXDequantize") == (3, 1, 0b110, 0)
    # min_a..max_b, min/max_freezed_output host; min_out/max_out host (gpu/quantized_matmul.cc:53-102)
    assert ops.op_signature("_ITEXQuantizedMatMulWithBias") == (7, 3, 0b1111000, 0b110)
    assert ops.op_signature("_ITEXQuantizedMatMulWithBiasAndDequantize") == (9, 1, 0b111111000, 0)
    assert ops.op_signature("_ITEXQuantizedConv2DWithBiasAndReluAndRequantize") == (9, 3, 0b111111000, 0b110)
    # perm / shape and the ranges are HostMemory (gpu/transpose_op.cc:48-56, gpu/quantized_reshape_op.cc); the concat's
    # arity depends on N (common/quantized_concat_op.cc:251-268)
    assert ops.op_signature("_ITEXQuantizedTranspose") == ops.op_signature("_QuantizedTranspose") == (4, 3, 0b1110, 0b110)
    assert ops.op_signature("_ITEXQuantizedReshape") == ops.op_signature("QuantizedReshape") == (4, 3, 0b1110, 0b110)
    assert ops.op_signature("_ITEXQuantizedConcatV2") == ops.op_signature("QuantizedConcatV2") == (-1, 3, 0, 0b110)
    with pytest.raises(itex.ItexError) as e:
        ops.op_signature("NoSuchOp")
    assert e.value.code == itex._lib.NOT_FOUND


def test_layout_kernels_reject_bad_arguments_before_touching_a_device(itex):
    """itexb_transpose / itexb_copy_rows validate on the host: these calls return without a CUDA call."""
    lib, L = itex.load(), itex._lib

    class Transpose(ctypes.Structure):
        _fields_ = [("x", ctypes.c_void_p), ("y", ctypes.c_void_p), ("rank", ctypes.c_int32), ("elem_size", ctypes.c_int32),
                    ("dims", ctypes.c_int64 * 8), ("perm", ctypes.c_int32 * 8)]

    def call(rank, dims, perm, esz=1):
        p = Transpose()
        p.rank, p.elem_size = rank, esz
        for i, d in enumerate(dims):
            p.dims[i] = d
        for i, a in enumerate(perm):
            p.perm[i] = a
        return lib.itexb_transpose(ctypes.byref(p), None)

    assert call(9, [1] * 8, list(range(8))) == L.INVALID_ARGUMENT            # rank above ITEXB_TRANSPOSE_MAX_RANK
    assert call(3, [2, 3, 4], [0, 1, 1]) == L.INVALID_ARGUMENT                # not a permutation
    assert call(3, [2, 3, 4], [0, 1, 3]) == L.INVALID_ARGUMENT
    assert call(2, [2, 3], [1, 0], esz=3) == L.INVALID_ARGUMENT
    assert call(3, [2, 0, 4], [2, 1, 0]) == L.OK                              # empty: nothing to do
    assert call(2, [2, 3], [1, 0]) == L.INVALID_ARGUMENT                      # NULL tensors
    lib.itexb_copy_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    assert lib.itexb_copy_rows(None, None, 4, 32, 16, 0, None) == L.INVALID_ARGUMENT   # rows longer than the pitch
    assert lib.itexb_copy_rows(None, None, 4, 16, 32, 24, None) == L.INVALID_ARGUMENT  # past the end of a row
    assert lib.itexb_copy_rows(None, None, 0, 16, 32, 0, None) == L.OK
    assert lib.itexb_copy_rows(None, None, 4, 16, 32, 0, None) == L.INVALID_ARGUMENT   # NULL pointers


@pytest.mark.parametrize("attrs,fragment", [
    (dict(T="qint8", mode="MIN_COMBINED"), "only supports SCALED and MIN_FIRST MODE"),
    (dict(T="qint8", mode="BOGUS"), "Mode string must be 'MIN_COMBINED', 'MIN_FIRST', or 'SCALED', is 'BOGUS'"),
    (dict(T="qint8", mode="SCALED", round_mode="UP"), "Round mode string must be"),
    (dict(T="qint8", mode="MIN_FIRST", round_mode="HALF_TO_EVEN"), "only supported for mode 'SCALED'"),
    (dict(T="qint32", mode="SCALED"), "no kernel registered for T=qint32"),
])
def test_quantize_constructor_errors(itex, attrs, fragment):
    import importlib
    ops = importlib.import_module("itex_b200.ops")
    with pytest.raises(itex.ItexError) as e:
        ops.Op("_ITEXQuantizeV2", **attrs)
    assert e.value.code == itex._lib.INVALID_ARGUMENT and fragment in str(e.value)


def test_matmul_and_conv_constructor_errors(itex):
    import importlib
    ops = importlib.import_module("itex_b200.ops")
    with pytest.raises(itex.ItexError) as e:
        ops.Op("_ITEXQuantizedMatMulWithBias", T1="quint8", T2="qint8", Toutput="qint32", input_quant_mode="SYMMETRIC")
    assert "Quantization mode must be either MIN_FIRST or SCALED, but received SYMMETRIC" in str(e.value)
    with pytest.raises(itex.ItexError) as e:  # T1 is quint8-only on these ops (cpu/quantized_matmul.cc:27)
        ops.Op("_ITEXQuantizedMatMulWithBias", T1="qint8", T2="qint8", Toutput="qint32")
    assert "no kernel registered" in str(e.value)
    with pytest.raises(itex.ItexError) as e:
        ops.Op("_ITEXQuantizedMatMulWithBiasAndDequantize", Toutput="quint8")
    assert "no kernel registered for Toutput=quint8" in str(e.value)
    conv = "_ITEXQuantizedConv2DWithBiasAndReluAndRequantize"
    with pytest.raises(itex.ItexError) as e:
        ops.Op(conv, strides=[1, 1, 1], padding="SAME")
    assert "Sliding window strides field must specify 4 dimensions" in str(e.value)
    with pytest.raises(itex.ItexError) as e:
        ops.Op(conv, strides=[2, 1, 1, 1], padding="SAME")
    assert e.value.code == itex._lib.UNIMPLEMENTED and "strides in the batch and depth dimensions" in str(e.value)
    with pytest.raises(itex.ItexError) as e:
        ops.Op(conv, strides=[1, 0, 1, 1], padding="SAME")
    assert "Row and column strides should be larger than 0." in str(e.value)
    with pytest.raises(itex.ItexError) as e:
        ops.Op(conv, strides=[1, 1, 1, 1], padding="SAME", dilations=[1, 0, 1, 1])
    assert "Dilated rates should be larger than 0." in str(e.value)
    with pytest.raises(itex.ItexError) as e:
        ops.Op("Fp8Quantize", fp8_meta_index=0, fp8_dtype="E3M4")
    assert "Unsupported fp8_dtype" in str(e.value)
    ops.Op(conv, strides=[1, 1, 1, 1], padding="SAME")  # defaults as in the op def


def test_fp8_recipe_rejects_what_the_reference_rejects(itex):
    import importlib
    fp8 = importlib.import_module("itex_b200.fp8")
    fp8.DelayedScaling(margin=0, amax_history_len=16, amax_compute_algo="most_recent")
    with pytest.raises(ValueError):
        fp8.DelayedScaling(amax_compute_algo=lambda h: h)
    with pytest.raises(ValueError):
        fp8.DelayedScaling(scaling_factor_compute_algo=lambda *a: a)


def test_fp8_autocast_state_nests_and_restores(itex):
    """fp8_autocast (itex/python/fp8/autocast.py:122-151): flag and recipe inside the block, outer state back on exit -
    also when the block raises; the default recipe when none is given."""
    import importlib
    fp8 = importlib.import_module("itex_b200.fp8")
    assert not fp8.is_fp8_enabled() and fp8.get_fp8_recipe() is None
    outer = fp8.DelayedScaling(margin=1, amax_history_len=16)
    with fp8.fp8_autocast(enabled=True, fp8_recipe=outer):
        assert fp8.is_fp8_enabled() and fp8.get_fp8_recipe() is outer
        with fp8.fp8_autocast(enabled=False):
            assert not fp8.is_fp8_enabled()
            assert fp8.get_fp8_recipe() == fp8.get_default_fp8_recipe()
        assert fp8.is_fp8_enabled() and fp8.get_fp8_recipe() is outer
        with pytest.raises(RuntimeError):
            with fp8.fp8_autocast(enabled=True):
                raise RuntimeError("inside")
        assert fp8.get_fp8_recipe() is outer
    assert not fp8.is_fp8_enabled() and fp8.get_fp8_recipe() is None
    assert fp8.get_fp8_dtype(outer, fwd=True) == "E4M3" and fp8.get_fp8_dtype(outer, fwd=False) == "E5M2"


def test_op_definitions_match_the_reference_registrations(itex, golden_dir):
    """itexb_op_def for every registered name: the names the plugin has to define itself carry exactly the input, output
    and attr specification strings the reference hands to TF_OpDefinitionBuilder (tests/golden/op_defs.json, extracted
    from itex/core/ops/nn_ops.cc and fp8_ops.cc by tests/golden/make_opdef_fixture.py); the others are TensorFlow's ops."""
    import importlib
    import json
    ops = importlib.import_module("itex_b200.ops")
    lib, L = itex.load(), itex._lib
    fixture = json.load(open(os.path.join(golden_dir, "op_defs.json")))
    assert sorted(ops.op_list()) == json.load(open(os.path.join(golden_dir, "op_names.json")))
    seen = 0
    for name in ops.op_list():
        d = L.OpDef()
        assert lib.itexb_op_def(name.encode(), ctypes.byref(d)) == L.OK
        got = {k: [getattr(d, k)[i].decode() for i in range(getattr(d, "num_" + k))] for k in ("inputs", "outputs", "attrs")}
        if name in fixture["ops"]:
            want = fixture["ops"][name]
            assert d.defined_by_plugin == 1 and d.name.decode() == name
            assert got == {k: want[k] for k in ("inputs", "outputs", "attrs")}, name
            seen += 1
        else:
            # TensorFlow's own op (or a name the reference gives kernels but no definition): the argument names come from
            # the twin the reference defines, for the HostMemory registration
            assert name in fixture["defined_by_tensorflow"] and d.defined_by_plugin == 0
            twin = {"QuantizedAvgPool": "ITEXQuantizedAvgPool", "_ITEXQuantizedAvgPool": "ITEXQuantizedAvgPool"}.get(
                name, "_ITEX" + (name[1:] if name.startswith("_Quantized") else name))
            if twin in fixture["ops"]:
                assert got["inputs"] == fixture["ops"][twin]["inputs"], name
            assert got["inputs"], name          # every kernel can name its HostMemory arguments
    assert seen == len(fixture["ops"]) >= 40
    # what the kernels read is what the definitions declare: every attr the quantized matmul reads exists in its definition
    mm = fixture["ops"]["_ITEXQuantizedMatMulWithBiasAndDequantize"]
    assert mm["inputs"][:3] == ["a: T1", "b: T2", "bias: Tbias"] and "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'MIN_FIRST'" in mm["attrs"]
    d = L.OpDef()
    assert lib.itexb_op_def(b"NoSuchOp", ctypes.byref(d)) == L.NOT_FOUND


def test_debug_hooks_reject_unknown_keys(itex):
    lib, L = itex.load(), itex._lib
    assert lib.itexb_debug_set(b"gemm_skip_kblock", ctypes.c_int64(-1)) == L.OK
    assert lib.itexb_debug_set(b"gemm_wait_limit_cycles", ctypes.c_int64(0)) == L.OK
    assert lib.itexb_debug_set(b"gemm_wait_limit_cycles", ctypes.c_int64(-5)) == L.INVALID_ARGUMENT
    assert lib.itexb_debug_set(b"gemm_cta_pair", ctypes.c_int64(2)) == L.INVALID_ARGUMENT
    assert lib.itexb_debug_set(b"gemm_cta_pair", ctypes.c_int64(-1)) == L.OK
    assert lib.itexb_debug_set(b"bogus", ctypes.c_int64(1)) == L.NOT_FOUND
    assert lib.itexb_op_check(None, 1) == L.INVALID_ARGUMENT


def _rewrite(itex, op, on_gpu=False, all_deq=False, **attrs):
    import importlib
    ops = importlib.import_module("itex_b200.ops")
    lib, L = itex.load(), itex._lib
    arr, keep = ops.make_attrs(attrs)
    q = L.RewriteQuery(op.encode(), ctypes.cast(arr, ctypes.POINTER(L.Attr)), len(attrs), int(on_gpu), int(all_deq))
    r = L.RewriteResult()
    st = lib.itexb_rewrite_node(ctypes.byref(q), ctypes.byref(r))
    if st != L.OK:
        return st, None, None
    added = {}
    for i in range(r.num_added):
        a = r.added[i]
        added[a.name.decode()] = a.s.decode() if a.type == 3 else int(a.i)
    return st, (r.new_op.decode() if r.new_op else None), added


def test_rewrite_rules_match_the_reference_table(itex, golden_dir):
    """itexb_rewrite_node against the reference's rename table (tests/golden/rewrite_table.json, extracted from
    native_layout.cc:113-199) for every entry whose target this library implements, and the predicate / attr-copy rules
    of layout_utils.cc:315-354,471-542 case by case."""
    import importlib
    import json
    ops = importlib.import_module("itex_b200.ops")
    lib, L = itex.load(), itex._lib
    table = json.load(open(os.path.join(golden_dir, "rewrite_table.json")))
    registered = set(ops.op_list())
    mine = {}
    i = 0
    while True:
        f, t = ctypes.c_char_p(), ctypes.c_char_p()
        if lib.itexb_rewrite_rule(i, ctypes.byref(f), ctypes.byref(t)) != L.OK:
            break
        mine[f.value.decode()] = t.value.decode()
        i += 1
    want = {e["from"]: e for e in table if e["to"] in registered}
    assert len(want) >= 25 and mine == {k: v["to"] for k, v in want.items()}
    need = {"CopyAttrsQuantizedConv2D": dict(out_type="qint32"), "CopyAttrsQuantizedMatMul": dict(Toutput="qint32"),
            "CopyAttrsQuantize": dict(mode="SCALED", round_mode="HALF_TO_EVEN"), "CopyAttrsAll": {}}
    for f, e in want.items():
        attrs = dict(need[e["copy"]])
        if e["rule"] == "RewriteQuantize":
            attrs.setdefault("mode", "SCALED")
        if e["rule"] == "RewriteQuantizeReshape":
            attrs["T"] = "qint8"
        st, new_op, added = _rewrite(itex, f, **attrs)
        assert st == L.OK and new_op == e["to"], f
        if e["copy"] == "CopyAttrsQuantizedConv2D":
            assert added == {"data_format": "NHWC"}
    # ops the table does not hold stay as they are
    assert _rewrite(itex, "Conv2D") == (L.OK, None, {})
    assert _rewrite(itex, "QuantizedConcatV2") == (L.OK, None, {})        # disabled in the reference's table
    # RewriteQuantizeReshape (layout_utils.cc:392-400): only a qint8 reshape is taken over
    assert _rewrite(itex, "QuantizedReshape", T="qint8")[1] == "_ITEXQuantizedReshape"
    assert _rewrite(itex, "QuantizedReshape", T="quint8")[1] is None
    assert _rewrite(itex, "QuantizedReshape")[0] == L.INVALID_ARGUMENT
    # RewriteQuantize
    assert _rewrite(itex, "QuantizeV2", mode="MIN_COMBINED", round_mode="HALF_AWAY_FROM_ZERO")[1] is None
    assert _rewrite(itex, "QuantizeV2", mode="SCALED", round_mode="HALF_AWAY_FROM_ZERO")[1] is None
    assert _rewrite(itex, "QuantizeV2", mode="MIN_FIRST", round_mode="HALF_AWAY_FROM_ZERO")[1] == "_ITEXQuantizeV2"
    assert _rewrite(itex, "Dequantize", mode="MIN_FIRST", on_gpu=True)[1] is None
    assert _rewrite(itex, "Dequantize", mode="MIN_FIRST", on_gpu=False)[1] == "_ITEXDequantize"
    assert _rewrite(itex, "Dequantize", mode="SCALED", on_gpu=True)[1] == "_ITEXDequantize"
    assert _rewrite(itex, "QuantizeV2")[0] == L.INVALID_ARGUMENT           # no `mode`
    # CopyAttrsQuantize: dtype defaults to float when absent; classic_asymmetric_algorithm follows the consumers
    st, new_op, added = _rewrite(itex, "QuantizeV2", mode="SCALED", round_mode="HALF_TO_EVEN", all_deq=True)
    assert added == {"dtype": L.DT_FLOAT, "classic_asymmetric_algorithm": 1}
    st, new_op, added = _rewrite(itex, "QuantizeV2", mode="SCALED", round_mode="HALF_TO_EVEN", dtype="bfloat16")
    assert added == {"classic_asymmetric_algorithm": 0}
    # CopyAttrsQuantizedConv2D / MatMul: Tbias carried over when present; out_type / Toutput required
    st, new_op, added = _rewrite(itex, "QuantizedConv2DWithBiasAndReluAndRequantize", out_type="quint8", Tbias="float")
    assert new_op == "_ITEXQuantizedConv2DWithBiasAndReluAndRequantize" and added == {"data_format": "NHWC", "Tbias": L.DT_FLOAT}
    assert _rewrite(itex, "QuantizedConv2D")[0] == L.INVALID_ARGUMENT
    st, new_op, added = _rewrite(itex, "QuantizedMatMulWithBiasAndDequantize", Toutput="float", Tbias="qint32")
    assert new_op == "_ITEXQuantizedMatMulWithBiasAndDequantize" and added == {"Tbias": L.DT_QINT32}
    assert _rewrite(itex, "QuantizedMatMulWithBias")[0] == L.INVALID_ARGUMENT
