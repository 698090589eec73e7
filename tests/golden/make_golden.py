"""Generates the committed golden fixtures under tests/golden/.

Two kinds of fixture:

1. reference_kat.json - known-answer vectors transcribed from the reference's
   own tests (inputs, attrs and expected outputs exactly as those tests state
   them), so the oracle and the CUDA path can be pinned without TensorFlow:
     test/tensorflow/python/kernel_tests/block_layout/quantized_ops_test.py
     test/tensorflow/python/kernel_tests/block_layout/dequantize_op_test.py
     test/sanity/quantization/quantized_matmul_op_test.py

2. onednn_matmul.npz / onednn_conv.npz - outputs of REAL oneDNN (the library the
   reference calls; here v3.10.2 reached through torch.ops.onednn.q*_pointwise,
   while the reference pins commit 242d4d9) on small seeded inputs.  The
   combined scale is passed as the weight scale and the pre-scaled bias as the
   bias, exactly how the reference drives dnnl::inner_product_forward /
   dnnl::convolution_forward (scale on DNNL_ARG_WEIGHTS, bias added after).

Run from the repository root on a machine with PyTorch (CPU is enough):
    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import itex_oracle as o  # noqa: E402  (host scale math only; outputs come from oneDNN)


def write_reference_kat():
    kat = {
        "source": "intel/intel-extension-for-tensorflow test suite (values transcribed)",
        "quantize_axis": {  # quantized_ops_test.py:141-212
            "shape": [2, 3, 4, 5],
            "values": [-1, -0.5, 0, 0.3, 0.8, 0.555, 0.5],
            "quant_values": [-127, -64, 0, 38, 102, 70, 64],
            "axes": [1, 2, 3, None],
            "min_per_slice": -1.0, "max_per_slice": 0.8,
            "T": "qint8", "mode": "SCALED", "round_mode": "HALF_TO_EVEN", "narrow_range": True,
            "compare": "exact",
        },
        "quantize_min_first": {  # quantized_ops_test.py:49-90
            "x": [1.0, 1.25, 1.75, 127.0, 255.0, 500.0], "min": 0.0, "max": 255.0,
            "T": "quint8", "expected": [1, 1, 2, 127, 255, 255], "atol": 0.1,
        },
        "quantize_asymmetric_legacy": {  # quantized_ops_test.py:93-124
            "x": [-1.0, 1.25, 1.75, 2.5, 2.75, 3.0], "min": -1.0, "max": 3.0, "T": "quint8",
            "expected": [0, 143, 175, 223, 239, 255], "atol": 0.1,
        },
        "quantize_asymmetric_classic": {  # quantized_ops_test.py:228-267
            "x": [-1.0, 1.25, 1.75, 2.5, 2.75, 3.0], "min": -1.0, "max": 3.0, "T": "quint8",
            "expected": [0, 144, 176, 223, 239, 255], "atol": 0.1,
        },
        "dequantize_min_first": {  # quantized_ops_test.py:126-138
            "q": [1, 2, 4, 8, 16, 255], "min": 0.0, "max": 255.0, "T": "quint8",
            "expected": [1.0, 2.0, 4.0, 8.0, 16.0, 255.0], "atol": 0.1,
        },
        "dequantize_axis": {  # dequantize_op_test.py:120-169
            "shape": [2, 3, 4, 5],
            "values": [-128, -64, 0, 38, 102, 71, 64],
            "dequant_values": [-2.015748, -1.007874, 0, 0.5984252, 1.6062992, 1.1181102, 1.007874],
            "axes": [0, 1, 2, 3, None],
            "min_per_slice": -2.0, "max_per_slice": 1.6,
            "T": "qint8", "mode": "SCALED", "narrow_range": True, "rtol": 1e-5, "atol": 1e-5,
        },
        "dequantize_scaled": {  # dequantize_op_test.py:48-118 (closed form: q * max(min/-127|-128, max/127))
            "cases": [
                {"q": [-128, 0, 127], "min": -1.0, "max": 2.0},
                {"q": [-2, 4, -17], "min": -5.0, "max": -3.0},
                {"q": [0, -4, 42, -108], "min": 5.0, "max": 40.0},
            ],
            "T": "qint8", "rtol": 1e-2, "atol": 1e-2,
        },
        "matmul_min_first": {  # quantized_matmul_op_test.py:41-236 (fp32 matmul at rtol=atol=0.2)
            "x_f32": [[1.51, 1.13, -0.66], [0.79, 0.98, 1.88]],
            "y_f32": [[-1.71, 3.05, 2.05, 0.64], [0.73, 0.23, 1.42, 3.57], [-0.61, 2.24, 2.69, 2.90]],
            "bias_f32": [-1.42, 2.05, -1.00, 0.94],
            "x_quant": {"T": "quint8", "mode": "MIN_FIRST"},
            "y_quant": {"T": "qint8", "mode": "SCALED", "round_mode": "HALF_TO_EVEN"},
            "input_quant_mode": "MIN_FIRST", "rtol": 0.2, "atol": 0.2,
        },
        "fused_matmul_min_first": {  # kernel_tests/native_quantized_fused_matmul_test.py:46-203 (fp32 math at rtol=atol=0.2)
            "x_f32": [[1.51, 1.13, -0.66], [0.79, 0.98, 1.88]],
            "y_f32": [[-1.71, 3.05, 2.05, 0.64], [0.73, 0.23, 1.42, 3.57], [-0.61, 2.24, 2.69, 2.90]],
            "bias_f32": [-1.42, 2.05, -1.00, 0.94],
            "z_f32": [[0.92, 1.43, 1.84, -1.01], [-1.83, -1.39, -0.50, 0.32]],  # the test feeds z + z as the addend
            "x_quant": {"T": "quint8", "mode": "MIN_FIRST"},
            "y_quant": {"T": "qint8", "mode": "SCALED", "round_mode": "HALF_TO_EVEN", "narrow_range": True},
            "cases": [
                {"fused_ops": ["BiasAdd", "GeluApproximate"], "per_channel": False},
                {"fused_ops": ["BiasAdd", "GeluApproximate"], "per_channel": True},
                {"fused_ops": ["BiasAdd", "Add"], "per_channel": False},
            ],
            "input_quant_mode": "MIN_FIRST", "Toutput": "float", "rtol": 0.2, "atol": 0.2,
        },
        "batch_matmul": {  # test/sanity/array/quantized_batch_matmul_test.py:48-190 (fp32 math at rtol=atol=0.5)
            "x_f32": [[[-0.33, 1.33, 1.44], [-0.23, 0.60, -0.08]], [[0.97, 0.70, 0.90], [-0.56, -1.84, -1.27]]],
            "y_f32": [[[0.14, 0.78], [1.51, -1.36], [0.56, -0.29]], [[1.05, 1.82], [1.72, 0.36], [0.16, -0.10]]],
            "mul": 0.5,
            "add_f32": [[[0.19, -0.35], [0.03, -0.41]], [[0.72, -0.12], [0.87, -0.84]]],
            "quant": {"T": "qint8", "mode": "SCALED", "round_mode": "HALF_TO_EVEN", "narrow_range": True},
            "cases": [[], ["Mul"], ["Mul", "Add"]],
            "rtol": 0.5, "atol": 0.5,
        },
    }
    with open(os.path.join(HERE, "reference_kat.json"), "w") as f:
        json.dump(kat, f, indent=1)


def onednn_linear(qa, qb_kn, scale, bias_p, relu, out_dtype):
    import torch
    n = qb_kn.shape[1]
    qw = torch.from_numpy(np.ascontiguousarray(qb_kn.T))
    pw = torch.ops.onednn.qlinear_prepack(qw, None)
    ws = torch.from_numpy(np.broadcast_to(np.asarray(scale, np.float32), (n,)).copy())
    wz = torch.zeros(n, dtype=torch.int64)
    y = torch.ops.onednn.qlinear_pointwise(torch.from_numpy(qa), 1.0, 0, pw, ws, wz,
                                           torch.from_numpy(bias_p), 1.0, 0, out_dtype,
                                           "relu" if relu else "none", [], "")
    return y.float().numpy() if y.dtype == torch.bfloat16 else y.numpy()


def onednn_conv(x_nhwc, f_hwio, scale, bias_p, stride, pad, relu, out_dtype):
    import torch
    qx = torch.from_numpy(np.ascontiguousarray(x_nhwc.transpose(0, 3, 1, 2))).contiguous(
        memory_format=torch.channels_last)
    qw = torch.from_numpy(np.ascontiguousarray(f_hwio.transpose(3, 2, 0, 1)))  # OIHW
    co = f_hwio.shape[3]
    ws = torch.from_numpy(np.asarray(scale, np.float32).copy())
    wz = torch.zeros(co, dtype=torch.int64)
    pw = torch.ops.onednn.qconv_prepack(qw, ws, 1.0, 0, list(stride), list(pad), [1, 1], 1, None)
    y = torch.ops.onednn.qconv2d_pointwise(qx, 1.0, 0, pw, ws, wz, torch.from_numpy(bias_p),
                                           list(stride), list(pad), [1, 1], 1, 1.0, 0, out_dtype,
                                           "relu" if relu else "none", [], "")
    y = y.float() if y.dtype == torch.bfloat16 else y
    return np.ascontiguousarray(y.permute(0, 2, 3, 1).numpy())


def write_onednn_matmul():
    import torch
    rng = np.random.default_rng(20240501)
    out = {}
    M, K, N = 24, 160, 72
    x = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    qa, mna, mxa = o.quantize_v2(x, x.min(), x.max(), T="quint8")
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    qb, mnb, mxb = o.quantize_v2(w, w.min(), w.max(), T="qint8")
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    mnf, mxf = np.float32(0.0), np.float32(1.5)
    out.update(a=qa, b=qb, bias=bias, min_a=mna, max_a=mxa, min_b=mnb, max_b=mxb,
               min_freezed=mnf, max_freezed=mxf)
    for tout, tdt in (("float", torch.float32), ("quint8", torch.uint8), ("bfloat16", torch.bfloat16)):
        for mode in ("SCALED", "MIN_FIRST"):
            for sbm in ("literal", "intended"):
                for relu in (False, True):
                    sc = o.matmul_output_scale(mna, mxa, mnb, mxb, tout, mnf, mxf)
                    bp = o.matmul_scaled_bias(bias, qb, mna, mxa, mnb, mxb, mode, tout, sc, "float", sbm)
                    y = onednn_linear(qa, qb, sc, bp, relu, tdt)
                    out["y_%s_%s_%s_%d" % (tout, mode, sbm, relu)] = y
    np.savez_compressed(os.path.join(HERE, "onednn_matmul.npz"), **out)


def write_onednn_conv():
    import torch
    rng = np.random.default_rng(20240502)
    out = {}
    cases = {"c3s1": (2, 9, 10, 16, 3, 24, 1), "c3s2": (2, 9, 10, 16, 3, 24, 2), "c1s1": (1, 6, 6, 32, 1, 16, 1)}
    for name, (n, h, w, c, k, co, s) in cases.items():
        x = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
        f32f = (rng.standard_normal((k, k, c, co)) * 0.05).astype(np.float32)
        amax = np.abs(f32f).reshape(-1, co).max(axis=0)
        qf = np.clip(np.rint(f32f * (127.0 / amax)), -127, 127).astype(np.int8)
        bias = (rng.standard_normal(co) * 0.1).astype(np.float32)
        mni, mxi = np.float32(0.0), np.float32(12.75)
        mnf, mxf = (-amax).astype(np.float32), amax.astype(np.float32)
        mno, mxo = np.float32(0.0), np.float32(20.0)
        oh, pt, pb = o.same_padding(h, k, s)
        ow, pl, pr = o.same_padding(w, k, s)
        out.update({name + "_x": x, name + "_f": qf, name + "_bias": bias, name + "_min_f": mnf,
                    name + "_max_f": mxf, name + "_stride": np.int32(s)})
        if pt != pb or pl != pr:
            # torch's binding takes symmetric padding only; pad the input ourselves.
            xp = np.zeros((n, h + pt + pb, w + pl + pr, c), np.uint8)
            xp[:, pt:pt + h, pl:pl + w] = x
            xin, pad = xp, (0, 0)
        else:
            xin, pad = x, (pt, pl)
        for tout, tdt in (("quint8", torch.uint8), ("float", torch.float32)):
            sc = o.conv_output_scale(mni, mxi, mnf, mxf, "quint8", tout, mno, mxo)
            bp = o.conv_scaled_bias(bias, mni, mxi, mnf, mxf, "quint8", tout, sc)
            y = onednn_conv(xin, qf, sc, bp, (s, s), pad, True, tdt)
            out["%s_y_%s" % (name, tout)] = y
    out.update(min_input=np.float32(0.0), max_input=np.float32(12.75), min_out=np.float32(0.0),
               max_out=np.float32(20.0))
    np.savez_compressed(os.path.join(HERE, "onednn_conv.npz"), **out)


def write_onednn_conv_sum():
    """The sum post-op (the residual additions of a quantized ResNet: _ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize,
    quantized_conv_ops.h:398-434) through real oneDNN.  Whether  f + sum_scale * summand  is one rounding or two only
    shows on rounding ties, a few elements in ten million: a large seeded 1x1 convolution is run once, the pixels where
    the two models disagree are found, and the fixture keeps exactly those pixels (plus as many ordinary ones) as a
    [1,1,P,64] input, re-run through oneDNN on its own."""
    import torch
    rng = np.random.default_rng(20240503)
    n, h, w, c, co = 16, 56, 56, 64, 256
    x = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
    f32f = (rng.standard_normal((1, 1, c, co)) * 0.05).astype(np.float32)
    amax = np.abs(f32f).reshape(-1, co).max(axis=0).astype(np.float32)
    qf = np.clip(np.rint(f32f * (127.0 / amax)), -127, 127).astype(np.int8)
    bias = (rng.standard_normal(co) * 0.1).astype(np.float32)
    summand = rng.integers(0, 256, (n, h, w, co)).astype(np.uint8)
    rng_in, rng_out, rng_sum = (np.float32(0.0), np.float32(12.75)), (np.float32(0.0), np.float32(37.3)), (np.float32(0.0), np.float32(5.123))
    sc = o.conv_output_scale(rng_in[0], rng_in[1], -amax, amax, "quint8", "quint8", rng_out[0], rng_out[1])
    bp = o.conv_scaled_bias(bias, rng_in[0], rng_in[1], -amax, amax, "quint8", "quint8", sc)
    sum_scale = np.float32(rng_sum[1] / rng_out[1])
    qw = torch.from_numpy(np.ascontiguousarray(qf.transpose(3, 2, 0, 1)))
    ws, wz = torch.from_numpy(sc.copy()), torch.zeros(co, dtype=torch.int64)
    pw = torch.ops.onednn.qconv_prepack(qw, ws, 1.0, 0, [1, 1], [0, 0], [1, 1], 1, None)

    def nchw(a):
        return torch.from_numpy(np.ascontiguousarray(a.transpose(0, 3, 1, 2))).contiguous(memory_format=torch.channels_last)

    def run_sum(xa, sa):
        y = torch.ops.onednn.qconv2d_pointwise.binary(nchw(xa), 1.0, 0, pw, ws, wz, nchw(sa), torch.from_numpy(bp), [1, 1], [0, 0], [1, 1], 1,
                                                      1.0, 0, torch.uint8, float(sum_scale), 0, "sum", 1.0, "relu", [], "")
        return np.ascontiguousarray(y.permute(0, 2, 3, 1).numpy())

    yf = torch.ops.onednn.qconv2d_pointwise(nchw(x), 1.0, 0, pw, ws, wz, torch.from_numpy(bp), [1, 1], [0, 0], [1, 1], 1, 1.0, 0,
                                            torch.float32, "none", [], "").permute(0, 2, 3, 1).numpy()
    two = np.clip(np.rint(np.maximum(yf + (sum_scale * summand.astype(np.float32)).astype(np.float32), 0)), 0, 255)
    one = np.clip(np.rint(np.maximum((np.float64(sum_scale) * summand.astype(np.float64) + yf.astype(np.float64)).astype(np.float32), 0)), 0, 255)
    tie_pix = np.argwhere((two != one).any(axis=3))
    assert len(tie_pix) >= 3, "no distinguishing element in the sample"
    pick = [tuple(p) for p in tie_pix[:32]]
    pick += [(int(a), int(b), int(d)) for a, b, d in zip(rng.integers(0, n, 32), rng.integers(0, h, 32), rng.integers(0, w, 32))]
    xs = np.stack([x[p] for p in pick])[None, None]                 # [1,1,P,64]
    ss = np.stack([summand[p] for p in pick])[None, None]           # [1,1,P,256]
    y = run_sum(xs, ss)
    full = run_sum(x, summand)
    assert all(np.array_equal(y[0, 0, i], full[p]) for i, p in enumerate(pick))
    np.savez_compressed(os.path.join(HERE, "onednn_conv_sum.npz"), x=xs, summand=ss, f=qf, bias=bias, min_f=-amax, max_f=amax,
                        min_input=rng_in[0], max_input=rng_in[1], min_out=rng_out[0], max_out=rng_out[1],
                        min_summand=rng_sum[0], max_summand=rng_sum[1], y=y, n_tie_pixels=np.int32(min(32, len(tie_pix))))


if __name__ == "__main__":
    write_reference_kat()
    write_onednn_matmul()
    write_onednn_conv()
    write_onednn_conv_sum()
    print("golden fixtures written to", HERE)
