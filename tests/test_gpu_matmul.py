"""GPU parity of the fused int8 matmul family through the C-ABI op layer."""
import ctypes as C
import json
import os

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import Canary, dev, host, modules

pytestmark = pytest.mark.gpu


def _cfg1(m=64, k=1024, n=1024, seed=1235):
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    qa, mna, mxa = o.quantize_v2(x, x.min(), x.max(), T="quint8")
    qb, mnb, mxb = o.quantize_v2(w, w.min(), w.max(), T="qint8")
    return x, w, bias, qa, mna, mxa, qb, mnb, mxb


@pytest.mark.parametrize("sbm", ["literal", "intended"])
@pytest.mark.parametrize("tout", ["float", "bfloat16", "half"])
def test_config1_matmul_with_bias_and_dequantize(sbm, tout):
    """fp32 [64,1024] -> QuantizeV2 quint8 SCALED -> _ITEXQuantizedMatMulWithBiasAndDequantize -> [64,1024].
    1e-5 relative is the bar; the restated epilogue order makes it bit-exact."""
    itex, K, ops = modules()
    x, w, bias, qa_ref, mna, mxa, qb, mnb, mxb = _cfg1()
    qa, mn, mx = ops._ITEXQuantizeV2(dev(x), float(x.min()), float(x.max()), T="quint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    np.testing.assert_array_equal(host(qa), qa_ref)
    out = ops._ITEXQuantizedMatMulWithBiasAndDequantize(qa, dev(qb), dev(bias), mn, mx, float(mnb), float(mxb), 0.0, 0.0,
                                                         Toutput=tout, input_quant_mode="SCALED", scaled_bias_mode=sbm)
    ref, _, _ = o.quantized_matmul_with_bias(qa_ref, qb, bias, mna, mxa, mnb, mxb, 0.0, 0.0, toutput=tout,
                                             input_quant_mode="SCALED", scaled_bias_mode=sbm)
    got = host(out)
    np.testing.assert_allclose(got, ref.astype(np.float32), rtol=1e-5, atol=0)
    np.testing.assert_array_equal(got, ref.astype(np.float32))
    if sbm == "intended" and tout == "float":  # close to the fp32 math the quantization approximates
        f = np.maximum(x, 0) @ w + bias
        assert np.abs(got - f).max() < 0.05


def test_reference_sanity_cases_min_first(golden_dir):
    """test/sanity/quantization/quantized_matmul_op_test.py: the four ops on the 2x3 . 3x4 constants, MIN_FIRST
    input, against fp32 math at rtol=atol=0.2 - and bit-exact against the oracle."""
    itex, K, ops = modules()
    k = json.load(open(os.path.join(golden_dir, "reference_kat.json")))["matmul_min_first"]
    x = np.array(k["x_f32"], np.float32)
    y = np.array(k["y_f32"], np.float32)
    b = np.array(k["bias_f32"], np.float32)
    tol = dict(rtol=k["rtol"], atol=k["atol"])
    qx, xmin, xmax = ops._ITEXQuantizeV2(dev(x), float(x.min()), float(x.max()), T="quint8", mode="MIN_FIRST")
    qy, ymin, ymax = ops._ITEXQuantizeV2(dev(y), float(y.min()), float(y.max()), T="qint8", mode="SCALED",
                                         round_mode="HALF_TO_EVEN", narrow_range=True)
    f = x @ y + b
    fr = np.maximum(f, 0)
    out, mn, mx = ops._ITEXQuantizedMatMulWithBiasAndReluAndRequantize(qx, qy, dev(b), xmin, xmax, ymin, ymax,
                                                                       float(fr.min()), float(fr.max()), Toutput="quint8")
    deq = ops._ITEXDequantize(out, mn, mx, mode="SCALED", narrow_range=True)
    np.testing.assert_allclose(host(deq), fr, **tol)
    ref, _, _ = o.quantized_matmul_with_bias(host(qx), host(qy), b, xmin, xmax, ymin, ymax, fr.min(), fr.max(),
                                             toutput="quint8", relu=True)
    np.testing.assert_array_equal(host(out), ref)
    out = ops._ITEXQuantizedMatMulWithBiasAndDequantize(qx, qy, dev(b), xmin, xmax, ymin, ymax, float(f.min()), float(f.max()))
    np.testing.assert_allclose(host(out), f, **tol)
    for relu, fn in ((False, ops._ITEXQuantizedMatMulWithBias), (True, ops._ITEXQuantizedMatMulWithBiasAndRelu)):
        out, mn, mx = fn(qx, qy, dev(b), xmin, xmax, ymin, ymax)
        ref, rmn, rmx = o.quantized_matmul_with_bias(host(qx), host(qy), b, xmin, xmax, ymin, ymax, toutput="qint32", relu=relu)
        np.testing.assert_array_equal(host(out), ref)
        assert (mn, mx) == (rmn, rmx)
        np.testing.assert_allclose(host(out).astype(np.float64) * (float(mx) / (2 ** 31 - 1)), fr if relu else f, **tol)


def test_against_onednn_fixtures(golden_dir):
    """Outputs of real oneDNN (tests/golden/onednn_matmul.npz) for every output type, input mode, bias mode, ReLU."""
    itex, K, ops = modules()
    g = np.load(os.path.join(golden_dir, "onednn_matmul.npz"))
    a, b, bias = dev(g["a"]), dev(g["b"]), dev(g["bias"])
    rng = (float(g["min_a"]), float(g["max_a"]), float(g["min_b"]), float(g["max_b"]))
    fz = (float(g["min_freezed"]), float(g["max_freezed"]))
    for tout in ("float", "quint8", "bfloat16"):
        for mode in ("SCALED", "MIN_FIRST"):
            for sbm in ("literal", "intended"):
                for relu in (0, 1):
                    ref = g["y_%s_%s_%s_%d" % (tout, mode, sbm, relu)]
                    kw = dict(Toutput=tout, input_quant_mode=mode, scaled_bias_mode=sbm)
                    if tout == "quint8":
                        fn = ops._ITEXQuantizedMatMulWithBiasAndReluAndRequantize if relu else ops._ITEXQuantizedMatMulWithBiasAndRequantize
                        out, mn, mx = fn(a, b, bias, *rng, *fz, **kw)
                        np.testing.assert_array_equal(host(out), ref)
                        assert (mn, mx) == fz
                    elif not relu:
                        out = ops._ITEXQuantizedMatMulWithBiasAndDequantize(a, b, bias, *rng, *fz, **kw)
                        np.testing.assert_allclose(host(out), ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("m,k,n", [(1, 16, 1), (77, 144, 200), (300, 160, 72), (129, 1040, 257), (5, 37, 19), (256, 100, 64)])
def test_odd_shapes_transposes_bias_types(m, k, n):
    itex, K, ops = modules()
    rng = np.random.default_rng(m * 1000 + n)
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    b = rng.integers(-127, 128, (k, n)).astype(np.int8)
    bias = rng.standard_normal(n).astype(np.float32)
    bias32 = rng.integers(-50000, 50000, n).astype(np.int32)
    mna, mxa, mnb, mxb, mnf, mxf = -0.3, 2.1, -0.4, 0.4, -30.0, 55.0
    for mode in ("MIN_FIRST", "SCALED"):
        for ta, tb in ((False, False), (True, False), (False, True), (True, True)):
            aa = np.ascontiguousarray(a.T) if ta else a
            bb = np.ascontiguousarray(b.T) if tb else b
            for bvec, tbias in ((bias, "float"), (bias32, "qint32")):
                out, mn, mx = ops._ITEXQuantizedMatMulWithBiasAndRequantize(
                    dev(aa), dev(bb), dev(bvec), mna, mxa, mnb, mxb, mnf, mxf, Toutput="qint8", transpose_a=ta, transpose_b=tb,
                    input_quant_mode=mode)
                ref, _, _ = o.quantized_matmul_with_bias(aa, bb, bvec, mna, mxa, mnb, mxb, mnf, mxf, toutput="qint8", tbias=tbias,
                                                         transpose_a=ta, transpose_b=tb, input_quant_mode=mode)
                np.testing.assert_array_equal(host(out), ref)
            out = ops._ITEXQuantizedMatMulWithBiasAndDequantize(dev(aa), dev(bb), dev(bias), mna, mxa, mnb, mxb, mnf, mxf,
                                                                 transpose_a=ta, transpose_b=tb, input_quant_mode=mode)
            ref, _, _ = o.quantized_matmul_with_bias(aa, bb, bias, mna, mxa, mnb, mxb, mnf, mxf, toutput="float", transpose_a=ta,
                                                     transpose_b=tb, input_quant_mode=mode)
            np.testing.assert_array_equal(host(out), ref)


def test_per_channel_min_b_uses_channel_zero_and_emits_vector_ranges():
    """The ...WithBias* ops read element 0 of min_b/max_b for the output scale (quantized_matmul_common.h:409-421)
    and emit per-channel min_out/max_out for qint32 output (quantized_ops.h:178-195)."""
    itex, K, ops = modules()
    rng = np.random.default_rng(3)
    m, k, n = 40, 64, 48
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    b = rng.integers(-127, 128, (k, n)).astype(np.int8)
    bias = rng.standard_normal(n).astype(np.float32)
    mnb = -np.linspace(0.1, 0.9, n).astype(np.float32)
    mxb = -mnb
    out, mn, mx = ops._ITEXQuantizedMatMulWithBias(dev(a), dev(b), dev(bias), 0.0, 3.0, mnb, mxb, input_quant_mode="SCALED")
    ref, rmn, rmx = o.quantized_matmul_with_bias(a, b, bias, 0.0, 3.0, mnb, mxb, toutput="qint32", input_quant_mode="SCALED")
    np.testing.assert_array_equal(host(out), ref)
    np.testing.assert_array_equal(mn, rmn)
    np.testing.assert_array_equal(mx, rmx)
    out = ops._ITEXQuantizedMatMulWithBiasAndDequantize(dev(a), dev(b), dev(bias), 0.0, 3.0, mnb, mxb, 0.0, 0.0, input_quant_mode="MIN_FIRST")
    ref, _, _ = o.quantized_matmul_with_bias(a, b, bias, 0.0, 3.0, mnb, mxb, 0.0, 0.0, toutput="float", input_quant_mode="MIN_FIRST")
    np.testing.assert_array_equal(host(out), ref)


def test_object_cache_second_run_and_changed_range():
    """Run twice 'to check object cache' (native_quantized_fused_matmul_test.py:83-90), then change min_a/max_a:
    the cached scaled bias must be rebuilt (IsCachedBiasValid, quantized_matmul_common.h:458-464)."""
    itex, K, ops = modules()
    x, w, bias, qa, mna, mxa, qb, mnb, mxb = _cfg1(m=96, k=256, n=320, seed=8)
    op = ops.Op("_ITEXQuantizedMatMulWithBiasAndDequantize", T1="quint8", T2="qint8", Tbias="float", Toutput="float",
                input_quant_mode="MIN_FIRST")
    A, B, Bi = dev(qa), dev(qb), dev(bias)
    for (lo, hi) in ((mna, mxa), (mna, mxa), (-0.5, 2.0), (mna, mxa)):
        out = op(A, B, Bi, float(lo), float(hi), float(mnb), float(mxb), 0.0, 0.0)
        ref, _, _ = o.quantized_matmul_with_bias(qa, qb, bias, lo, hi, mnb, mxb, 0.0, 0.0, toutput="float")
        np.testing.assert_array_equal(host(out), ref)
    with pytest.raises(itex.ItexError) as e:
        op(A, dev(qb[:100]), Bi, 0.0, 1.0, -1.0, 1.0, 0.0, 0.0)
    assert "Matrix size-incompatible" in str(e.value)


def test_non_const_bias_rewritten_in_place_is_not_served_from_the_cache():
    """is_bias_const=false: the bias tensor may change between calls while its address stays (an allocator reuses it);
    the scaled bias is then rebuilt every call, as the reference only caches when bias AND weight are constant
    (quantized_matmul_common.h:459,637,1146).  Per-channel weight ranges: a change in a range other than element 0
    rebuilds the cached scaled bias of a constant-bias instance too."""
    itex, K, ops = modules()
    x, w, bias, qa, mna, mxa, qb, mnb, mxb = _cfg1(m=64, k=128, n=192, seed=9)
    A, B, Bi = dev(qa), dev(qb), dev(bias)
    op = ops.Op("_ITEXQuantizedMatMulWithBiasAndDequantize", T1="quint8", T2="qint8", Tbias="float", Toutput="float",
                input_quant_mode="MIN_FIRST", is_bias_const=False)
    for step in range(3):
        b_now = (bias * (1.0 + step)).astype(np.float32)
        Bi.copy_(torch.from_numpy(b_now))                      # same address, new values
        out = op(A, B, Bi, float(mna), float(mxa), float(mnb), float(mxb), 0.0, 0.0)
        ref, _, _ = o.quantized_matmul_with_bias(qa, qb, b_now, mna, mxa, mnb, mxb, 0.0, 0.0, toutput="float")
        np.testing.assert_array_equal(host(out), ref)
    # fused flavour, per-channel ranges: only the LAST channel's range changes between the two calls
    n = qb.shape[1]
    rw = np.abs(w).max(axis=0).astype(np.float32)
    qbc = np.clip(np.rint(w * (127.0 / rw)), -127, 127).astype(np.int8)
    qs, smn, smx = o.quantize_v2(x, x.min(), x.max(), T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    fop = ops.Op("_ITEXQuantizedFusedMatMulAndDequantize", T1="qint8", T2="qint8", Targs="float", Toutput="float", fused_ops=["BiasAdd"],
                 input_quant_mode="SCALED", is_filter_const=True, is_bias_const=True, _scaled_bias_mode="literal")
    Bc, Bi2 = dev(qbc), dev(bias)
    for scale_last in (1.0, 3.0):
        r = rw.copy()
        r[-1] *= scale_last
        out = fop(dev(qs), Bc, Bi2, float(smn), float(smx), -r, r)
        ref, _, _ = o.quantized_fused_matmul(qs, qbc, bias, smn, smx, -r, r, fused_ops=["BiasAdd"], t1="qint8", toutput="float",
                                             scaled_bias_mode="literal")
        np.testing.assert_array_equal(host(out), ref)


def test_raw_accumulators_exact_large_and_canaries():
    """int32 accumulators bit-exact (u8 x s8 and s8 x s8) at a BERT-sized shape, exact check by f64 matmul on the GPU;
    no write outside the output."""
    itex, K, ops = modules()
    L = itex._lib
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for signed in (False, True):
        m, n, k = 1536, 1024, 4096
        a = torch.randint(-128 if signed else 0, 128 if signed else 256, (m, k), device="cuda").to(torch.int8 if signed else torch.uint8)
        b = torch.randint(-127, 128, (n, k), device="cuda").to(torch.int8)
        c = Canary(m * n * 4)
        out = K.gemm(a, b, L.DT_QINT32, ep=K.make_epilogue(raw_acc=True), out=c.view(torch.int32, (m, n)), status_word=status)
        ref = (a.double() @ b.double().t()).to(torch.int64)
        assert bool((out.to(torch.int64) == ref).all())
        c.check()
        assert int(status.item()) == 0
    # linearity property at the full 8192^3 size: gemm(a, b1 + b2) == gemm(a, b1) + gemm(a, b2)
    m = n = k = 8192
    a = torch.randint(0, 256, (m, k), device="cuda").to(torch.uint8)
    b1 = torch.randint(-60, 61, (n, k), device="cuda").to(torch.int8)
    b2 = torch.randint(-60, 61, (n, k), device="cuda").to(torch.int8)
    ep = K.make_epilogue(raw_acc=True)
    s = K.gemm(a, b1 + b2, L.DT_QINT32, ep=ep, status_word=status)
    s -= K.gemm(a, b1, L.DT_QINT32, ep=ep, status_word=status)
    s -= K.gemm(a, b2, L.DT_QINT32, ep=ep, status_word=status)
    assert int(s.abs().max()) == 0 and int(status.item()) == 0
    # and one 128-row slice of it against exact arithmetic
    ref = (a[4096:4224].double() @ b1.double().t()).to(torch.int64)
    got = K.gemm(a[4096:4224], b1, L.DT_QINT32, ep=ep).to(torch.int64)
    assert bool((got == ref).all())


@pytest.mark.parametrize("n,k,summand", [(256, 64, False), (256, 64, True), (64, 256, False)], ids=["n256-plain", "n256-sum", "n64-plain"])
def test_epilogue_bound_shape(n, k, summand):
    """ResNet-sized 1x1 convolutions as GEMMs (200704 pixels; 256 channels from K = 64: one 64-byte k-block per tile, so
    the epilogue is all there is; 64 channels from K = 256: 64-column tiles, one slice per epilogue warp and tile) with
    per-channel scale, bias, ReLU[, a u8 summand] and u8 output, three launches.
    Checked in full against the same arithmetic in separate fp32 steps on the raw accumulators (themselves exact by
    the test above): multiply, add[, ONE fused multiply-add of the summand - oneDNN's sum post-op, formed here in float64
    where byte x float is exact - ], clamp, round half to even."""
    itex, K, ops = modules()
    L = itex._lib
    m = 200704
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randint(0, 256, (m, k), device="cuda", generator=g).to(torch.uint8)
    b = torch.randint(-127, 128, (n, k), device="cuda", generator=g).to(torch.int8)
    scale = (torch.rand(n, device="cuda", generator=g) * 2e-3 + 1e-4).float()
    bias = (torch.randn(n, device="cuda", generator=g) * 20).float()
    sm = torch.randint(0, 256, (m, n), device="cuda", generator=g).to(torch.uint8) if summand else None
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    raw = K.gemm(a, b, L.DT_QINT32, ep=K.make_epilogue(raw_acc=True), status_word=status)
    want = raw.float() * scale
    want = want + bias
    if summand:
        want = (want.double() + sm.double() * float(np.float32(0.37))).float()
    want = torch.round(torch.clamp(want, 0.0, 255.0)).to(torch.uint8)
    ep = K.make_epilogue(scale=scale, bias=bias, relu=True, summand=sm, sum_scale=0.37)
    for _ in range(3):
        out = K.gemm(a, b, L.DT_QUINT8, ep=ep, status_word=status)
        assert torch.equal(out, want)
    assert int(status.item()) == 0


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (512, 768, 1024), (1024, 300, 400), (2304, 1024, 4096 + 48), (256 * 5, 512, 64)])
def test_cta_pair_kernel_equals_single_cta_kernel(m, n, k):
    """The kernel that runs a pair of CTAs per 256-row tile (each loading half of the B tile) against the one-CTA kernel
    and against exact arithmetic: raw accumulators (u8 x s8), the plain u8 epilogue with preset accumulators, the general
    bf16 epilogue, a narrow last k-block (k % 128 = 48) and a ragged last tile column (n = 300).  The pair is forced with
    the debug key; without it only launches with at least two waves of pair tiles take it."""
    itex, K, ops = modules()
    L = itex._lib
    lib = L.load()
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randint(0, 256, (m, k), device="cuda", generator=g).to(torch.uint8)
    b = torch.randint(-127, 128, (n, k), device="cuda", generator=g).to(torch.int8)
    scale = (torch.rand(n, device="cuda", generator=g) * 2e-4 + 1e-5).float()
    bias = (torch.randn(n, device="cuda", generator=g) * 20).float()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    eps = [(L.DT_QINT32, dict(raw_acc=True)), (L.DT_QUINT8, dict(scale=scale, bias=bias, relu=True)),
           (L.DT_BFLOAT16, dict(scale=scale, bias=bias, activation=L.ACT_GELU_TANH))]
    results = {}
    try:
        for pair in (0, 1):
            assert lib.itexb_debug_set(b"gemm_cta_pair", C.c_int64(pair)) == 0
            results[pair] = [K.gemm(a, b, dt, ep=K.make_epilogue(**kw), status_word=status) for dt, kw in eps for _ in range(2)]
    finally:
        assert lib.itexb_debug_set(b"gemm_cta_pair", C.c_int64(-1)) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for x, y in zip(results[0], results[1]):
        assert torch.equal(x, y)
    ref = (a.double() @ b.double().t()).to(torch.int64)
    assert bool((results[1][0].to(torch.int64) == ref).all())


@pytest.mark.parametrize("n,k,summand", [(64, 64, False), (64, 160, True), (128, 128, False)])
def test_stacked_subtiles_with_a_partial_last_group(n, k, summand):
    """Narrow tiles with one or two k-blocks run with several consecutive tile rows stacked in one accumulator stage, each
    handed over through its own barriers.  590 tile rows (the last one ragged) are 147 full groups of four and one group
    with two tile rows that do not exist: their hand-overs still have to take place and nothing may be stored for them.
    Checked in full against separate fp32 steps on the raw accumulators; a canary guards the end of the output."""
    itex, K, ops = modules()
    L = itex._lib
    m = 590 * 128 - 57
    g = torch.Generator(device="cuda").manual_seed(11 + n + k)
    a = torch.randint(0, 256, (m, k), device="cuda", generator=g).to(torch.uint8)
    b = torch.randint(-127, 128, (n, k), device="cuda", generator=g).to(torch.int8)
    scale = (torch.rand(n, device="cuda", generator=g) * 2e-3 + 1e-4).float()
    bias = (torch.randn(n, device="cuda", generator=g) * 20).float()
    sm = torch.randint(0, 256, (m, n), device="cuda", generator=g).to(torch.uint8) if summand else None
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    raw = K.gemm(a, b, L.DT_QINT32, ep=K.make_epilogue(raw_acc=True), status_word=status)
    assert bool((raw.to(torch.int64) == (a.double() @ b.double().t()).to(torch.int64)).all())
    want = raw.float() * scale
    want = want + bias
    if summand:
        want = (want.double() + sm.double() * float(np.float32(0.37))).float()
    want = torch.round(torch.clamp(want, 0.0, 255.0)).to(torch.uint8)
    ep = K.make_epilogue(scale=scale, bias=bias, relu=True, summand=sm, sum_scale=0.37)
    c = Canary(m * n)
    for _ in range(2):
        out = K.gemm(a, b, L.DT_QUINT8, ep=ep, out=c.view(torch.uint8, (m, n)), status_word=status)
        assert torch.equal(out, want)
    c.check()
    assert int(status.item()) == 0


def test_kernel_level_argument_errors():
    itex, K, ops = modules()
    L = itex._lib
    a = torch.zeros((8, 24), dtype=torch.uint8, device="cuda")
    b = torch.zeros((8, 24), dtype=torch.int8, device="cuda")
    with pytest.raises(itex.ItexError) as e:  # K pitch not a multiple of 16: the op layer pads, the raw call refuses
        K.gemm(a, b, L.DT_QINT32)
    assert "multiples of 16" in str(e.value)
    a = torch.zeros((8, 32), dtype=torch.uint8, device="cuda")
    b = torch.zeros((8, 32), dtype=torch.int8, device="cuda")
    sc = torch.ones(3, device="cuda")
    with pytest.raises(itex.ItexError) as e:
        K.gemm(a, b, L.DT_FLOAT, ep=K.make_epilogue(scale=sc))
    assert "scale_count" in str(e.value)
    with pytest.raises(itex.ItexError):
        K.gemm(a, b, L.DT_FLOAT, ep=K.make_epilogue(raw_acc=True))


@pytest.mark.parametrize("shape", [(5, 100, 72, 64), (16, 384, 384, 64), (3, 130, 300, 272)])
def test_batched_gemm(shape):
    """Batched products through the third tensor-map coordinate: every batch is an exact int32 product, rows past m and
    columns past n of one batch never reach the next one (ragged m, n, k included)."""
    itex, K, ops = modules()
    L = itex._lib
    bsz, m, n, k = shape
    rng = np.random.default_rng(sum(shape))
    kp = (k + 15) // 16 * 16
    a = np.zeros((bsz, m, kp), np.int8)
    b = np.zeros((bsz, n, kp), np.int8)
    a[:, :, :k] = rng.integers(-127, 128, (bsz, m, k))
    b[:, :, :k] = rng.integers(-127, 128, (bsz, n, k))
    want = np.einsum("bmk,bnk->bmn", a.astype(np.int64), b.astype(np.int64)).astype(np.int32)
    guard = Canary(bsz * m * n * 4)
    out = guard.view(torch.int32, (bsz, m, n))
    K.gemm(dev(a), dev(b), L.DT_QINT32, ep=K.make_epilogue(raw_acc=True), out=out, k=k)
    np.testing.assert_array_equal(host(out), want)
    guard.check()
    scale = rng.uniform(1e-4, 3e-4, n).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    got = K.gemm(dev(a), dev(b), L.DT_FLOAT, ep=K.make_epilogue(scale=dev(scale), bias=dev(bias)), k=k)
    ref = (want.astype(np.float32) * scale).astype(np.float32) + bias
    np.testing.assert_array_equal(host(got), ref)
