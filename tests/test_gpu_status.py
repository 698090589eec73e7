"""A bounded device wait that runs out is reported, the kernel returns, and the next launch works.

The failure is made on the host's request, without a fault or a hang: the test hook "gemm_skip_kblock" makes the TMA
producer leave out one k-block (neither its expect_tx arrival nor its copies are issued), so the barrier the MMA issuer
waits on is a flag that nothing sets, and "gemm_wait_limit_cycles" shortens the wait limit from ~2 s to ~1 ms.  The
kernel must notice, write the role code into the status word, release its tensor memory and return; the op layer must
turn the word into an error for the caller."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import dev, host, modules

pytestmark = pytest.mark.gpu

K_ERR_MMA = 2


def _hooks(lib, limit, skip):
    assert lib.itexb_debug_set(b"gemm_wait_limit_cycles", C.c_int64(limit)) == 0
    assert lib.itexb_debug_set(b"gemm_skip_kblock", C.c_int64(skip)) == 0


def test_expired_wait_sets_the_status_word_and_the_next_launch_is_exact():
    itex, K, ops = modules()
    lib, L = itex.load(), itex._lib
    m, n, k = 512, 512, 1024                    # 8 k-blocks per tile, 16 tiles
    rng = np.random.default_rng(77)
    a = dev(rng.integers(0, 256, (m, k), dtype=np.uint8))
    b = dev(rng.integers(-127, 128, (n, k)).astype(np.int8))
    ref = (a.double() @ b.double().t()).to(torch.int32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ep = K.make_epilogue(raw_acc=True)
    try:
        _hooks(lib, 2_000_000, 3)               # ~1 ms at 2 GHz; k-block 3 of every CTA's first tile never arrives
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        K.gemm(a, b, L.DT_QINT32, ep=ep, status_word=status)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        _hooks(lib, 0, -1)
    assert int(status.item()) == K_ERR_MMA       # the starved role reports, not a bystander
    assert elapsed < 0.5                         # milliseconds, not the 2 s default (generous for a cold first launch)
    # tensor memory was released and nothing is left hanging: the same launch now runs and is exact
    status.zero_()
    out = K.gemm(a, b, L.DT_QINT32, ep=ep, status_word=status)
    assert int(status.item()) == 0 and bool((out == ref).all())
    assert lib.itexb_debug_set(b"no_such_key", C.c_int64(1)) == L.NOT_FOUND


def test_the_op_layer_surfaces_an_expired_wait():
    itex, K, ops = modules()
    lib, L = itex.load(), itex._lib
    rng = np.random.default_rng(78)
    m, k, n = 256, 512, 384
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    qa, mna, mxa = o.quantize_v2(x, x.min(), x.max(), T="quint8")
    qb, mnb, mxb = o.quantize_v2(w, w.min(), w.max(), T="qint8")
    ref, _, _ = o.quantized_matmul_with_bias(qa, qb, bias, mna, mxa, mnb, mxb, 0.0, 0.0, toutput="float", input_quant_mode="SCALED")
    args = (dev(qa), dev(qb), dev(bias), float(mna), float(mxa), float(mnb), float(mxb), 0.0, 0.0)
    mk = lambda: ops.Op("_ITEXQuantizedMatMulWithBiasAndDequantize", T1="quint8", T2="qint8", Tbias="float", Toutput="float",
                        input_quant_mode="SCALED", is_weight_const=True)
    # (1) asynchronous: the failing Compute itself returns OK, itexb_op_check / the next Compute report it
    op = mk()
    np.testing.assert_array_equal(host(op(*args)), ref)      # healthy first call (packs the weight)
    op.check()
    try:
        _hooks(lib, 2_000_000, 1)
        op(*args)
    finally:
        _hooks(lib, 0, -1)
    with pytest.raises(itex.ItexError) as e:
        op.check(wait=True)
    assert e.value.code == L.ABORTED and "MMA issuer" in str(e.value) and "status 2" in str(e.value)
    op.check()                                               # reported once, then clear
    np.testing.assert_array_equal(host(op(*args)), ref)      # the instance keeps working, bit-exact
    op.check()
    # (2) the next Compute reports what the previous one left behind, and does not run
    op2 = mk()
    op2(*args)
    try:
        _hooks(lib, 2_000_000, 1)
        op2(*args)
    finally:
        _hooks(lib, 0, -1)
    torch.cuda.synchronize()
    with pytest.raises(itex.ItexError) as e:
        op2(*args)
    assert e.value.code == L.ABORTED
    np.testing.assert_array_equal(host(op2(*args)), ref)
    # (3) a convolution instance does the same
    xc = rng.integers(0, 256, (2, 14, 14, 64), dtype=np.uint8)
    f = (rng.standard_normal((3, 3, 64, 64)) * 0.05).astype(np.float32)
    amax = np.abs(f).reshape(-1, 64).max(axis=0).astype(np.float32)
    qf = np.clip(np.rint(f * (127.0 / amax)), -127, 127).astype(np.int8)
    cb = (rng.standard_normal(64) * 0.1).astype(np.float32)
    cop = ops.Op("_ITEXQuantizedConv2DWithBiasAndReluAndRequantize", Tinput="quint8", Tfilter="qint8", Tbias="float", out_type="quint8",
                 strides=[1, 1, 1, 1], padding="SAME", dilations=[1, 1, 1, 1], data_format="NHWC")
    cargs = (dev(xc), dev(qf), dev(cb), 0.0, 12.75, -amax, amax, 0.0, 9.0)
    yref, _, _ = o.quantized_conv2d(xc, qf, cb, 0.0, 12.75, -amax, amax, 0.0, 9.0, out_type="quint8", relu=True)
    np.testing.assert_array_equal(host(cop(*cargs)[0]), yref)
    try:
        _hooks(lib, 2_000_000, 2)
        cop(*cargs)
    finally:
        _hooks(lib, 0, -1)
    with pytest.raises(itex.ItexError):
        cop.check()
    np.testing.assert_array_equal(host(cop(*cargs)[0]), yref)
    cop.check()
