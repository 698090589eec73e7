"""The allocation-free convolution entry point gives the bytes the ordinary one gives.

itexb_conv2d_static_scratch serves hosts that cannot call cudaMalloc when the convolution is
due (a plugin inside another framework's memory arena, code inside a stream capture, an
allocation-free serving loop): its scratch is an array inside the library's device image.
The test calls it through the C-ABI twice in a row - the second call finds the first call's
leftovers in the shared array - and compares with itexb_conv2d run on caller scratch; it
also checks the size limit is enforced with a clear status.  The file name sorts last so
that a run stopping at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import dev, host, modules

pytestmark = pytest.mark.gpu


def _params(L, x, fpk, out, scale, bias, n, h, w, c, kh, kw, co, stride, pad, oh, ow, workspace=None):
    p = L.ConvParams()
    p.n, p.h, p.w, p.c, p.kh, p.kw, p.co = n, h, w, c, kh, kw, co
    p.stride_h = p.stride_w = stride
    p.dil_h = p.dil_w = 1
    p.pad_top = p.pad_left = pad
    p.oh, p.ow, p.c_pad = oh, ow, c
    p.x_dtype, p.out_dtype = L.DT_QUINT8, L.DT_QUINT8
    p.x, p.filter_packed, p.out = x.data_ptr(), fpk.data_ptr(), out.data_ptr()
    p.ep.scale, p.ep.scale_count, p.ep.bias, p.ep.relu = scale.data_ptr(), co, bias.data_ptr(), 1
    p.workspace = 0 if workspace is None else workspace.data_ptr()
    return p


def _run_case(itex, seed, n, h, w, c, kh, co, stride, first_call_on_device=False):
    lib, L = itex.load(), itex._lib
    lib.itexb_conv2d_workspace_bytes.restype = C.c_size_t
    rng = np.random.default_rng(seed)
    pad = kh // 2
    oh, ow = (h + stride - 1) // stride, (w + stride - 1) // stride
    x = dev(rng.integers(0, 256, (n, h, w, c), dtype=np.uint8))
    f = dev(rng.integers(-127, 128, (kh, kh, c, co)).astype(np.int8))
    scale = dev(rng.uniform(2e-4, 6e-4, co).astype(np.float32))
    bias = dev(rng.standard_normal(co).astype(np.float32))
    c_pad = c
    fpk = torch.empty((co, (kh * kh * c_pad + 15) // 16 * 16), dtype=torch.int8, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    L.check(lib.itexb_pack_filter_hwio(C.c_void_p(f.data_ptr()), C.c_void_p(fpk.data_ptr()), kh, kh, c, co, c_pad, stream))
    ref = torch.empty((n, oh, ow, co), dtype=torch.uint8, device="cuda")
    p = _params(L, x, fpk, ref, scale, bias, n, h, w, c, kh, kh, co, stride, pad, oh, ow)
    ws = torch.empty(max(1, lib.itexb_conv2d_workspace_bytes(C.byref(p))), dtype=torch.uint8, device="cuda")
    p.workspace = ws.data_ptr()
    L.check(lib.itexb_conv2d(C.byref(p), stream))
    out = torch.full((n, oh, ow, co), 77, dtype=torch.uint8, device="cuda")
    q = _params(L, x, fpk, out, scale, bias, n, h, w, c, kh, kh, co, stride, pad, oh, ow)  # workspace left NULL
    torch.cuda.synchronize()
    # "allocates nothing": neither this library's allocator nor the driver's free-memory figure may move across the call
    st0, st1 = L.AllocatorStats(), L.AllocatorStats()
    L.check(lib.itexb_rt_allocator_stats(0, C.byref(st0)))
    free0 = torch.cuda.mem_get_info()[0]
    L.check(lib.itexb_conv2d_static_scratch(C.byref(q), stream))
    torch.cuda.synchronize()
    free1 = torch.cuda.mem_get_info()[0]
    L.check(lib.itexb_rt_allocator_stats(0, C.byref(st1)))
    assert (st1.num_allocs, st1.bytes_in_use, st1.bytes_reserved) == (st0.num_allocs, st0.bytes_in_use, st0.bytes_reserved)
    if not first_call_on_device:
        assert free1 == free0, "device free memory changed across an allocation-free call"
    assert int(ref.max()) > 0
    np.testing.assert_array_equal(host(out), host(ref))  # integer output: identical bytes are the tolerance


def test_static_scratch_conv_matches_caller_scratch_conv_twice_in_a_row():
    itex, K, ops = modules()
    # channel counts that are not a multiple of 16 are the ones whose patch matrix is staged in scratch
    # (the very first launch of a kernel in a process may make the driver load its code: the free-memory figure is
    # compared from the second call on)
    _run_case(itex, 1, 2, 28, 28, 24, 3, 64, 1, first_call_on_device=True)   # 2*28*28 x 224 patch matrix = 0.35 MB
    _run_case(itex, 1, 2, 28, 28, 24, 3, 64, 1)
    _run_case(itex, 2, 4, 32, 32, 3, 7, 48, 2)    # an RGB stem: runs over the first call's leftovers


def test_static_scratch_rejects_bad_dimensions_as_an_argument_error():
    itex, K, ops = modules()
    lib, L = itex.load(), itex._lib
    x = torch.zeros(1, dtype=torch.uint8, device="cuda")
    p = _params(L, x, x, x, x, x, 1, 8, 8, 24, 3, 3, 64, 0, 1, 8, 8)     # stride 0
    st = lib.itexb_conv2d_static_scratch(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == L.INVALID_ARGUMENT


def test_static_scratch_limit_is_enforced():
    itex, K, ops = modules()
    lib, L = itex.load(), itex._lib
    x = torch.zeros(1, dtype=torch.uint8, device="cuda")
    p = _params(L, x, x, x, x, x, 32, 112, 112, 24, 3, 3, 64, 1, 1, 112, 112)  # needs 32*112*112*224 B = 89.9 MB of scratch
    st = lib.itexb_conv2d_static_scratch(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == L.RESOURCE_EXHAUSTED
    msg = lib.itexb_last_error().decode()
    assert "89915392" in msg and "16777216" in msg and "itexb_conv2d" in msg
