"""The device runtime behind the StreamExecutor-style callbacks: allocator, streams, events, copies."""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import modules

pytestmark = pytest.mark.gpu


def test_allocator_caches_and_reports():
    itex, K, ops = modules()
    lib, L = itex.load(), itex._lib
    st0 = L.AllocatorStats()
    L.check(lib.itexb_rt_allocator_stats(0, C.byref(st0)))
    p1, p2 = C.c_void_p(), C.c_void_p()
    L.check(lib.itexb_rt_allocate(0, C.c_size_t(1000), C.byref(p1)))
    L.check(lib.itexb_rt_allocate(0, C.c_size_t(3 << 20), C.byref(p2)))
    assert p1.value % 256 == 0 and p2.value % 256 == 0
    st = L.AllocatorStats()
    L.check(lib.itexb_rt_allocator_stats(0, C.byref(st)))
    assert st.bytes_in_use - st0.bytes_in_use == 1024 + (4 << 20) and st.num_allocs == st0.num_allocs + 2
    L.check(lib.itexb_rt_deallocate(0, p1))
    q = C.c_void_p()
    L.check(lib.itexb_rt_allocate(0, C.c_size_t(600), C.byref(q)))   # same size class: served from the cache
    assert q.value == p1.value
    L.check(lib.itexb_rt_deallocate(0, q))
    L.check(lib.itexb_rt_deallocate(0, p2))
    assert lib.itexb_rt_deallocate(0, C.c_void_p(12345)) == L.INVALID_ARGUMENT
    L.check(lib.itexb_rt_trim(0))
    L.check(lib.itexb_rt_allocator_stats(0, C.byref(st)))
    assert st.bytes_in_use == st0.bytes_in_use
    free, total = C.c_int64(), C.c_int64()
    L.check(lib.itexb_rt_device_memory_usage(0, C.byref(free), C.byref(total)))
    assert 0 < free.value <= total.value


def test_streams_events_copies_callbacks():
    itex, K, ops = modules()
    lib, L = itex.load(), itex._lib
    s1, s2 = C.c_void_p(), C.c_void_p()
    L.check(lib.itexb_rt_create_stream(0, C.byref(s1)))
    L.check(lib.itexb_rt_create_stream(0, C.byref(s2)))
    n = 1 << 20
    hp, dp, dp2 = C.c_void_p(), C.c_void_p(), C.c_void_p()
    L.check(lib.itexb_rt_host_allocate(C.c_size_t(n), C.byref(hp)))
    L.check(lib.itexb_rt_allocate(0, C.c_size_t(n), C.byref(dp)))
    L.check(lib.itexb_rt_allocate(0, C.c_size_t(n), C.byref(dp2)))
    src = np.ctypeslib.as_array(C.cast(hp, C.POINTER(C.c_uint8)), shape=(n,))
    src[:] = np.arange(n, dtype=np.uint32).astype(np.uint8)
    e0, e1 = C.c_void_p(), C.c_void_p()
    L.check(lib.itexb_rt_create_event(C.byref(e0)))
    L.check(lib.itexb_rt_create_event(C.byref(e1)))
    L.check(lib.itexb_rt_record_event(s1, e0))
    L.check(lib.itexb_rt_memcpy_h2d(dp, hp, C.c_size_t(n), s1))
    L.check(lib.itexb_rt_memset32(dp2, C.c_uint32(0x01020304), C.c_size_t(n), s1))
    L.check(lib.itexb_rt_record_event(s1, e1))
    L.check(lib.itexb_rt_stream_dependency(s2, s1))          # s2 waits for what s1 has queued
    L.check(lib.itexb_rt_memcpy_d2d(dp2, dp, C.c_size_t(n // 2), s2))
    fired = []
    cb = C.CFUNCTYPE(None, C.c_void_p)(lambda arg: fired.append(arg))
    L.check(lib.itexb_rt_host_callback(s2, cb, C.c_void_p(7)))
    out = np.zeros(n, np.uint8)
    L.check(lib.itexb_rt_block_host_until_done(s2))
    L.check(lib.itexb_rt_sync_memcpy_d2h(out.ctypes.data_as(C.c_void_p), dp2, C.c_size_t(n)))
    assert fired == [7]
    np.testing.assert_array_equal(out[:n // 2], src[:n // 2])
    np.testing.assert_array_equal(out[n // 2:].view(np.uint32), np.full(n // 8, 0x01020304, np.uint32))
    done, ms = C.c_int(), C.c_float()
    L.check(lib.itexb_rt_block_host_for_event(e1))
    L.check(lib.itexb_rt_event_status(e1, C.byref(done)))
    L.check(lib.itexb_rt_event_elapsed_ms(e0, e1, C.byref(ms)))
    assert done.value == 1 and ms.value >= 0
    assert lib.itexb_rt_stream_status(s1) == L.OK
    L.check(lib.itexb_rt_mem_zero(dp, C.c_size_t(n), s1))
    L.check(lib.itexb_rt_synchronize_all_activity(0))
    for ev in (e0, e1):
        L.check(lib.itexb_rt_destroy_event(ev))
    for s in (s1, s2):
        L.check(lib.itexb_rt_destroy_stream(s))
    L.check(lib.itexb_rt_host_deallocate(hp))
    L.check(lib.itexb_rt_deallocate(0, dp))
    L.check(lib.itexb_rt_deallocate(0, dp2))


def test_simple_context_runs_an_op_without_python_allocation():
    """The library's own context (outputs/temps from the caching allocator) drives an op end to end."""
    itex, K, ops = modules()
    lib, L = itex.load(), itex._lib
    lib.itexb_simple_context_begin.restype = C.POINTER(L.OpContext)
    lib.itexb_simple_context_output.restype = C.POINTER(L.Tensor)
    lib.itexb_simple_context_begin.argtypes = [C.c_void_p, C.POINTER(L.Tensor), C.c_int]
    lib.itexb_simple_context_output.argtypes = [C.c_void_p, C.c_int]
    op = ops.Op("_ITEXQuantizeV2", T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    x = torch.linspace(-1, 1, 1000, device="cuda")
    sctx = C.c_void_p()
    L.check(lib.itexb_simple_context_create(0, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(sctx)))
    tens = (L.Tensor * 3)()
    tens[0].dtype, tens[0].rank, tens[0].data = L.DT_FLOAT, 1, x.data_ptr()
    tens[0].dims[0] = 1000
    mn, mx = np.array(-1.0, np.float32), np.array(1.0, np.float32)
    for t, a in ((tens[1], mn), (tens[2], mx)):
        t.dtype, t.rank, t.data, t.on_host = L.DT_FLOAT, 0, a.ctypes.data, 1
    ctx = lib.itexb_simple_context_begin(sctx, tens, 3)
    L.check(lib.itexb_op_compute(op._h, ctx))
    assert lib.itexb_simple_context_num_outputs(sctx) == 3
    o0 = lib.itexb_simple_context_output(sctx, 0).contents
    o2 = lib.itexb_simple_context_output(sctx, 2).contents
    assert o0.dtype == L.DT_QINT8 and o0.dims[0] == 1000 and not o0.on_host and o2.on_host
    got = np.zeros(1000, np.int8)
    torch.cuda.synchronize()
    L.check(lib.itexb_rt_sync_memcpy_d2h(got.ctypes.data_as(C.c_void_p), C.c_void_p(o0.data), C.c_size_t(1000)))
    np.testing.assert_array_equal(got, np.rint(np.clip(x.cpu().numpy() * np.float32(127.0), -128, 127)).astype(np.int8))
    assert C.cast(o2.data, C.POINTER(C.c_float))[0] == 1.0
    L.check(lib.itexb_simple_context_reset(sctx))
    lib.itexb_simple_context_destroy.restype = None
    lib.itexb_simple_context_destroy(sctx)


def test_verbose_prints_one_timing_line_per_op_call():
    """ITEXB_VERBOSE=1 (the reference's ITEX_VERBOSE): every op call runs to completion and prints
    "type,instance,nanoseconds" on stderr.  The switch is read once per process, hence the child process."""
    import os
    import re
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import importlib, torch\n"
        "from conftest import load_package\n"
        "load_package(); ops = importlib.import_module('itex_b200.ops')\n"
        "x = torch.rand(1000, device='cuda')\n"
        "for _ in range(2): ops._ITEXQuantizeV2(x, 0.0, 1.0, T='quint8')\n"
        "print('done')\n" % here)
    env = dict(os.environ, ITEXB_VERBOSE="1")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "done" in r.stdout, r.stderr[-2000:]
    lines = [l for l in r.stderr.splitlines() if l.startswith("_ITEXQuantizeV2,")]
    assert len(lines) == 2
    for l in lines:
        assert re.fullmatch(r"_ITEXQuantizeV2,0x[0-9a-f]+,\d+", l), l
