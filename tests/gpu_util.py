"""Helpers shared by the GPU parity tests."""
import importlib

import numpy as np
import torch


def modules():
    from conftest import load_package
    itex = load_package()
    ops = importlib.import_module("itex_b200.ops")
    return itex, importlib.import_module("itex_b200.kernels"), ops


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def host(t):
    if t.dtype == torch.bfloat16 or t.dtype == torch.float16:
        return t.float().cpu().numpy()
    return t.cpu().numpy()


def scale_per_slice(shape, axis, values):
    """The generator the reference's _testAxis uses (quantized_ops_test.py:145-154)."""
    out = np.take(values, np.remainder(np.arange(np.prod(shape)), len(values))).reshape(shape)
    if axis is not None:
        ss = [1] * len(shape)
        ss[axis] = shape[axis]
        out = out * np.arange(1, shape[axis] + 1).reshape(ss)
    return out


class Canary:
    """Device buffer with guard bytes on both sides of the payload; check() fails if a
    kernel wrote outside its output."""

    def __init__(self, nbytes, guard=256):
        self.guard = guard
        self.buf = torch.full((nbytes + 2 * guard,), 0xA5, dtype=torch.uint8, device="cuda")
        self.payload = self.buf[guard:guard + nbytes]

    def view(self, dtype, shape):
        return self.payload.view(dtype).view(shape)

    def check(self):
        g = self.guard
        assert bool((self.buf[:g] == 0xA5).all()) and bool((self.buf[-g:] == 0xA5).all()), "write outside the output buffer"
