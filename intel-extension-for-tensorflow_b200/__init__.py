"""itex_b200: B200 (sm_100a) implementation of the quantized-inference hot path of
intel/intel-extension-for-tensorflow - QuantizeV2 / Dequantize, the fused int8 matmul
family, the fused int8 Conv2D and the FP8 e4m3 matmul with delayed scaling.

The directory name contains hyphens, so it is imported by path under the module name
`itex_b200` (see tests/conftest.py: load_package()).  All compute goes through
lib/libitexb200.so; importing the kernel or op modules fails loudly if it is not built.
"""
from . import _lib  # noqa: F401
from ._lib import ItexError, load  # noqa: F401

__all__ = ["_lib", "ItexError", "load"]
