"""FP8 delayed-scaling surface: DelayedScaling recipe, per-layer meta tensors, the
once-per-step amax -> scale update and the Dense forward built on Fp8Quantize / Fp8Matmul.

Mirrors itex/python/fp8/recipe.py:30-93 (DelayedScaling), itex/python/fp8/autocast.py:44-121
(amax_and_scale_update) and the forward half of itex/python/transformer/base.py:48-93 and
layer.py:65-100,170-194 (meta layout: slot 0 = input, 1 = weight, 2 = output per GEMM).
State lives in three device tensors per direction, updated by one small kernel
(itexb_fp8_amax_and_scale_update) instead of a chain of TF ops.
"""
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Optional

import torch

from . import kernels as K
from . import ops

FP8_MAX_FWD = 448.0     # e4m3 (Format.HYBRID max_fwd, recipe.py:27)
FP8_MAX_BWD = 57344.0   # e5m2


@dataclass
class DelayedScaling:
    margin: int = 0
    fp8_format: str = "HYBRID"
    amax_history_len: int = 1024
    amax_compute_algo: str = "max"
    scaling_factor_compute_algo: Optional[object] = None

    def __post_init__(self):
        if self.fp8_format != "HYBRID":
            raise ValueError("only Format.HYBRID is supported")
        if callable(self.amax_compute_algo) or self.scaling_factor_compute_algo is not None \
                or self.amax_compute_algo not in ("max", "most_recent"):
            raise ValueError("We only support the fp8 recipe with 'max' or 'most_recent' amax_compute_algo and default "
                             "scaling_factor_compute_algo at this moment.")


# ---- fp8_autocast (itex/python/fp8/autocast.py:26-68,122-151): a process-wide "FP8 on" flag and recipe that layers
# consult when they are built and called; nesting restores the outer state on exit.
_FP8_ENABLED = False
_FP8_RECIPE = None


def get_default_fp8_recipe():
    """Margin 0, HYBRID format, 'max' over the default history (autocast.py:42-47)."""
    return DelayedScaling()


def get_fp8_dtype(fp8_recipe, fwd=True):
    """HYBRID: e4m3 forward, e5m2 backward (autocast.py:49-52)."""
    assert fp8_recipe.fp8_format == "HYBRID"
    return "E4M3" if fwd else "E5M2"


def is_fp8_enabled():
    return _FP8_ENABLED


def get_fp8_recipe():
    return _FP8_RECIPE


@contextmanager
def fp8_autocast(enabled: bool = False, fp8_recipe: Optional[DelayedScaling] = None):
    """with fp8_autocast(enabled=True, fp8_recipe=DelayedScaling(...)): y = layer(x)"""
    global _FP8_ENABLED, _FP8_RECIPE
    saved = (_FP8_ENABLED, _FP8_RECIPE)
    try:
        _FP8_ENABLED = enabled
        _FP8_RECIPE = get_default_fp8_recipe() if fp8_recipe is None else fp8_recipe
        yield
    finally:
        _FP8_ENABLED, _FP8_RECIPE = saved


class Fp8Meta:
    """amax_history [H, n], scale [n], scale_inv [n] on one device (n = 3 * num_gemms forward)."""

    def __init__(self, recipe: DelayedScaling, num_gemms: int = 1, device="cuda", fwd: bool = True):
        n = num_gemms * (3 if fwd else 2)
        self.recipe = recipe
        self.fp8_max = FP8_MAX_FWD if fwd else FP8_MAX_BWD
        self.scale = torch.ones(n, dtype=torch.float32, device=device)
        self.scale_inv = torch.ones(n, dtype=torch.float32, device=device)
        self.amax_history = torch.zeros((recipe.amax_history_len, n), dtype=torch.float32, device=device)

    def amax_and_scale_update(self):
        """Run before the forward of each step (base.py:197-200)."""
        K.fp8_amax_and_scale_update(self.amax_history, self.scale, self.scale_inv, self.fp8_max,
                                    float(self.recipe.margin), self.recipe.amax_compute_algo)

    def state_dict(self):
        return {"scale": self.scale.clone(), "scale_inv": self.scale_inv.clone(), "amax_history": self.amax_history.clone()}

    def load_state_dict(self, sd):
        self.scale.copy_(sd["scale"])
        self.scale_inv.copy_(sd["scale_inv"])
        self.amax_history.copy_(sd["amax_history"])


class Fp8Dense:
    """Forward of the FP8 Dense layer: y = x @ kernel (+ bias), e4m3 operands, `out_dtype` result.

    kernel is [in, out] like the Keras layer's weight; with `weight_layout="nk"` the caller
    keeps it as [out, in] and the op runs with transpose_b=True (no per-call transposition).
    """

    def __init__(self, kernel: torch.Tensor, bias: Optional[torch.Tensor] = None, recipe: Optional[DelayedScaling] = None,
                 out_dtype="bfloat16", weight_layout="kn"):
        self.kernel = kernel
        self.bias = bias
        self.recipe = recipe or (get_fp8_recipe() if is_fp8_enabled() else None) or DelayedScaling()  # explicit, autocast's, default
        self.meta = Fp8Meta(self.recipe, 1, kernel.device, fwd=True)
        self.out_dtype = out_dtype
        self.transpose_b = weight_layout == "nk"
        self._dummy = torch.zeros(1, dtype=torch.bfloat16 if out_dtype == "bfloat16" else torch.float32, device=kernel.device)

    def __call__(self, x: torch.Tensor, update_meta: bool = True) -> torch.Tensor:
        m = self.meta
        if update_meta:
            m.amax_and_scale_update()
        amax_row0 = m.amax_history[0]
        xq = ops.Fp8Quantize(x, amax_row0, m.scale, 0, "E4M3")
        wq = ops.Fp8Quantize(self.kernel, amax_row0, m.scale, 1, "E4M3")
        bias = self.bias if self.bias is not None else self._dummy
        return ops.Fp8Matmul(xq, wq, bias, self._dummy, m.scale_inv, m.scale_inv, amax_row0, m.scale, 0, 1, -1,
                             transpose_b=self.transpose_b, use_bias=self.bias is not None, sum_dtype=self.out_dtype,
                             out_dtype=self.out_dtype)
