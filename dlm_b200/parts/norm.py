"""Normalisation parts."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import Norm, ParamSpec, Runtime


class RMSNorm(Norm):
    """``out = (x / sqrt(mean(x^2) + eps)) * weight`` with 32-bit statistics
    (src/forward/cpu.rs:934-942); the result is stored in the activation dtype."""

    def __init__(self, size: int, eps: float, param: str = "weight", scale: float = 1.0):
        """``param``: the weight tensor's name relative to the part's prefix ("" when the prefix is the
        whole name).  ``scale``: a factor on the output (it joins the 32-bit weight at load): a model whose logits
        are its head's product times a constant gives that constant to its final norm."""
        self.size, self.eps, self.param, self.scale = int(size), float(eps), str(param), float(scale)
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return [ParamSpec(self.param, (self.size,), init="norm")]

    def load(self, tensors, rt: Runtime):
        self.weight = rt.vector(tensors[self.param])
        if self.scale != 1.0:
            self.weight = (self.weight * self.scale).contiguous()

    def forward(self, x, rt: Runtime, rows=None, out_dtype=None):
        return rt.ops.rmsnorm(x, self.weight, self.eps, out_dtype or rt.dtype, rows)

    def fusable_rms(self):
        return self.weight, self.eps


class DynamicTanh(Norm):
    """A norm that takes no statistics: ``out = tanh(alpha * x) * weight + bias`` entry by entry, with one learned
    scalar ``alpha``; all of it 32-bit, the result stored in the activation dtype.  Tensors: the weight (``param``),
    ``<param>.b`` and ``<param>.alpha`` (a tensor without dimensions)."""

    def __init__(self, size: int, param: str = "weight"):
        self.size, self.param = int(size), str(param)
        self.weight = self.bias = None
        self.alpha = 1.0

    def param_specs(self):
        return [ParamSpec(self.param, (self.size,), init="norm"), ParamSpec(self.param + ".b", (self.size,), init="bias"),
                ParamSpec(self.param + ".alpha", (), init="norm")]

    def load(self, tensors, rt: Runtime):
        self.weight, self.bias = rt.vector(tensors[self.param]), rt.vector(tensors[self.param + ".b"])
        self.alpha = float(tensors[self.param + ".alpha"].to(torch.float32).reshape(()))

    def forward(self, x, rt: Runtime, rows=None, out_dtype=None):
        return rt.ops.dyt_norm(x, self.weight, self.bias, self.alpha, out_dtype or rt.dtype, rows)

    def pair_with(self, other):
        if not isinstance(other, DynamicTanh) or other.size != self.size:
            return None

        def both(x, rt: Runtime, want_f32: bool):
            return rt.ops.dyt_norm_pair(x, self.weight, self.bias, self.alpha, other.weight, other.bias, other.alpha,
                                        rt.dtype, want_f32=want_f32)
        return both


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
