"""Parts that make the input of a pass when a run of layers is repeated with the same weights."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import ParamSpec, Part, Runtime


class InputInjection(Part):
    """Before pass t of a repeated run: ``x <- W [x; x0] + step[t]`` with x the residual as the layers before left
    it, x0 the embedded tokens, ``W`` ``[hidden, 2 hidden]`` (x's half first) and ``step`` ``[passes, hidden]``.
    The product reads x and x0 in the activation dtype; the sum and the added vector are 32-bit."""

    def __init__(self, hidden_size: int, passes: int, weight: str = "in", step: str = "step"):
        self.hidden, self.passes = int(hidden_size), int(passes)
        self.n_w, self.n_step = str(weight), str(step)
        self.w = self.step = None

    def param_specs(self):
        return [ParamSpec(self.n_w, (self.hidden, 2 * self.hidden)),
                ParamSpec(self.n_step, (self.passes, self.hidden), init="bias")]

    def load(self, tensors, rt: Runtime):
        self.w = rt.matrix(tensors[self.n_w])
        self.step = rt.vector(tensors[self.n_step])

    def forward(self, x: torch.Tensor, x0: torch.Tensor, t: int, rt: Runtime) -> torch.Tensor:
        if not (0 <= t < self.passes):
            raise ValueError(f"pass {t} of {self.passes}")
        both = rt.ops.concat_rows(x, x0, rt.dtype)
        return rt.ops.linear(both, self.w, self.step[t], torch.float32)


class AdditiveEntry(Part):
    """Before pass t of a repeated run: ``x <- x + x0 + step[t]`` for t > 0 and ``x <- x + step[0]`` for the first pass,
    with x0 the embedded tokens and ``step`` ``[passes, hidden]``; all of it 32-bit, in place.  With
    ``add_embedded`` False the embedded tokens are never added: ``x <- x + step[t]`` in every pass."""

    def __init__(self, hidden_size: int, passes: int, step: str = "step", add_embedded: bool = True):
        self.hidden, self.passes, self.n_step = int(hidden_size), int(passes), str(step)
        self.needs_embedded = bool(add_embedded)      # False: the model need not keep the embedded tokens
        self.step = None

    def param_specs(self):
        return [ParamSpec(self.n_step, (self.passes, self.hidden), init="bias")]

    def load(self, tensors, rt: Runtime):
        self.step = rt.vector(tensors[self.n_step])

    def forward(self, x: torch.Tensor, x0: torch.Tensor, t: int, rt: Runtime) -> torch.Tensor:
        if not (0 <= t < self.passes):
            raise ValueError(f"pass {t} of {self.passes}")
        rt.ops.add_vec_rows(x, x0 if (t > 0 and self.needs_embedded) else None, self.step[t])
        return x


register_part("entry", "input_injection", InputInjection)
register_part("entry", "additive", AdditiveEntry)
