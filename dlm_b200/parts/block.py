"""How a mixer, a feed-forward and their norms are arranged in one layer."""
from __future__ import annotations

from dataclasses import replace

from ..registry import build_part, register_part
import torch

from .base import ParamSpec, Part, PartSpec, RequestState, StepContext


class PreNormBlock(Part):
    """``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/forward/cpu.rs:1171-1212).  The
    residual ``x`` stays 32-bit; each sub-part adds into it."""

    # sub-part -> name prefix inside the layer
    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, ffn: PartSpec,
                 names: dict[str, str] | None = None):
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.norm2 = build_part("norm", norm2)
        self.ffn = build_part("ffn", ffn)
        self.names = {"norm1": "norm1.", "mixer": "mixer.", "norm2": "norm2.", "ffn": "ffn."}
        if names:
            self.names.update(names)

    def children(self):
        return [(self.names["norm1"], self.norm1), (self.names["mixer"], self.mixer),
                (self.names["norm2"], self.norm2), (self.names["ffn"], self.ffn)]

    def param_specs(self):
        out = []
        for prefix, part in self.children():
            for s in part.param_specs():
                out.append(replace(s, name=prefix + s.name))
        return out

    def load(self, tensors, rt):
        for prefix, part in self.children():
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, rt)

    def forward(self, resid, ctx: StepContext, call: int):
        rt = ctx.rt
        self.mixer.forward(self.norm1.forward(resid, rt), resid, ctx, call)
        self.ffn.forward(self.norm2.forward(resid, rt), resid, ctx, pre_norm=self.norm2)


class ParallelBlock(PreNormBlock):
    """``x += mixer(norm1(x)) + ffn(norm2(x))``: both sublayers read the same x, each through a norm of its own.
    ``ffn`` None: the layer has no feed-forward (and no second norm).  The feed-forward runs first: its router may
    read the residual itself (through ``norm2``), which must still be the layer's input then; the mixer's input was
    normed before anything was added."""

    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec | None = None, ffn: PartSpec | None = None,
                 names: dict[str, str] | None = None):
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.norm2 = build_part("norm", norm2) if ffn is not None else None
        self.names = {"norm1": "norm1.", "mixer": "mixer.", "norm2": "norm2.", "ffn": "ffn."}
        if names:
            self.names.update(names)

    def children(self):
        out = [(self.names["norm1"], self.norm1), (self.names["mixer"], self.mixer)]
        if self.ffn is not None:
            out += [(self.names["norm2"], self.norm2), (self.names["ffn"], self.ffn)]
        return out

    def load(self, tensors, rt):
        for prefix, part in self.children():
            mine = {prefix + s.name for s in part.param_specs()}
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k in mine}, rt)

    def forward(self, resid, ctx: StepContext, call: int):
        rt = ctx.rt
        if self.ffn is None:
            self.mixer.forward(self.norm1.forward(resid, rt), resid, ctx, call)
            return
        a, b = self.norm1.fusable_rms(), self.norm2.fusable_rms()
        both = self.norm1.pair_with(self.norm2)
        extra = {}
        if a is not None and b is not None and a[1] == b[1]:
            # two RMS norms of the same rows: one statistic, one pass
            h1, h2 = rt.ops.rmsnorm_pair(resid, a[0], b[0], a[1], rt.dtype)
        elif both is not None:
            # two norms that can share a pass over the rows; a feed-forward that wants its input in 32-bit as well
            # (a router) gets it from the same pass
            h1, h2, h32 = both(resid, rt, self.ffn.takes_normed32)
            if self.ffn.takes_normed32:
                extra["normed32"] = h32
        else:
            h1, h2 = self.norm1.forward(resid, rt), self.norm2.forward(resid, rt)
        self.ffn.forward(h2, resid, ctx, pre_norm=self.norm2, **extra)
        self.mixer.forward(h1, resid, ctx, call)


class SandwichBlock(ParallelBlock):
    """A norm before and after each sublayer: ``x += norm1b(mixer(norm1(x)))``, then ``x += norm2b(ffn(norm2(x)))``.
    ``ffn`` None: only the first sublayer.  When the norms are RMS norms the mixer's closing norm, the add and the
    feed-forward's opening norm are one pass over the rows (``norm_add_norm``); otherwise each norm runs by itself."""

    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm1b: PartSpec, norm2: PartSpec | None = None,
                 ffn: PartSpec | None = None, norm2b: PartSpec | None = None, names: dict[str, str] | None = None):
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.norm1b = build_part("norm", norm1b)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.norm2 = build_part("norm", norm2) if ffn is not None else None
        self.norm2b = build_part("norm", norm2b) if ffn is not None else None
        self.names = {"norm1": "norm1.", "mixer": "mixer.", "norm1b": "norm1b.", "norm2": "norm2.", "ffn": "ffn.",
                      "norm2b": "norm2b."}
        if names:
            self.names.update(names)

    def children(self):
        out = [(self.names["norm1"], self.norm1), (self.names["mixer"], self.mixer), (self.names["norm1b"], self.norm1b)]
        if self.ffn is not None:
            out += [(self.names["norm2"], self.norm2), (self.names["ffn"], self.ffn), (self.names["norm2b"], self.norm2b)]
        return out

    @staticmethod
    def _close(resid, y, post, nxt, rt):
        """``resid += post(y)``; returns ``nxt(resid)`` in the activation dtype when ``nxt`` is given."""
        a = post.fusable_rms()
        b = nxt.fusable_rms() if nxt is not None else None
        if a is not None and (nxt is None or (b is not None and b[1] == a[1])):
            return rt.ops.norm_add_norm(resid, y, a[0], b[0] if b is not None else None, a[1], rt.dtype)
        resid += post.forward(y, rt, out_dtype=torch.float32)
        return nxt.forward(resid, rt) if nxt is not None else None

    def forward(self, resid, ctx: StepContext, call: int):
        rt = ctx.rt
        y = torch.zeros_like(resid)
        self.mixer.forward(self.norm1.forward(resid, rt), y, ctx, call)
        h = self._close(resid, y, self.norm1b, self.norm2, rt)
        if self.ffn is None:
            return
        y.zero_()
        self.ffn.forward(h, y, ctx, pre_norm=None)
        self._close(resid, y, self.norm2b, None, rt)


class HyperConnectionBlock(Part):
    """A pre-norm layer over S residual streams ``xs[:, s]`` instead of one.  For sublayer q (1: the mixer,
    2: the feed-forward) with learned ``in_q[S]``, ``mix_q[S, S]`` (indexed [from, to]) and ``out_q[S]``::

        u  = sum_s in_q[s] xs[:, s]
        y  = sublayer(norm_q(u))
        xs[:, r] <- sum_s mix_q[s, r] xs[:, s] + out_q[r] y        (all streams from the old ones)

    With ``input_taps`` the mixer reads ``h + conv(h)`` instead of ``h = norm_1(u)``: a causal convolution
    over time on every channel (weights ``[hidden, taps]``, no bias, the last tap meets the current token);
    the last ``taps - 1`` values of h are part of a request's state.  ``ffn`` None: the layer has no second
    sublayer.  The streams, the sums and the norms are 32-bit."""

    def __init__(self, hidden_size: int, streams: int, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec | None = None,
                 ffn: PartSpec | None = None, input_taps: int | None = None, names: dict[str, str] | None = None):
        self.hidden, self.S = int(hidden_size), int(streams)
        self.taps = int(input_taps) if input_taps else 0
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.norm2 = build_part("norm", norm2) if ffn is not None else None
        self.names = {"norm1": "norm1.", "mixer": "mixer.", "norm2": "norm2.", "ffn": "ffn.", "hc1": "hc1.",
                      "hc2": "hc2.", "input_conv": "input_conv"}
        if names:
            self.names.update(names)
        self.hc = {}            # q -> (in, mix, out)
        self.conv_w = None

    def children(self):
        out = [(self.names["norm1"], self.norm1), (self.names["mixer"], self.mixer)]
        if self.ffn is not None:
            out += [(self.names["norm2"], self.norm2), (self.names["ffn"], self.ffn)]
        return out

    def _own_specs(self):
        S = self.S
        out = []
        for q in ("hc1", "hc2") if self.ffn is not None else ("hc1",):
            pre = self.names[q]
            out += [ParamSpec(pre + "in", (S,), init="norm"), ParamSpec(pre + "out", (S,), init="norm"),
                    ParamSpec(pre + "mix", (S, S), init="eye")]
        if self.taps:
            out.append(ParamSpec(self.names["input_conv"], (self.hidden, self.taps)))
        return out

    def param_specs(self):
        out = self._own_specs()
        for prefix, part in self.children():
            for s in part.param_specs():
                out.append(replace(s, name=prefix + s.name))
        return out

    def load(self, tensors, rt):
        for prefix, part in self.children():
            mine = {prefix + s.name for s in part.param_specs()}
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k in mine}, rt)
        for q in ("hc1", "hc2") if self.ffn is not None else ("hc1",):
            pre = self.names[q]
            self.hc[q] = tuple(rt.vector(tensors[pre + n]) for n in ("in", "mix", "out"))
        if self.taps:
            self.conv_w = rt.vector(tensors[self.names["input_conv"]])

    def state_need(self):
        need = {}
        m = self.mixer.state_need()
        if isinstance(m, dict):
            need.update(m)
        elif m is not None:
            need[""] = m
        if self.taps > 1:
            need["input_conv"] = RequestState((self.taps - 1, self.hidden))
        return need or None

    def _read(self, xs, w_in, norm, rt, out_dtype):
        rms = norm.fusable_rms()
        if rms is not None:
            return rt.ops.streams_reduce(xs, w_in, rms[0], rms[1], out_dtype)
        return norm.forward(rt.ops.streams_reduce(xs, w_in, None, 0.0, torch.float32), rt, out_dtype=out_dtype)

    def forward(self, xs, ctx: StepContext, call: int):
        rt, ops = ctx.rt, ctx.rt.ops
        T = xs.shape[0]
        w_in, w_mix, w_out = self.hc["hc1"]
        if self.taps:
            h = self._read(xs, w_in, self.norm1, rt, torch.float32)
            state = ctx.state(call, "input_conv") if self.taps > 1 else torch.empty((0, 0, self.hidden), device=xs.device)
            h = ops.causal_conv(h, self.conv_w, None, state, ctx.batch, True, False, rt.dtype)
        else:
            h = self._read(xs, w_in, self.norm1, rt, rt.dtype)
        y = torch.zeros((T, self.hidden), dtype=torch.float32, device=xs.device)
        self.mixer.forward(h, y, ctx, call)
        if self.ffn is None:
            ops.streams_update(xs, w_mix, w_out, y)
        else:
            # the mixer's update of the streams and the feed-forward's read of them, in one pass where the norm
            # is an RMS norm
            rms = self.norm2.fusable_rms()
            w_in2 = self.hc["hc2"][0]
            if rms is not None:
                h = ops.streams_update_reduce(xs, w_mix, w_out, y, w_in2, rms[0], rms[1], rt.dtype)
            else:
                ops.streams_update(xs, w_mix, w_out, y)
                h = self._read(xs, w_in2, self.norm2, rt, rt.dtype)
            w_in, w_mix, w_out = self.hc["hc2"]
            y = torch.zeros((T, self.hidden), dtype=torch.float32, device=xs.device)
            self.ffn.forward(h, y, ctx, pre_norm=None)
            ops.streams_update(xs, w_mix, w_out, y)


register_part("block", "prenorm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "hyper_connections", HyperConnectionBlock)
