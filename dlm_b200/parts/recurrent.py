"""Mixers that carry a state of fixed size per request instead of keys and values."""
from __future__ import annotations

import math

import torch

from dataclasses import replace

from ..registry import build_part, register_part
from .base import Mixer, ParamSpec, PartSpec, RequestState, Runtime, StepContext
from .rope import rope_inv_freqs


class Mamba2Mixer(Mixer):
    """State-space mixer with a scalar decay per head.  ``inner = heads * vdim``; ``W_in h`` is laid out
    ``[z: inner | x: inner | B: groups * state | C: groups * state | dt: heads]``.  x, B and C together pass a
    causal convolution per channel (``conv_taps`` taps with bias, the last tap meets the current token) and silu.
    Per head n (group ``n // (heads / groups)``), with ``dt = softplus(dt + dt_bias)`` (no clamp)::

        S_t = exp(-exp(A_log_n) dt) S_(t-1) + dt B_t x_t^T          (S: state x vdim, 32-bit, zero at the start)
        y_t = S_t^T C_t + D_n x_t

    then ``y * silu(z)``, an RMS norm over ``norm_groups`` equal parts of the channels (the gate comes before the
    norm), times ``norm``, then ``W_o``.  A request's state: S of every head and the convolution's last
    ``conv_taps - 1`` inputs.  Everything between the two projections is 32-bit."""

    def __init__(self, hidden_size: int, heads: int, vdim: int, state: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float):
        self.hidden, self.H, self.P, self.N, self.G = int(hidden_size), int(heads), int(vdim), int(state), int(groups)
        self.taps, self.ng, self.eps = int(conv_taps), int(norm_groups), float(eps)
        self.inner = self.H * self.P
        self.C = self.inner + 2 * self.G * self.N          # channels that pass the convolution
        if self.H % self.G:
            raise ValueError("heads must be a multiple of groups")
        if self.inner % self.ng:
            raise ValueError("heads * vdim must be a multiple of norm_groups")
        if self.taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.A_log = self.D = self.norm_w = None

    def param_specs(self):
        return [ParamSpec("in", (2 * self.inner + 2 * self.G * self.N + self.H, self.hidden)),
                ParamSpec("conv", (self.C, self.taps)), ParamSpec("conv.b", (self.C,), init="bias"),
                ParamSpec("dt_bias", (self.H,), init="bias"), ParamSpec("A_log", (self.H,), init="bias"),
                ParamSpec("D", (self.H,), init="norm"), ParamSpec("norm", (self.inner,), init="norm"),
                ParamSpec("o", (self.hidden, self.inner))]

    def load(self, tensors, rt: Runtime):
        self.w_in, self.w_o = rt.matrix(tensors["in"]), rt.matrix(tensors["o"])
        self.conv_w, self.conv_b = rt.vector(tensors["conv"]), rt.vector(tensors["conv.b"])
        self.dt_bias, self.A_log, self.D = (rt.vector(tensors[n]) for n in ("dt_bias", "A_log", "D"))
        self.norm_w = rt.vector(tensors["norm"])

    def state_need(self):
        need = {"ssm": RequestState((self.H, self.N, self.P))}
        if self.taps > 1:
            need["conv"] = RequestState((self.taps - 1, self.C))
        return need

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        proj = ops.linear(h, self.w_in, None, torch.float32)
        z = proj[:, :self.inner]
        dt = proj[:, self.inner + self.C:]
        conv_state = ctx.state(call, "conv") if self.taps > 1 else torch.empty((0, 0, self.C), device=h.device)
        xbc = ops.causal_conv(proj[:, self.inner:self.inner + self.C], self.conv_w, self.conv_b, conv_state, b,
                              False, True, torch.float32)
        y = ops.ssm_scan(xbc, dt, self.dt_bias, self.A_log, self.D, ctx.state(call, "ssm"), b, self.H, self.P, self.N,
                         self.G)
        g = ops.gated_rmsnorm(y, z, self.norm_w, self.ng, self.eps, "silu_before", rt.dtype)
        ops.linear_add(g, self.w_o, resid)


class GeneralDeltaMixer(Mixer):
    """Delta-rule recurrence with a decay and a removal rate per head and key channel.  ``r, k, v = W h`` (heads x
    dim each); decay ``w = exp(-decay_coef * sigmoid(W_w2 tanh(W_w1 h) + w0))``; removal rate
    ``a = sigmoid(W_a h + a.b)``; unit key ``u = k / sqrt(sum k^2 + unit_eps)`` per head::

        S_t = diag(w) S_(t-1) - (a * u)(u^T S_(t-1)) + k v^T       (S: dim x dim, 32-bit, zero at the start)
        o_t = S_t^T r

    Each head's o is divided by its root mean square, the heads side by side are multiplied by ``norm`` and by
    ``sigmoid(W_g h)``, then ``W_o``.  The width of the decay's bottleneck is whatever ``w1`` has."""

    def __init__(self, hidden_size: int, heads: int, dim: int, eps: float, decay_coef: float = math.exp(-0.5),
                 unit_eps: float = 1e-6, decay_rank: int = 16):
        self.hidden, self.H, self.d, self.eps = int(hidden_size), int(heads), int(dim), float(eps)
        self.decay_coef, self.unit_eps, self.decay_rank = float(decay_coef), float(unit_eps), int(decay_rank)
        self.HD = self.H * self.d
        self.w_in = self.w2 = self.w0 = self.a_b = self.norm_w = self.w_o = None

    def param_specs(self):
        HD, hid = self.HD, self.hidden
        # -1: the size is the checkpoint's (random weights take `arg`)
        return [ParamSpec("r", (HD, hid)), ParamSpec("k", (HD, hid)), ParamSpec("v", (HD, hid)),
                ParamSpec("a", (HD, hid)), ParamSpec("a.b", (HD,), init="bias"), ParamSpec("g", (HD, hid)),
                ParamSpec("w1", (-1, hid), arg=self.decay_rank), ParamSpec("w2", (HD, -1), arg=self.decay_rank),
                ParamSpec("w0", (HD,), init="bias"), ParamSpec("norm", (HD,), init="norm"), ParamSpec("o", (hid, HD))]

    def load(self, tensors, rt: Runtime):
        if tensors["w1"].shape[0] != tensors["w2"].shape[1]:
            raise ValueError("w1 and w2 disagree about the width of the decay's bottleneck")
        self.w_in = torch.cat([rt.matrix(tensors[n]) for n in ("r", "k", "v", "a", "g", "w1")], dim=0).contiguous()
        self.w2, self.w_o = rt.matrix(tensors["w2"]), rt.matrix(tensors["o"])
        self.w0, self.a_b, self.norm_w = rt.vector(tensors["w0"]), rt.vector(tensors["a.b"]), rt.vector(tensors["norm"])

    def state_need(self):
        return {"delta": RequestState((self.H, self.d, self.d))}

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        HD = self.HD
        proj = ops.linear(h, self.w_in, None, torch.float32)        # [r | k | v | a | g | w1 h]
        bottleneck = ops.activation(proj[:, 5 * HD:], "tanh", rt.dtype)
        lw = ops.linear(bottleneck, self.w2, self.w0, torch.float32)
        o = ops.delta_scan(proj, (0, HD, 2 * HD, 3 * HD), lw, self.a_b, ctx.state(call, "delta"), b, self.H, self.d,
                           self.unit_eps, self.decay_coef)
        g = ops.gated_rmsnorm(o, proj[:, 4 * HD:5 * HD], self.norm_w, self.H, self.eps, "sigmoid_after", rt.dtype)
        ops.linear_add(g, self.w_o, resid)


class Mamba1Mixer(Mixer):
    """Selective state-space mixer with a decay per channel and state and a step size per channel.
    ``W_in h = [x: inner | z: inner]``; x passes a causal convolution per channel (``conv_taps`` taps with bias, the
    last tap meets the current token) and silu.  ``W_x x = [dt: dt_rank | B: state | C: state]``;
    ``dt = softplus(W_dt dt + dt.b)`` per channel; ``A = -exp(A_log)`` (inner x state).  Per channel c and state n::

        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n          (S 32-bit, zero at a request's start)
        y_c = sum_n S[c, n] C_n + D_c x_c

    then ``y * silu(z)`` and ``W_o``.  A request's state: S and the convolution's last ``conv_taps - 1`` inputs.
    Between the projections everything is 32-bit; the scan reads the 32-bit x, the projections its rounding."""

    def __init__(self, hidden_size: int, inner: int, state: int, dt_rank: int, conv_taps: int):
        self.hidden, self.inner, self.N, self.R = int(hidden_size), int(inner), int(state), int(dt_rank)
        self.taps = int(conv_taps)
        if self.taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.w_in = self.w_x = self.w_dt = self.w_o = None
        self.conv_w = self.conv_b = self.dt_b = self.A_log = self.D = None

    def param_specs(self):
        return [ParamSpec("in", (2 * self.inner, self.hidden)), ParamSpec("conv", (self.inner, self.taps)),
                ParamSpec("conv.b", (self.inner,), init="bias"), ParamSpec("x", (self.R + 2 * self.N, self.inner)),
                ParamSpec("dt", (self.inner, self.R)), ParamSpec("dt.b", (self.inner,), init="bias"),
                ParamSpec("A_log", (self.inner, self.N), init="bias"), ParamSpec("D", (self.inner,), init="norm"),
                ParamSpec("o", (self.hidden, self.inner))]

    def load(self, tensors, rt: Runtime):
        self.w_in, self.w_x, self.w_o = (rt.matrix(tensors[n]) for n in ("in", "x", "o"))
        self.w_dt = rt.matrix(tensors["dt"])
        self.conv_w, self.conv_b = rt.vector(tensors["conv"]), rt.vector(tensors["conv.b"])
        self.dt_b, self.A_log, self.D = (rt.vector(tensors[n]) for n in ("dt.b", "A_log", "D"))

    def state_need(self):
        need = {"scan": RequestState((self.inner, self.N))}
        if self.taps > 1:
            need["conv"] = RequestState((self.taps - 1, self.inner))
        return need

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        xz = ops.linear(h, self.w_in, None, torch.float32)
        conv_state = ctx.state(call, "conv") if self.taps > 1 else torch.empty((0, 0, self.inner), device=h.device)
        x = ops.causal_conv(xz[:, :self.inner], self.conv_w, self.conv_b, conv_state, b, False, True, torch.float32)
        low = ops.linear(x if rt.dtype == torch.float32 else ops.activation(x, "copy", rt.dtype), self.w_x, None,
                         torch.float32)
        dt_in = low[:, :self.R]
        dt_in = dt_in.contiguous() if rt.dtype == torch.float32 else ops.activation(dt_in, "copy", rt.dtype)
        dt_raw = ops.linear(dt_in, self.w_dt, None, torch.float32)
        y = ops.selective_scan(x, dt_raw, low[:, self.R:], xz[:, self.inner:], self.dt_b, self.A_log, self.D,
                               ctx.state(call, "scan"), b, rt.dtype)
        ops.linear_add(y, self.w_o, resid)


class RetentionMixer(Mixer):
    """Linear attention with a constant decay per head, no softmax and no denominator.  ``q, k = W h`` (heads x
    dim), ``v = W h`` (heads x vdim), no biases; rotary positions on the first ``rope_dims`` entries of every q and k
    head (entry i with i + rope_dims / 2, angle ``position * rope_base^(-2i / rope_dims)``); k is multiplied by
    ``dim^(-1/2)`` after the rotation.  Per head n::

        S <- decay_n S + k v^T          (S: dim x vdim, 32-bit, zero at a request's start)
        o = S^T q

    Each head's o is divided by its root mean square (no weight), the heads side by side are multiplied by
    ``silu(W_g h)``, then ``W_o``.  The scan is the state-space scan with constant decays and step size 1 (keys as
    its B, queries as its C, one group per head)."""

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, decay: list[float], eps: float,
                 rope_base: float | None = None, rope_dims: int = 0):
        self.hidden, self.H, self.d, self.dv, self.eps = int(hidden_size), int(heads), int(dim), int(vdim), float(eps)
        self.decay = [float(v) for v in decay]
        if len(self.decay) != self.H:
            raise ValueError(f"{self.H} heads need {self.H} decays, got {len(self.decay)}")
        self.rope_dims = int(rope_dims) if rope_base is not None else 0
        self.rope_base = float(rope_base) if rope_base is not None else 0.0
        if self.rope_dims % 2 or not (0 <= self.rope_dims <= self.d):
            raise ValueError(f"rope_dims must be even and at most dim, got {self.rope_dims}")
        self.w_in = self.w_o = self._freq = self._decay = None

    def param_specs(self):
        H, d, dv = self.H, self.d, self.dv
        return [ParamSpec("q", (H * d, self.hidden)), ParamSpec("k", (H * d, self.hidden)),
                ParamSpec("v", (H * dv, self.hidden)), ParamSpec("g", (H * dv, self.hidden)),
                ParamSpec("o", (self.hidden, H * dv))]

    def load(self, tensors, rt: Runtime):
        # rows [v | k | q | g]: the scan reads values, keys and queries side by side in that order
        self.w_in = torch.cat([rt.matrix(tensors[n]) for n in ("v", "k", "q", "g")], dim=0).contiguous()
        self.w_o = rt.matrix(tensors["o"])
        self._decay = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(rt.device)
        self._freq = rope_inv_freqs(self.rope_dims, self.rope_base, self.rope_dims).to(rt.device) \
            if self.rope_dims else None

    def state_need(self):
        return {"retention": RequestState((self.H, self.d, self.dv))}

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        H, d, dv = self.H, self.d, self.dv
        proj = ops.linear(h, self.w_in, None, torch.float32)               # [v | k | q | g]
        ops.rotate_heads(proj, b.positions, self._freq, self.rope_dims, H, d, H * dv, d ** -0.5, H * dv + H * d, 1.0)
        o = ops.ssm_scan(proj[:, :H * dv + 2 * H * d], None, None, None, None, ctx.state(call, "retention"), b, H, dv,
                         d, H, fixed_decay=self._decay)
        g = ops.gated_rmsnorm(o, proj[:, H * dv + 2 * H * d:], None, H, self.eps, "silu_after", rt.dtype)
        ops.linear_add(g, self.w_o, resid)


class GatedDeltaMixer(Mixer):
    """Delta-rule recurrence with one decay per head.  ``q, k = W h`` (``kv_heads`` x ``dim``), ``v = W h``
    (``heads`` x ``vdim``), no biases; head n reads q/k head ``n // (heads / kv_heads)``.  Each of q, k, v passes a
    causal convolution over time per channel (``conv_taps`` taps, no bias, the last tap meets the current token) and
    silu; q and k then become unit vectors per head, ``x / sqrt(sum x^2 + unit_eps)``, and q is multiplied by
    ``dim^(-1/2)``.  With ``beta = sigmoid(W_b h)`` and ``g = exp(-exp(A_log_n) softplus(W_a h + dt_bias))`` per head::

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q      (S: dim x vdim, 32-bit, zero at the start)

    Each head's o is divided by its root mean square over ``vdim`` and multiplied by ``norm`` (``[vdim]``, the same
    for all heads) and by ``silu(W_g h)``; then ``W_o``.  A request's state: S of every head and the convolutions'
    last ``conv_taps - 1`` inputs.  Everything between the two projections is 32-bit."""

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, conv_taps: int, eps: float,
                 unit_eps: float = 1e-6):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.hidden, self.H, self.G, self.d, self.dv = int(hidden_size), int(heads), int(kv_heads), int(dim), int(vdim)
        self.taps, self.eps, self.unit_eps = int(conv_taps), float(eps), float(unit_eps)
        if self.taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.C = 2 * self.G * self.d + self.H * self.dv          # channels that pass the convolution: q, k, v
        self.w_in = self.w_o = self.conv_w = self.A_log = self.dt_bias = self.norm_w = None

    def param_specs(self):
        H, G, d, dv, hid, taps = self.H, self.G, self.d, self.dv, self.hidden, self.taps
        return [ParamSpec("q", (G * d, hid)), ParamSpec("q.conv", (G * d, taps)),
                ParamSpec("k", (G * d, hid)), ParamSpec("k.conv", (G * d, taps)),
                ParamSpec("v", (H * dv, hid)), ParamSpec("v.conv", (H * dv, taps)),
                ParamSpec("b", (H, hid)), ParamSpec("a", (H, hid)), ParamSpec("A_log", (H,), init="bias"),
                ParamSpec("dt_bias", (H,), init="bias"), ParamSpec("norm", (dv,), init="norm"),
                ParamSpec("g", (H * dv, hid)), ParamSpec("o", (hid, H * dv))]

    def load(self, tensors, rt: Runtime):
        self.w_in = torch.cat([rt.matrix(tensors[n]) for n in ("q", "k", "v", "b", "a", "g")], dim=0).contiguous()
        self.conv_w = torch.cat([rt.vector(tensors[n + ".conv"]) for n in ("q", "k", "v")], dim=0).contiguous()
        self.A_log, self.dt_bias = rt.vector(tensors["A_log"]), rt.vector(tensors["dt_bias"])
        self.norm_w = rt.vector(tensors["norm"]).repeat(self.H).contiguous()      # one weight for every head
        self.w_o = rt.matrix(tensors["o"])

    def state_need(self):
        need = {"delta": RequestState((self.H, self.d, self.dv))}
        if self.taps > 1:
            need["conv"] = RequestState((self.taps - 1, self.C))
        return need

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        H, C, Gd = self.H, self.C, self.G * self.d
        proj = ops.linear(h, self.w_in, None, torch.float32)               # [q | k | v | beta | a | gate]
        conv_state = ctx.state(call, "conv") if self.taps > 1 else torch.empty((0, 0, C), device=h.device)
        qkv = ops.causal_conv(proj[:, :C], self.conv_w, None, conv_state, b, False, True, torch.float32)
        o = ops.gated_scan(qkv[:, :Gd], qkv[:, Gd:2 * Gd], qkv[:, 2 * Gd:], proj[:, C + H:C + 2 * H], proj[:, C:C + H],
                           ctx.state(call, "delta"), b, H, self.G, self.d, self.dv, unit_eps=self.unit_eps,
                           q_scale=self.d ** -0.5, A_log=self.A_log, decay_bias=self.dt_bias)
        g = ops.gated_rmsnorm(o, proj[:, C + 2 * H:], self.norm_w, H, self.eps, "silu_after", rt.dtype)
        ops.linear_add(g, self.w_o, resid)


class GatedLinearAttention(Mixer):
    """Linear attention whose state decays per key channel by a factor made from the input.  ``q = W h * dim^(-1/2)``,
    ``k = W h`` (heads x dim), ``v = W h`` (heads x vdim); ``alpha = sigmoid(W_a2 (W_a1 h) + a2.b)^(1 / tau)`` laid out
    heads x dim (the width of the bottleneck is whatever ``a1`` has).  Per head::

        S <- diag(alpha) S + k v^T;   o = S^T q                      (S: dim x vdim, 32-bit, zero at the start)

    Each head's o is RMS-normed over ``vdim`` with ``norm`` (``[vdim]``, the same for all heads); the heads side by
    side are multiplied by ``silu(W_g h)``; the output is ``out_scale * W_o`` of that.  The decay is worked out in
    32-bit as ``exp(log sigmoid(z) / tau)``."""

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, tau: float, eps: float,
                 decay_rank: int = 16, out_scale: float = 1.0):
        self.hidden, self.H, self.d, self.dv = int(hidden_size), int(heads), int(dim), int(vdim)
        self.tau, self.eps, self.decay_rank, self.out_scale = float(tau), float(eps), int(decay_rank), float(out_scale)
        if self.tau <= 0:
            raise ValueError("tau must be positive")
        self.w_in = self.w_a2 = self.b_a2 = self.norm_w = self.w_o = None
        self.rank = self.decay_rank

    def param_specs(self):
        H, d, dv, hid = self.H, self.d, self.dv, self.hidden
        return [ParamSpec("q", (H * d, hid)), ParamSpec("k", (H * d, hid)), ParamSpec("v", (H * dv, hid)),
                ParamSpec("g", (H * dv, hid)), ParamSpec("a1", (-1, hid), arg=self.decay_rank),
                ParamSpec("a2", (H * d, -1), arg=self.decay_rank), ParamSpec("a2.b", (H * d,), init="bias"),
                ParamSpec("norm", (dv,), init="norm"), ParamSpec("o", (hid, H * dv))]

    def load(self, tensors, rt: Runtime):
        if tensors["a1"].shape[0] != tensors["a2"].shape[1]:
            raise ValueError("a1 and a2 disagree about the width of the decay's bottleneck")
        self.rank = int(tensors["a1"].shape[0])
        self.w_in = torch.cat([rt.matrix(tensors[n]) for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.w_a2, self.b_a2 = rt.matrix(tensors["a2"]), rt.vector(tensors["a2.b"])
        self.norm_w = (rt.vector(tensors["norm"]) * self.out_scale).repeat(self.H).contiguous()
        self.w_o = rt.matrix(tensors["o"])

    def state_need(self):
        return {"gla": RequestState((self.H, self.d, self.dv))}

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        H, Hd, Hv = self.H, self.H * self.d, self.H * self.dv
        proj = ops.linear(h, self.w_in, None, torch.float32)               # [q | k | v | gate | a1 h]
        low = proj[:, 2 * Hd + 2 * Hv:]
        low = low.contiguous() if rt.dtype == torch.float32 else ops.activation(low, "copy", rt.dtype)
        z = ops.linear(low, self.w_a2, self.b_a2, torch.float32)
        o = ops.gated_scan(proj[:, :Hd], proj[:, Hd:2 * Hd], proj[:, 2 * Hd:2 * Hd + Hv], z, None,
                           ctx.state(call, "gla"), b, H, H, self.d, self.dv, q_scale=self.d ** -0.5, tau=self.tau)
        g = ops.gated_rmsnorm(o, proj[:, 2 * Hd + Hv:2 * Hd + 2 * Hv], self.norm_w, H, self.eps, "silu_after", rt.dtype)
        ops.linear_add(g, self.w_o, resid)


class MatrixMemory(Mixer):
    """A matrix memory per head with exponential input gates, kept in range by a running maximum of the log gates.
    ``q = W h * dim^(-1/2)``, ``k = W h`` (heads x dim), ``v = W h`` (heads x vdim), no biases.  Per head a log input
    gate ``i = c tanh((W_i h + i.b) / c)`` and a log forget gate ``f = log sigmoid(c tanh((W_f h + f.b) / c))`` with
    ``c = gate_cap``.  With S, n and the running maximum m all zero at the start::

        m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n <- exp(f + m - m') n + exp(i - m') k
        o = S^T q / (max(|n . q|, exp(-m')) + den_eps)                    (S: dim x vdim, n: dim; 32-bit)

    Each head's o is divided by its root mean square over ``vdim``; the heads side by side are multiplied by ``norm``
    (``[heads * vdim]``) and by ``sigmoid(W_g h)``; the output is ``out_scale * W_o`` of that.  A request's state: S, n
    and m of every head (m in ``vdim + 1`` equal copies, so that every block of the scan kernel, which shares out the
    columns of ``[S | n]``, carries one of its own).  Everything between the two projections is 32-bit."""

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 den_eps: float = 1e-6, out_scale: float = 1.0):
        self.hidden, self.H, self.d, self.dv = int(hidden_size), int(heads), int(dim), int(vdim)
        self.cap, self.eps, self.den_eps, self.out_scale = float(gate_cap), float(eps), float(den_eps), float(out_scale)
        if self.cap <= 0:
            raise ValueError("gate_cap must be positive")
        self.w_in = self.i_bias = self.f_bias = self.norm_w = self.w_o = None

    def param_specs(self):
        H, d, dv, hid = self.H, self.d, self.dv, self.hidden
        return [ParamSpec("q", (H * d, hid)), ParamSpec("k", (H * d, hid)), ParamSpec("v", (H * dv, hid)),
                ParamSpec("g", (H * dv, hid)), ParamSpec("i", (H, hid)), ParamSpec("i.b", (H,), init="bias"),
                ParamSpec("f", (H, hid)), ParamSpec("f.b", (H,), init="bias"),
                ParamSpec("norm", (H * dv,), init="norm"), ParamSpec("o", (hid, H * dv))]

    def load(self, tensors, rt: Runtime):
        self.w_in = torch.cat([rt.matrix(tensors[n]) for n in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous()
        self.i_bias, self.f_bias = rt.vector(tensors["i.b"]), rt.vector(tensors["f.b"])
        self.norm_w = (rt.vector(tensors["norm"]) * self.out_scale).contiguous()
        self.w_o = rt.matrix(tensors["o"])

    def state_need(self):
        return {"memory": RequestState((self.H, self.d, self.dv)), "memory_norm": RequestState((self.H, self.d)),
                "memory_max": RequestState((self.H, self.dv + 1))}     # equal copies of m: one per column block of the scan

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        H, Hd, Hv = self.H, self.H * self.d, self.H * self.dv
        proj = ops.linear(h, self.w_in, None, torch.float32)               # [q | k | v | gate | i | f]
        gates = 2 * Hd + 2 * Hv
        o, rden = ops.memory_scan(proj[:, :Hd], proj[:, Hd:2 * Hd], proj[:, 2 * Hd:2 * Hd + Hv],
                                  proj[:, gates:gates + H], proj[:, gates + H:gates + 2 * H], self.i_bias, self.f_bias,
                                  self.cap, ctx.state(call, "memory"), ctx.state(call, "memory_norm"),
                                  ctx.state(call, "memory_max"), b, H, self.d, self.dv, q_scale=self.d ** -0.5,
                                  den_eps=self.den_eps)
        g = ops.gated_rmsnorm(o, proj[:, 2 * Hd + Hv:gates], self.norm_w, H, self.eps, "sigmoid_after", rt.dtype,
                              row_scale=rden)
        ops.linear_add(g, self.w_o, resid)


class ParallelMixers(Mixer):
    """Two mixers side by side that read the same input.  ``combine`` ``"norm_mean"``: each output is RMS-normed over
    the model width with a weight of its own (``<name>.out``); the result is ``coef`` times their sum (a half: the
    mean).  ``combine`` ``"sum"``: the outputs are added as they are (a mixer that is to count with a factor takes it
    as its own ``out_scale``); there are no tensors beside the children's.  The children's tensors lie under
    ``<name>.``; their caches and states are the pair's."""

    def __init__(self, hidden_size: int, left: PartSpec, right: PartSpec, eps: float, coef: float = 0.5,
                 names: tuple[str, str] = ("left", "right"), combine: str = "norm_mean"):
        self.hidden, self.eps, self.coef = int(hidden_size), float(eps), float(coef)
        if combine not in ("norm_mean", "sum"):
            raise ValueError(f"unknown way to combine two mixers: {combine!r}")
        self.combine = combine
        self.names = tuple(names)
        self.parts = (build_part("mixer", left), build_part("mixer", right))
        self.w_out = [None, None]
        if sum(p.cache_need() is not None for p in self.parts) > 1:
            raise ValueError("only one of two mixers side by side may keep paged keys and values")

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def param_specs(self):
        out = []
        for name, part in zip(self.names, self.parts):
            out += [replace(s, name=f"{name}.{s.name}") for s in part.param_specs()]
            if self.combine == "norm_mean":
                out.append(ParamSpec(f"{name}.out", (self.hidden,), init="norm"))
        return out

    def load(self, tensors, rt: Runtime):
        for i, (name, part) in enumerate(zip(self.names, self.parts)):
            mine = {f"{name}.{s.name}" for s in part.param_specs()}
            part.load({k[len(name) + 1:]: v for k, v in tensors.items() if k in mine}, rt)
            if self.combine == "norm_mean":
                self.w_out[i] = rt.vector(tensors[f"{name}.out"])

    def cache_need(self):
        return next((p.cache_need() for p in self.parts if p.cache_need() is not None), None)

    def state_need(self):
        need = {}
        for part in self.parts:
            s = part.state_need()
            if s is None:
                continue
            s = s if isinstance(s, dict) else {"": s}
            clash = set(s) & set(need)
            if clash:
                raise ValueError(f"two mixers side by side both name a state {sorted(clash)}")
            need.update(s)
        return need or None

    def forward(self, h, resid, ctx: StepContext, call: int):
        ops = ctx.rt.ops
        if self.combine == "sum":
            # both add into the same rows, one after the other (an add is a read and a write of the same place)
            self.parts[0].forward(h, resid, ctx, call)
            self.parts[1].forward(h, resid, ctx, call)
            return
        outs = [torch.zeros_like(resid), torch.zeros_like(resid)]
        # neither mixer needs anything of the other: in a small step the second runs beside the first
        branch = ops.branch(h.shape[0])
        with branch:
            self.parts[1].forward(h, outs[1], ctx, call)
        self.parts[0].forward(h, outs[0], ctx, call)
        branch.join()
        ops.branch_norm_add(resid, outs[0], self.w_out[0], outs[1], self.w_out[1], self.eps, self.coef)


register_part("mixer", "gated_delta", GatedDeltaMixer)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "mamba1", Mamba1Mixer)
register_part("mixer", "matrix_memory", MatrixMemory)
register_part("mixer", "retention", RetentionMixer)
register_part("mixer", "parallel_mixers", ParallelMixers)
register_part("mixer", "mamba2", Mamba2Mixer)
register_part("mixer", "general_delta", GeneralDeltaMixer)
