"""Feed-forward parts: a dense SwiGLU MLP and a routed mixture of SwiGLU experts."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import FeedForward, ParamSpec, Runtime, StepContext


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows ``2i`` = gate row i, ``2i + 1`` = up row i, so that a SwiGLU epilogue finds both
    halves of an output in neighbouring accumulator columns."""
    out = torch.empty((2 * gate.shape[0], gate.shape[1]), dtype=gate.dtype, device=gate.device)
    out[0::2] = gate
    out[1::2] = up
    return out


class DenseSwiGLU(FeedForward):
    """``resid += down · (silu(gate·h) ⊙ up·h)`` without biases (src/forward/cpu.rs:966-971, 1198)."""

    def __init__(self, hidden_size: int, intermediate_size: int, names: dict[str, str] | None = None):
        """``names``: the three tensors' names, by default the ones of Qwen2-MoE checkpoints."""
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        if names:
            self.names.update(names)
        self.w_gate_up = self.w_down = None

    def param_specs(self):
        nm = self.names
        return [ParamSpec(nm["gate"], (self.inter, self.hidden)), ParamSpec(nm["up"], (self.inter, self.hidden)),
                ParamSpec(nm["down"], (self.hidden, self.inter))]

    def load(self, tensors, rt: Runtime):
        nm = self.names
        self.w_gate_up = interleave_gate_up(rt.matrix(tensors[nm["gate"]]), rt.matrix(tensors[nm["up"]]))
        self.w_down = rt.matrix(tensors[nm["down"]])

    def forward(self, h, resid, ctx: StepContext, pre_norm=None):
        ops = ctx.rt.ops
        act = ops.linear_swiglu(h, self.w_gate_up)
        ops.linear_add(act, self.w_down, resid)


class DenseActMLP(FeedForward):
    """``resid += down · act(up · h)`` without biases; ``activation``: "gelu_tanh" (the tanh form), "gelu" (the exact
    form) or "silu".  Either gelu sits in the first product's epilogue; silu is a kernel behind it."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh"):
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        if activation not in ("gelu_tanh", "gelu", "silu"):
            raise ValueError(f"unknown activation {activation!r}")
        self.act = activation
        self.w_up = self.w_down = None

    def param_specs(self):
        return [ParamSpec("up", (self.inter, self.hidden)), ParamSpec("down", (self.hidden, self.inter))]

    def load(self, tensors, rt: Runtime):
        self.w_up, self.w_down = rt.matrix(tensors["up"]), rt.matrix(tensors["down"])

    def forward(self, h, resid, ctx: StepContext, pre_norm=None):
        ops = ctx.rt.ops
        act = ops.linear_act(h, self.w_up, self.act)
        ops.linear_add(act, self.w_down, resid)


class SoftmaxTopKMoE(FeedForward):
    """Routed experts as the reference computes them (src/forward/cpu.rs:980-1048): router
    logits in 32-bit from the 32-bit normalised residual, softmax over all experts, the k largest probabilities (ties: lower
    expert first), optionally renormalised; each chosen expert's SwiGLU output scaled by its
    weight and summed from zero in routing order; then an optional shared expert scaled by
    ``sigmoid(shared_gate · h)``; the sum goes to the residual.  ``shared_gate``: True, the gate
    tensor is required; False, there is none and the factor is 1; None, the checkpoint decides:
    a missing gate tensor means the factor 1 (src/forward/cpu.rs:1032-1041).

    At load the experts are stacked into ``[E, 2I, H]`` (gate and up rows interleaved) and
    ``[E, H, I]``; the router and the shared gate become one ``[E (+1), H]`` matrix."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, expert_intermediate_size: int,
                 norm_topk_prob: bool, shared_intermediate_size: int | None = None,
                 shared_gate: bool | None = True, router_bias: bool = False, names: dict[str, str] | None = None):
        """``router_bias``: the router has a bias (tensor ``names["router_bias"]``) that is added to its logits; with
        ``norm_topk_prob`` the weights are then the softmax over the chosen logits.  ``names``: the tensors' names
        (``{e}`` stands for the expert's number), by default the ones of Qwen2-MoE checkpoints."""
        self.names = {"router": "gate.weight", "router_bias": "gate.bias",
                      "gate": "experts.{e}.gate_proj.weight", "up": "experts.{e}.up_proj.weight",
                      "down": "experts.{e}.down_proj.weight", "shared_gate_proj": "shared_expert.gate_proj.weight",
                      "shared_up": "shared_expert.up_proj.weight", "shared_down": "shared_expert.down_proj.weight",
                      "shared_gate": "shared_expert_gate.weight"}
        if names:
            self.names.update(names)
        self.router_bias = bool(router_bias)
        self.b_router = None
        self.hidden, self.E, self.k, self.I = int(hidden_size), int(num_experts), int(top_k), int(expert_intermediate_size)
        if not (1 <= self.k <= self.E):
            raise ValueError("top_k must be in 1..num_experts")
        self.norm = bool(norm_topk_prob)
        self.Is = int(shared_intermediate_size) if shared_intermediate_size else None
        self.shared_gate = shared_gate if self.Is is not None else False
        self.has_gate = bool(self.shared_gate)      # None: settled when the tensors are loaded
        self.w_router = self.w_gate_up = self.w_down = self.ws_gate_up = self.ws_down = None

    def param_specs(self):
        nm = self.names
        specs = [ParamSpec(nm["router"], (self.E, self.hidden))]
        if self.router_bias:
            specs.append(ParamSpec(nm["router_bias"], (self.E,), init="bias"))
        for e in range(self.E):
            specs += [ParamSpec(nm["gate"].format(e=e), (self.I, self.hidden)),
                      ParamSpec(nm["up"].format(e=e), (self.I, self.hidden)),
                      ParamSpec(nm["down"].format(e=e), (self.hidden, self.I))]
        if self.Is:
            specs += [ParamSpec(nm["shared_gate_proj"], (self.Is, self.hidden)),
                      ParamSpec(nm["shared_up"], (self.Is, self.hidden)),
                      ParamSpec(nm["shared_down"], (self.hidden, self.Is))]
            if self.shared_gate is not False:
                specs.append(ParamSpec(nm["shared_gate"], (1, self.hidden), optional=self.shared_gate is None))
        return specs

    def load(self, tensors, rt: Runtime):
        nm = self.names
        rows = [rt.matrix(tensors[nm["router"]])]
        self.b_router = rt.vector(tensors[nm["router_bias"]]) if self.router_bias else None
        self.has_gate = (self.shared_gate is True
                         or (self.shared_gate is None and nm["shared_gate"] in tensors))
        if self.has_gate:
            rows.append(rt.matrix(tensors[nm["shared_gate"]]).reshape(1, self.hidden))
        self.w_router = torch.cat(rows, dim=0).contiguous()
        self.w_gate_up = torch.empty((self.E, 2 * self.I, self.hidden), dtype=rt.dtype, device=rt.device)
        self.w_down = torch.empty((self.E, self.hidden, self.I), dtype=rt.dtype, device=rt.device)
        for e in range(self.E):
            self.w_gate_up[e, 0::2] = rt.matrix(tensors[nm["gate"].format(e=e)])
            self.w_gate_up[e, 1::2] = rt.matrix(tensors[nm["up"].format(e=e)])
            self.w_down[e] = rt.matrix(tensors[nm["down"].format(e=e)])
        if self.Is:
            self.ws_gate_up = interleave_gate_up(rt.matrix(tensors[nm["shared_gate_proj"]]),
                                                 rt.matrix(tensors[nm["shared_up"]]))
            self.ws_down = rt.matrix(tensors[nm["shared_down"]])

    def forward(self, h, resid, ctx: StepContext, pre_norm=None):
        ops = ctx.rt.ops
        rms = pre_norm.fusable_rms() if pre_norm is not None else None
        shared = None
        bias = {"logit_bias": self.b_router} if self.b_router is not None else {}
        branch = ops.branch(h.shape[0])
        if self.Is:
            # the shared expert needs nothing from the router: it may run beside the routed experts
            with branch:
                sact = ops.linear_swiglu(h, self.ws_gate_up)
                shared = ops.linear(sact, self.ws_down, None, torch.float32)
        # router logits (and the shared expert's gate) from the 32-bit normalised residual: an RMS norm is
        # applied again inside the router's kernel, any other norm is asked for a 32-bit result
        if rms is not None:
            # (the residual was last written before ``pre_norm`` ran: the kernel launched just before this
            # one, the norm's or the shared expert's, only reads it)
            ids, wts, gate, offsets, rows, dest = ops.route(resid, self.w_router, self.E, self.k, self.norm,
                                                            self.has_gate, norm_weight=rms[0], eps=rms[1],
                                                            input_settled=True, **bias)
        else:
            x = h if pre_norm is None else pre_norm.forward(resid, ctx.rt, out_dtype=torch.float32)
            ids, wts, gate, offsets, rows, dest = ops.route(x, self.w_router, self.E, self.k, self.norm, self.has_gate,
                                                            **bias)
        act = ops.grouped_swiglu(h, self.w_gate_up, offsets, rows)
        y = ops.grouped_linear(act, self.w_down, offsets)
        branch.join()
        ops.moe_combine(y, dest, wts, shared, gate, resid)


class RoutedActExperts(FeedForward):
    """Routed two-matrix experts, some of which hand their input through, and an optional shared expert.

    Router logits ``z = W_router x`` in 32-bit from the 32-bit normalised residual x; scores ``s = softmax(z)`` over
    all ``experts + identity`` router outputs.  The ``top`` experts with the largest ``s + correction`` are chosen
    (``correction`` a stored vector; ties: the lower expert); their weights are their scores s divided by the chosen
    scores' sum (``+ 1e-20``).  Expert e < ``experts`` gives ``down_e · act(up_e · h)`` (no biases; ``activation``
    "gelu", the exact form, "gelu_tanh" or "silu"); the last ``identity`` router outputs are identity experts without
    tensors whose output is x itself.  The shared expert (``shared_size`` given) has the same form, runs for every
    token and is added unweighted.  ``resid += out_scale * (weighted sum + shared)``.  Tensors: ``router``
    ``[experts + identity, hidden]``, ``correction`` ``[experts + identity]``, ``e<i>.up`` ``[ff, hidden]``,
    ``e<i>.down`` ``[hidden, ff]``, ``shared.up``, ``shared.down``; the experts are stacked at load."""

    def __init__(self, hidden_size: int, num_experts: int, top: int, expert_size: int, identity: int = 0,
                 shared_size: int | None = None, activation: str = "gelu", shared_activation: str | None = None,
                 out_scale: float = 1.0):
        self.hidden, self.E, self.k, self.I = int(hidden_size), int(num_experts), int(top), int(expert_size)
        self.ident = int(identity)
        if not (1 <= self.k <= self.E + self.ident):
            raise ValueError("top must be in 1..experts + identity")
        self.Is = int(shared_size) if shared_size else None
        self.act = activation
        self.shared_act = shared_activation or activation
        for a in (self.act, self.shared_act):
            if a not in ("gelu", "gelu_tanh", "silu"):
                raise ValueError(f"unknown expert activation {a!r}")
        self.out_scale = float(out_scale)
        self.w_router = self.correction = self.w_up = self.w_down = self.ws_up = self.ws_down = None

    def param_specs(self):
        n = self.E + self.ident
        specs = [ParamSpec("router", (n, self.hidden)), ParamSpec("correction", (n,), init="bias")]
        for e in range(self.E):
            specs += [ParamSpec(f"e{e}.up", (self.I, self.hidden)), ParamSpec(f"e{e}.down", (self.hidden, self.I))]
        if self.Is:
            specs += [ParamSpec("shared.up", (self.Is, self.hidden)), ParamSpec("shared.down", (self.hidden, self.Is))]
        return specs

    def load(self, tensors, rt: Runtime):
        self.w_router = rt.matrix(tensors["router"])
        self.correction = rt.vector(tensors["correction"])
        if self.E:
            self.w_up = torch.stack([rt.matrix(tensors[f"e{e}.up"]) for e in range(self.E)]).contiguous()
            self.w_down = torch.stack([rt.matrix(tensors[f"e{e}.down"]) for e in range(self.E)]).contiguous()
        if self.Is:
            self.ws_up, self.ws_down = rt.matrix(tensors["shared.up"]), rt.matrix(tensors["shared.down"])

    takes_normed32 = True

    def forward(self, h, resid, ctx: StepContext, pre_norm=None, normed32=None):
        ops = ctx.rt.ops
        shared = None
        branch = ops.branch(h.shape[0])
        if self.Is:
            # the shared expert needs nothing from the router: it may run beside the routed experts
            with branch:
                sact = ops.linear_act(h, self.ws_up, self.shared_act)
                shared = ops.linear(sact, self.ws_down, None, torch.float32)
        # the router (and the identity experts) read the normalised residual in 32-bit
        rms = pre_norm.fusable_rms() if pre_norm is not None else None
        if normed32 is not None:
            x = normed32
        elif rms is not None:
            x = ops.rmsnorm(resid, rms[0], rms[1], torch.float32)
        elif pre_norm is not None:
            x = pre_norm.forward(resid, ctx.rt, out_dtype=torch.float32)
        else:
            x = h if h.dtype == torch.float32 else h.float()
        n = self.E + self.ident
        ids, wts, _, offsets, rows, dest = ops.route(x, self.w_router, n, self.k, 2, False, select_bias=self.correction,
                                                     scale=self.out_scale)
        y = None
        if self.E:
            act = ops.grouped_act(h, self.w_up, offsets, rows, self.act)
            y = ops.grouped_linear(act, self.w_down, offsets)
        branch.join()
        ops.moe_combine(y, dest, wts, shared, None, resid, ids=ids, num_real=self.E, passthrough=x,
                        shared_scale=self.out_scale)


class TableRoutedExperts(FeedForward):
    """A mixture of small two-matrix experts without a router: row ``token id`` of an integer table
    ``[vocab, top]`` names the token's experts (the entries of a row differ), each weighted ``1 / top``:
    ``resid += (1 / top) sum_e down_e · act(up_e · h)``, no biases.  ``activation``: "gelu" (the exact, erf
    form) or "silu".  Tensors: ``table``, ``e<i>.up`` ``[ff, hidden]``, ``e<i>.down`` ``[hidden, ff]``; at load
    the experts are stacked ``[E, ff, hidden]`` and ``[E, hidden, ff]``."""

    def __init__(self, hidden_size: int, num_experts: int, top: int, expert_size: int, vocab_size: int,
                 activation: str = "gelu"):
        self.hidden, self.E, self.k, self.I, self.V = (int(hidden_size), int(num_experts), int(top), int(expert_size),
                                                      int(vocab_size))
        if not (1 <= self.k <= self.E):
            raise ValueError("top must be in 1..experts")
        if activation not in ("gelu", "silu"):
            raise ValueError(f"unknown expert activation {activation!r}")
        self.act = activation
        self.table = self.w_up = self.w_down = None

    def param_specs(self):
        specs = [ParamSpec("table", (self.V, self.k), init="ids", arg=self.E)]
        for e in range(self.E):
            specs += [ParamSpec(f"e{e}.up", (self.I, self.hidden)), ParamSpec(f"e{e}.down", (self.hidden, self.I))]
        return specs

    def load(self, tensors, rt: Runtime):
        self.table = rt.table(tensors["table"])
        self.w_up = torch.stack([rt.matrix(tensors[f"e{e}.up"]) for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([rt.matrix(tensors[f"e{e}.down"]) for e in range(self.E)]).contiguous()

    def forward(self, h, resid, ctx: StepContext, pre_norm=None):
        ops = ctx.rt.ops
        _, wts, offsets, rows, dest = ops.table_route(ctx.batch.tokens, self.table, self.E)
        act = ops.grouped_act(h, self.w_up, offsets, rows, self.act)
        y = ops.grouped_linear(act, self.w_down, offsets)
        ops.moe_combine(y, dest, wts, None, None, resid)


register_part("ffn", "table_experts", TableRoutedExperts)
register_part("ffn", "routed_act_experts", RoutedActExperts)
register_part("ffn", "swiglu_dense", DenseSwiGLU)
register_part("ffn", "dense_act", DenseActMLP)
register_part("ffn", "moe_softmax_topk", SoftmaxTopKMoE)
