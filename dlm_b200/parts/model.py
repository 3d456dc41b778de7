"""A decoder model put together from parts according to a ``ModelSpec``.

The spec is data: which block each layer is, which tensors' names it reads, and
the *order* in which layers run.  The order is a list of ``LayerCall``; it may
name a layer twice, and a call may read the cache an earlier call wrote instead
of writing one of its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace

import torch

from ..registry import build_part
from .base import PagedView, ParamSpec, PartSpec, Runtime, StepBatch, StepContext


@dataclass(frozen=True)
class LayerCall:
    layer: int
    reads_cache_of: int | None = None   # index (in the order) of an earlier call whose cache is read
    enters_pass: int | None = None      # t: this call opens pass t of a run of layers that is repeated; the model's
                                        # ``pass_entry`` part makes the pass's input first


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: list[PartSpec]               # block specs
    layer_prefixes: list[str]            # tensor-name prefix of each layer ("model.layers.0.")
    final_norm: PartSpec
    final_norm_prefix: str = "model.norm."
    embed_name: str = "model.embed_tokens.weight"
    lm_head_name: str | None = "lm_head.weight"   # None: the design has no head tensor (the embedding is the head)
    tie_word_embeddings: bool = False    # True: the embedding is the head; False: tied iff the head is absent
    order: list[LayerCall] | None = None # None: every layer once, in index order
    embed_position: PartSpec | None = None   # a position encoding that acts on the embedded tokens
    embed_position_prefix: str = ""          # tensor-name prefix of that encoding's own tensors (if it has any)
    embed_scale: float = 1.0                 # the embedded tokens are multiplied by this
    residual_streams: int | None = None      # S: blocks get ``[T, S, hidden]`` (S equal copies at the start, summed at the end)
    pass_entry: PartSpec | None = None       # what makes the input of a repeated run's pass (calls with ``enters_pass``)
    pass_entry_prefix: str = ""              # tensor-name prefix of that part's tensors
    logit_softcap: float = 0.0               # c > 0: the logits are ``c tanh(head product / c)``
    dependent_launch: bool = True            # False: this model's steps launch every kernel in the ordinary way (each
                                             # starts when the one before it has ended) where the backend has the choice


class WeightError(ValueError):
    """Lists, in one message, every missing tensor, unexpected tensor and wrong shape."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = ["the checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing[:40])
                         + (" ..." if len(self.missing) > 40 else ""))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected[:40])
                         + (" ..." if len(self.unexpected) > 40 else ""))
        for name, got, want in self.wrong_shape[:40]:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype[:40]:
            lines.append(f"  unsupported dtype: {name} is {got}")
        super().__init__("\n".join(lines))


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec, self.rt = spec, rt
        self.blocks = [build_part("block", bs) for bs in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.embed_position = build_part("position", spec.embed_position) if spec.embed_position else None
        self.pass_entry = build_part("entry", spec.pass_entry) if spec.pass_entry else None
        self.order = list(spec.order) if spec.order is not None else [LayerCall(i) for i in range(len(self.blocks))]
        for ci, c in enumerate(self.order):
            if not (0 <= c.layer < len(self.blocks)):
                raise ValueError(f"order names layer {c.layer}, the model has {len(self.blocks)}")
            if c.enters_pass is not None and self.pass_entry is None:
                raise ValueError(f"call {ci} opens a pass but the model has no pass_entry part")
            if c.reads_cache_of is not None:
                if not (0 <= c.reads_cache_of < ci) or self.order[c.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"call {ci} must read the cache of an earlier call that owns one")
                a = self.blocks[c.layer].mixer.cache_need()
                b = self.blocks[self.order[c.reads_cache_of].layer].mixer.cache_need()
                if a is None or b is None or not a.same_layout(b):
                    raise ValueError(f"call {ci} cannot read call {c.reads_cache_of}'s cache: their shapes differ")
        self.embed: torch.Tensor | None = None
        self.lm_head: torch.Tensor | None = None
        # called as ``after_layer(call, x)`` with the residual rows after every call of the order, when set (for
        # comparing a model layer by layer; steps replayed from a graph do not call it)
        self.after_layer = None

    # ------------------------------------------------------------- tensors
    def param_specs(self) -> dict[str, ParamSpec]:
        s = self.spec
        out = {s.embed_name: ParamSpec(s.embed_name, (s.vocab_size, s.hidden_size))}
        if self.embed_position is not None:
            for p in self.embed_position.param_specs():
                out[s.embed_position_prefix + p.name] = replace(p, name=s.embed_position_prefix + p.name)
        if self.pass_entry is not None:
            for p in self.pass_entry.param_specs():
                out[s.pass_entry_prefix + p.name] = replace(p, name=s.pass_entry_prefix + p.name)
        for prefix, block in zip(s.layer_prefixes, self.blocks):
            for p in block.param_specs():
                out[prefix + p.name] = replace(p, name=prefix + p.name)
        for p in self.final_norm.param_specs():
            out[s.final_norm_prefix + p.name] = replace(p, name=s.final_norm_prefix + p.name)
        if s.lm_head_name is not None:
            out[s.lm_head_name] = ParamSpec(s.lm_head_name, (s.vocab_size, s.hidden_size), optional=True)
        return out

    def check(self, available: dict[str, tuple[torch.dtype, tuple[int, ...]]]) -> None:
        """Raises ``WeightError`` unless ``available`` (name -> dtype, shape) fits the model."""
        specs = self.param_specs()
        missing = [n for n, p in specs.items() if not p.optional and n not in available]
        unexpected = [n for n in available if n not in specs]
        wrong, wrong_dt = [], []
        for n, (dt, shape) in available.items():
            if n in specs:
                want = tuple(specs[n].shape)      # -1: any size (the checkpoint's)
                if len(shape) != len(want) or any(w != -1 and int(g) != w for g, w in zip(shape, want)):
                    wrong.append((n, shape, want))
                ok = (torch.int32, torch.int64) if specs[n].init == "ids" else \
                    (torch.float32, torch.bfloat16, torch.float16, torch.float64)
                if dt not in ok:
                    wrong_dt.append((n, dt))
        if missing or unexpected or wrong or wrong_dt:
            raise WeightError(sorted(missing), sorted(unexpected), wrong, wrong_dt)

    def load(self, get, names) -> None:
        """``get(name) -> tensor`` for every name in ``names`` (already checked)."""
        s, rt = self.spec, self.rt
        names = set(names)
        self.embed = rt.matrix(get(s.embed_name))
        if s.tie_word_embeddings or s.lm_head_name is None or s.lm_head_name not in names:
            self.lm_head = self.embed                  # an alias, not a copy
        else:
            self.lm_head = rt.matrix(get(s.lm_head_name))
        if self.embed_position is not None:
            mine = {s.embed_position_prefix + p.name for p in self.embed_position.param_specs()}
            self.embed_position.load({n[len(s.embed_position_prefix):]: get(n) for n in names if n in mine}, rt)
        if self.pass_entry is not None:
            mine = {s.pass_entry_prefix + p.name for p in self.pass_entry.param_specs()}
            self.pass_entry.load({n[len(s.pass_entry_prefix):]: get(n) for n in names if n in mine}, rt)
        for prefix, block in zip(s.layer_prefixes, self.blocks):
            block.load({n[len(prefix):]: get(n) for n in names if n.startswith(prefix)}, rt)
        self.final_norm.load({n[len(s.final_norm_prefix):]: get(n) for n in names
                              if n.startswith(s.final_norm_prefix)}, rt)

    # --------------------------------------------------------------- cache
    def cache_needs(self):
        """Per call of the order: (PagedCache or None, RequestState or None, owner call index)."""
        out = []
        for ci, c in enumerate(self.order):
            block = self.blocks[c.layer]
            owner = ci if c.reads_cache_of is None else c.reads_cache_of
            # a block with state of its own (beside its mixer's) says so itself
            state = block.state_need() if hasattr(block, "state_need") else block.mixer.state_need()
            out.append((block.mixer.cache_need(), state, owner))
        return out

    # ---------------------------------------------------------------- step
    def step(self, batch: StepBatch, cache) -> torch.Tensor:
        """Runs the batch's tokens through every call of the order, reading and writing
        ``cache``; returns 32-bit logits ``[len(batch.logit_rows), vocab]``."""
        rt, ops = self.rt, self.rt.ops
        if not self.spec.dependent_launch and hasattr(ops, "dependent_launch"):
            with ops.dependent_launch(False):
                return self._step(batch, cache)
        return self._step(batch, cache)

    def _step(self, batch: StepBatch, cache) -> torch.Tensor:
        rt, ops = self.rt, self.rt.ops

        def paged(call):
            return cache.paged_view(call, batch)

        ctx = StepContext(rt, batch, paged, cache.state_tensor)
        s = self.spec
        x = ops.embed(batch.tokens, self.embed, s.embed_scale) if s.embed_scale != 1.0 else ops.embed(batch.tokens, self.embed)
        if self.embed_position is not None:
            self.embed_position.on_embed(x, batch.positions, rt)
        if s.residual_streams is not None:
            x = ops.streams_expand(x, s.residual_streams)
        # a model with repeated passes keeps the embedded tokens: blocks change x in place
        x0 = x.clone() if self.pass_entry is not None and getattr(self.pass_entry, "needs_embedded", True) else None
        for ci, c in enumerate(self.order):
            if c.enters_pass is not None:
                x = self.pass_entry.forward(x, x0, c.enters_pass, rt)
            self.blocks[c.layer].forward(x, ctx, ci)
            if self.after_layer is not None:
                self.after_layer(ci, x)
        if s.residual_streams is not None:
            x = ops.streams_reduce(x, None, None, 0.0, torch.float32)
        n = self.final_norm.forward(x, rt, rows=batch.logit_rows)
        logits = ops.linear(n, self.lm_head, None, torch.float32)
        if s.logit_softcap > 0.0:
            ops.tanh_cap(logits, s.logit_softcap)
        return logits
