"""Typed configuration of the Faguzen decoder.

``config.json`` of this design is nested: ``layers`` is a list with one entry per layer, each naming its mixer
(``type``: ``parallel``), the mixer's sizes (``mixer``, with the sections ``left``, softmax attention, and ``right``, a
matrix memory, and the factors ``left_scale`` / ``right_scale``) and its feed-forward (``mlp``: ``kind`` ``moe`` with the
sections ``router``, ``expert`` and optionally ``shared``, or null for none).  ``loop`` (optional) names a run of layers
``start .. stop - 1`` that is repeated ``times`` times with the same weights.  Model-wide: ``vocab``, ``width``,
``norm.eps``, ``residual_mult``, ``logit_softcap``.  Every size and constant is read from here (or from a tensor's
shape); the class checks what each kind needs and keeps the layer entries as they were written, so that ``to_dict``
gives the file back.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, as_float, as_int

LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim")
RIGHT_KEYS = ("heads", "dim", "vdim")
SCALING_KEYS = ("factor", "low", "high", "original")
LAYER_TYPES = ("parallel",)


def _section(raw: dict, key: str, where: str = "config.json") -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where} lacks the section {key!r}")
    return v


def _positive(v: Any, key: str) -> float:
    x = as_float(v, key)
    if not x > 0:
        raise ConfigError(f"{key} must be positive, got {x}")
    return x


def _cap(section: dict, key: str, where: str) -> None:
    """A tanh cap: absent, null or 0 for none, else a positive number."""
    v = section.get(key)
    if v is None:
        return
    if as_float(v, f"{where}.{key}") < 0:
        raise ConfigError(f"{where}.{key} must not be negative")


def _rotation(section: dict, where: str, most: int) -> None:
    rot = section.get("rot")
    if rot is None:
        return
    if not isinstance(rot, dict):
        raise ConfigError(f"{where}.rot must be a section")
    _positive(rot.get("base"), f"{where}.rot.base")
    dims = as_int(rot.get("dims", most), f"{where}.rot.dims", minimum=0)
    if dims % 2 or dims > most:
        raise ConfigError(f"{where}.rot.dims must be even and at most {most}, got {dims}")
    sc = rot.get("scaling")
    if sc is None:
        return
    if not isinstance(sc, dict):
        raise ConfigError(f"{where}.rot.scaling must be a section")
    for key in SCALING_KEYS:
        _positive(sc.get(key), f"{where}.rot.scaling.{key}")
    if not sc["high"] > sc["low"]:
        raise ConfigError(f"{where}.rot.scaling: high must be above low")


@dataclass
class FaguzenConfig:
    vocab: int
    width: int
    layers: list[dict[str, Any]]
    norm_eps: float = 1e-6
    residual_mult: float = 1.0
    logit_softcap: float = 0.0              # 0: the logits are the head's product as it is
    loop: dict[str, int] | None = None       # {"start", "stop", "times"}
    max_positions: int = 32768               # the design has no table of positions; this is the context an engine is
                                             # made for when its caller names none (the key `max_positions` overrides it)
    eos_token_ids: list[int] = field(default_factory=list)

    architecture = "Faguzen"
    model_type = "faguzen"

    # what the engine and the command line ask of any config
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, raw: dict) -> "FaguzenConfig":
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError("config.json lacks 'layers' (a list with one entry per layer)")
        for key in ("vocab", "width"):
            if key not in raw:
                raise ConfigError(f"config.json lacks required key {key!r}")
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("'loop' must be a section with start, stop and times")
            loop = {k: as_int(loop.get(k), f"loop.{k}", minimum=(1 if k == "times" else 0))
                    for k in ("start", "stop", "times")}
        cap = raw.get("logit_softcap")
        cfg = cls(vocab=as_int(raw["vocab"], "vocab", minimum=1), width=as_int(raw["width"], "width", minimum=1),
                  layers=copy.deepcopy(raw["layers"]),
                  norm_eps=as_float(_section(raw, "norm").get("eps", 1e-6), "norm.eps"),
                  residual_mult=as_float(raw.get("residual_mult", 1.0), "residual_mult"),
                  logit_softcap=as_float(cap, "logit_softcap") if cap is not None else 0.0, loop=loop,
                  max_positions=as_int(raw.get("max_positions", 32768), "max_positions", minimum=1))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        n = len(self.layers)
        if self.logit_softcap < 0:
            raise ConfigError("logit_softcap must not be negative")
        if self.loop is not None and not (0 <= self.loop["start"] < self.loop["stop"] <= n):
            raise ConfigError(f"loop: start < stop <= {n} layers is needed, got {self.loop['start']} .. {self.loop['stop']}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                raise ConfigError(f"{where}: 'type' must be one of {list(LAYER_TYPES)}, got "
                                  f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = _section(layer, "mixer", where)
            w = where + ".mixer"
            left, right = _section(m, "left", w), _section(m, "right", w)
            for key in LEFT_KEYS:
                as_int(left.get(key), f"{w}.left.{key}", minimum=1)
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"{w}.left: heads must be a multiple of kv_heads")
            as_float(left.get("scale"), f"{w}.left.scale")
            _cap(left, "softcap", w + ".left")
            _rotation(left, w + ".left", left["dim"])
            for key in RIGHT_KEYS:
                as_int(right.get(key), f"{w}.right.{key}", minimum=1)
            _positive(right.get("gate_cap"), f"{w}.right.gate_cap")
            as_float(m.get("left_scale"), f"{w}.left_scale")
            as_float(m.get("right_scale"), f"{w}.right_scale")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                raise ConfigError(f"{where}: 'mlp' must be null or of kind 'moe'")
            w = where + ".mlp"
            router = _section(mlp, "router", w)
            experts = as_int(router.get("experts"), f"{w}.router.experts", minimum=0)
            ident = as_int(router.get("identity", 0), f"{w}.router.identity", minimum=0)
            top = as_int(router.get("top"), f"{w}.router.top", minimum=1)
            if top > experts + ident:
                raise ConfigError(f"{w}.router.top must be at most experts + identity = {experts + ident}, got {top}")
            if experts:
                as_int(_section(mlp, "expert", w).get("ff"), f"{w}.expert.ff", minimum=1)
            if mlp.get("shared") is not None:
                as_int(_section(mlp, "shared", w).get("ff"), f"{w}.shared.ff", minimum=1)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "logit_softcap": self.logit_softcap, "layers": copy.deepcopy(self.layers)}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        if self.max_positions != 32768:
            out["max_positions"] = self.max_positions
        return out
