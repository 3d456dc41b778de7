"""Typed configuration of the Salolorn decoder.

``config.json`` of this design is nested: ``layers`` is a list with one entry per layer, each naming its mixer
(``type``: ``delta``, ``latent_attention`` or ``parallel``), the mixer's sizes (``mixer``; a ``parallel`` mixer has the
sections ``left``, chunked softmax attention, and ``right``, gated linear attention, and the factors ``left_scale`` /
``right_scale``) and its feed-forward (``mlp``: ``kind`` ``dense`` with ``ff``, or null for none).  ``loop`` (optional)
names a run of layers ``start .. stop - 1`` that is repeated ``times`` times with the same weights.  Model-wide:
``vocab``, ``width``, ``norm.eps``, ``logit_scale``.  Every size and constant is read from here (or from a tensor's
shape); the class checks what each kind needs and keeps the layer entries as they were written, so that ``to_dict``
gives the file back.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, as_float, as_int

DELTA_KEYS = ("heads", "kv_heads", "dim", "vdim", "conv")
LATENT_KEYS = ("heads", "dim", "rot_dim", "vdim", "kv_rank")
LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim")
RIGHT_KEYS = ("heads", "dim", "vdim")
LAYER_TYPES = ("delta", "latent_attention", "parallel")


def _section(raw: dict, key: str, where: str = "config.json") -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where} lacks the section {key!r}")
    return v


def _rotation(section: dict, where: str, most: int, dims_default: int | None = None) -> None:
    rot = _section(section, "rot", where)
    as_float(rot.get("base"), f"{where}.rot.base")
    dims = rot.get("dims", dims_default)
    dims = as_int(dims, f"{where}.rot.dims", minimum=0)
    if dims % 2 or dims > most:
        raise ConfigError(f"{where}.rot.dims must be even and at most {most}, got {dims}")


@dataclass
class SalolornConfig:
    vocab: int
    width: int
    layers: list[dict[str, Any]]
    norm_eps: float = 1e-6
    logit_scale: float = 1.0
    loop: dict[str, int] | None = None       # {"start", "stop", "times"}
    max_positions: int = 32768               # the design has no table of positions; this is the context an engine is
                                             # made for when its caller names none (the key `max_positions` overrides it)
    eos_token_ids: list[int] = field(default_factory=list)

    architecture = "Salolorn"
    model_type = "salolorn"

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
    def from_dict(cls, raw: dict) -> "SalolornConfig":
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
        cfg = cls(vocab=as_int(raw["vocab"], "vocab", minimum=1), width=as_int(raw["width"], "width", minimum=1),
                  layers=copy.deepcopy(raw["layers"]),
                  norm_eps=as_float(_section(raw, "norm").get("eps", 1e-6), "norm.eps"),
                  logit_scale=as_float(raw.get("logit_scale", 1.0), "logit_scale"), loop=loop,
                  max_positions=as_int(raw.get("max_positions", 32768), "max_positions", minimum=1))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        n = len(self.layers)
        if self.loop is not None and not (0 <= self.loop["start"] < self.loop["stop"] <= n):
            raise ConfigError(f"loop: start < stop <= {n} layers is needed, got {self.loop['start']} .. {self.loop['stop']}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                raise ConfigError(f"{where}: 'type' must be one of {list(LAYER_TYPES)}, got "
                                  f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = _section(layer, "mixer", where)
            w = where + ".mixer"
            if layer["type"] == "delta":
                for key in DELTA_KEYS:
                    as_int(m.get(key), f"{w}.{key}", minimum=1)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{w}: heads must be a multiple of kv_heads")
            elif layer["type"] == "latent_attention":
                for key in LATENT_KEYS:
                    as_int(m.get(key), f"{w}.{key}", minimum=1)
                as_float(m.get("scale"), f"{w}.scale")
                _rotation(m, w, m["rot_dim"], m["rot_dim"])
                if m["rot"].get("dims", m["rot_dim"]) != m["rot_dim"]:
                    raise ConfigError(f"{w}: the rotated part is rotated as a whole (rot.dims = rot_dim)")
            else:
                left, right = _section(m, "left", w), _section(m, "right", w)
                for key in LEFT_KEYS:
                    as_int(left.get(key), f"{w}.left.{key}", minimum=1)
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{w}.left: heads must be a multiple of kv_heads")
                as_float(left.get("scale"), f"{w}.left.scale")
                as_int(_section(left, "mask", w + ".left").get("size"), f"{w}.left.mask.size", minimum=1)
                _rotation(left, w + ".left", left["dim"], left["dim"])
                for key in RIGHT_KEYS:
                    as_int(right.get(key), f"{w}.right.{key}", minimum=1)
                if as_float(right.get("tau"), f"{w}.right.tau") <= 0:
                    raise ConfigError(f"{w}.right.tau must be positive")
                as_float(m.get("left_scale"), f"{w}.left_scale")
                as_float(m.get("right_scale"), f"{w}.right_scale")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"{where}: 'mlp' must be null or of kind 'dense'")
            as_int(mlp.get("ff"), f"{where}.mlp.ff", minimum=1)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "layers": copy.deepcopy(self.layers)}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        if self.max_positions != 32768:
            out["max_positions"] = self.max_positions
        return out
