"""Salolorn as a ``ModelSpec`` of parts.

Token embedding that is also the output matrix (logits times a constant); layers with an RMS norm before and after
each sublayer; per layer one of three mixers: a delta-rule recurrence with one decay per head behind short
convolutions, softmax attention through one cached latent per token (rotation on neighbouring pairs), or two mixers
side by side whose outputs are added with a factor each (grouped-query attention inside chunks of positions with
per-head query/key norms, a sink in the softmax and a gate per head; linear attention with a decay per key channel);
a gated (silu) feed-forward or none; optionally a run of layers repeated several times, each pass with a cache and
state of its own, opened by adding the embedded tokens (from the second pass on) and a learned vector per pass.
Tensor names are the checkpoint's own: ``embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.salolorn import SalolornConfig
from ..parts.base import PartSpec
from ..parts.model import ModelSpec
from ..registry import register_architecture
from .zasazen import layer_order

_NAMES = {"norm1": "norm1", "norm1b": "norm1b", "mixer": "mix.", "norm2": "norm2", "norm2b": "norm2b", "ffn": "mlp."}
_FF_NAMES = {"gate": "gate", "up": "up", "down": "down"}
UNIT_EPS = 1e-6          # inside the root when the delta rule's queries and keys are made unit vectors


def _mixer(cfg: SalolornConfig, layer: dict) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    if kind == "delta":
        return PartSpec("gated_delta", {"hidden_size": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"],
                                        "dim": m["dim"], "vdim": m["vdim"], "conv_taps": m["conv"], "eps": cfg.norm_eps,
                                        "unit_eps": UNIT_EPS})
    if kind == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
            "kv_rank": m["kv_rank"], "q_rank": None, "eps": cfg.norm_eps, "rope_base": m["rot"]["base"],
            "rope_dims": m["rot"].get("dims", m["rot_dim"]), "window": None, "scale": m["scale"], "sink": False,
            "gate": False, "interleaved": True})
    left, right = m["left"], m["right"]
    rot = left["rot"]
    return PartSpec("parallel_mixers", {
        "hidden_size": cfg.width, "eps": cfg.norm_eps, "names": ("left", "right"), "combine": "sum",
        "left": PartSpec("head_normed_attention", {
            "hidden_size": cfg.width, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"],
            "vdim": left["vdim"], "scale": left["scale"], "eps": cfg.norm_eps, "qk_norm": True,
            "position": PartSpec("rope_neox", {"head_dim": left["dim"], "theta": rot["base"],
                                               "rotary_dim": rot.get("dims", left["dim"])})
            if rot.get("dims", left["dim"]) else None,
            "chunk": left["mask"]["size"], "sink": True, "gate": True, "out_scale": m["left_scale"]}),
        "right": PartSpec("gated_linear_attention", {
            "hidden_size": cfg.width, "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"],
            "tau": right["tau"], "eps": cfg.norm_eps, "out_scale": m["right_scale"]})})


def build_spec(cfg: SalolornConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "param": ""})
    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        mlp = layer.get("mlp")
        ffn = PartSpec("swiglu_dense", {"hidden_size": cfg.width, "intermediate_size": mlp["ff"],
                                        "names": _FF_NAMES}) if mlp is not None else None
        layers.append(PartSpec("sandwich", {"norm1": norm, "mixer": _mixer(cfg, layer), "norm1b": norm,
                                            "norm2": norm if ffn is not None else None, "ffn": ffn,
                                            "norm2b": norm if ffn is not None else None, "names": _NAMES}))
        prefixes.append(f"l{i}.")
    entry = None
    if cfg.loop:
        entry = PartSpec("additive", {"hidden_size": cfg.width, "passes": cfg.loop["times"], "step": "step"})
    final = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "param": "", "scale": cfg.logit_scale})
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, layer_prefixes=prefixes,
                     final_norm=final, final_norm_prefix="final.norm", embed_name="embed", lm_head_name=None,
                     tie_word_embeddings=True, order=layer_order(len(cfg.layers), cfg.loop),
                     pass_entry=entry, pass_entry_prefix="loop.")


register_architecture(SalolornConfig.architecture, SalolornConfig, build_spec, model_type=SalolornConfig.model_type)
