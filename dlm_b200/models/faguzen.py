"""Faguzen as a ``ModelSpec`` of parts.

Token embedding and a separate head whose logits pass ``c tanh(. / c)``; a norm without statistics
(``tanh(alpha x) w + b``) wherever the design norms; layers that add ``residual_mult`` times the sum of a mixer and a
feed-forward of the same input, each through a norm of its own.  The mixer is two mixers side by side whose outputs
are added with a factor each: grouped-query softmax attention over all earlier positions (biases, a rotation over
part of each head whose long waves are slowed, scores squashed by a tanh, a gate per output entry) and a matrix
memory per head with exponential gates and a running maximum.  The feed-forward is a mixture of two-matrix gelu
experts chosen on score plus a stored correction, of which the last few hand their input through, plus a shared
expert; or absent.  Optionally a run of layers is repeated several times, each pass with a cache and state of its
own, opened by adding a learned vector per pass.  ``residual_mult`` rides on the parts' own output factors (the
attention's gate and output bias, the memory's norm weight, the router's weights and the shared expert), so a layer
adds to the residual once per part and no pass over the rows is spent on it.
Tensor names are the checkpoint's own: ``embed``, ``head``, ``loop.step``, ``l<i>.norm1`` (``.b``, ``.alpha``),
``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.faguzen import FaguzenConfig
from ..parts.base import PartSpec
from ..parts.model import ModelSpec
from ..registry import register_architecture
from .zasazen import layer_order

_NAMES = {"norm1": "norm1", "mixer": "mix.", "norm2": "norm2", "ffn": "mlp."}
DEN_EPS = 1e-6           # added to the matrix memory's denominator


def _mixer(cfg: FaguzenConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    left, right = m["left"], m["right"]
    rot = left.get("rot") or {}
    dims = rot.get("dims", left["dim"]) if rot else 0
    mult = cfg.residual_mult
    return PartSpec("parallel_mixers", {
        "hidden_size": cfg.width, "eps": cfg.norm_eps, "names": ("left", "right"), "combine": "sum",
        "left": PartSpec("head_normed_attention", {
            "hidden_size": cfg.width, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"],
            "vdim": left["vdim"], "scale": left["scale"], "eps": cfg.norm_eps, "qk_norm": False,
            "position": PartSpec("rope_scaled_neox", {"head_dim": left["dim"], "theta": rot["base"], "rotary_dim": dims,
                                                      "scaling": rot.get("scaling")}) if dims else None,
            "gate": "entry", "qkv_bias": True, "o_bias": True, "softcap": left.get("softcap") or None,
            "out_scale": mult * m["left_scale"]}),
        "right": PartSpec("matrix_memory", {
            "hidden_size": cfg.width, "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"],
            "gate_cap": right["gate_cap"], "eps": cfg.norm_eps, "den_eps": DEN_EPS,
            "out_scale": mult * m["right_scale"]})})


def _ffn(cfg: FaguzenConfig, mlp: dict | None) -> PartSpec | None:
    if mlp is None:
        return None
    router = mlp["router"]
    return PartSpec("routed_act_experts", {
        "hidden_size": cfg.width, "num_experts": router["experts"], "top": router["top"],
        "expert_size": mlp["expert"]["ff"] if router["experts"] else 1, "identity": router.get("identity", 0),
        "shared_size": mlp["shared"]["ff"] if mlp.get("shared") else None, "activation": "gelu",
        "out_scale": cfg.residual_mult})


def build_spec(cfg: FaguzenConfig) -> ModelSpec:
    norm = PartSpec("dynamic_tanh", {"size": cfg.width, "param": ""})
    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        ffn = _ffn(cfg, layer.get("mlp"))
        layers.append(PartSpec("parallel", {"norm1": norm, "mixer": _mixer(cfg, layer),
                                            "norm2": norm if ffn is not None else None, "ffn": ffn, "names": _NAMES}))
        prefixes.append(f"l{i}.")
    entry = None
    if cfg.loop:
        entry = PartSpec("additive", {"hidden_size": cfg.width, "passes": cfg.loop["times"], "step": "step",
                                      "add_embedded": False})
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, layer_prefixes=prefixes,
                     final_norm=norm, final_norm_prefix="final.norm", embed_name="embed", lm_head_name="head",
                     order=layer_order(len(cfg.layers), cfg.loop), pass_entry=entry, pass_entry_prefix="loop.",
                     logit_softcap=cfg.logit_softcap,
                     # This design's steps stopped answering now and then when the clocks were polled beside them and
                     # its kernels were launched dependently; with ordinary launches they did not, so it takes those.
                     dependent_launch=False)


register_architecture(FaguzenConfig.architecture, FaguzenConfig, build_spec, model_type=FaguzenConfig.model_type)
