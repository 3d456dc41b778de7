"""Small Faguzen configurations and random weights for the tests.

The weights are drawn so that every mechanism matters to the logits: norm weights away from 1 with biases and an
alpha of their own, attention biases of the size of the projections, scores large enough for the cap to bend them,
gate projections on both sides of zero, forget gates between slow and fast, input gates that move the running
maximum, a correction that changes which experts are chosen, pass vectors of the size of the embedding.  Matrices are
stored in bfloat16 (so that a bfloat16 engine and the 64-bit plain implementation read the same numbers).

A, B, C and D differ in every size and option; sizes that a config could make equal by accident (dim and vdim, the
heads of the two sides, the experts' and the shared expert's width) are unequal, and none is a power of two unless a
kernel's fast path needs it.  A: a loop over the middle, a rotation over part of the head with slowed long waves, a
layer without feed-forward, identity experts.  B: no loop, sizes that are multiples of neither 4 nor 8, as many
key/value heads as query heads, one memory head, no identity experts, no shared expert in one layer, top 1, no cap on
the logits, a rotation over the whole head without scaling.  C: sizes of the tensor-core paths (64- and 128-wide
heads), a loop that starts at the first layer and runs three times, more identity experts than others, no score cap
in one layer.  D: a loop of one pass over all layers, no rotation at all, only identity experts in one layer, top 3.
"""
from __future__ import annotations

import json
import math
import os

import torch

SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}


def left(heads, kv, dim, vdim, scale, cap=None, base=None, dims=None, scaling=None):
    out = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if cap is not None:
        out["softcap"] = cap
    if base is not None:
        out["rot"] = {"base": base, "dims": dims if dims is not None else dim}
        if scaling:
            out["rot"]["scaling"] = dict(scaling)
    return out


def right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def moe(experts, identity, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(lf, rt, ls, rs, mlp=None):
    return {"type": "parallel", "mixer": {"left": lf, "right": rt, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


CONFIGS = {
    "A": {"architecture": "Faguzen", "vocab": 131, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
          "logit_softcap": 9.0, "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [layer(left(6, 3, 24, 40, 0.3, 6.0, 5000.0, 16, SCALING), right(3, 10, 14, 9.0), 0.7, 1.4, moe(5, 2, 2, 30, 44)),
                     layer(left(4, 2, 20, 12, 0.35, 4.0, 300.0, 20, SCALING), right(2, 18, 26, 5.0), 1.2, 0.6),
                     layer(left(3, 1, 28, 36, 0.25, 10.0, 1e4, 8), right(4, 6, 10, 15.0), 0.9, 1.1, moe(6, 3, 3, 20, 28)),
                     layer(left(2, 2, 16, 24, 0.4, 5.0, 50.0, 12, SCALING), right(1, 30, 22, 7.0), 1.0, 0.8, moe(4, 1, 1, 50))]},
    "B": {"architecture": "Faguzen", "vocab": 77, "width": 62, "norm": {"eps": 3e-6}, "residual_mult": 1.0,
          "layers": [layer(left(4, 4, 10, 6, 0.5, 3.0, 300.0), right(1, 46, 38, 4.0), 1.0, 0.5, moe(7, 0, 1, 26)),
                     layer(left(5, 1, 14, 18, 0.3, 8.0, 77.0, 6), right(3, 7, 5, 20.0), 0.4, 1.3, moe(3, 2, 2, 34, 18))]},
    "C": {"architecture": "Faguzen", "vocab": 260, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.6,
          "logit_softcap": 20.0, "loop": {"start": 0, "stop": 2, "times": 3},
          "layers": [layer(left(8, 2, 64, 64, 0.15, 12.0, 1e6, 32, {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 128}),
                           right(2, 64, 128, 12.0), 1.3, 0.9, moe(8, 2, 2, 64, 96)),
                     layer(left(4, 1, 128, 96, 0.1, None, 1e4, 128), right(4, 32, 64, 6.0), 0.8, 1.2, moe(2, 5, 3, 48, 32)),
                     layer(left(2, 2, 96, 128, 0.12, 30.0, 500.0, 64), right(1, 128, 64, 8.0), 0.5, 1.0)]},
    "D": {"architecture": "Faguzen", "vocab": 53, "width": 48, "norm": {"eps": 2e-5}, "residual_mult": 1.3,
          "logit_softcap": 4.0, "loop": {"start": 0, "stop": 2, "times": 1},
          "layers": [layer(left(2, 1, 12, 20, 0.45, 2.5), right(3, 8, 12, 10.0), 1.0, 1.0, moe(0, 4, 3, 1, 22)),
                     layer(left(6, 3, 8, 4, 0.5, 7.0), right(2, 20, 9, 3.0), 0.7, 0.9, moe(9, 1, 3, 14, 10))]},
}


def one_layer(lyr, width=64, vocab=53, loop=None, mult=0.9, cap=7.0):
    """A model of a single layer (for a mechanism alone)."""
    cfg = {"architecture": "Faguzen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": mult,
           "logit_softcap": cap, "layers": [lyr]}
    if loop:
        cfg["loop"] = loop
    return cfg


def make_weights(cfg, seed=0):
    """name -> tensor (bfloat16) for a config dict."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(*shape, generator=g)).to(torch.bfloat16)

    def lin(o, i, gain=1.0):
        return rnd(o, i, std=gain / math.sqrt(i))

    def norm(name):
        out[name] = rnd(W, std=0.2, mean=1.1)
        out[name + ".b"] = rnd(W, std=0.15)
        out[name + ".alpha"] = rnd(1, std=0.1, mean=0.7).reshape(())

    out["embed"] = rnd(V, W, std=0.8)
    out["head"] = lin(V, W, gain=3.0)
    norm("final.norm")
    if cfg.get("loop"):
        out["loop.step"] = rnd(cfg["loop"]["times"], W, std=0.4)
    for i, L in enumerate(cfg["layers"]):
        norm(f"l{i}.norm1")
        p, m = f"l{i}.mix.left.", L["mixer"]["left"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "q"], out[p + "k"], out[p + "v"] = lin(H * d, W, 2.0), lin(G * d, W, 2.0), lin(G * dv, W, 1.2)
        out[p + "q.b"], out[p + "k.b"], out[p + "v.b"] = rnd(H * d, std=0.5), rnd(G * d, std=0.5), rnd(G * dv, std=0.4)
        out[p + "g"], out[p + "o"], out[p + "o.b"] = lin(H * dv, W, 2.0), lin(W, H * dv, 1.0), rnd(W, std=0.2)
        p, m = f"l{i}.mix.right.", L["mixer"]["right"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        out[p + "q"], out[p + "k"], out[p + "v"] = lin(H * d, W, 1.5), lin(H * d, W, 1.5), lin(H * dv, W, 1.2)
        out[p + "g"], out[p + "o"] = lin(H * dv, W, 2.0), lin(W, H * dv, 1.0)
        out[p + "norm"] = rnd(H * dv, std=0.3, mean=1.2)
        out[p + "i"], out[p + "f"] = lin(H, W, 2.0), lin(H, W, 2.5)
        out[p + "i.b"], out[p + "f.b"] = rnd(H, std=1.0, mean=-0.5), rnd(H, std=1.0, mean=2.0)
        mlp = L["mlp"]
        if mlp is None:
            continue
        norm(f"l{i}.norm2")
        p = f"l{i}.mlp."
        E, ident, ff = mlp["router"]["experts"], mlp["router"].get("identity", 0), mlp["expert"]["ff"]
        out[p + "router"] = lin(E + ident, W, 3.0)
        out[p + "correction"] = rnd(E + ident, std=0.25)
        for e in range(E):
            out[p + f"e{e}.up"], out[p + f"e{e}.down"] = lin(ff, W, 1.5), lin(W, ff, 1.5)
        if mlp.get("shared"):
            out[p + "shared.up"], out[p + "shared.down"] = lin(mlp["shared"]["ff"], W, 1.5), lin(W, mlp["shared"]["ff"], 1.0)
    return out


def write_model(cfg, folder, seed=0, tensors=None):
    from dlm_b200.weights.safetensors_io import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = make_weights(cfg, seed) if tensors is None else tensors
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return tensors


def tokens(seed, length, vocab):
    g = torch.Generator().manual_seed(9000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def row_error(got, ref):
    """Per row: root mean square of the difference (its mean taken off) over that of the reference."""
    got, ref = got.double(), ref.double()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return torch.sqrt((d * d).mean(-1)) / torch.sqrt((r * r).mean(-1))


# what a correct engine stays within (rounding of the format; measured values are printed by the tests)
TOL = {"float32": 2e-4, "bfloat16": 6e-2}
# A choice of experts is clear when the last chosen expert's score + correction is this far above the next one's;
# where it is not, two correct computations may choose differently, and the position is not compared.  In bfloat16 the
# positions right behind such a one are left out as well: keys, values and the memory carry the other choice on for
# a while.  (Measured on these weights with the plain model, exact against rounded: choices differ only where the lead
# is below 3e-3, and the error is back to that of rounding within five positions.)
GAP = {"float32": 2e-5, "bfloat16": 5e-3}
CARRY = {"float32": 0, "bfloat16": 6}


def references(oracle, reqs, dtype, gap=None, carry=None):
    """Per request the exact logits, a limit for every position, and which positions are compared.  The limit is TOL,
    or in bfloat16 three times the error that rounding alone causes (the plain model with bfloat16 where an engine
    must round) where that is more; the error that rounding causes at a position is taken as the larger of the
    rounded run's error there and its root mean square over the request's compared positions."""
    import plain_faguzen as plain
    ref, lim, ok = {}, {}, {}
    for rid, t in reqs.items():
        ref[rid] = oracle.forward(t)
        gaps = oracle.last_gaps
        clear = gaps >= (GAP[dtype] if gap is None else gap)
        for at in (~clear).nonzero().flatten().tolist():
            clear[at:at + 1 + (CARRY[dtype] if carry is None else carry)] = False
        ok[rid] = clear
        lim[rid] = torch.full((len(t),), TOL[dtype], dtype=torch.float64)
    if dtype == "bfloat16":
        rounded = plain.PlainFaguzen(oracle.cfg, oracle.t, rounded=True)
        for rid, t in reqs.items():
            err = row_error(rounded.forward(t), ref[rid])
            if bool(ok[rid].any()):
                err = torch.maximum(err, torch.sqrt((err[ok[rid]] ** 2).mean()))
            lim[rid] = torch.maximum(lim[rid], 3.0 * err)
    return ref, lim, ok


def ratios(got, ref, lim, ok):
    return [float(row_error(row, ref[rid][p]) / lim[rid][p]) for (rid, p), row in got.items() if bool(ok[rid][p])]


def worst_ratio(got, ref, lim, ok):
    """Largest error / limit over the compared rows of ``{(request, position): logits}``."""
    return max(ratios(got, ref, lim, ok), default=0.0)


def within_limits(got, ref, lim, ok):
    """A limit made from one rounded run is itself a noisy number, so a few rows may pass it by a little: no row is
    beyond one and a half times its limit and at most one in fifty is beyond it."""
    r = ratios(got, ref, lim, ok)
    return max(r, default=0.0) < 1.5 and sum(x > 1.0 for x in r) <= len(r) // 50


def mostly_within_limits(got, ref, lim, ok):
    """For a model wide enough that rounding now and then turns a choice of experts which the lead did not mark as
    close: such a turn shows at a few positions behind it and nowhere else, a fault of a kernel shows everywhere.  At
    most one row in fifty is beyond its limit, and the median row is within half of it."""
    r = sorted(ratios(got, ref, lim, ok))
    return sum(x > 1.0 for x in r) <= len(r) // 50 and r[len(r) // 2] < 0.5
