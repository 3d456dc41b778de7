"""Small Salolorn configurations and random weights for the tests.

The weights are drawn so that every mechanism matters to the logits: norm weights away from 1, sinks of the size of the
scores, decays between slow and fast, write strengths on both sides of a half, pass vectors of the size of the
embedding.  Matrices are stored in bfloat16 (so that a bfloat16 engine and the 64-bit plain implementation read the
same numbers).

A, B, C and D differ in every size and option; sizes that a config could make equal by accident (dim and vdim, the
heads of the two halves, query/key heads and value heads of the delta rule) are unequal, and none is a power of two
unless a kernel's fast path needs it.  A: a loop over the middle, chunks of 37 positions, a rotation over part of the
head, a layer without feed-forward.  B: no loop, sizes that are multiples of neither 4 nor 8, a convolution of a single
tap, chunks of 5, as many key/value heads as query heads, one linear-attention head, tau 1.  C: sizes of the
tensor-core paths (64- and 128-wide heads, a latent of 128), chunks of exactly a page, a loop that starts at the first
layer and runs three times.  D: a loop of one pass over all layers, chunks longer than any request, no rotation in the
chunked attention.
"""
from __future__ import annotations

import json
import math
import os

import torch


def delta(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, scale, base, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}}, "mlp": mlp}


def left(heads, kv, dim, vdim, scale, size, base, dims):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size},
            "rot": {"base": base, "dims": dims}}


def right(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def parallel(lf, rt, ls, rs, mlp=None):
    return {"type": "parallel", "mixer": {"left": lf, "right": rt, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


CONFIGS = {
    "A": {"architecture": "Salolorn", "vocab": 131, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [delta(4, 2, 12, 20, 3),
                     parallel(left(6, 3, 24, 40, 0.2, 37, 5000.0, 16), right(3, 10, 14, 8.0), 0.7, 1.4, dense(120)),
                     latent(3, 20, 12, 28, 40, 0.15, 1000.0, dense(72)),
                     delta(2, 2, 16, 8, 2, dense(50))]},
    "B": {"architecture": "Salolorn", "vocab": 77, "width": 62, "norm": {"eps": 3e-6}, "logit_scale": 1.0,
          "layers": [latent(5, 6, 2, 10, 18, 0.4, 50.0),
                     parallel(left(4, 4, 10, 6, 0.3, 5, 300.0, 10), right(1, 46, 38, 1.0), 1.0, 0.5, dense(50)),
                     delta(3, 1, 6, 10, 1, dense(30))]},
    "C": {"architecture": "Salolorn", "vocab": 260, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 2.0,
          "loop": {"start": 0, "stop": 2, "times": 3},
          "layers": [parallel(left(8, 2, 64, 64, 0.1, 64, 1e6, 32), right(2, 64, 128, 4.0), 1.3, 0.9, dense(256)),
                     latent(8, 32, 16, 32, 128, 0.14, 1e4, dense(192)),
                     delta(4, 2, 64, 64, 4),
                     parallel(left(4, 1, 128, 96, 0.08, 200, 1e4, 128), right(4, 32, 64, 32.0), 0.8, 1.2, dense(128))]},
    "D": {"architecture": "Salolorn", "vocab": 53, "width": 48, "norm": {"eps": 2e-5}, "logit_scale": 0.3,
          "loop": {"start": 0, "stop": 2, "times": 1},
          "layers": [parallel(left(2, 1, 12, 20, 0.25, 100000, 100.0, 0), right(3, 8, 12, 2.5), 1.0, 1.0, dense(40)),
                     delta(6, 3, 8, 4, 5)]},
}


def one_layer(layer, width=64, vocab=53, loop=None):
    """A model of a single layer (for a mechanism alone)."""
    cfg = {"architecture": "Salolorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
           "layers": [layer]}
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

    out["embed"] = rnd(V, W, std=0.5)
    out["final.norm"] = rnd(W, std=0.1, mean=1.0)
    if cfg.get("loop"):
        out["loop.step"] = rnd(cfg["loop"]["times"], W, std=0.3)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        out[f"l{i}.norm1"] = rnd(W, std=0.1, mean=1.0)
        out[f"l{i}.norm1b"] = rnd(W, std=0.1, mean=0.8)
        if L["type"] == "delta":
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                out[p + n] = lin(rows, W, gain=1.5)
                out[p + n + ".conv"] = rnd(rows, taps, std=0.6)
            out[p + "b"], out[p + "a"] = lin(H, W, gain=2.0), lin(H, W, gain=2.0)
            out[p + "A_log"] = (3.0 * torch.rand(H, generator=g) - 2.5).to(torch.bfloat16)
            out[p + "dt_bias"] = rnd(H, std=1.0, mean=-1.0)
            out[p + "norm"] = rnd(dv, std=0.2, mean=1.2)
            out[p + "g"], out[p + "o"] = lin(H * dv, W, gain=2.0), lin(W, H * dv)
        elif L["type"] == "latent_attention":
            H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out[p + "q"] = lin(H * (d + dr), W, gain=2.0)
            out[p + "dkv"] = lin(rank + dr, W, gain=2.0)
            out[p + "dkv.norm"] = rnd(rank, std=0.2, mean=1.5)
            out[p + "uk"], out[p + "uv"] = lin(H * d, rank, gain=1.5), lin(H * dv, rank)
            out[p + "o"] = lin(W, H * dv)
        else:
            lf, rt = m["left"], m["right"]
            H, G, d, dv = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
            out[p + "left.q"], out[p + "left.k"] = lin(H * d, W, 1.5), lin(G * d, W, 1.5)
            out[p + "left.v"], out[p + "left.o"] = lin(G * dv, W), lin(W, H * dv)
            out[p + "left.q.norm"] = rnd(d, std=0.3, mean=2.0)
            out[p + "left.k.norm"] = rnd(d, std=0.3, mean=2.0)
            out[p + "left.sink"] = rnd(H, std=1.5, mean=0.5)
            out[p + "left.g"] = lin(H, W, gain=2.0)
            H2, d2, dv2 = rt["heads"], rt["dim"], rt["vdim"]
            out[p + "right.q"], out[p + "right.k"] = lin(H2 * d2, W, 1.5), lin(H2 * d2, W, 1.5)
            out[p + "right.v"], out[p + "right.g"] = lin(H2 * dv2, W), lin(H2 * dv2, W, 2.0)
            out[p + "right.o"] = lin(W, H2 * dv2)
            out[p + "right.norm"] = rnd(dv2, std=0.2, mean=1.2)
            r = 5 + i                                           # the bottleneck's width is the tensors' own
            out[p + "right.a1"], out[p + "right.a2"] = lin(r, W, 1.5), lin(H2 * d2, r, 2.0)
            out[p + "right.a2.b"] = rnd(H2 * d2, std=1.5, mean=2.0)
        mlp = L["mlp"]
        if mlp is None:
            continue
        out[f"l{i}.norm2"] = rnd(W, std=0.1, mean=1.0)
        out[f"l{i}.norm2b"] = rnd(W, std=0.1, mean=0.9)
        ff = mlp["ff"]
        out[f"l{i}.mlp.gate"], out[f"l{i}.mlp.up"], out[f"l{i}.mlp.down"] = lin(ff, W, 1.5), lin(ff, W, 1.5), lin(W, ff, 1.5)
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
    g = torch.Generator().manual_seed(7000 + seed)
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


def references(oracle, reqs, dtype):
    """Per request the exact logits and a limit for every position: TOL, or in bfloat16 three times the error that
    rounding alone causes (the plain model with bfloat16 where an engine must round) where that is more.  Rounding
    error at one position is a draw from a distribution (a norm behind a small mixer output magnifies it at some
    positions and not at others, and an engine that rounds in other places draws other ones), so the error that
    rounding causes at a position is taken as the larger of the rounded run's error there and its root mean square
    over the request."""
    import plain_salolorn as plain
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    lim = {rid: torch.full((len(t),), TOL[dtype], dtype=torch.float64) for rid, t in reqs.items()}
    if dtype == "bfloat16":
        rounded = plain.PlainSalolorn(oracle.cfg, oracle.t, rounded=True)
        for rid, t in reqs.items():
            err = row_error(rounded.forward(t), ref[rid])
            err = torch.maximum(err, torch.sqrt((err * err).mean()))
            lim[rid] = torch.maximum(lim[rid], 3.0 * err)
    return ref, lim


def worst_ratio(got, ref, lim):
    """Largest error / limit over the rows ``{(request, position): logits}``."""
    return max(float(row_error(row, ref[rid][p]) / lim[rid][p]) for (rid, p), row in got.items())


def within_limits(got, ref, lim):
    """A limit made from one rounded run is itself a noisy number, so a few rows may pass it by a little: no row is
    beyond one and a half times its limit and at most one in fifty is beyond it."""
    ratios = [float(row_error(row, ref[rid][p]) / lim[rid][p]) for (rid, p), row in got.items()]
    return max(ratios) < 1.5 and sum(r > 1.0 for r in ratios) <= len(ratios) // 50
