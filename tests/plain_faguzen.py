"""A plain, slow statement of the Faguzen design in PyTorch, one function per mechanism.

It shares no code with the package: it reads ``config.json`` as a dict and the
tensors by their stored names, walks the recurrence token by token, and keeps
nothing between calls.  Everything is computed in ``dtype`` (float64 by default)
from the weights as they are stored.  With ``rounded=True`` whatever a 16-bit
engine hands to a matrix product or keeps in its cache is rounded to bfloat16
first.

Notation: ``h`` is a sublayer's input ``[T, width]``; ``p(name)`` gives a tensor of
the current layer's mixer or feed-forward; positions count from 0.
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ small pieces
def as_stored(x, rounded):
    return x.to(torch.bfloat16).to(x.dtype) if rounded else x


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def log_sigmoid(z):
    """ln(1 / (1 + e^-z)) without overflow on either side."""
    return torch.minimum(z, torch.zeros_like(z)) - torch.log1p(torch.exp(-z.abs()))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def tanh_cap(z, cap):
    """cap * tanh(z / cap); ``cap`` None or 0: z itself."""
    return cap * torch.tanh(z / cap) if cap else z


def dynamic_tanh(x, w, b, alpha):
    """A norm without statistics: tanh(alpha x) w + b, entry by entry."""
    return torch.tanh(alpha * x) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scaled_frequencies(base, dims, scaling):
    """f_i = base^(-2i / dims), i < dims / 2, in 64-bit; with ``scaling`` (factor, low, high, original) long waves
    are slowed: wavelength L = 2 pi / f; L < original / high keeps f; L > original / low gives f / factor; between
    them s = (original / L - low) / (high - low) blends (1 - s) f / factor + s f."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return torch.tensor(f, dtype=torch.float64)
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for x in f:
        wave = 2.0 * math.pi / x
        if wave < orig / high:
            out.append(x)
        elif wave > orig / low:
            out.append(x / factor)
        else:
            s = (orig / wave - low) / (high - low)
            out.append((1.0 - s) * x / factor + s * x)
    return torch.tensor(out, dtype=torch.float64)


def rotate_halves(x, positions, freqs, dims):
    """First ``dims`` entries of the last dimension, entry i with entry i + dims / 2.  x: [T, heads, D]."""
    if dims == 0:
        return x
    half = dims // 2
    a = (positions.to(x.dtype)[:, None] * freqs.to(x.dtype)[None, :])[:, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------ mixers
def capped_gated_attention(h, p, m, rounded=False):
    """Grouped-query softmax attention over all earlier positions with biases, a rotation over part of each head,
    scores squashed by a tanh and an output gate per entry."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    hh = as_stored(h, rounded)
    q = (hh @ p("q").T + p("q.b")).reshape(T, H, d)
    k = (hh @ p("k").T + p("k.b")).reshape(T, G, d)
    v = as_stored((hh @ p("v").T + p("v.b")).reshape(T, G, dv), rounded)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        f = scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q, k = (rotate_halves(x, pos, f, rot["dims"]) for x in (q, k))
    q, k = as_stored(q, rounded), as_stored(k, rounded)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    scores = tanh_cap(torch.einsum("ihd,jhd->hij", q, k) * m["scale"], m.get("softcap"))
    visible = pos[None, :] <= pos[:, None]
    w = torch.softmax(scores.masked_fill(~visible[None], float("-inf")), dim=-1)
    o = torch.einsum("hij,jhv->ihv", w, v).reshape(T, H * dv)
    o = o * sigmoid(hh @ p("g").T)
    return as_stored(o, rounded) @ p("o").T + p("o.b")


def matrix_memory(h, p, m, eps, rounded=False, state=None):
    """A matrix memory per head with exponential input gates, kept in range by a running maximum of the log gates.
    ``state`` (S, n, mx) continues an earlier call; the new one is returned beside the output."""
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    T = h.shape[0]
    hh = as_stored(h, rounded)
    q = (hh @ p("q").T).reshape(T, H, d) * d ** -0.5
    k = (hh @ p("k").T).reshape(T, H, d)
    v = (hh @ p("v").T).reshape(T, H, dv)
    li = tanh_cap(hh @ p("i").T + p("i.b"), cap)                              # log input gate [T, H]
    lf = log_sigmoid(tanh_cap(hh @ p("f").T + p("f.b"), cap))                 # log forget gate
    if state is None:
        S = torch.zeros(H, d, dv, dtype=h.dtype)
        n = torch.zeros(H, d, dtype=h.dtype)
        mx = torch.zeros(H, dtype=h.dtype)
    else:
        S, n, mx = (x.clone() for x in state)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        new = torch.maximum(lf[t] + mx, li[t])
        keep, put = torch.exp(lf[t] + mx - new), torch.exp(li[t] - new)
        S = keep[:, None, None] * S + put[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + put[:, None] * k[t]
        mx = new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    y = unit_rms(o, eps).reshape(T, H * dv) * p("norm") * sigmoid(hh @ p("g").T)
    return as_stored(y, rounded) @ p("o").T, (S, n, mx)


def parallel_mixer(h, p, m, eps, rounded=False):
    left = capped_gated_attention(h, lambda n: p("left." + n), m["left"], rounded)
    right, _ = matrix_memory(h, lambda n: p("right." + n), m["right"], eps, rounded)
    return m["left_scale"] * left + m["right_scale"] * right


# ------------------------------------------------------------------ feed-forward
def two_matrix_expert(hh, up, down, rounded):
    return as_stored(gelu_erf(hh @ up.T), rounded) @ down.T


def route(h, p, mlp):
    """Chosen experts ``[T, top]`` and their weights.  Scores are a softmax over every expert (identity experts
    too); the choice looks at score + correction, the weights at the scores alone, divided by their sum."""
    top = mlp["router"]["top"]
    s = torch.softmax(h @ p("router").T, dim=-1)
    pick = torch.sort(s + p("correction"), dim=-1, descending=True, stable=True)
    ids = pick.indices[:, :top]
    w = torch.gather(s, 1, ids)
    # how clear the choice was: the last chosen expert's lead over the first one left out
    gap = pick.values[:, top - 1] - pick.values[:, top] if top < s.shape[1] else torch.full_like(s[:, 0], math.inf)
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20), gap


def expert_mixture(h, p, mlp, rounded=False, gaps=None):
    """Routed two-matrix experts, of which the last ``identity`` hand their input through, plus a shared expert."""
    E, ident = mlp["router"]["experts"], mlp["router"].get("identity", 0)
    hh = as_stored(h, rounded)
    ids, w, gap = route(h, p, mlp)
    if gaps is not None:
        gaps.append(gap)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), w[t]):
            if e >= E:
                assert e < E + ident
                out[t] += g * h[t]
            else:
                out[t] += g * two_matrix_expert(hh[t:t + 1], p(f"e{e}.up"), p(f"e{e}.down"), rounded)[0]
    if mlp.get("shared"):
        out = out + two_matrix_expert(hh, p("shared.up"), p("shared.down"), rounded)
    return out


# ------------------------------------------------------------------------- model
def layer_runs(cfg):
    """(layer, pass it opens or None) for every layer run, in order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for r in range(loop["times"]):
        runs += [(i, r if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


class PlainFaguzen:
    """``tensors``: name -> tensor as stored.  ``forward(tokens)`` gives logits at every position and, with
    ``trace=True``, also the residual after every layer run; ``last_gaps`` then holds, per position, how clear the
    least clear choice of experts was."""

    def __init__(self, config: dict, tensors: dict, dtype=torch.float64, rounded=False):
        self.cfg, self.dtype, self.rounded = config, dtype, rounded
        self.t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self._gaps, self.last_gaps = [], None

    def norm(self, name, x):
        t = self.t
        return dynamic_tanh(x, t[name], t[name + ".b"], t[name + ".alpha"])

    def layer(self, i, x):
        cfg, t = self.cfg, self.t
        spec = cfg["layers"][i]
        assert spec["type"] == "parallel"
        y = parallel_mixer(self.norm(f"l{i}.norm1", x), lambda n: t[f"l{i}.mix.{n}"], spec["mixer"],
                           cfg["norm"]["eps"], self.rounded)
        if spec.get("mlp") is not None:
            assert spec["mlp"]["kind"] == "moe"
            y = y + expert_mixture(self.norm(f"l{i}.norm2", x), lambda n: t[f"l{i}.mlp.{n}"], spec["mlp"], self.rounded,
                                   self._gaps)
        return x + cfg.get("residual_mult", 1.0) * y

    def forward(self, tokens, trace=False):
        cfg, t = self.cfg, self.t
        x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)].clone()
        after = []
        self._gaps = []
        for i, opens in layer_runs(cfg):
            if opens is not None:
                x = x + t["loop.step"][opens]
            x = self.layer(i, x)
            after.append(x)
        # per position, the least clear choice of experts over all layer runs
        self.last_gaps = torch.stack(self._gaps).min(0).values if self._gaps else torch.full((x.shape[0],), math.inf,
                                                                                              dtype=self.dtype)
        y = as_stored(self.norm("final.norm", x), self.rounded)
        logits = tanh_cap(y @ t["head"].T, cfg.get("logit_softcap"))
        return (logits, torch.stack(after)) if trace else logits
