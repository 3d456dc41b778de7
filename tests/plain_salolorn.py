"""A plain, slow statement of the Salolorn design in PyTorch, one function per mechanism.

It shares no code with the package: it reads ``config.json`` as a dict and the
tensors by their stored names, walks recurrences token by token, and keeps nothing
between calls.  Everything is computed in ``dtype`` (float64 by default) from the
weights as they are stored.  With ``rounded=True`` whatever a 16-bit engine hands
to a matrix product or keeps in its cache is rounded to bfloat16 first.

Notation: ``h`` is a sublayer's input ``[T, width]``; ``p(name)`` gives a tensor of
the current layer's mixer or feed-forward; positions count from 0.
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ small pieces
def as_stored(x, rounded):
    return x.to(torch.bfloat16).to(x.dtype) if rounded else x


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_conv(x, w):
    """``out[t, c] = sum_j w[c, j] * x[t - taps + 1 + j, c]``, zeros before the start, no bias."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += x[:T - back] * w[:, j]
    return out


def rotation_angles(positions, base, dims, dtype):
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = (float(base) ** (-2.0 * i / dims)).to(dtype)
    return (positions.to(dtype)[:, None] * f[None, :])[:, None, :]          # [T, 1, dims/2]


def rotate_halves(x, positions, base, dims):
    """First ``dims`` entries of the last dimension: entry i with entry i + dims/2.  x: [T, heads, D]."""
    if dims == 0:
        return x
    half = dims // 2
    a = rotation_angles(positions, base, dims, x.dtype)
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def rotate_neighbours(x, positions, base, dims):
    """First ``dims`` entries of the last dimension: entry 2i with entry 2i + 1.  x: [T, heads, D]."""
    if dims == 0:
        return x
    a = rotation_angles(positions, base, dims, x.dtype)
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    rot = torch.stack([u * c - v * s, v * c + u * s], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([rot, x[..., dims:]], dim=-1)


def masked_softmax_mix(scores, visible, values, sink=None):
    """``scores [H, T, T]`` (query, key), ``visible [T, T]`` bool, ``values [H, T, dv]``.  With ``sink [H]`` the
    denominator also holds exp(sink) (no key, no value)."""
    s = scores.masked_fill(~visible[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None].expand_as(m))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return (e / den) @ values


# ------------------------------------------------------------------------ mixers
def delta_mixer(h, p, m, eps, rounded=False):
    """Gated delta rule with one decay per head."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    hh = as_stored(h, rounded)
    q = silu(short_conv(hh @ p("q").T, p("q.conv"))).reshape(T, G, d)
    k = silu(short_conv(hh @ p("k").T, p("k.conv"))).reshape(T, G, d)
    v = silu(short_conv(hh @ p("v").T, p("v.conv"))).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigmoid(hh @ p("b").T)                                            # [T, H]
    g = torch.exp(-torch.exp(p("A_log")) * softplus(hh @ p("a").T + p("dt_bias")))   # [T, H]
    gate = silu(hh @ p("g").T).reshape(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for n in range(H):
            kk, qq = k[t, n // (H // G)], q[t, n // (H // G)]
            S[n] = g[t, n] * S[n]
            u = beta[t, n] * (v[t, n] - S[n].T @ kk)
            S[n] = S[n] + torch.outer(kk, u)
            o[t, n] = S[n].T @ qq
    y = unit_rms(o, eps) * p("norm") * gate
    return as_stored(y.reshape(T, H * dv), rounded) @ p("o").T


def latent_attention(h, p, m, eps, rounded=False):
    """Attention whose keys and values are projections of one cached latent per token."""
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base = m["rot"]["base"]
    T = h.shape[0]
    pos = torch.arange(T)
    hh = as_stored(h, rounded)
    q = (hh @ p("q").T).reshape(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_neighbours(q[..., d:], pos, base, dr)
    low = hh @ p("dkv").T
    c = as_stored(rms_norm(low[:, :rank], p("dkv.norm"), eps), rounded)
    k_rot = as_stored(rotate_neighbours(low[:, None, rank:], pos, base, dr)[:, 0], rounded)
    k_plain = (c @ p("uk").T).reshape(T, H, d)
    v = (c @ p("uv").T).reshape(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    visible = pos[None, :] <= pos[:, None]
    o = masked_softmax_mix(scores, visible, v.transpose(0, 1)).transpose(0, 1)
    return as_stored(o.reshape(T, H * dv), rounded) @ p("o").T


def chunked_sink_attention(h, p, m, eps, rounded=False):
    """Grouped-query attention inside chunks of positions, with per-head norms of queries and keys, a sink in the
    softmax and an output gate per head."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    hh = as_stored(h, rounded)
    q = rms_norm((hh @ p("q").T).reshape(T, H, d), p("q.norm"), eps)
    k = rms_norm((hh @ p("k").T).reshape(T, G, d), p("k.norm"), eps)
    v = as_stored((hh @ p("v").T).reshape(T, G, dv), rounded)
    rot = m.get("rot")
    if rot:
        q, k = (rotate_halves(x, pos, rot["base"], rot["dims"]) for x in (q, k))
    q, k = as_stored(q, rounded), as_stored(k, rounded)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    size = m["mask"]["size"]
    visible = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    o = masked_softmax_mix(scores, visible, v.transpose(0, 1), sink=p("sink")).transpose(0, 1)     # [T, H, dv]
    o = o * sigmoid(hh @ p("g").T)[:, :, None]
    return as_stored(o.reshape(T, H * dv), rounded) @ p("o").T


def gated_linear_attention(h, p, m, eps, rounded=False):
    """Linear attention whose state decays per key channel by a data-dependent factor."""
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    hh = as_stored(h, rounded)
    q = (hh @ p("q").T).reshape(T, H, d) * d ** -0.5
    k = (hh @ p("k").T).reshape(T, H, d)
    v = (hh @ p("v").T).reshape(T, H, dv)
    z = as_stored(hh @ p("a1").T, rounded) @ p("a2").T + p("a2.b")
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, d)
    gate = silu(hh @ p("g").T)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = (rms_norm(o, p("norm"), eps)).reshape(T, H * dv) * gate
    return as_stored(y, rounded) @ p("o").T


def parallel_mixer(h, p, m, eps, rounded=False):
    left = chunked_sink_attention(h, lambda n: p("left." + n), m["left"], eps, rounded)
    right = gated_linear_attention(h, lambda n: p("right." + n), m["right"], eps, rounded)
    return m["left_scale"] * left + m["right_scale"] * right


def dense_ff(h, p, rounded=False):
    hh = as_stored(h, rounded)
    return as_stored(silu(hh @ p("gate").T) * (hh @ p("up").T), rounded) @ p("down").T


MIXERS = {"delta": delta_mixer, "latent_attention": latent_attention, "parallel": parallel_mixer}


# ------------------------------------------------------------------------- model
class PlainSalolorn:
    """``tensors``: name -> tensor as stored.  ``forward(tokens)`` gives logits at every position and, with
    ``trace=True``, also the residual after every layer run."""

    def __init__(self, config: dict, tensors: dict, dtype=torch.float64, rounded=False):
        self.cfg, self.dtype, self.rounded = config, dtype, rounded
        self.t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}

    def layer(self, i, x):
        cfg, eps = self.cfg, self.cfg["norm"]["eps"]
        spec = cfg["layers"][i]
        t = self.t
        mix = MIXERS[spec["type"]](rms_norm(x, t[f"l{i}.norm1"], eps), lambda n: t[f"l{i}.mix.{n}"], spec["mixer"], eps,
                                   self.rounded)
        x = x + rms_norm(mix, t[f"l{i}.norm1b"], eps)
        if spec.get("mlp") is not None:
            ff = dense_ff(rms_norm(x, t[f"l{i}.norm2"], eps), lambda n: t[f"l{i}.mlp.{n}"], self.rounded)
            x = x + rms_norm(ff, t[f"l{i}.norm2b"], eps)
        return x

    def forward(self, tokens, trace=False):
        cfg, t = self.cfg, self.t
        x0 = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        x = x0.clone()
        n = len(cfg["layers"])
        loop = cfg.get("loop")
        runs = []
        if loop:
            runs += [(i, None) for i in range(loop["start"])]
            for r in range(loop["times"]):
                runs += [(i, r if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
            runs += [(i, None) for i in range(loop["stop"], n)]
        else:
            runs = [(i, None) for i in range(n)]
        after = []
        for i, opens in runs:
            if opens is not None:
                if opens > 0:
                    x = x + x0
                x = x + t["loop.step"][opens]
            x = self.layer(i, x)
            after.append(x)
        y = as_stored(rms_norm(x, t["final.norm"], cfg["norm"]["eps"]), self.rounded)
        logits = (y @ t["embed"].T) * cfg.get("logit_scale", 1.0)
        return (logits, torch.stack(after)) if trace else logits
