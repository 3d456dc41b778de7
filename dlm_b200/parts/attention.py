"""Attention mixers."""
from __future__ import annotations

import math

import torch

from ..registry import build_part, register_part
from .base import CacheTensor, Mixer, PagedCache, PagedKV, ParamSpec, PartSpec, Runtime, StepContext
from .rope import rope_inv_freqs


class GroupedQueryAttention(Mixer):
    """Softmax attention over paged keys and values with grouped query heads
    (src/forward/cpu.rs:1171-1193, 1126-1151): q/k/v projections (bias optional, added
    before the rotation), position encoding on q and k, keys stored rotated, query head h
    reads kv head ``h // (heads / kv_heads)``, scores scaled by ``1/sqrt(head_dim)``,
    output projection without bias added to the residual.  With ``window`` W a query at
    position p sees key j iff ``j <= p`` and ``p - j < W``.

    The three projections are concatenated at load into one ``[Q + 2KV, hidden]`` matrix.
    """

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool | None = None, window: int | None = None,
                 position: PartSpec | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.qkv_bias = qkv_bias          # None: decided by the presence of the bias tensors
        self.window = int(window) if window else None
        self.position = build_part("position", position) if position is not None else None
        self.q_dim, self.kv_dim = self.nh * self.hd, self.nkv * self.hd
        self.scale = 1.0 / math.sqrt(self.hd)
        self.w_qkv = self.b_qkv = self.w_o = None

    def param_specs(self):
        opt = self.qkv_bias is None
        specs = [ParamSpec("q_proj.weight", (self.q_dim, self.hidden)),
                 ParamSpec("k_proj.weight", (self.kv_dim, self.hidden)),
                 ParamSpec("v_proj.weight", (self.kv_dim, self.hidden)),
                 ParamSpec("o_proj.weight", (self.hidden, self.q_dim))]
        if self.qkv_bias is not False:
            specs += [ParamSpec("q_proj.bias", (self.q_dim,), init="bias", optional=opt),
                      ParamSpec("k_proj.bias", (self.kv_dim,), init="bias", optional=opt),
                      ParamSpec("v_proj.bias", (self.kv_dim,), init="bias", optional=opt)]
        return specs

    def load(self, tensors, rt: Runtime):
        self.w_qkv = torch.cat([rt.matrix(tensors[f"{n}_proj.weight"]) for n in "qkv"], dim=0).contiguous()
        self.w_o = rt.matrix(tensors["o_proj.weight"])
        have = [f"{n}_proj.bias" in tensors for n in "qkv"]
        if any(have):
            parts = []
            for n, size in zip("qkv", (self.q_dim, self.kv_dim, self.kv_dim)):
                key = f"{n}_proj.bias"
                parts.append(rt.vector(tensors[key]) if key in tensors
                             else torch.zeros(size, dtype=torch.float32, device=rt.device))
            self.b_qkv = torch.cat(parts).contiguous()
        else:
            self.b_qkv = None
        if self.position is not None:
            self.position.rotary(rt)        # the table is made now: no copy from the host in the middle of a step

    def cache_need(self):
        return PagedKV(self.nkv, self.hd, self.window)

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        view = ctx.paged(call)
        qkv = ops.linear(h, self.w_qkv, self.b_qkv, torch.float32)
        rot = self.position.rotary(rt) if self.position is not None else None
        inv_freq, rotary_dim = rot if rot is not None else (None, 0)
        q = ops.rope_kv_write(qkv, b.positions, inv_freq, rotary_dim,
                              view.group.slots if view.write else None,
                              view.k, view.v, self.nh, self.nkv, self.hd, rt.dtype,
                              interleaved=bool(rot is not None and self.position.interleaved))
        o = ops.attention(q, view.k, view.v, view.group.block_table, b.cu_q, b.kv_len,
                          self.window or 0, self.scale, self.nh, self.nkv, self.hd,
                          b.max_q_len, b.max_kv_len, b.num_single)
        ops.linear_add(o, self.w_o, resid)


class LatentAttention(Mixer):
    """Softmax attention whose keys and values are projections of one cached latent per token.

    ``c_q = rmsnorm(W_dq h)``, ``q = W_uq c_q`` laid out per head ``[dim plain | rot_dim rotated]``;
    ``W_dkv h = [c_raw: kv_rank | k_rot: rot_dim]``, ``c = rmsnorm(c_raw)``; head n has key ``[W_uk,n c | k_rot]``
    (the rotated part is shared by all heads) and value ``W_uv,n c``; score ``= (q . key) * scale``.  The
    rotation acts on the first ``rope_dims`` entries of the rotated parts of q and k, pairs ``(i, i + rope_dims / 2)``,
    angle ``position * base^(-2i / rope_dims)``.  A query at p sees keys j with ``0 <= p - j < window`` (None:
    all).  The softmax's denominator also holds ``exp(sink_n)``, a learned logit per head without key or value.
    Head n's output is multiplied by ``sigmoid(W_g h)_n``; then ``W_o``.

    ``q_rank`` None: there is no query latent and ``q = W_q h`` (tensor ``q``).  ``interleaved``: the rotation
    pairs entries ``(2i, 2i + 1)`` instead.

    Only ``[c | rotated k_rot]`` is cached (one paged tensor, ``kv_rank + rot_dim`` wide).  The kernels work on
    the latent: ``q' = W_uk,n^T q_plain`` meets c directly and the weighted sum of latents goes through
    ``W_uv,n`` at the end, so neither keys nor values of a head are ever built.  Both per-head products are one
    grouped matrix product each, with the heads as groups (``latent_attend``)."""

    def __init__(self, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 q_rank: int | None, eps: float, rope_base: float, rope_dims: int | None = None,
                 window: int | None = None, scale: float | None = None, sink: bool = True, gate: bool = True,
                 interleaved: bool = False):
        self.hidden, self.H, self.dn, self.dr, self.dv = int(hidden_size), int(heads), int(dim), int(rot_dim), int(vdim)
        self.rank, self.q_rank, self.eps = int(kv_rank), int(q_rank) if q_rank else 0, float(eps)
        self.interleaved = bool(interleaved)
        self.rope_base = float(rope_base)
        self.rope_dims = int(rope_dims) if rope_dims is not None else self.dr
        if self.rope_dims % 2 or not (0 <= self.rope_dims <= self.dr):
            raise ValueError(f"rope_dims must be even and at most rot_dim, got {self.rope_dims}")
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.dn + self.dr)
        self.has_sink, self.has_gate = bool(sink), bool(gate)
        self.w_in = self.w_uq = self.w_uk = self.w_uv = self.w_o = None
        self.qn = self.kvn = self.sink = self._freq = None

    def param_specs(self):
        H, dn, dr, dv = self.H, self.dn, self.dr, self.dv
        if self.q_rank:
            specs = [ParamSpec("dq", (self.q_rank, self.hidden)), ParamSpec("dq.norm", (self.q_rank,), init="norm"),
                     ParamSpec("uq", (H * (dn + dr), self.q_rank))]
        else:
            specs = [ParamSpec("q", (H * (dn + dr), self.hidden))]
        specs += [ParamSpec("dkv", (self.rank + dr, self.hidden)), ParamSpec("dkv.norm", (self.rank,), init="norm"),
                 ParamSpec("uk", (H * dn, self.rank)), ParamSpec("uv", (H * dv, self.rank)),
                 ParamSpec("o", (self.hidden, H * dv))]
        if self.has_sink:
            specs.append(ParamSpec("sink", (H,), init="bias"))
        if self.has_gate:
            specs.append(ParamSpec("g", (H, self.hidden)))
        return specs

    def load(self, tensors, rt: Runtime):
        # rows [query latent, or the queries themselves | key/value latent and rotated key part | gate]
        rows = [rt.matrix(tensors["dq" if self.q_rank else "q"]), rt.matrix(tensors["dkv"])]
        if self.has_gate:
            rows.append(rt.matrix(tensors["g"]))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_uq = rt.matrix(tensors["uq"]) if self.q_rank else None
        # per head: W_uk transposed ([rank, dim]: the product's rows are latent entries) and W_uv as it is
        self.w_ukT = rt.matrix(tensors["uk"]).reshape(self.H, self.dn, self.rank).transpose(1, 2).contiguous()
        self.w_uv = rt.matrix(tensors["uv"]).reshape(self.H, self.dv, self.rank).contiguous()
        self.w_o = rt.matrix(tensors["o"])
        self.qn = rt.vector(tensors["dq.norm"]) if self.q_rank else None
        self.kvn = rt.vector(tensors["dkv.norm"])
        self.sink = rt.vector(tensors["sink"]) if self.has_sink else None
        self._freq = rope_inv_freqs(self.rope_dims, self.rope_base, self.rope_dims).to(rt.device) \
            if self.rope_dims else torch.zeros(1, device=rt.device)

    def cache_need(self):
        return PagedCache((CacheTensor("latent", 1, self.rank + self.dr),), self.window)

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        view = ctx.paged(call)
        cache = view.tensors["latent"]
        proj = ops.linear(h, self.w_in, None, torch.float32)
        q_cols = self.q_rank or self.H * (self.dn + self.dr)
        cq = ops.latent_prep(proj, 0, self.q_rank, self.qn, q_cols, self.rank, self.kvn, self.dr, self._freq,
                             self.rope_dims, b.positions, view.group.slots if view.write else None, self.eps, cache,
                             rt.dtype, interleaved=self.interleaved)
        q = ops.linear(cq, self.w_uq, None, torch.float32) if self.q_rank else proj[:, :q_cols]
        gate = proj[:, q_cols + self.rank + self.dr:] if self.has_gate else None
        o = latent_attend(ops, q, gate, self.w_ukT, self.w_uv, self.sink, cache, view.group.block_table, b, self._freq,
                          self.rope_dims, self.window or 0, self.scale, interleaved=self.interleaved)
        ops.linear_add(o, self.w_o, resid)


def latent_attend(ops, q, gate, w_ukT, w_uv, sink, cache, block_table, batch, inv_freq, rot_dims, window, scale,
                  interleaved=False):
    """From projected queries to gated head outputs ``[T, H * vdim]`` over a cache of latents ``[c | k_rot]``.
    ``q [T, H * (dim + rot_dim)]`` 32-bit, ``gate [T, H]`` raw or None, ``w_ukT [H, rank, dim]``,
    ``w_uv [H, vdim, rank]``: split and rotate the queries; take the plain parts through W_uk (a grouped product,
    heads as groups); attend over the latent rows; take the weighted latents through W_uv (grouped again); gate."""
    H, rank, dn = w_ukT.shape
    dv = w_uv.shape[1]
    T = q.shape[0]
    dr = q.shape[1] // H - dn
    qn, q_rot = ops.latent_q_split(q, batch.positions, inv_freq, rot_dims, H, dn, dr, cache.dtype,
                                   interleaved=interleaved)
    offsets = ops.head_offsets(H, T, q.device)
    q_lat = ops.grouped_linear(qn.reshape(H * T, dn), w_ukT, offsets).reshape(H, T, rank)
    lat = ops.latent_attention(q_lat, q_rot, sink, cache, block_table, batch, H, dr, rank, window, scale)
    val = ops.grouped_linear(lat.reshape(H * T, rank), w_uv, offsets)
    return ops.latent_gate_out(val, gate, H, dv, cache.dtype)


class NormedBiasedAttention(Mixer):
    """Softmax attention without rotation whose positions enter through a distance penalty and a query temperature.

    ``q, k, v = W h (+ bias)`` with ``heads`` query heads and ``kv_heads`` key/value heads (query head n reads
    key/value head ``n // (heads / kv_heads)``), keys ``dim`` wide, values ``vdim`` wide.  With ``qk_norm`` the whole
    query projection (all heads at once) is divided by its root mean square and multiplied by ``q.norm``; the key
    projection likewise with ``k.norm``.  The query at position p is multiplied by
    ``1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)`` (``temp_every`` None: no temperature).  A score is
    ``(q . k) * scale - slope_n * (p - j)`` with ``slope_n = 2^(-slope_bits (n + 1) / heads)`` (``slope_bits`` None:
    no penalty); position p sees every ``j <= p`` (the last ``window`` of them when that is given); plain softmax;
    ``W_o`` on the heads side by side.

    Keys and values are cached with one head size ``max(dim, vdim)`` rounded up to a size the tensor-core kernels
    take; entries beyond a head's own size are zeros, which change neither scores nor outputs, and ``W_o`` gets
    zero columns for them at load."""

    _HEAD_SIZES = (16, 32, 48, 64, 96, 128)

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float,
                 qkv_bias: bool = True, qk_norm: bool = True, temp_coef: float = 0.0, temp_every: int | None = None,
                 slope_bits: float | None = 8.0, window: int | None = None):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.hidden, self.H, self.G, self.d, self.dv = int(hidden_size), int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.eps = float(scale), float(eps)
        self.qkv_bias, self.qk_norm = bool(qkv_bias), bool(qk_norm)
        self.temp_coef = float(temp_coef)
        self.temp_every = int(temp_every) if temp_every else 0
        self.slope_bits = None if slope_bits is None else float(slope_bits)
        self.window = int(window) if window else None
        need = max(self.d, self.dv)
        self.D = next((s for s in self._HEAD_SIZES if s >= need), -(-need // 8) * 8)
        self.w_qkv = self.b_qkv = self.w_o = self.qn = self.kn = self.slopes = None

    def param_specs(self):
        H, G, d, dv = self.H, self.G, self.d, self.dv
        specs = [ParamSpec("q", (H * d, self.hidden)), ParamSpec("k", (G * d, self.hidden)),
                 ParamSpec("v", (G * dv, self.hidden)), ParamSpec("o", (self.hidden, H * dv))]
        if self.qkv_bias:
            specs += [ParamSpec("q.b", (H * d,), init="bias"), ParamSpec("k.b", (G * d,), init="bias"),
                      ParamSpec("v.b", (G * dv,), init="bias")]
        if self.qk_norm:
            specs += [ParamSpec("q.norm", (H * d,), init="norm"), ParamSpec("k.norm", (G * d,), init="norm")]
        return specs

    def load(self, tensors, rt: Runtime):
        self.w_qkv = torch.cat([rt.matrix(tensors[n]) for n in "qkv"], dim=0).contiguous()
        self.b_qkv = torch.cat([rt.vector(tensors[n + ".b"]) for n in "qkv"]).contiguous() if self.qkv_bias else None
        w_o = rt.matrix(tensors["o"])
        if self.D != self.dv:       # zero columns where the stored heads are wider than the values
            wide = torch.zeros((self.hidden, self.H, self.D), dtype=w_o.dtype, device=w_o.device)
            wide[:, :, :self.dv] = w_o.reshape(self.hidden, self.H, self.dv)
            w_o = wide.reshape(self.hidden, self.H * self.D).contiguous()
        self.w_o = w_o
        if self.qk_norm:
            self.qn, self.kn = rt.vector(tensors["q.norm"]), rt.vector(tensors["k.norm"])
        if self.slope_bits is not None:
            self.slopes = torch.tensor([2.0 ** (-self.slope_bits * (n + 1) / self.H) for n in range(self.H)],
                                       dtype=torch.float64).to(torch.float32).to(rt.device)

    def cache_need(self):
        return PagedKV(self.G, self.D, self.window)

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        view = ctx.paged(call)
        qkv = ops.linear(h, self.w_qkv, self.b_qkv, torch.float32)
        q = ops.qk_norm_write(qkv, b.positions, self.qn, self.kn, self.eps, self.temp_coef, self.temp_every,
                              view.group.slots if view.write else None, view.k, view.v, self.H, self.G, self.d, self.dv,
                              self.D, rt.dtype)
        o = ops.attention(q, view.k, view.v, view.group.block_table, b.cu_q, b.kv_len, self.window or 0, self.scale,
                          self.H, self.G, self.D, b.max_q_len, b.max_kv_len, b.num_single, slopes=self.slopes)
        ops.linear_add(o, self.w_o, resid)


class HeadNormedAttention(Mixer):
    """Grouped-query softmax attention with a norm per head, a choice of masks, an optional sink and an optional gate.

    ``q, k, v = W h`` (with ``qkv_bias`` plus the biases ``q.b``, ``k.b``, ``v.b``, added in the projection) with
    ``heads`` query heads and ``kv_heads`` key/value heads (query head n reads key/value head
    ``n // (heads / kv_heads)``), keys ``dim`` wide, values ``vdim`` wide.  With ``qk_norm`` every query
    head is divided by its root mean square over ``dim`` and multiplied by ``q.norm`` (``[dim]``, the same for all
    heads), every key head likewise with ``k.norm``; then the rotation (``position``: any registered rotary encoding;
    its table, how many entries it turns and how it pairs them are the encoding's).  A score is ``(q . k) * scale``,
    and with ``softcap`` c then ``c tanh(score / c)``.
    A query at p sees key ``j <= p`` iff ``p - j < window`` (when a window is given) and
    ``floor(j / chunk) == floor(p / chunk)`` (when a chunk size is given; chunks are counted from position 0 of the
    request).  With ``sink`` the softmax's denominator also holds ``exp(sink_n)``, a learned logit per head that has
    no key and no value and is not scaled.  ``gate`` True or ``"head"``: head n's output is multiplied by
    ``sigmoid(W_g h)_n`` (``g`` is ``[heads, hidden]``); ``"entry"``: the heads side by side are multiplied entry by
    entry by ``sigmoid(W_g h)`` (``g`` is ``[heads * vdim, hidden]``).  The gate reads the same input as the
    projections.  The output is ``out_scale * (W_o [heads side by side] + o.b)`` (the bias with ``o_bias``).

    Keys and values are cached with one head size (the larger of ``dim`` and ``vdim``, rounded up to a size the
    tensor-core kernels take; zeros beyond a head's own, zero columns in ``W_o``).  A chunked mask never looks back
    further than ``chunk - 1`` positions, so its pages live in a windowed group of that length and go back to the
    pool as the chunks pass."""

    _HEAD_SIZES = (16, 32, 48, 64, 96, 128)

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float,
                 qk_norm: bool = True, position: PartSpec | None = None, window: int | None = None,
                 chunk: int | None = None, sink: bool = False, gate: bool | str = False, out_scale: float = 1.0,
                 qkv_bias: bool = False, o_bias: bool = False, softcap: float | None = None):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if gate not in (False, True, "head", "entry"):
            raise ValueError(f"gate must be False, True, 'head' or 'entry', got {gate!r}")
        self.hidden, self.H, self.G, self.d, self.dv = int(hidden_size), int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.eps, self.out_scale = float(scale), float(eps), float(out_scale)
        self.qk_norm, self.has_sink, self.has_gate = bool(qk_norm), bool(sink), bool(gate)
        self.gate_rows = self.H * self.dv if gate == "entry" else self.H          # rows of W_g
        self.qkv_bias, self.o_bias = bool(qkv_bias), bool(o_bias)
        self.softcap = float(softcap) if softcap else 0.0
        self.window = int(window) if window else None
        self.chunk = int(chunk) if chunk else None
        self.position = build_part("position", position) if position is not None else None
        need = max(self.d, self.dv)
        self.D = next((s for s in self._HEAD_SIZES if s >= need), -(-need // 8) * 8)
        self.w_in = self.b_in = self.w_o = self.b_o = self.qn = self.kn = self.sink = None

    def param_specs(self):
        H, G, d, dv = self.H, self.G, self.d, self.dv
        specs = [ParamSpec("q", (H * d, self.hidden)), ParamSpec("k", (G * d, self.hidden)),
                 ParamSpec("v", (G * dv, self.hidden)), ParamSpec("o", (self.hidden, H * dv))]
        if self.qkv_bias:
            specs += [ParamSpec("q.b", (H * d,), init="bias"), ParamSpec("k.b", (G * d,), init="bias"),
                      ParamSpec("v.b", (G * dv,), init="bias")]
        if self.o_bias:
            specs.append(ParamSpec("o.b", (self.hidden,), init="bias"))
        if self.qk_norm:
            specs += [ParamSpec("q.norm", (d,), init="norm"), ParamSpec("k.norm", (d,), init="norm")]
        if self.has_sink:
            specs.append(ParamSpec("sink", (H,), init="bias"))
        if self.has_gate:
            specs.append(ParamSpec("g", (self.gate_rows, self.hidden)))
        return specs

    def load(self, tensors, rt: Runtime):
        names = ("q", "k", "v", "g") if self.has_gate else ("q", "k", "v")
        self.w_in = torch.cat([rt.matrix(tensors[n]) for n in names], dim=0).contiguous()
        if self.qkv_bias:       # the gate has no bias: zeros for its rows
            parts = [rt.vector(tensors[n + ".b"]) for n in "qkv"]
            if self.has_gate:
                parts.append(torch.zeros(self.gate_rows, dtype=torch.float32, device=rt.device))
            self.b_in = torch.cat(parts).contiguous()
        w_o = tensors["o"].to(device=rt.device, dtype=torch.float32)
        if not self.has_gate and self.out_scale != 1.0:
            w_o = w_o * self.out_scale             # with a gate the factor rides on the gate instead
        if self.D != self.dv:       # zero columns where the stored heads are wider than the values
            wide = torch.zeros((self.hidden, self.H, self.D), dtype=w_o.dtype, device=w_o.device)
            wide[:, :, :self.dv] = w_o.reshape(self.hidden, self.H, self.dv)
            w_o = wide.reshape(self.hidden, self.H * self.D)
        self.w_o = rt.matrix(w_o)
        self.b_o = (rt.vector(tensors["o.b"]) * self.out_scale).contiguous() if self.o_bias else None
        if self.qk_norm:
            self.qn, self.kn = rt.vector(tensors["q.norm"]), rt.vector(tensors["k.norm"])
        self.sink = rt.vector(tensors["sink"]) if self.has_sink else None
        if self.position is not None:
            self.position.rotary(rt)        # the table is made now: no copy from the host in the middle of a step

    def _span(self):
        """How far back a query can see (None: to the start)."""
        spans = [s for s in (self.window, self.chunk) if s]
        return min(spans) if spans else None

    def cache_need(self):
        return PagedKV(self.G, self.D, self._span())

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        H, G, d, dv = self.H, self.G, self.d, self.dv
        view = ctx.paged(call)
        proj = ops.linear(h, self.w_in, self.b_in, torch.float32)          # [q | k | v | gate]
        rot = self.position.rotary(rt) if self.position is not None else None
        inv_freq, rot_dims = rot if rot is not None else (None, 0)
        q = ops.head_norm_rope_write(proj, b.positions, self.qn, self.kn, self.eps, inv_freq, rot_dims,
                                     bool(rot is not None and self.position.interleaved),
                                     view.group.slots if view.write else None, view.k, view.v, H, G, d, dv, self.D,
                                     rt.dtype)
        extra = {"softcap": self.softcap} if self.softcap else {}
        o = ops.attention(q, view.k, view.v, view.group.block_table, b.cu_q, b.kv_len, self.window or 0, self.scale,
                          H, G, self.D, b.max_q_len, b.max_kv_len, b.num_single, chunk=self.chunk or 0, sinks=self.sink,
                          **extra)
        bias = self.b_o                                # the output bias still to be added (None: none, or done)
        if self.has_gate:
            g = proj[:, (H + G) * d + G * dv:]
            if self.gate_rows == H:
                ops.head_gate(o, g, H, self.D, self.out_scale)
            else:
                # the output bias rides along: the same launch adds it to the token's residual row
                ops.entry_gate(o, g, H, dv, self.D, self.out_scale, resid=resid if bias is not None else None, bias=bias)
                bias = None
        ops.linear_add(o, self.w_o, resid)
        if bias is not None:
            ops.add_vec_rows(resid, None, bias)


register_part("mixer", "gqa_attention", GroupedQueryAttention)
register_part("mixer", "head_normed_attention", HeadNormedAttention)
register_part("mixer", "normed_biased_attention", NormedBiasedAttention)
register_part("mixer", "latent_attention", LatentAttention)
