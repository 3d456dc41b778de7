"""Plain PyTorch statement of every kernel's contract (same call signatures as
``dlm_b200.ops.native.NativeOps``).  Two uses, both in tests only:

* the reference each kernel is compared with, alone, at sizes of the test's choosing;
* a stand-in backend that lets the host-side logic (cache, step function, scheduler,
  replay) run on a machine without a GPU.

It is not part of the package and the package never falls back to it.
"""
from __future__ import annotations

import torch


def _f(t):
    return t.to(torch.float32)


class _InOrder:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def join(self):
        pass


class PlainOps:
    def check_errors(self):
        pass

    def branch(self, rows):
        return _InOrder()

    # ----------------------------------------------------------------- basic
    def embed(self, tokens, table, scale=1.0):
        return _f(table[tokens.long()]) * scale

    def add_rows(self, x, table, idx):
        x += _f(table[idx.long()])

    # ------------------------------------------------------ residual streams
    def streams_expand(self, x, S):
        return x[:, None, :].repeat(1, S, 1).contiguous()

    def streams_reduce(self, xs, a, norm_w, eps, out_dtype):
        u = xs.sum(1) if a is None else torch.einsum("s,tsh->th", a, xs)
        if norm_w is not None:
            u = (u * (1.0 / torch.sqrt((u * u).mean(-1, keepdim=True) + eps))) * norm_w
        return u.to(out_dtype)

    def streams_update(self, xs, mix, outw, y):
        xs.copy_(torch.einsum("sr,tsh->trh", mix, xs) + outw[None, :, None] * y[:, None, :])

    def streams_update_reduce(self, xs, mix, outw, y, in_next, norm_w, eps, out_dtype):
        self.streams_update(xs, mix, outw, y)
        return self.streams_reduce(xs, in_next, norm_w, eps, out_dtype)

    # ------------------------------------------- convolutions and recurrences
    def causal_conv(self, x, w, bias, state, batch, add_input, silu, out_dtype):
        T, C = x.shape
        taps = w.shape[1]
        out = torch.zeros((T, C), dtype=torch.float32, device=x.device)
        cu, slots = batch.cu_q.tolist(), batch.state_slot.tolist()
        for r in range(batch.num_requests):
            a, b = cu[r], cu[r + 1]
            if b == a:
                continue
            full = torch.cat([state[slots[r]], x[a:b]], dim=0) if taps > 1 else x[a:b]   # [taps - 1 + n, C]
            for j in range(taps):
                out[a:b] += w[:, j] * full[j:j + (b - a)]
            if taps > 1:
                state[slots[r]] = full[-(taps - 1):]
        if bias is not None:
            out += bias
        if add_input:
            out += x
        if silu:
            out = out / (1.0 + torch.exp(-out))
        return out.to(out_dtype)

    def activation(self, x, op, out_dtype):
        if op == "tanh":
            v = torch.tanh(x)
        elif op == "gelu":
            v = 0.5 * x * (1.0 + torch.erf(x * 0.7071067811865476))
        elif op == "gelu_tanh":
            v = 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))
        elif op == "copy":
            v = x
        else:
            v = x / (1.0 + torch.exp(-x))
        return v.to(out_dtype)

    def gated_rmsnorm(self, y, gate, w, groups, eps, mode, out_dtype, row_scale=None):
        T, C = y.shape
        if row_scale is not None:          # a factor per token and group, before anything else
            y = (y.reshape(T, groups, C // groups) * row_scale[:, :, None]).reshape(T, C)
        v = y * (gate / (1.0 + torch.exp(-gate))) if mode == "silu_before" else y
        v = v.reshape(T, groups, C // groups)
        v = (v * (1.0 / torch.sqrt((v * v).mean(-1, keepdim=True) + eps))).reshape(T, C)
        if w is not None:
            v = v * w
        if mode == "sigmoid_after":
            v = v * torch.sigmoid(gate)
        elif mode == "silu_after":
            v = v * (gate / (1.0 + torch.exp(-gate)))
        return v.to(out_dtype)

    def ssm_scan(self, xbc, dt_raw, dt_bias, A_log, D, state, batch, heads, P, N, groups, fixed_decay=None):
        T = xbc.shape[0]
        inner = heads * P
        y = torch.zeros((T, inner), dtype=torch.float32, device=xbc.device)
        cu, slots = batch.cu_q.tolist(), batch.state_slot.tolist()
        if fixed_decay is not None:
            dt = torch.ones((T, heads), dtype=torch.float32, device=xbc.device)
            decay = fixed_decay[None, :].expand(T, heads)
        else:
            dt = torch.nn.functional.softplus(dt_raw + dt_bias, threshold=30.0)
            decay = torch.exp(-torch.exp(A_log) * dt)                 # [T, heads]
        if D is None:
            D = torch.zeros(heads, dtype=torch.float32, device=xbc.device)
        per = heads // groups
        for r in range(batch.num_requests):
            S = state[slots[r]]                                        # [heads, N, P]
            for t in range(cu[r], cu[r + 1]):
                x = xbc[t, :inner].reshape(heads, P)
                B = xbc[t, inner:inner + groups * N].reshape(groups, N).repeat_interleave(per, 0)
                C = xbc[t, inner + groups * N:].reshape(groups, N).repeat_interleave(per, 0)
                S.copy_(decay[t][:, None, None] * S + (dt[t][:, None] * B)[:, :, None] * x[:, None, :])
                y[t] = (torch.einsum("hnp,hn->hp", S, C) + D[:, None] * x).reshape(inner)
        return y

    def selective_scan(self, x, dt_raw, bc, z, dt_bias, A_log, D, state, batch, out_dtype):
        T, inner = x.shape
        N = A_log.shape[1]
        out = torch.zeros((T, inner), dtype=torch.float32, device=x.device)
        cu, slots = batch.cu_q.tolist(), batch.state_slot.tolist()
        dt = torch.nn.functional.softplus(dt_raw + dt_bias, threshold=30.0)
        A = -torch.exp(A_log)
        for r in range(batch.num_requests):
            S = state[slots[r]]                                        # [inner, N]
            for t in range(cu[r], cu[r + 1]):
                S.copy_(torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * bc[t, :N][None, :])
                out[t] = S @ bc[t, N:2 * N] + D * x[t]
        return (out * (z / (1.0 + torch.exp(-z)))).to(out_dtype)

    def qk_norm_write(self, qkv, positions, qn_w, kn_w, eps, temp_coef, temp_every, slots, k_cache, v_cache, nh, nkv, d,
                      dv, D, out_dtype):
        T = qkv.shape[0]
        Q, K = nh * d, nkv * d
        q, k, v = qkv[:, :Q], qkv[:, Q:Q + K], qkv[:, Q + K:Q + K + nkv * dv]
        if qn_w is not None:
            q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * qn_w
        if kn_w is not None:
            k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * kn_w
        if temp_every > 0:
            steps = torch.div(positions + 1, temp_every, rounding_mode="floor").to(torch.float32)
            q = q * (1.0 + temp_coef * torch.log(steps + 1.0))[:, None]
        pad = torch.nn.functional.pad
        qo = pad(q.reshape(T, nh, d), (0, D - d)).reshape(T, nh * D)
        if slots is not None:
            ps = k_cache.shape[2]
            sl = slots.long()
            ok = sl >= 0
            page, off = sl[ok] // ps, sl[ok] % ps
            k_cache[page, :, off, :] = pad(k.reshape(T, nkv, d), (0, D - d))[ok].to(k_cache.dtype)
            v_cache[page, :, off, :] = pad(v.reshape(T, nkv, dv), (0, D - dv))[ok].to(v_cache.dtype)
        return qo.to(out_dtype)

    def rotate_heads(self, x, positions, inv_freq, rot_dims, heads, dim, off_a, scale_a, off_b, scale_b):
        T = x.shape[0]
        for off, f in ((off_a, scale_a), (off_b, scale_b)):
            v = x[:, off:off + heads * dim].reshape(T, heads, dim).clone()
            if rot_dims:
                v = self._rotate(v, positions, inv_freq, rot_dims)
            x[:, off:off + heads * dim] = (v * f).reshape(T, heads * dim)

    def branch_norm_add(self, resid, a, wa, b, wb, eps, coef):
        v = a / torch.sqrt((a * a).mean(-1, keepdim=True) + eps) * wa
        if b is not None:
            v = v + b / torch.sqrt((b * b).mean(-1, keepdim=True) + eps) * wb
        resid += coef * v

    def rmsnorm_pair(self, x, wa, wb, eps, out_dtype):
        v = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
        return (v * wa).to(out_dtype), (v * wb).to(out_dtype)

    def concat_rows(self, a, b, out_dtype):
        return torch.cat([a, b], dim=-1).to(out_dtype)

    def delta_scan(self, proj, offsets, lw, a_bias, state, batch, heads, d, unit_eps, decay_coef):
        T = proj.shape[0]
        HD = heads * d
        o_r, o_k, o_v, o_a = offsets
        r_, k_, v_ = (proj[:, o:o + HD].reshape(T, heads, d) for o in (o_r, o_k, o_v))
        a_ = torch.sigmoid(proj[:, o_a:o_a + HD] + a_bias).reshape(T, heads, d)
        w_ = torch.exp(-decay_coef * torch.sigmoid(lw)).reshape(T, heads, d)
        u_ = k_ / torch.sqrt((k_ * k_).sum(-1, keepdim=True) + unit_eps)
        out = torch.zeros((T, HD), dtype=torch.float32, device=proj.device)
        cu, slots = batch.cu_q.tolist(), batch.state_slot.tolist()
        for r in range(batch.num_requests):
            S = state[slots[r]]                                        # [heads, d(key), d(value)]
            for t in range(cu[r], cu[r + 1]):
                uS = torch.einsum("hi,hij->hj", u_[t], S)
                S.copy_(w_[t][:, :, None] * S - (a_[t] * u_[t])[:, :, None] * uS[:, None, :]
                        + k_[t][:, :, None] * v_[t][:, None, :])
                out[t] = torch.einsum("hij,hi->hj", S, r_[t]).reshape(HD)
        return out

    # ------------------------------------------------------- latent attention
    @staticmethod
    def _rotate(x, positions, inv_freq, rot_dims):
        half = rot_dims // 2
        if half == 0:
            return x
        ang = positions.to(torch.float32)[:, None] * inv_freq[None, :half]
        while ang.dim() < x.dim():
            ang = ang.unsqueeze(1)
        sin, cos = torch.sin(ang), torch.cos(ang)
        a, b = x[..., :half], x[..., half:rot_dims]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rot_dims:]], dim=-1)

    @staticmethod
    def _rotate_neighbours(x, positions, inv_freq, rot_dims):
        if rot_dims == 0:
            return x
        ang = positions.to(torch.float32)[:, None] * inv_freq[None, :rot_dims // 2]
        while ang.dim() < x.dim():
            ang = ang.unsqueeze(1)
        sin, cos = torch.sin(ang), torch.cos(ang)
        a, b = x[..., 0:rot_dims:2], x[..., 1:rot_dims:2]
        rot = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).reshape(*x.shape[:-1], rot_dims)
        return torch.cat([rot, x[..., rot_dims:]], dim=-1)

    def latent_prep(self, proj, off_q, q_rank, qn_w, off_kv, rank, kvn_w, dr, inv_freq, rot_dims, positions, slots,
                    eps, cache, out_dtype, interleaved=False):
        def rms(v, w):
            return (v * (1.0 / torch.sqrt((v * v).mean(-1, keepdim=True) + eps))) * w
        cq = rms(proj[:, off_q:off_q + q_rank], qn_w).to(out_dtype) if q_rank else None
        if slots is not None:
            c = rms(proj[:, off_kv:off_kv + rank], kvn_w)
            rotate = self._rotate_neighbours if interleaved else self._rotate
            kr = rotate(proj[:, off_kv + rank:off_kv + rank + dr], positions, inv_freq, rot_dims)
            ps = cache.shape[2]
            sl = slots.long()
            ok = sl >= 0
            cache[sl[ok] // ps, 0, sl[ok] % ps, :] = torch.cat([c, kr], dim=-1)[ok].to(cache.dtype)
        return cq

    def latent_q_split(self, q, positions, inv_freq, rot_dims, H, dn, dr, out_dtype, interleaved=False):
        T = q.shape[0]
        q = q.reshape(T, H, dn + dr)
        qn = q[..., :dn].transpose(0, 1).contiguous().to(out_dtype)
        rotate = self._rotate_neighbours if interleaved else self._rotate
        return qn, rotate(q[..., dn:], positions, inv_freq, rot_dims).contiguous()

    # ------------------------------------- gated recurrences, per-head norms, norms on both sides of a sublayer
    def gated_scan(self, q, k, v, decay, beta, state, batch, heads, qk_heads, dk, dv, *, unit_eps=None, q_scale=1.0,
                   A_log=None, decay_bias=None, tau=None):
        T = v.shape[0]
        rep = heads // qk_heads
        q_ = q.reshape(T, qk_heads, dk)
        k_ = k.reshape(T, qk_heads, dk)
        if unit_eps is not None:
            q_ = q_ / torch.sqrt((q_ * q_).sum(-1, keepdim=True) + unit_eps)
            k_ = k_ / torch.sqrt((k_ * k_).sum(-1, keepdim=True) + unit_eps)
        q_ = (q_ * q_scale).repeat_interleave(rep, dim=1)
        k_ = k_.repeat_interleave(rep, dim=1)
        v_ = v.reshape(T, heads, dv)
        sp = torch.nn.functional.softplus
        if A_log is not None:
            raw = decay + (decay_bias if decay_bias is not None else 0.0)
            a_ = torch.exp(-torch.exp(A_log) * sp(raw))[:, :, None].expand(T, heads, dk)
        else:
            a_ = torch.exp(-sp(-decay) / tau).reshape(T, heads, dk)
        b_ = torch.sigmoid(beta) if beta is not None else None
        out = torch.zeros((T, heads * dv), dtype=torch.float32, device=v.device)
        cu, slots = batch.cu_q.tolist(), batch.state_slot.tolist()
        for r in range(batch.num_requests):
            S = state[slots[r]]                                        # [heads, dk, dv]
            for t in range(cu[r], cu[r + 1]):
                S.mul_(a_[t][:, :, None])
                u = v_[t]
                if b_ is not None:
                    u = b_[t][:, None] * (u - torch.einsum("hij,hi->hj", S, k_[t]))
                S.add_(k_[t][:, :, None] * u[:, None, :])
                out[t] = torch.einsum("hij,hi->hj", S, q_[t]).reshape(heads * dv)
        return out

    def head_norm_rope_write(self, qkv, positions, qn_w, kn_w, eps, inv_freq, rot_dims, interleaved, slots, k_cache,
                             v_cache, nh, nkv, d, dv, D, out_dtype):
        T = qkv.shape[0]
        Q, K = nh * d, nkv * d
        q, k = qkv[:, :Q].reshape(T, nh, d), qkv[:, Q:Q + K].reshape(T, nkv, d)
        v = qkv[:, Q + K:Q + K + nkv * dv].reshape(T, nkv, dv)
        if qn_w is not None:
            q = (q * (1.0 / torch.sqrt((q * q).mean(-1, keepdim=True) + eps))) * qn_w
        if kn_w is not None:
            k = (k * (1.0 / torch.sqrt((k * k).mean(-1, keepdim=True) + eps))) * kn_w
        if rot_dims:
            rotate = self._rotate_neighbours if interleaved else self._rotate
            q, k = rotate(q, positions, inv_freq, rot_dims), rotate(k, positions, inv_freq, rot_dims)
        pad = torch.nn.functional.pad
        if slots is not None:
            ps = k_cache.shape[2]
            sl = slots.long()
            ok = sl >= 0
            page, off = sl[ok] // ps, sl[ok] % ps
            k_cache[page, :, off, :] = pad(k, (0, D - d))[ok].to(k_cache.dtype)
            v_cache[page, :, off, :] = pad(v, (0, D - dv))[ok].to(v_cache.dtype)
        return pad(q, (0, D - d)).reshape(T, nh * D).to(out_dtype)

    def head_gate(self, o, gate, nh, D, factor=1.0):
        T = o.shape[0]
        g = factor * torch.sigmoid(gate)
        o.copy_((_f(o).reshape(T, nh, D) * g[:, :, None]).reshape(T, nh * D).to(o.dtype))

    def norm_add_norm(self, resid, y, w_post, w_next, eps, out_dtype):
        resid += (y * (1.0 / torch.sqrt((y * y).mean(-1, keepdim=True) + eps))) * w_post
        if w_next is None:
            return None
        return ((resid * (1.0 / torch.sqrt((resid * resid).mean(-1, keepdim=True) + eps))) * w_next).to(out_dtype)

    def add_vec_rows(self, x, x0, vec):
        if x0 is not None:
            x += x0
        x += vec

    def head_offsets(self, H, T, device):
        return torch.arange(0, (H + 1) * T, T, dtype=torch.int32, device=device)

    def latent_attention(self, q_lat, q_rot, sink, cache, block_table, batch, H, dr, rank, window, scale):
        T = q_rot.shape[0]
        ps = cache.shape[2]
        out = torch.zeros((H, T, rank), dtype=torch.float32, device=q_lat.device)
        req, pos = batch.token_req.tolist(), batch.positions.tolist()
        for t in range(T):
            lo = max(0, pos[t] - window + 1) if window > 0 else 0
            js = torch.arange(lo, pos[t] + 1, device=q_lat.device)
            pages = block_table[req[t], (js // ps).long()].long()
            assert int(pages.min()) >= 0, "a visible key has no page"
            rows = _f(cache[pages, 0, js % ps, :])                     # [n, rank + dr]
            s = (q_lat[:, t] @ rows[:, :rank].T + q_rot[t] @ rows[:, rank:].T) * scale      # [H, n]
            if sink is not None:
                s = torch.cat([s, sink[:, None]], dim=1)
            p = torch.softmax(s, dim=-1)[:, :js.numel()]
            out[:, t] = p @ rows[:, :rank]
        return out.to(cache.dtype)

    def latent_gate_out(self, val, gate, H, dv, out_dtype):
        T = val.shape[0] // H
        out = val.reshape(H, T, dv).transpose(0, 1)
        if gate is not None:
            out = out * torch.sigmoid(gate)[:, :, None]
        return out.reshape(T, H * dv).to(out_dtype)

    def rmsnorm(self, x, w, eps, out_dtype, rows=None):
        if rows is not None:
            x = x[rows.long()]
        ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
        return ((x * (1.0 / torch.sqrt(ms + eps))) * w).to(out_dtype)

    # -------------------------------------------------------------- products
    def linear(self, a, w, bias, out_dtype):
        out = _f(a) @ _f(w).T
        if bias is not None:
            out = out + bias
        return out.to(out_dtype)

    def linear_act(self, a, w, act):
        return self.activation(_f(a) @ _f(w).T, act, a.dtype)

    def linear_add(self, a, w, resid):
        resid += _f(a) @ _f(w).T

    @staticmethod
    def _swiglu(acc, dtype):
        g, u = acc[:, 0::2], acc[:, 1::2]
        return ((g / (1.0 + torch.exp(-g))) * u).to(dtype)

    def linear_swiglu(self, a, w_gate_up):
        return self._swiglu(_f(a) @ _f(w_gate_up).T, a.dtype)

    def grouped_swiglu(self, a, w_gate_up, offsets, rows):
        E, N, K = w_gate_up.shape
        out = torch.zeros((rows.numel(), N // 2), dtype=a.dtype, device=a.device)
        off = offsets.tolist()
        for e in range(E):
            if off[e + 1] > off[e]:
                x = _f(a[rows[off[e]:off[e + 1]].long()])
                out[off[e]:off[e + 1]] = self._swiglu(x @ _f(w_gate_up[e]).T, a.dtype)
        return out

    def grouped_act(self, a, w_up, offsets, rows, act):
        E, N, K = w_up.shape
        out = torch.zeros((rows.numel(), N), dtype=a.dtype, device=a.device)
        off = offsets.tolist()
        for e in range(E):
            if off[e + 1] > off[e]:
                x = _f(a[rows[off[e]:off[e + 1]].long()])
                out[off[e]:off[e + 1]] = self.activation(x @ _f(w_up[e]).T, act, a.dtype)
        return out

    def table_route(self, tokens, table, E):
        ids = table[tokens.long()].to(torch.int32)
        wts = torch.full(ids.shape, 1.0 / ids.shape[1], dtype=torch.float32, device=ids.device)
        offsets, rows, dest = self.moe_permute(ids, E)
        return ids, wts, offsets, rows, dest

    def grouped_linear(self, a, w, offsets):
        E, N, K = w.shape
        out = torch.zeros((a.shape[0], N), dtype=torch.float32, device=a.device)
        off = offsets.tolist()
        for e in range(E):
            if off[e + 1] > off[e]:
                out[off[e]:off[e + 1]] = _f(a[off[e]:off[e + 1]]) @ _f(w[e]).T
        return out

    # ------------------------------------------------------------- attention
    def rope_kv_write(self, qkv, positions, inv_freq, rotary_dim, slots, k_cache, v_cache, nh, nkv, hd, out_dtype,
                      interleaved=False):
        T = qkv.shape[0]
        Q, KV = nh * hd, nkv * hd
        q = qkv[:, :Q].reshape(T, nh, hd).clone()
        k = qkv[:, Q:Q + KV].reshape(T, nkv, hd).clone()
        v = qkv[:, Q + KV:].reshape(T, nkv, hd)
        if inv_freq is not None:
            half = rotary_dim // 2
            ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
            sin, cos = torch.sin(ang)[:, None, :], torch.cos(ang)[:, None, :]
            for x in (q, k):
                if interleaved:
                    a, b = x[..., 0:rotary_dim:2].clone(), x[..., 1:rotary_dim:2].clone()
                    x[..., 0:rotary_dim:2] = a * cos - b * sin
                    x[..., 1:rotary_dim:2] = a * sin + b * cos
                else:
                    a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
                    x[..., :half] = a * cos - b * sin
                    x[..., half:rotary_dim] = a * sin + b * cos
        if slots is not None:
            ps = k_cache.shape[2]
            sl = slots.long()
            ok = sl >= 0
            page, off = sl[ok] // ps, sl[ok] % ps
            k_cache[page, :, off, :] = k[ok].to(k_cache.dtype)
            v_cache[page, :, off, :] = v[ok].to(v_cache.dtype)
        return q.reshape(T, Q).to(out_dtype)

    def attention(self, q, k_cache, v_cache, block_table, cu_q, kv_len, window, scale, nh, nkv, hd, max_q_len,
                  max_kv_len, num_single=0, slopes=None, chunk=0, sinks=None, softcap=0.0):
        T = q.shape[0]
        ps = k_cache.shape[2]
        out = torch.zeros((T, nh * hd), dtype=torch.float32, device=q.device)
        cu, lens = cu_q.tolist(), kv_len.tolist()
        group = nh // nkv
        for r in range(block_table.shape[0]):
            q_len, n = cu[r + 1] - cu[r], lens[r]
            if q_len == 0:
                continue
            first = n - q_len
            lo = max(0, first - window + 1) if window > 0 else 0
            if chunk > 0:
                lo = max(lo, (first // chunk) * chunk)
            pos = torch.arange(lo, n, device=q.device)
            pages = block_table[r, (pos // ps).long()].long()
            assert int(pages.min()) >= 0, "a visible key has no page"
            k = _f(k_cache[pages, :, pos % ps, :])          # [n - lo, nkv, hd]
            v = _f(v_cache[pages, :, pos % ps, :])
            qs = _f(q[cu[r]:cu[r + 1]]).reshape(q_len, nh, hd)
            qpos = torch.arange(first, n, device=q.device)
            ok = pos[None, :] <= qpos[:, None]
            if window > 0:
                ok &= (qpos[:, None] - pos[None, :]) < window
            if chunk > 0:
                ok &= torch.div(pos, chunk, rounding_mode="floor")[None, :] == torch.div(qpos, chunk, rounding_mode="floor")[:, None]
            for h in range(nh):
                s = (qs[:, h, :] @ k[:, h // group, :].T) * scale
                if softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                if slopes is not None:
                    s = s - slopes[h] * (qpos[:, None] - pos[None, :]).to(torch.float32)
                s = s.masked_fill(~ok, float("-inf"))
                if sinks is not None:
                    s = torch.cat([s, sinks[h].expand(q_len, 1)], dim=1)
                p = torch.softmax(s, dim=-1)[:, :pos.numel()]
                out[cu[r]:cu[r + 1], h * hd:(h + 1) * hd] = p @ v[:, h // group, :]
        return out.to(q.dtype)

    def dyt_norm(self, x, w, b, alpha, out_dtype, rows=None):
        if rows is not None:
            x = x[rows.long()]
        return (torch.tanh(alpha * x) * w + b).to(out_dtype)

    def dyt_norm_pair(self, x, wa, ba, alpha_a, wb, bb, alpha_b, out_dtype, want_f32=False):
        b32 = torch.tanh(alpha_b * x) * wb + bb
        return (torch.tanh(alpha_a * x) * wa + ba).to(out_dtype), b32.to(out_dtype), (b32 if want_f32 else None)

    def tanh_cap(self, x, cap):
        x.copy_(cap * torch.tanh(x / cap))

    def entry_gate(self, o, gate, nh, dv, D, factor=1.0, resid=None, bias=None):
        T = o.shape[0]
        if resid is not None:
            resid += bias
        v = _f(o).reshape(T, nh, D).clone()
        v[:, :, :dv] = v[:, :, :dv] * (factor * torch.sigmoid(gate.reshape(T, nh, dv)))
        o.copy_(v.reshape(T, nh * D).to(o.dtype))

    def memory_scan(self, q, k, v, igate, fgate, i_bias, f_bias, cap, S, n, m, batch, heads, dk, dv, q_scale=1.0,
                    den_eps=1e-6):
        T = v.shape[0]
        q_ = q.reshape(T, heads, dk) * q_scale
        k_ = k.reshape(T, heads, dk)
        v_ = v.reshape(T, heads, dv)
        li = cap * torch.tanh((igate + i_bias) / cap)
        lf = torch.nn.functional.logsigmoid(cap * torch.tanh((fgate + f_bias) / cap))
        out = torch.zeros((T, heads * dv), dtype=torch.float32, device=v.device)
        rden = torch.zeros((T, heads), dtype=torch.float32, device=v.device)
        cu, slots = batch.cu_q.tolist(), batch.state_slot.tolist()
        for r in range(batch.num_requests):
            Sr, nr, mall = S[slots[r]], n[slots[r]], m[slots[r]]       # [heads, dk, dv], [heads, dk], [heads, dv + 1]
            mr = mall[:, 0].clone()                                    # the copies of m are equal
            for t in range(cu[r], cu[r + 1]):
                new = torch.maximum(lf[t] + mr, li[t])
                keep, put = torch.exp(lf[t] + mr - new), torch.exp(li[t] - new)
                kp = put[:, None] * k_[t]
                Sr.copy_(keep[:, None, None] * Sr + kp[:, :, None] * v_[t][:, None, :])
                nr.copy_(keep[:, None] * nr + kp)
                mr = new
                mall.copy_(new[:, None].expand_as(mall))
                out[t] = torch.einsum("hij,hi->hj", Sr, q_[t]).reshape(heads * dv)
                rden[t] = 1.0 / (torch.maximum((nr * q_[t]).sum(-1).abs(), torch.exp(-new)) + den_eps)
        return out, rden

    # ------------------------------------------------------------------- moe
    def router_topk(self, h, w, E, k, norm, has_gate, norm_weight=None, eps=0.0, score="softmax", scale=1.0,
                    select_bias=None, logit_bias=None):
        if norm_weight is not None:
            h = self.rmsnorm(h, norm_weight, eps, torch.float32)
        logits = _f(h) @ _f(w).T
        gate = None
        if has_gate:
            gate = 1.0 / (1.0 + torch.exp(-logits[:, E]))
            logits = logits[:, :E]
        if logit_bias is not None:
            logits = logits + logit_bias[None, :]
        probs = torch.softmax(logits, dim=-1) if score == "softmax" else 1.0 / (1.0 + torch.exp(-logits))
        pick = probs if select_bias is None else probs + select_bias[None, :].to(probs.dtype)
        ids = torch.sort(pick, dim=-1, descending=True, stable=True).indices[:, :k]
        wts = torch.gather(probs, 1, ids)
        if norm:
            s = wts.sum(-1, keepdim=True)
            wts = torch.where(s > 0, wts / (s + 1e-20 if norm == 2 else s), wts)
        return ids.to(torch.int32), wts * scale, gate

    def route(self, h, w, E, k, norm, has_gate, input_settled=False, **kw):
        ids, wts, gate = self.router_topk(h, w, E, k, norm, has_gate, **kw)
        return (ids, wts, gate) + tuple(self.moe_permute(ids, E))

    def moe_permute(self, ids, E):
        T, k = ids.shape
        flat = ids.reshape(-1).long()
        order = torch.sort(flat, stable=True).indices
        counts = torch.bincount(flat, minlength=E)
        offsets = torch.zeros(E + 1, dtype=torch.int32, device=ids.device)
        offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
        rows = (order // k).to(torch.int32)
        dest = torch.empty(T * k, dtype=torch.int32, device=ids.device)
        dest[order] = torch.arange(T * k, dtype=torch.int32, device=ids.device)
        return offsets, rows, dest.reshape(T, k)

    def moe_combine(self, y, dest, wts, shared, gate, resid, ids=None, num_real=0, passthrough=None, shared_scale=1.0):
        T, k = dest.shape
        acc = torch.zeros_like(resid)
        for j in range(k):
            if ids is None:
                src = y[dest[:, j].long()]
            else:                               # experts from num_real on hand the token's own row through
                real = ids[:, j] < num_real
                src = passthrough.clone()
                if y is not None and bool(real.any()):
                    src[real] = y[dest[real, j].long()]
            acc = acc + wts[:, j:j + 1] * src
        if shared is not None:
            g = gate[:, None] if gate is not None else 1.0
            acc = acc + (g * shared_scale) * shared
        resid += acc

    # -------------------------------------------------------------- sampling
    def argmax(self, logits):
        # the first maximum
        mx = logits.max(dim=-1, keepdim=True).values
        first = torch.argmax((logits == mx).to(torch.int32), dim=-1)
        return first.to(torch.int32)

    def sample(self, logits, params, top_k, u, seen_offsets, seen_tokens):
        """Same candidate order and cuts as the kernel, in double precision."""
        N, V = logits.shape
        out = torch.zeros(N, dtype=torch.int32, device=logits.device)
        for i in range(N):
            temp, top_p, min_p, pen = [float(x) for x in params[i]]
            z = logits[i].clone()
            if pen != 1.0 and seen_offsets is not None:
                seen = seen_tokens[int(seen_offsets[i]):int(seen_offsets[i + 1])].long()
                z[seen] = torch.where(z[seen] > 0, z[seen] / pen, z[seen] * pen)
            if not temp > 0:
                out[i] = int(self.argmax(z[None])[0])
                continue
            order = torch.sort(z, descending=True, stable=True).indices
            k = int(top_k[i])
            if 0 < k < V:
                order = order[:k]
            p = torch.exp((z[order] - z[order[0]]).double() / temp)
            if 0.0 < top_p < 1.0:
                cum = torch.cumsum(p, 0)
                cut = int(torch.nonzero(cum >= top_p * cum[-1])[0]) + 1
                order, p = order[:cut], p[:cut]
            if min_p > 0:
                keep = max(int((p >= min(min_p, 1.0)).sum()), 1)
                order, p = order[:keep], p[:keep]
            cum = torch.cumsum(p, 0)
            hit = torch.nonzero(cum > float(u[i]) * cum[-1])
            out[i] = int(order[int(hit[0])]) if hit.numel() else int(order[-1])
        return out
