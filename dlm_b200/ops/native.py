"""The kernel backend: thin, shape-checking wrappers around the sm_100a launchers.

There is no other backend in the package and no fallback: constructing
``NativeOps`` without a CUDA device, or without a kernel library that builds and
loads, raises.  Every method takes and returns torch tensors on the CUDA device;
outputs are allocated with torch's caching allocator (which is also what makes
the calls capturable in a CUDA graph).
"""
from __future__ import annotations

import os

import torch

from ..build import load_kernels

_F32, _BF16 = 0, 1


def _dt(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise TypeError(f"kernels take float32 or bfloat16, got {dtype}")


def _p(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


class KernelError(RuntimeError):
    pass


class _Branch:
    """A piece of a step that may run beside the launching stream.  ``with branch:`` launches
    what is inside on a second stream that starts after everything launched so far;
    ``branch.join()`` makes the launching stream wait for it.  Inactive, it does nothing and the
    work stays in order on the launching stream."""

    def __init__(self, side):
        self.side = side
        self.main = None
        self.ctx = None

    def __enter__(self):
        if self.side is not None:
            self.main = torch.cuda.current_stream()
            self.side.wait_stream(self.main)
            self.ctx = torch.cuda.stream(self.side)
            self.ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)
            self.ctx = None
        return False

    def join(self):
        if self.side is not None and self.main is not None:
            self.main.wait_stream(self.side)


class NativeOps:
    """``fast=False`` keeps every product and the attention on the plain FMA kernels
    (the path the 32-bit mode always takes)."""

    def __init__(self, fast: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("dlm_b200 needs a CUDA device: there is no CPU path")
        self.k = load_kernels()
        self.fast = 1 if fast else 0
        self.launches = 0        # kernels launched through this object (for the benchmark's count)
        self.tc = bool(self.k.gemm_tc_enabled()) if fast else False
        self.branches = os.environ.get("DLM_B200_NO_BRANCH", "") in ("", "0")
        self._side = None        # second stream for branches of a step (made at first use)

    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def branch(self, rows: int) -> _Branch:
        """A branch for work on ``rows`` tokens that is independent of what the caller launches
        next.  With few rows the kernels stream weights and leave most of the machine idle
        between them, so two chains side by side fill it better; with many rows each kernel
        fills the machine alone and the branch stays inactive."""
        if not self.fast or rows > 64 or not self.branches:
            return _Branch(None)
        if self._side is None:
            self._side = torch.cuda.Stream()
        return _Branch(self._side)

    def dependent_launch(self, on: bool):
        """A context in which the short kernels are (on) or are not (off) launched with programmatic dependent
        launch; the library's setting is put back at the end."""
        import contextlib

        @contextlib.contextmanager
        def scope():
            before = bool(self.k.dep_launch_enabled())
            self.k.set_dep_launch(bool(on) and before)      # never switched on where the process has it off
            try:
                yield
            finally:
                self.k.set_dep_launch(before)
        return scope()

    def check_errors(self) -> None:
        """Raises if a kernel refused an access (page or token id outside its table)."""
        flag = self.k.take_error_flag()
        if flag == 5:
            # a kernel gave up on a wait: the decode attention's split counters may not be back at zero
            self.k.reset_decode_merge_counters(self._stream())
        if flag:
            what = {1: "token id outside the vocabulary", 2: "cache slot outside the pool",
                    3: "a visible key has no page", 4: "expert id outside the table",
                    5: "a wait inside a kernel ran out (copy or tensor-core pipeline)",
                    6: "position outside the table of learned positions"}.get(flag, "unknown")
            raise KernelError(f"a kernel reported error {flag}: {what}")

    # ----------------------------------------------------------------- basic
    def embed(self, tokens, table, scale=1.0):
        T, (V, H) = tokens.numel(), table.shape
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
        self.launches += 1
        self.k.embed(_p(tokens), _p(table), _p(out), T, H, V, float(scale), _dt(table.dtype), self._stream())
        return out

    def add_rows(self, x, table, idx):
        """``x[t] += table[idx[t]]`` in place (x 32-bit): learned position vectors."""
        T, H = x.shape
        assert x.dtype == torch.float32 and table.shape[1] == H and x.is_contiguous()
        self.launches += 1
        self.k.add_rows(_p(x), _p(table), _p(idx), T, H, table.shape[0], _dt(table.dtype), self._stream())

    # ------------------------------------------------------ residual streams
    def streams_expand(self, x, S):
        """``[T, H] -> [T, S, H]``: S equal copies of the residual."""
        T, H = x.shape
        xs = torch.empty((T, S, H), dtype=torch.float32, device=x.device)
        self.launches += 1
        self.k.streams_expand(_p(x), _p(xs), T, S, H, self._stream())
        return xs

    def streams_reduce(self, xs, a, norm_w, eps, out_dtype):
        """``u = sum_s a[s] xs[:, s]`` (``a`` None: plain sum), RMS-normed with ``norm_w`` unless that is None."""
        T, S, H = xs.shape
        assert xs.dtype == torch.float32 and xs.is_contiguous()
        out = torch.empty((T, H), dtype=out_dtype, device=xs.device)
        self.launches += 1
        self.k.streams_reduce(_p(xs), _p(a), _p(norm_w), float(eps), _p(out), T, S, H, _dt(out_dtype), self._stream())
        return out

    def streams_update(self, xs, mix, outw, y):
        """``xs[:, r] <- sum_s mix[s, r] xs[:, s] + outw[r] * y`` in place."""
        T, S, H = xs.shape
        assert mix.shape == (S, S) and outw.shape == (S,) and y.shape == (T, H) and y.dtype == torch.float32
        self.launches += 1
        self.k.streams_update(_p(xs), _p(mix), _p(outw), _p(y), T, S, H, self._stream())

    def streams_update_reduce(self, xs, mix, outw, y, in_next, norm_w, eps, out_dtype):
        """``streams_update`` and the next sublayer's ``streams_reduce`` in one pass over the streams."""
        T, S, H = xs.shape
        if S > 8:
            self.streams_update(xs, mix, outw, y)
            return self.streams_reduce(xs, in_next, norm_w, eps, out_dtype)
        assert mix.shape == (S, S) and outw.shape == (S,) and in_next.shape == (S,) and y.shape == (T, H)
        out = torch.empty((T, H), dtype=out_dtype, device=xs.device)
        self.launches += 1
        self.k.streams_update_reduce(_p(xs), _p(mix), _p(outw), _p(y), _p(in_next), _p(norm_w), float(eps), _p(out), T, S,
                                     H, _dt(out_dtype), self._stream())
        return out

    # ------------------------------------------- convolutions and recurrences
    def causal_conv(self, x, w, bias, state, batch, add_input, silu, out_dtype):
        """Causal convolution over time per channel and request; ``x`` is 32-bit ``[T, C]`` (may be a column
        slice of a wider tensor), ``state`` ``[slots, taps - 1, C]`` holds each request's last inputs and is
        brought up to date."""
        T, C = x.shape
        taps = w.shape[1]
        assert x.dtype == torch.float32 and x.stride(1) == 1 and w.shape[0] == C
        assert state.shape[1:] == (taps - 1, C) and state.dtype == torch.float32
        out = torch.empty((T, C), dtype=out_dtype, device=x.device)
        self.launches += 2 if taps > 1 else 1
        self.k.causal_conv(_p(x), x.stride(0), _p(w), _p(bias), _p(state), _p(batch.cu_q), _p(batch.token_req),
                           _p(batch.state_slot), T, batch.num_requests, C, taps, int(bool(add_input)), int(bool(silu)),
                           _p(out), C, _dt(out_dtype), self._stream())
        return out

    _ACTS = {"tanh": 0, "gelu": 1, "silu": 2, "gelu_tanh": 3, "copy": 4}

    def activation(self, x, op, out_dtype):
        """Element-wise ``tanh`` / ``gelu`` (erf) / ``silu`` of 32-bit ``x`` (may be a column slice)."""
        R, C = x.shape
        assert x.dtype == torch.float32 and x.stride(1) == 1
        out = torch.empty((R, C), dtype=out_dtype, device=x.device)
        self.launches += 1
        self.k.activation(_p(x), x.stride(0), _p(out), C, R, C, self._ACTS[op], _dt(out_dtype), self._stream())
        return out

    def gated_rmsnorm(self, y, gate, w, groups, eps, mode, out_dtype, row_scale=None):
        """Norm over ``groups`` equal parts of the channels with a gate; ``mode`` ``"silu_before"``:
        ``rms(y * silu(gate)) * w``; ``"sigmoid_after"``: ``rms(y) * w * sigmoid(gate)``.  ``row_scale`` (32-bit
        ``[T, groups]``, with a gate after the norm): y is multiplied by it first, group by group."""
        T, C = y.shape
        assert C % groups == 0 and gate.shape == (T, C) and y.stride(1) == 1 and gate.stride(1) == 1
        assert row_scale is None or (row_scale.shape == (T, groups) and row_scale.is_contiguous()
                                     and row_scale.dtype == torch.float32 and mode != "silu_before")
        out = torch.empty((T, C), dtype=out_dtype, device=y.device)
        self.launches += 1
        self.k.gated_rmsnorm(_p(y), y.stride(0), _p(gate), gate.stride(0), _p(w), _p(out), C, T, groups, C // groups,
                             float(eps), {"silu_before": 0, "sigmoid_after": 1, "silu_after": 2}[mode], _dt(out_dtype),
                             _p(row_scale), self._stream())
        return out

    def ssm_scan(self, xbc, dt_raw, dt_bias, A_log, D, state, batch, heads, P, N, groups, fixed_decay=None):
        """State-space scan over each request's tokens; ``state`` ``[slots, heads, N, P]`` is read and left
        up to date.  Returns y ``[T, heads * P]`` in 32-bit."""
        T = xbc.shape[0]
        assert xbc.shape[1] == heads * P + 2 * groups * N and xbc.dtype == torch.float32 and xbc.stride(1) == 1
        assert state.shape[1:] == (heads, N, P)
        assert fixed_decay is not None or (dt_raw.shape == (T, heads) and dt_raw.stride(1) == 1)
        y = torch.empty((T, heads * P), dtype=torch.float32, device=xbc.device)
        self.launches += 1
        self.k.ssm_scan(_p(xbc), xbc.stride(0), _p(dt_raw), 0 if dt_raw is None else dt_raw.stride(0), _p(dt_bias),
                        _p(A_log), _p(D), _p(state), _p(batch.cu_q), _p(batch.state_slot), _p(y), batch.num_requests,
                        heads, P, N, groups, _p(fixed_decay), self._stream())
        return y

    def delta_scan(self, proj, offsets, lw, a_bias, state, batch, heads, d, unit_eps, decay_coef):
        """Delta-rule scan; ``proj`` 32-bit rows hold r, k, v and the raw removal rate at column ``offsets``
        (r, k, v, a); ``lw`` the raw decay ``[T, heads * d]``; ``state`` ``[slots, heads, d, d]``."""
        T = proj.shape[0]
        assert proj.dtype == torch.float32 and lw.shape == (T, heads * d) and state.shape[1:] == (heads, d, d)
        o = torch.empty((T, heads * d), dtype=torch.float32, device=proj.device)
        self.launches += 1
        self.k.delta_scan(_p(proj), proj.stride(0), *[int(v) for v in offsets], _p(lw), lw.stride(0), _p(a_bias),
                          _p(state), _p(batch.cu_q), _p(batch.state_slot), _p(o), batch.num_requests, heads, d,
                          float(unit_eps), float(decay_coef), self._stream())
        return o

    def selective_scan(self, x, dt_raw, bc, z, dt_bias, A_log, D, state, batch, out_dtype):
        """Diagonal state-space scan with a step size per channel: ``x, dt_raw, z [T, inner]``, ``bc [T, 2 N]`` (B then
        C), all 32-bit and possibly column slices; ``state [slots, inner, N]`` is read and left up to date.  Returns
        ``y * silu(z)`` in ``out_dtype``."""
        T, inner = x.shape
        N = A_log.shape[1]
        for t in (x, dt_raw, bc, z):
            assert t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[0] == T
        assert dt_raw.shape[1] == inner and z.shape[1] == inner and bc.shape[1] == 2 * N
        assert A_log.shape == (inner, N) and state.shape[1:] == (inner, N) and A_log.is_contiguous()
        out = torch.empty((T, inner), dtype=out_dtype, device=x.device)
        self.launches += 1
        self.k.selective_scan(_p(x), x.stride(0), _p(dt_raw), dt_raw.stride(0), _p(bc), bc.stride(0), _p(z), z.stride(0),
                              _p(dt_bias), _p(A_log), _p(D), _p(state), _p(batch.cu_q), _p(batch.state_slot), _p(out),
                              inner, batch.num_requests, inner, N, _dt(out_dtype), self._stream())
        return out

    def qk_norm_write(self, qkv, positions, qn_w, kn_w, eps, temp_coef, temp_every, slots, k_cache, v_cache, nh, nkv, d,
                      dv, D, out_dtype):
        """Norms over the whole query and key projections, the query temperature, and the write of k and v at the
        tokens' slots, every head ``D`` wide (zeros beyond its own size).  Returns q ``[T, nh * D]``."""
        T = qkv.shape[0]
        assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] >= (nh + nkv) * d + nkv * dv
        total_pages, nkv_c, page_size, D_c = k_cache.shape
        assert (nkv_c, D_c) == (nkv, D) and k_cache.dtype == out_dtype and v_cache.shape == k_cache.shape
        q = torch.empty((T, nh * D), dtype=out_dtype, device=qkv.device)
        self.launches += 1
        self.k.qk_norm_write(_p(qkv), qkv.stride(0), _p(positions), _p(qn_w), _p(kn_w), float(eps), float(temp_coef),
                             int(temp_every), _p(slots), _p(q), _p(k_cache), _p(v_cache), T, nh, nkv, d, dv, D,
                             page_size, total_pages, _dt(out_dtype), self._stream())
        return q

    def rotate_heads(self, x, positions, inv_freq, rot_dims, heads, dim, off_a, scale_a, off_b, scale_b):
        """Rotary positions in place on two runs of heads of the 32-bit rows ``x`` (columns ``off_a`` and ``off_b``),
        each run then multiplied by its factor."""
        T = x.shape[0]
        assert x.dtype == torch.float32 and x.stride(1) == 1
        assert max(off_a, off_b) + heads * dim <= x.shape[1]
        self.launches += 1
        self.k.rotate_heads(_p(x), x.stride(0), _p(positions), _p(inv_freq), int(rot_dims), T, heads, dim, int(off_a),
                            float(scale_a), int(off_b), float(scale_b), self._stream())

    def branch_norm_add(self, resid, a, wa, b, wb, eps, coef):
        """``resid += coef * (rms_norm(a) * wa + rms_norm(b) * wb)`` (``b`` None: one branch); all 32-bit ``[T, H]``."""
        T, H = resid.shape
        assert a.shape == (T, H) and a.is_contiguous() and resid.is_contiguous() and (b is None or b.shape == (T, H))
        self.launches += 1
        self.k.branch_norm_add(_p(resid), _p(a), _p(wa), _p(b), _p(wb), float(eps), float(coef), T, H, self._stream())

    def rmsnorm_pair(self, x, wa, wb, eps, out_dtype):
        """Two RMS norms of the same 32-bit rows with one statistic: ``(x / rms(x) * wa, x / rms(x) * wb)``."""
        T, H = x.shape
        assert x.dtype == torch.float32 and x.is_contiguous() and wa.shape == (H,) and wb.shape == (H,)
        a = torch.empty((T, H), dtype=out_dtype, device=x.device)
        b = torch.empty((T, H), dtype=out_dtype, device=x.device)
        self.launches += 1
        self.k.rmsnorm_pair(_p(x), _p(wa), _p(wb), _p(a), _p(b), T, H, float(eps), _dt(out_dtype), self._stream())
        return a, b

    def concat_rows(self, a, b, out_dtype):
        """``[a | b]`` in ``out_dtype`` (a, b 32-bit ``[T, H]``)."""
        T, H = a.shape
        assert a.dtype == torch.float32 and b.shape == (T, H) and a.is_contiguous() and b.is_contiguous()
        out = torch.empty((T, 2 * H), dtype=out_dtype, device=a.device)
        self.launches += 1
        self.k.concat_rows(_p(a), _p(b), _p(out), T, H, _dt(out_dtype), self._stream())
        return out

    # ------------------------------------------------------- latent attention
    def latent_prep(self, proj, off_q, q_rank, qn_w, off_kv, rank, kvn_w, dr, inv_freq, rot_dims, positions, slots,
                    eps, cache, out_dtype, interleaved=False):
        """Normalises the query latent (returned, activation dtype; None when ``q_rank`` is 0: the design has none)
        and writes the token's cache row ``[normalised latent | rotated key part]`` at its slot.  ``interleaved``:
        rotary pairs are entries (2i, 2i + 1) instead of (i, i + rot_dims / 2)."""
        T = proj.shape[0]
        total_pages, one, page_size, width = cache.shape
        assert one == 1 and width == rank + dr and cache.dtype == out_dtype and proj.dtype == torch.float32
        cq = torch.empty((T, q_rank), dtype=out_dtype, device=proj.device) if q_rank else None
        self.launches += 1
        self.k.latent_prep(_p(proj), proj.stride(0), int(off_q), int(q_rank), _p(qn_w), int(off_kv), int(rank),
                           _p(kvn_w), int(dr), _p(inv_freq), int(rot_dims), int(bool(interleaved)), _p(positions),
                           _p(slots), float(eps), _p(cq), _p(cache), page_size, total_pages, T, _dt(out_dtype),
                           self._stream())
        return cq

    def latent_q_split(self, q, positions, inv_freq, rot_dims, H, dn, dr, out_dtype, interleaved=False):
        """Per head ``[dn plain | dr to be rotated]`` of ``q [T, H * (dn + dr)]`` (32-bit, may be a column slice) ->
        the plain parts head by head ``[H, T, dn]`` in ``out_dtype`` and the rotated parts ``[T, H, dr]`` in 32-bit."""
        T = q.shape[0]
        assert q.dtype == torch.float32 and q.shape[1] == H * (dn + dr) and q.stride(1) == 1
        qn = torch.empty((H, T, dn), dtype=out_dtype, device=q.device)
        qr = torch.empty((T, H, dr), dtype=torch.float32, device=q.device)
        self.launches += 1
        self.k.latent_q_split(_p(q), q.stride(0), _p(positions), _p(inv_freq), int(rot_dims), int(bool(interleaved)),
                              _p(qn), _p(qr), T, H, dn, dr, _dt(out_dtype), self._stream())
        return qn, qr

    # ------------------------------------- gated recurrences, per-head norms, norms on both sides of a sublayer
    def gated_scan(self, q, k, v, decay, beta, state, batch, heads, qk_heads, dk, dv, *, unit_eps=None, q_scale=1.0,
                   A_log=None, decay_bias=None, tau=None):
        """Recurrence with a state ``S [dk, dv]`` per head over each request's tokens: ``S <- diag(a) S``;
        ``u = beta (v - S^T k)`` (``beta`` raw ``[T, heads]``, sigmoid applied) or ``u = v`` (``beta`` None);
        ``S += k u^T``; ``o = S^T q``.  ``q, k [T, qk_heads * dk]``, ``v [T, heads * dv]``, all 32-bit and possibly
        column slices.  ``unit_eps`` given: q and k become unit vectors per head first; q is multiplied by
        ``q_scale``.  The decay is one per head, ``exp(-exp(A_log) softplus(decay + decay_bias))`` with ``decay``
        ``[T, heads]`` (``A_log`` given), or one per key channel, ``sigmoid(decay)^(1 / tau)`` with ``decay``
        ``[T, heads * dk]`` (``tau`` given).  ``state [slots, heads, dk, dv]`` is read and left up to date.  Returns o
        ``[T, heads * dv]`` in 32-bit."""
        T = v.shape[0]
        per_head = A_log is not None
        assert per_head != (tau is not None), "one decay per head (A_log) or one per key channel (tau)"
        for t in (q, k, v, decay) + ((beta,) if beta is not None else ()):
            assert t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[0] == T
        assert q.shape[1] == qk_heads * dk and k.shape[1] == qk_heads * dk and v.shape[1] == heads * dv
        assert decay.shape[1] == (heads if per_head else heads * dk) and (beta is None or beta.shape[1] == heads)
        assert state.shape[1:] == (heads, dk, dv) and state.dtype == torch.float32
        o = torch.empty((T, heads * dv), dtype=torch.float32, device=v.device)
        self.launches += 1
        self.k.gated_scan(_p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(decay), decay.stride(0),
                          _p(beta), 0 if beta is None else beta.stride(0), _p(A_log), _p(decay_bias), _p(state),
                          _p(batch.cu_q), _p(batch.state_slot), _p(o), heads * dv, batch.num_requests, heads, qk_heads,
                          dk, dv, int(unit_eps is not None), float(unit_eps or 0.0), float(q_scale),
                          0 if per_head else 1, float(tau or 0.0), self._stream())
        return o

    def head_norm_rope_write(self, qkv, positions, qn_w, kn_w, eps, inv_freq, rot_dims, interleaved, slots, k_cache,
                             v_cache, nh, nkv, d, dv, D, out_dtype):
        """RMS norm of every query and key head over its ``d`` entries (weights ``[d]`` shared by the heads; None: no
        norm), rotary positions on the first ``rot_dims`` entries, q returned ``[T, nh * D]`` and k, v written at the
        tokens' slots, every head ``D`` wide (zeros beyond its own size)."""
        T = qkv.shape[0]
        assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] >= (nh + nkv) * d + nkv * dv
        total_pages, nkv_c, page_size, D_c = k_cache.shape
        assert (nkv_c, D_c) == (nkv, D) and k_cache.dtype == out_dtype and v_cache.shape == k_cache.shape
        q = torch.empty((T, nh * D), dtype=out_dtype, device=qkv.device)
        self.launches += 1
        self.k.head_norm_rope_write(_p(qkv), qkv.stride(0), _p(positions), _p(qn_w), _p(kn_w), float(eps), _p(inv_freq),
                                    int(rot_dims), int(bool(interleaved)), _p(slots), _p(q), _p(k_cache), _p(v_cache), T,
                                    nh, nkv, d, dv, D, page_size, total_pages, _dt(out_dtype), self._stream())
        return q

    def head_gate(self, o, gate, nh, D, factor=1.0):
        """``o[t, h * D + i] *= factor * sigmoid(gate[t, h])`` in place (``gate`` 32-bit, may be a column slice)."""
        T = o.shape[0]
        assert o.shape[1] == nh * D and o.is_contiguous() and gate.dtype == torch.float32 and gate.shape == (T, nh)
        self.launches += 1
        self.k.head_gate(_p(o), _p(gate), gate.stride(0), T, nh, D, float(factor), _dt(o.dtype), self._stream())

    def norm_add_norm(self, resid, y, w_post, w_next, eps, out_dtype):
        """``resid += rms_norm(y) * w_post``; then, with ``w_next``, returns ``rms_norm(resid) * w_next`` in
        ``out_dtype`` (else None): a sublayer's closing norm, the add and the next sublayer's opening norm in one pass."""
        T, H = resid.shape
        assert resid.dtype == torch.float32 and resid.is_contiguous() and y.shape == (T, H) and y.is_contiguous()
        out = torch.empty((T, H), dtype=out_dtype, device=resid.device) if w_next is not None else None
        self.launches += 1
        self.k.norm_add_norm(_p(resid), _p(y), _p(w_post), _p(w_next), float(eps), _p(out), T, H, _dt(out_dtype),
                             self._stream())
        return out

    def add_vec_rows(self, x, x0, vec):
        """``x[t] += x0[t] + vec`` in place (``x0`` None: only the vector); all 32-bit."""
        T, H = x.shape
        assert x.dtype == torch.float32 and x.is_contiguous() and vec.shape == (H,) and vec.is_contiguous()
        assert x0 is None or (x0.shape == (T, H) and x0.is_contiguous() and x0.dtype == torch.float32)
        self.launches += 1
        self.k.add_vec_rows(_p(x), _p(x0), _p(vec), T, H, self._stream())

    # ------------------------------------- squashing norms and caps, a gate per entry, the max-gated matrix memory
    def dyt_norm(self, x, w, b, alpha, out_dtype, rows=None):
        """``tanh(alpha * x) * w + b`` of the 32-bit rows x (only ``rows`` of them when given) in ``out_dtype``."""
        H = x.shape[-1]
        assert x.dtype == torch.float32 and x.is_contiguous() and w.shape == (H,) and b.shape == (H,)
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, H), dtype=out_dtype, device=x.device)
        self.launches += 1
        self.k.dyt_norm(_p(x), _p(rows), _p(w), _p(b), float(alpha), _p(out), n, H, _dt(out_dtype), self._stream())
        return out

    def dyt_norm_pair(self, x, wa, ba, alpha_a, wb, bb, alpha_b, out_dtype, want_f32=False):
        """The same 32-bit rows through two such norms in one pass; with ``want_f32`` the second result also in
        32-bit: ``(a, b, b32 or None)``."""
        T, H = x.shape
        assert x.dtype == torch.float32 and x.is_contiguous()
        a = torch.empty((T, H), dtype=out_dtype, device=x.device)
        b = torch.empty((T, H), dtype=out_dtype, device=x.device)
        b32 = torch.empty((T, H), dtype=torch.float32, device=x.device) if want_f32 and out_dtype != torch.float32 else None
        self.launches += 1
        self.k.dyt_norm_pair(_p(x), _p(wa), _p(ba), float(alpha_a), _p(a), _p(wb), _p(bb), float(alpha_b), _p(b), _p(b32),
                             T, H, _dt(out_dtype), self._stream())
        return a, b, (b if want_f32 and b32 is None else b32)

    def tanh_cap(self, x, cap):
        """``x <- cap * tanh(x / cap)`` in place on a contiguous 32-bit tensor."""
        assert x.dtype == torch.float32 and x.is_contiguous()
        self.launches += 1
        self.k.tanh_cap(_p(x), x.numel(), float(cap), self._stream())

    def entry_gate(self, o, gate, nh, dv, D, factor=1.0, resid=None, bias=None):
        """``o[t, h * D + i] *= factor * sigmoid(gate[t, h * dv + i])`` for ``i < dv``, in place (``gate`` 32-bit,
        may be a column slice; heads stored ``D`` wide keep their padding).  With ``resid`` (32-bit ``[T, W]``) and
        ``bias`` (``[W]``) the same launch also does ``resid[t] += bias``."""
        T = o.shape[0]
        assert o.shape[1] == nh * D and o.is_contiguous() and gate.dtype == torch.float32
        assert gate.shape == (T, nh * dv) and gate.stride(1) == 1
        W = 0
        if resid is not None:
            W = resid.shape[1]
            assert resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape[0] == T
            assert bias is not None and bias.shape == (W,) and bias.dtype == torch.float32 and bias.is_contiguous()
        self.launches += 1
        self.k.entry_gate(_p(o), _p(gate), gate.stride(0), T, nh, dv, D, float(factor), _dt(o.dtype), _p(resid),
                          _p(bias if resid is not None else None), W, self._stream())

    def memory_scan(self, q, k, v, igate, fgate, i_bias, f_bias, cap, S, n, m, batch, heads, dk, dv, q_scale=1.0,
                    den_eps=1e-6):
        """Matrix memory with exponential gates and a running maximum over each request's tokens: with
        ``i = cap tanh((igate + i_bias) / cap)``, ``f = log sigmoid(cap tanh((fgate + f_bias) / cap))``:
        ``m' = max(f + m, i)``; ``S <- exp(f + m - m') S + exp(i - m') k v^T``; n likewise with k alone;
        ``o = S^T q`` (q times ``q_scale``).  ``q, k [T, heads * dk]``, ``v [T, heads * dv]``, ``igate, fgate
        [T, heads]``, all 32-bit and possibly column slices.  ``S [slots, heads, dk, dv]``, ``n [slots, heads, dk]``
        and ``m [slots, heads, dv + 1]`` (equal copies of the maximum) are read and left up to date.  Returns o
        ``[T, heads * dv]`` (not divided) and ``1 / (max(|n . q|, exp(-m')) + den_eps)`` ``[T, heads]``."""
        T = v.shape[0]
        for t in (q, k, v, igate, fgate):
            assert t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[0] == T
        assert q.shape[1] == heads * dk and k.shape[1] == heads * dk and v.shape[1] == heads * dv
        assert igate.shape[1] == heads and fgate.shape[1] == heads
        assert S.shape[1:] == (heads, dk, dv) and n.shape[1:] == (heads, dk) and m.shape[1:] == (heads, dv + 1)
        assert S.dtype == n.dtype == m.dtype == torch.float32
        o = torch.empty((T, heads * dv), dtype=torch.float32, device=v.device)
        rden = torch.empty((T, heads), dtype=torch.float32, device=v.device)
        self.launches += 1
        self.k.memory_scan(_p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(igate), igate.stride(0),
                           _p(fgate), fgate.stride(0), _p(i_bias), _p(f_bias), float(cap), _p(S), _p(n), _p(m),
                           _p(batch.cu_q), _p(batch.state_slot), _p(o), heads * dv, _p(rden), batch.num_requests, heads,
                           dk, dv, float(q_scale), float(den_eps), self._stream())
        return o, rden

    def head_offsets(self, H, T, device):
        """``[0, T, 2T, ..., H T]``: the groups of a grouped product whose groups are heads (kept: built once)."""
        key = (H, T, str(device))
        cache = self.__dict__.setdefault("_head_offsets", {})
        if key not in cache:
            if len(cache) > 4096:
                cache.clear()
            cache[key] = torch.arange(0, (H + 1) * T, T, dtype=torch.int32, device=device)
        return cache[key]

    def latent_attention(self, q_lat, q_rot, sink, cache, block_table, batch, H, dr, rank, window, scale):
        """Windowed attention over the cached latents with a sink per head.  ``q_lat [H, T, rank]`` (32-bit): the
        queries through W_uk; ``q_rot [T, H, dr]``.  Returns the normalised weighted sums of latent rows,
        ``[H, T, rank]`` in the cache's dtype."""
        T = q_rot.shape[0]
        total_pages, _, page_size, width = cache.shape
        assert q_lat.dtype == torch.float32 and q_lat.shape == (H, T, rank) and q_rot.shape == (T, H, dr)
        assert width == rank + dr and q_lat.is_contiguous() and q_rot.is_contiguous()
        lat = torch.empty((H, T, rank), dtype=cache.dtype, device=q_lat.device)
        # few tokens (a decode step): every token's keys are cut over several blocks and merged by a second kernel
        longest = getattr(batch, "max_kv_len", 0) or page_size * block_table.shape[1]
        max_keys = min(int(window), longest) if window else longest
        splits = self.k.latent_attention_splits(T, H, rank, dr, int(max_keys), _dt(cache.dtype), self.fast)
        partial = torch.empty((T * H * splits * (rank + 2),), dtype=torch.float32, device=q_lat.device) if splits > 1 else None
        self.launches += 2 if splits > 1 else 1
        self.k.latent_attention(_p(q_lat), _p(q_rot), _p(sink), _p(cache), _p(block_table), block_table.shape[1],
                                _p(batch.token_req), _p(batch.positions), _p(lat), _p(partial), splits, T, H, dr, rank,
                                page_size, total_pages, int(window), float(scale), _dt(cache.dtype), self.fast,
                                self._stream())
        return lat

    def latent_gate_out(self, val, gate, H, dv, out_dtype):
        """``out[t, h * dv + d] = val[h, t, d] * sigmoid(gate[t, h])`` (``gate`` None: 1) in ``out_dtype``."""
        T = val.shape[0] // H
        assert val.dtype == torch.float32 and val.shape == (H * T, dv) and val.is_contiguous()
        out = torch.empty((T, H * dv), dtype=out_dtype, device=val.device)
        self.launches += 1
        self.k.latent_gate_out(_p(val), _p(gate), 0 if gate is None else gate.stride(0), _p(out), T, H, dv,
                               _dt(out_dtype), self._stream())
        return out

    def rmsnorm(self, x, w, eps, out_dtype, rows=None):
        H = x.shape[-1]
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, H), dtype=out_dtype, device=x.device)
        self.launches += 1
        self.k.rmsnorm(_p(x), _p(w), _p(out), _p(rows), n, H, float(eps), _dt(out_dtype), self._stream())
        return out

    # -------------------------------------------------------------- products
    def _gemm(self, a, w, out, M, N, K, epilogue, *, bias=None, a_rows=None, offsets=None, num_experts=0,
              w_expert_stride=0, ldo=None):
        self.launches += 1
        self.k.gemm(_p(a), a.stride(0), _p(a_rows), _p(w), K, w_expert_stride, _p(offsets), num_experts, _p(bias),
                    _p(out), out.stride(0) if ldo is None else ldo, M, N, K, _dt(a.dtype), _dt(out.dtype), epilogue,
                    self.fast, self._stream())

    def linear(self, a, w, bias, out_dtype):
        (M, K), N = a.shape, w.shape[0]
        assert w.shape[1] == K and a.dtype == w.dtype
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        self._gemm(a, w, out, M, N, K, self.k.EPI_STORE, bias=bias)
        return out

    def linear_add(self, a, w, resid):
        (M, K), N = a.shape, w.shape[0]
        assert w.shape[1] == K and resid.shape == (M, N) and resid.dtype == torch.float32
        self._gemm(a, w, resid, M, N, K, self.k.EPI_ADD)

    def linear_act(self, a, w, act):
        """``act(a · w^T)`` in the activation dtype; ``act`` as in ``activation``.  Both forms of gelu are an epilogue
        of the product, the other activations a kernel behind a 32-bit product."""
        (M, K), N = a.shape, w.shape[0]
        assert w.shape[1] == K and a.dtype == w.dtype
        epi = {"gelu": self.k.EPI_GELU, "gelu_tanh": self.k.EPI_GELU_TANH}.get(act)
        if epi is not None:
            out = torch.empty((M, N), dtype=a.dtype, device=a.device)
            self._gemm(a, w, out, M, N, K, epi)
            return out
        return self.activation(self.linear(a, w, None, torch.float32), act, a.dtype)

    def linear_swiglu(self, a, w_gate_up):
        (M, K), N = a.shape, w_gate_up.shape[0]
        out = torch.empty((M, N // 2), dtype=a.dtype, device=a.device)
        self._gemm(a, w_gate_up, out, M, N, K, self.k.EPI_SWIGLU)
        return out

    def grouped_swiglu(self, a, w_gate_up, offsets, rows):
        E, N, K = w_gate_up.shape
        M = rows.numel()
        out = torch.empty((M, N // 2), dtype=a.dtype, device=a.device)
        if (self.fast and self.tc and a.dtype == torch.bfloat16 and 8 * M > 9 * E and K % 8 == 0
                and a.stride(0) == K):
            # more than about a row per expert (the kernels' own rule): put each expert's rows side by side, so that the TMA can fetch them as tiles
            gathered = torch.empty((M, K), dtype=a.dtype, device=a.device)
            self.launches += 1
            self.k.gather_rows(_p(a), _p(rows), _p(gathered), M, K, _dt(a.dtype), self._stream())
            self._gemm(gathered, w_gate_up, out, M, N, K, self.k.EPI_SWIGLU, offsets=offsets, num_experts=E,
                       w_expert_stride=N * K)
            return out
        self._gemm(a, w_gate_up, out, M, N, K, self.k.EPI_SWIGLU, a_rows=rows, offsets=offsets, num_experts=E,
                   w_expert_stride=N * K)
        return out

    def grouped_act(self, a, w_up, offsets, rows, act):
        """``act(a[rows] · w_up[e]^T)`` for each expert's rows, in the activation dtype (``act``: see
        ``activation``).  gelu sits in the product's epilogue; other activations are a kernel behind it."""
        E, N, K = w_up.shape
        M = rows.numel()
        fused = act == "gelu"
        out = torch.empty((M, N), dtype=a.dtype if fused else torch.float32, device=a.device)
        epi = self.k.EPI_GELU if fused else self.k.EPI_STORE
        if (self.fast and self.tc and a.dtype == torch.bfloat16 and 8 * M > 9 * E and K % 8 == 0
                and a.stride(0) == K):
            gathered = torch.empty((M, K), dtype=a.dtype, device=a.device)
            self.launches += 1
            self.k.gather_rows(_p(a), _p(rows), _p(gathered), M, K, _dt(a.dtype), self._stream())
            self._gemm(gathered, w_up, out, M, N, K, epi, offsets=offsets, num_experts=E, w_expert_stride=N * K)
        else:
            self._gemm(a, w_up, out, M, N, K, epi, a_rows=rows, offsets=offsets, num_experts=E, w_expert_stride=N * K)
        return out if fused else self.activation(out, act, a.dtype)

    def table_route(self, tokens, table, E):
        """Experts of each token from a table row of its id, each weighted ``1 / top``, grouped by expert:
        ``(ids, wts, offsets, rows, dest)`` as ``route`` gives them."""
        T = tokens.numel()
        V, top = table.shape
        assert table.dtype == torch.int32 and table.is_contiguous()
        ids = torch.empty((T, top), dtype=torch.int32, device=tokens.device)
        wts = torch.empty((T, top), dtype=torch.float32, device=tokens.device)
        self.launches += 1
        self.k.table_lookup(_p(tokens), _p(table), _p(ids), _p(wts), T, V, top, E, self._stream())
        offsets, rows, dest = self.moe_permute(ids, E)
        return ids, wts, offsets, rows, dest

    def grouped_linear(self, a, w, offsets):
        E, N, K = w.shape
        M = a.shape[0]
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
        self._gemm(a, w, out, M, N, K, self.k.EPI_STORE, offsets=offsets, num_experts=E, w_expert_stride=N * K)
        return out

    # ------------------------------------------------------------- attention
    def rope_kv_write(self, qkv, positions, inv_freq, rotary_dim, slots, k_cache, v_cache, nh, nkv, hd, out_dtype,
                      interleaved=False):
        """``interleaved``: rotary pairs are dims (2i, 2i + 1) instead of (i, i + rotary_dim / 2)."""
        T = qkv.shape[0]
        assert qkv.dtype == torch.float32 and qkv.shape[1] == (nh + 2 * nkv) * hd
        total_pages, nkv_c, page_size, hd_c = k_cache.shape
        assert (nkv_c, hd_c) == (nkv, hd) and k_cache.dtype == out_dtype
        q = torch.empty((T, nh * hd), dtype=out_dtype, device=qkv.device)
        self.launches += 1
        self.k.rope_kv_write(_p(qkv), _p(positions), _p(inv_freq), int(rotary_dim), int(bool(interleaved)), _p(slots),
                             _p(q), _p(k_cache),
                             _p(v_cache), T, nh, nkv, hd, page_size, total_pages, _dt(out_dtype), self._stream())
        return q

    def attention(self, q, k_cache, v_cache, block_table, cu_q, kv_len, window, scale, nh, nkv, hd, max_q_len,
                  max_kv_len, num_single=0, slopes=None, chunk=0, sinks=None, softcap=0.0):
        """``slopes`` (32-bit ``[nh]`` or None): a score loses ``slopes[head] * (query position - key position)``.
        ``chunk`` > 0: a query at p sees only keys from ``floor(p / chunk) * chunk`` on.  ``sinks`` (32-bit ``[nh]`` or
        None): the softmax's denominator also holds ``exp(sinks[head])``.  ``softcap`` c > 0: the scaled dot product
        becomes ``c tanh(. / c)`` first."""
        T = q.shape[0]
        R, width = block_table.shape
        total_pages, _, page_size, _ = k_cache.shape
        out = torch.empty_like(q)
        scratch = None
        if self.fast and num_single > 0:
            n = self.k.attention_scratch_floats(R, nh, nkv, hd, int(max_kv_len))
            if n > 0:
                scratch = torch.empty((n,), dtype=torch.float32, device=q.device)
        # the tensor-core decode kernel merges its key splits itself; the FMA one has a merge kernel behind it
        decode_kernels = 1 if (q.dtype == torch.bfloat16 and hd in (16, 32, 48, 64, 96, 128)) else 2
        self.launches += 1 if scratch is None else (decode_kernels if num_single == R else decode_kernels + 1)
        self.k.attention(_p(q), _p(k_cache), _p(v_cache), _p(block_table), width, _p(cu_q), _p(kv_len), _p(out), T, R,
                         nh, nkv, hd, page_size, total_pages, int(window), float(scale), _p(slopes), int(chunk), _p(sinks),
                         float(softcap), int(max_q_len), int(max_kv_len), int(num_single), _p(scratch), _dt(q.dtype), self.fast,
                         self._stream())
        return out

    # ------------------------------------------------------------------- moe
    def router_topk(self, h, w, E, k, norm, has_gate, norm_weight=None, eps=0.0, score="softmax", scale=1.0,
                    select_bias=None):
        """Scores (``score``: softmax over the experts, or a sigmoid of each logit), the k best (chosen on
        score + ``select_bias`` when that is given), optionally renormalised, times ``scale``.  ``h`` is one
        of: activations in the weights' dtype; the 32-bit residual together with ``norm_weight`` / ``eps``
        (the RMS norm then runs inside the kernel, in 32-bit); 32-bit activations that are already normalised."""
        T, H = h.shape
        assert w.shape == (E + (1 if has_gate else 0), H)
        assert h.dtype in (w.dtype, torch.float32) and (norm_weight is None or h.dtype == torch.float32)
        score_fn = {"softmax": 0, "sigmoid": 1}[score]
        h_is_f32 = int(norm_weight is None and h.dtype == torch.float32 and w.dtype != torch.float32)
        ids = torch.empty((T, k), dtype=torch.int32, device=h.device)
        wts = torch.empty((T, k), dtype=torch.float32, device=h.device)
        gate = torch.empty((T,), dtype=torch.float32, device=h.device) if has_gate else None
        logits = torch.empty((T, w.shape[0]), dtype=torch.float32, device=h.device)
        self.launches += 2
        self.k.router_topk(_p(h), _p(w), _p(norm_weight), float(eps), _p(logits), _p(ids), _p(wts), _p(gate), T, H,
                           E, k, int(norm), int(has_gate), _dt(w.dtype), h_is_f32, score_fn, float(scale),
                           _p(select_bias), self._stream())
        return ids, wts, gate

    def route(self, h, w, E, k, norm, has_gate, norm_weight=None, eps=0.0, score="softmax", scale=1.0,
              select_bias=None, input_settled=False, logit_bias=None):
        """``router_topk`` and ``moe_permute`` together: ``(ids, wts, gate, offsets, rows, dest)``.  A step
        of at most 48 tokens does all of it in one launch.  ``input_settled``: ``h`` was not written by the
        kernel launched just before this call (it is a step's residual and a norm kernel ran in between); a
        step of few tokens then works its logits out while that kernel ends."""
        T, H = h.shape
        assert w.shape == (E + (1 if has_gate else 0), H)
        assert h.dtype in (w.dtype, torch.float32) and (norm_weight is None or h.dtype == torch.float32)
        score_fn = {"softmax": 0, "sigmoid": 1}[score]
        if logit_bias is not None:
            # the router's own bias joins the logits before the softmax (and so the choice as well)
            assert score == "softmax" and select_bias is None and logit_bias.shape == (E,)
            score_fn, select_bias = 2, logit_bias
        h_is_f32 = int(norm_weight is None and h.dtype == torch.float32 and w.dtype != torch.float32)
        dev = h.device
        ids = torch.empty((T, k), dtype=torch.int32, device=dev)
        wts = torch.empty((T, k), dtype=torch.float32, device=dev)
        gate = torch.empty((T,), dtype=torch.float32, device=dev) if has_gate else None
        logits = torch.empty((T, w.shape[0]), dtype=torch.float32, device=dev)
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
        rows = torch.empty((T * k,), dtype=torch.int32, device=dev)
        dest = torch.empty((T, k), dtype=torch.int32, device=dev)
        self.launches += self.k.router_topk_permute(_p(h), _p(w), _p(norm_weight), float(eps), _p(logits), _p(ids), _p(wts), _p(gate),
                                   _p(offsets), _p(rows), _p(dest), T, H, E, k, int(norm), int(has_gate),
                                   _dt(w.dtype), h_is_f32, score_fn, float(scale), _p(select_bias),
                                                   int(bool(input_settled)), self._stream())
        return ids, wts, gate, offsets, rows, dest

    def moe_permute(self, ids, E):
        T, k = ids.shape
        n = T * k
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=ids.device)
        rows = torch.empty((n,), dtype=torch.int32, device=ids.device)
        dest = torch.empty((T, k), dtype=torch.int32, device=ids.device)
        self.launches += 1
        self.k.moe_permute(_p(ids), n, k, E, _p(offsets), _p(rows), _p(dest), self._stream())
        return offsets, rows, dest

    def moe_combine(self, y, dest, wts, shared, gate, resid, ids=None, num_real=0, passthrough=None, shared_scale=1.0):
        """``resid[t] += sum_j wts[t, j] y[dest[t, j]] + shared_scale * gate[t] * shared[t]`` (no gate: 1).  With
        ``ids``: a pair whose expert id is ``num_real`` or more reads ``passthrough[t]`` (32-bit ``[T, H]``) instead of
        a row of y (``y`` may be None when there are no other experts)."""
        T, H = resid.shape
        assert ids is None or (passthrough is not None and passthrough.shape == (T, H) and passthrough.is_contiguous()
                               and passthrough.dtype == torch.float32 and ids.shape == dest.shape)
        self.launches += 1
        self.k.moe_combine(_p(y), _p(dest), _p(wts), _p(shared), _p(gate), _p(resid), T, H, dest.shape[1], _p(ids),
                           int(num_real), _p(passthrough), float(shared_scale), self._stream())

    # -------------------------------------------------------------- sampling
    def argmax(self, logits):
        N, V = logits.shape
        out = torch.empty((N,), dtype=torch.int32, device=logits.device)
        nbytes = self.k.argmax_scratch_bytes(N, V)
        scratch = torch.empty((nbytes,), dtype=torch.uint8, device=logits.device) if nbytes else None
        self.launches += 2 if nbytes else 1
        self.k.argmax(_p(logits), _p(out), N, V, _p(scratch), self._stream())
        return out

    def sample(self, logits, params, top_k, u, seen_offsets, seen_tokens):
        N, V = logits.shape
        out = torch.empty((N,), dtype=torch.int32, device=logits.device)
        scratch = torch.empty((N, V), dtype=torch.float32, device=logits.device)
        self.launches += 1
        self.k.sample(_p(logits), _p(out), N, V, _p(params), _p(top_k), _p(u), _p(seen_offsets), _p(seen_tokens),
                      _p(scratch), self._stream())
        return out
