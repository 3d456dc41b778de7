"""Salolorn on the GPU.  Kernels alone against their plain PyTorch statements, with inputs made so that a fault shows
(one key that stands out just inside and just outside a chunk, at a page's border, far back; a sink that takes all the
weight; something written into a state hundreds of tokens ago, kept or removed); then the engine against the plain
model: every mixer alone, four configurations of unlike sizes under every cutting in both precisions, slots and pages
that are used again, long greedy decoding through the scheduler and the replayed graphs, the command line."""
import math
from types import SimpleNamespace

import pytest
import torch

import cuttings
import plain_salolorn as plain
from plain_ops import PlainOps
from salolorn_models import (CONFIGS, TOL, delta, dense, latent, left, one_layer, parallel, references, right, row_error,
                             tokens, within_limits, worst_ratio, write_model)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from dlm_b200.ops import native_ops
    return native_ops(fast=True)


@pytest.fixture(scope="module")
def slow_ops():
    from dlm_b200.ops import native_ops
    return native_ops(fast=False)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("salolorn_gpu")
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(base / name)
        tensors = write_model(cfg, folder, seed=len(name) + ord(name))
        out[name] = (folder, plain.PlainSalolorn(cfg, tensors))
    return out


def batch_of(lengths, slots, starts=None):
    """The fields of a step the kernels read, for requests that bring ``lengths`` tokens from ``starts`` on."""
    starts = starts or [0] * len(lengths)
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    i32 = dict(dtype=torch.int32, device=DEV)
    return SimpleNamespace(
        num_requests=len(lengths), cu_q=torch.tensor(cu, **i32), state_slot=torch.tensor(slots, **i32),
        token_req=torch.tensor([r for r, n in enumerate(lengths) for _ in range(n)], **i32),
        positions=torch.tensor([s + i for s, n in zip(starts, lengths) for i in range(n)], **i32))


def to_cpu(b):
    return SimpleNamespace(**{k: (v.cpu() if torch.is_tensor(v) else v) for k, v in vars(b).items()})


def randn(*shape, seed=0, std=1.0, dtype=torch.float32):
    return (std * torch.randn(*shape, generator=torch.Generator().manual_seed(seed))).to(DEV, dtype)


# ============================================================== kernels alone
@pytest.mark.parametrize("heads,qk_heads,dk,dv", [(4, 2, 12, 20), (2, 1, 32, 64), (3, 3, 64, 64), (4, 2, 128, 128),
                                                 (6, 3, 8, 4), (1, 1, 46, 38), (2, 2, 200, 24)])
def test_gated_scan_delta_rule(ops, heads, qk_heads, dk, dv):
    """The delta rule with a decay per head, unit vectors and shared query/key heads; inputs are column slices of a
    wider matrix; three requests whose states lie in slots of their own and are not zero at the start."""
    ref = PlainOps()
    lens = [9, 1, 37]
    T = sum(lens)
    Q, V = qk_heads * dk, heads * dv
    wide = randn(T, 2 * Q + V + 2 * heads + 3, seed=1)
    q, k, v = wide[:, 1:1 + Q], wide[:, 1 + Q:1 + 2 * Q], wide[:, 1 + 2 * Q:1 + 2 * Q + V]
    dec, beta = wide[:, 2 + 2 * Q + V:2 + 2 * Q + V + heads], wide[:, 2 + 2 * Q + V + heads:2 + 2 * Q + V + 2 * heads]
    A_log, bias = randn(heads, seed=2, std=0.7) - 1.0, randn(heads, seed=3)
    state = randn(5, heads, dk, dv, seed=4, std=0.2)
    b = batch_of(lens, [3, 0, 4])
    want_state = state.clone().cpu()
    c = lambda t: t.cpu()
    want = ref.gated_scan(c(q), c(k), c(v), c(dec), c(beta), want_state, to_cpu(b), heads, qk_heads, dk, dv, unit_eps=1e-6,
                          q_scale=dk ** -0.5, A_log=c(A_log), decay_bias=c(bias))
    got = ops.gated_scan(q, k, v, dec, beta, state, b, heads, qk_heads, dk, dv, unit_eps=1e-6, q_scale=dk ** -0.5,
                         A_log=A_log, decay_bias=bias)
    ops.check_errors()
    assert torch.allclose(got.cpu(), want, atol=2e-4, rtol=2e-4)
    assert torch.allclose(state.cpu(), want_state, atol=2e-4, rtol=2e-4)
    assert torch.equal(state[1].cpu(), want_state[1]) and torch.equal(state[2].cpu(), want_state[2])   # slots not named


@pytest.mark.parametrize("heads,dk,dv,tau", [(3, 10, 14, 8.0), (1, 46, 38, 1.0), (4, 32, 32, 16.0), (2, 64, 128, 4.0),
                                             (2, 128, 64, 2.5)])
def test_gated_scan_decay_per_key_channel(ops, heads, dk, dv, tau):
    """Linear attention whose state rows decay by sigmoid(z)^(1/tau), a factor per key channel; no removal."""
    ref = PlainOps()
    lens = [5, 40, 2]
    T = sum(lens)
    q, k, v = randn(T, heads * dk, seed=1), randn(T, heads * dk, seed=2), randn(T, heads * dv, seed=3)
    z = randn(T, heads * dk, seed=4, std=2.0) + 1.0
    state = randn(4, heads, dk, dv, seed=5, std=0.3)
    b = batch_of(lens, [2, 1, 3])
    want_state = state.clone().cpu()
    want = ref.gated_scan(q.cpu(), k.cpu(), v.cpu(), z.cpu(), None, want_state, to_cpu(b), heads, heads, dk, dv,
                          q_scale=dk ** -0.5, tau=tau)
    got = ops.gated_scan(q, k, v, z, None, state, b, heads, heads, dk, dv, q_scale=dk ** -0.5, tau=tau)
    ops.check_errors()
    assert torch.allclose(got.cpu(), want, atol=3e-4, rtol=3e-4)
    assert torch.allclose(state.cpu(), want_state, atol=3e-4, rtol=3e-4)


def test_gated_scan_keeps_and_removes_a_far_key(ops):
    """No decay (the raw decay very negative) and full write strength: the pair (k = e_5, v) written at token 0 is
    read back by q = e_5 at token 300, through three steps.  A later token with the same key direction and v = 0
    takes it out first; with write strength 0 it stays.  The read-out of token 0 already sees its own write."""
    heads, dk, dv, T = 1, 24, 20, 301
    q, k, v = torch.zeros(T, dk, device=DEV), torch.zeros(T, dk, device=DEV), torch.zeros(T, dv, device=DEV)
    q[:, 7] = 1.0                                      # most tokens ask for a direction that nothing is written to
    k[:, 9] = 1.0                                      # ... and write nothing (v = 0) somewhere else
    v0 = torch.arange(1, dv + 1, device=DEV).float()
    k[0] = 0
    k[0, 5], v[0] = 3.0, v0                            # unit vectors: the length of k does not matter
    q[0] = 0
    q[0, 5] = 1.0
    q[T - 1] = 0
    q[T - 1, 5] = 2.0
    dec = torch.full((T, 1), -60.0, device=DEV)        # softplus -> 0: g = 1
    beta = torch.full((T, 1), 40.0, device=DEV)        # sigmoid -> 1
    A_log, bias = torch.zeros(1, device=DEV), torch.zeros(1, device=DEV)
    state = torch.zeros(2, heads, dk, dv, device=DEV)

    def run(cuts):
        state.zero_()
        outs, at = [], 0
        for n in cuts:
            s = slice(at, at + n)
            outs.append(ops.gated_scan(q[s], k[s], v[s], dec[s], beta[s], state, batch_of([n], [1]), heads, heads, dk, dv,
                                       unit_eps=1e-6, q_scale=1.0, A_log=A_log, decay_bias=bias))
            at += n
        return torch.cat(outs)
    o = run((200, 2, 99))
    assert torch.allclose(o[T - 1], v0, rtol=1e-4) and torch.allclose(o[0], v0, rtol=1e-4)
    assert float(o[1:T - 1].abs().max()) == 0.0
    k[150] = 0
    k[150, 5] = 1.0                                    # the same direction, nothing to write: removal
    o = run((T,))
    assert float(o[T - 1].abs().max()) < 1e-4 * float(v0.max())
    beta[150] = -40.0                                  # write strength 0: nothing happens
    o = run((149, 3, 149))
    assert torch.allclose(o[T - 1], v0, rtol=1e-4)
    dec[150] = 3.0                                     # one token that decays: exp(-exp(0) softplus(3))
    o = run((T,))
    assert torch.allclose(o[T - 1], v0 * math.exp(-math.log1p(math.exp(3.0))), rtol=1e-4)


def test_gated_scan_channel_decay_remembers_and_forgets(ops):
    """Decay per key channel: channel 3 keeps (z large), channel 4 forgets (z very negative).  What token 0 wrote
    through channel 3 is there 250 tokens later, what it wrote through channel 4 is gone after one token."""
    heads, dk, dv, T = 1, 8, 6, 251
    q, k, v = torch.zeros(T, dk, device=DEV), torch.zeros(T, dk, device=DEV), torch.zeros(T, dv, device=DEV)
    z = torch.full((T, dk), 40.0, device=DEV)
    z[:, 4] = -40.0
    v0 = torch.arange(1, dv + 1, device=DEV).float()
    k[0, 3], k[0, 4], v[0] = 1.0, 1.0, v0
    q[0, 4] = q[1, 4] = 1.0
    q[T - 1, 3] = 1.0
    state = torch.zeros(1, heads, dk, dv, device=DEV)
    outs, at = [], 0
    for n in (1, 1, 120, 129):
        s = slice(at, at + n)
        outs.append(ops.gated_scan(q[s], k[s], v[s], z[s], None, state, batch_of([n], [0]), heads, heads, dk, dv,
                                   q_scale=1.0, tau=2.0))
        at += n
    o = torch.cat(outs)
    assert torch.allclose(o[0], v0, rtol=1e-5)          # the key's own step does not decay it
    assert float(o[1].abs().max()) < 1e-6               # sigmoid(-40)^(1/2) ~ 2e-9
    assert torch.allclose(o[T - 1], v0, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,D,rot,interleaved,normed", [
    (6, 3, 24, 40, 48, 16, False, True), (4, 4, 10, 6, 16, 10, False, True), (8, 2, 64, 64, 64, 32, False, True),
    (4, 1, 128, 96, 128, 128, True, True), (2, 1, 12, 20, 32, 0, False, True), (3, 1, 20, 20, 32, 8, True, False)])
def test_head_norms_rotation_and_paged_write(ops, dtype, nh, nkv, d, dv, D, rot, interleaved, normed):
    """Per-head RMS norms with a weight shared by the heads, the rotation on part of a head in either pairing, q out
    and k, v into their pages, heads padded to the stored size; tokens of two requests at positions of their own."""
    ref = PlainOps()
    ps, pages = 16, 6
    b = batch_of([5, 30], [0, 1], starts=[11, 0])
    T = 35
    proj = randn(T, (nh + nkv) * d + nkv * dv + nh, seed=1)              # a gate's columns behind q, k, v
    qn, kn = (randn(d, seed=2, std=0.3) + 2.0, randn(d, seed=3, std=0.3) + 1.0) if normed else (None, None)
    inv_freq = (1000.0 ** (-torch.arange(0, max(rot, 2), 2).float() / max(rot, 2))).to(DEV)
    slot_list = [3 * ps + 11 + i for i in range(5)] + [(5 if i < 16 else 1) * ps + i % ps for i in range(30)]
    slot_list[7] = -1                                                    # a token whose key is not kept
    slots = torch.tensor(slot_list, dtype=torch.int32, device=DEV)
    kc, vc = randn(pages, nkv, ps, D, seed=4, dtype=dtype), randn(pages, nkv, ps, D, seed=5, dtype=dtype)
    kw, vw = kc.clone().cpu(), vc.clone().cpu()
    cpu = lambda t: None if t is None else t.cpu()
    want = ref.head_norm_rope_write(proj.cpu(), b.positions.cpu(), cpu(qn), cpu(kn), 1e-5, inv_freq.cpu(), rot, interleaved,
                                    slots.cpu(), kw, vw, nh, nkv, d, dv, D, dtype)
    got = ops.head_norm_rope_write(proj, b.positions, qn, kn, 1e-5, inv_freq, rot, interleaved, slots, kc, vc, nh, nkv, d,
                                   dv, D, dtype)
    ops.check_errors()
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    for a, w in ((got, want), (kc, kw), (vc, vw)):
        assert torch.allclose(a.float().cpu(), w.float(), **tol)
    if D > d:
        assert float(got.reshape(T, nh, D)[:, :, d:].abs().max()) == 0.0


def test_rotation_makes_scores_a_function_of_the_distance(ops):
    """q at p and k at j, both rotated by the kernel: their product equals that of q at p - j and k at 0."""
    nh = nkv = 1
    d = 16
    inv_freq = (300.0 ** (-torch.arange(0, d, 2).float() / d)).to(DEV)
    x = randn(1, 3 * d, seed=7)
    for interleaved in (False, True):
        rows = []
        for p in (50, 37, 13, 0):
            pos = torch.tensor([p], dtype=torch.int32, device=DEV)
            kc, vc = torch.zeros(1, 1, 16, d, device=DEV), torch.zeros(1, 1, 16, d, device=DEV)
            q = ops.head_norm_rope_write(x, pos, None, None, 1e-5, inv_freq, d, interleaved,
                                         torch.tensor([0], dtype=torch.int32, device=DEV), kc, vc, nh, nkv, d, d, d,
                                         torch.float32)
            rows.append((q[0].clone(), kc[0, 0, 0].clone()))
        (q50, _), (_, k37), (q13, _), (_, k0) = rows
        assert abs(float(q50 @ k37) - float(q13 @ k0)) < 1e-4 * float(q13.norm() * k0.norm())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_per_head_norm_add_norm_and_pass_entry(ops, dtype):
    ref = PlainOps()
    T, nh, D, W = 9, 5, 24, 200
    o, gate = randn(T, nh * D, seed=1, dtype=dtype), randn(T, nh + 3, seed=2)[:, 2:2 + nh]
    want = o.clone().cpu()
    ref.head_gate(want, gate.cpu(), nh, D, 1.3)
    ops.head_gate(o, gate, nh, D, 1.3)
    assert torch.allclose(o.float().cpu(), want.float(), atol=1e-5 if dtype == torch.float32 else 3e-2, rtol=1e-2)
    # rows that stay in shared memory, rows that take a larger block, and rows too long to stay there
    for W in (200, 2304, 5400):
        _norm_add_norm_case(ops, ref, T, W, dtype)
    W = 200
    x, x0, vec = randn(T, W, seed=7), randn(T, W, seed=8), randn(W, seed=9)
    a = x.clone()
    ops.add_vec_rows(a, None, vec)
    assert torch.equal(a, x + vec)
    ops.add_vec_rows(a, x0, vec)
    assert torch.allclose(a, x + vec + x0 + vec, atol=1e-6)
    ops.check_errors()


def _norm_add_norm_case(ops, ref, T, W, dtype):
    resid, y = randn(T, W, seed=3), randn(T, W, seed=4, std=5.0)
    w1, w2 = randn(W, seed=5, std=0.2) + 1.0, randn(W, seed=6, std=0.2) + 0.7
    for nxt in (w2, None):
        r_want = resid.clone().cpu()
        n_want = ref.norm_add_norm(r_want, y.cpu(), w1.cpu(), None if nxt is None else nxt.cpu(), 1e-5, dtype)
        r_got = resid.clone()
        n_got = ops.norm_add_norm(r_got, y, w1, nxt, 1e-5, dtype)
        assert torch.allclose(r_got.cpu(), r_want, atol=1e-5, rtol=1e-5)
        assert (n_got is None) == (nxt is None)
        if nxt is not None:
            assert n_got.dtype == dtype
            assert torch.allclose(n_got.float().cpu(), n_want.float(), atol=1e-5 if dtype == torch.float32 else 2e-2, rtol=1e-2)


# ------------------------------------------------------------------ attention inside chunks, with a sink
def paged(reqs, nkv, hd, ps, dtype, seed, drop_before=None):
    """reqs: [(kv_len, q_len)].  Pages scattered over the pool; ``drop_before[r]``: positions below it have no page
    any more (the table holds -1 there).  Returns k, v, table, cu_q, kv_len."""
    total = sum(-(-n // ps) for n, _ in reqs) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    k, v = randn(total, nkv, ps, hd, seed=seed + 1, dtype=dtype), randn(total, nkv, ps, hd, seed=seed + 2, dtype=dtype)
    table = torch.full((len(reqs), max(-(-n // ps) for n, _ in reqs) + 1), -1, dtype=torch.int32)
    cu, it = [0], iter(perm)
    for r, (n, ql) in enumerate(reqs):
        for i in range(-(-n // ps)):
            page = next(it)
            if drop_before is None or (i + 1) * ps > drop_before[r]:
                table[r, i] = page
        cu.append(cu[-1] + ql)
    i32 = dict(dtype=torch.int32, device=DEV)
    return k, v, table.to(DEV), torch.tensor(cu, **i32), torch.tensor([n for n, _ in reqs], **i32)


CHUNK_CASES = [
    # nh, nkv, hd, page, chunk, [(kv_len, q_len)]
    (6, 3, 48, 16, 37, [(100, 100), (75, 1), (74, 1), (38, 2), (37, 37), (112, 40)]),
    (4, 4, 16, 16, 5, [(33, 33), (11, 1), (10, 1), (26, 7)]),
    (8, 2, 64, 64, 64, [(300, 300), (129, 1), (128, 1), (193, 66), (64, 64), (65, 65)]),
    (4, 1, 128, 64, 200, [(700, 700), (401, 1), (400, 1), (601, 203), (1000, 130)]),
    (6, 2, 64, 16, 120, [(500, 260), (121, 1), (120, 1), (240, 1), (241, 1), (1, 1)]),
    (2, 1, 32, 16, 100000, [(150, 150), (90, 1)]),
    (12, 2, 64, 64, 24, [(25, 1), (24, 1), (49, 1), (47, 1), (500, 1), (96, 1), (97, 1)]),       # single tokens only
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,ps,chunk,reqs", CHUNK_CASES)
@pytest.mark.parametrize("fast", [False, True])
@pytest.mark.parametrize("sink", [False, True])
def test_attention_inside_chunks(ops, slow_ops, dtype, nh, nkv, hd, ps, chunk, reqs, fast, sink):
    """Every attention kernel (FMA, warp-level prefill, both decode kernels) with a chunked mask and a sink, prompts'
    portions that start inside a chunk and cross several, single tokens at a chunk's first and last position; pages
    of chunks that have passed are gone."""
    o, ref = (ops if fast else slow_ops), PlainOps()
    drop = [((n - ql) // chunk) * chunk for n, ql in reqs]
    k, v, table, cu_q, kv_len = paged(reqs, nkv, hd, ps, dtype, 21, drop_before=drop)
    T = int(cu_q[-1])
    q = randn(T, nh * hd, seed=22, dtype=dtype)
    sinks = (randn(nh, seed=23, std=2.0) + 1.0) if sink else None
    scale = 0.9 / math.sqrt(hd)
    mq, mk = max(ql for _, ql in reqs), max(n for n, _ in reqs)
    ns = sum(1 for _, ql in reqs if ql == 1)
    got = o.attention(q, k, v, table, cu_q, kv_len, 0, scale, nh, nkv, hd, mq, mk, ns, chunk=chunk, sinks=sinks)
    want = ref.attention(q.cpu(), k.cpu(), v.cpu(), table.cpu(), cu_q.cpu(), kv_len.cpu(), 0, scale, nh, nkv, hd, mq, mk,
                         chunk=chunk, sinks=None if sinks is None else sinks.cpu())
    o.check_errors()
    tol = dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=1.5e-2)
    assert torch.allclose(got.float().cpu(), want.float(), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fast", [False, True])
@pytest.mark.parametrize("chunk,ps", [(16, 16), (17, 16), (5, 16), (64, 64), (40, 64), (120, 64), (33, 16), (128, 64)])
@pytest.mark.parametrize("q_len", [1, 2, 50])
def test_attention_finds_the_key_at_the_chunks_edge(ops, slow_ops, dtype, fast, chunk, ps, q_len):
    """The first key of the last query's chunk stands out and must be the answer; the key before it (the last of the
    chunk before) stands out even more and must not be seen.  The query is the last of a portion of 1, 2 or 50
    tokens, at a chunk's last position, so the loud key is as far back as the mask allows."""
    o = ops if fast else slow_ops
    nh, nkv, hd = 4, 2, 64
    n = 4 * chunk                                       # the last position is the last of the fourth chunk
    ql = min(q_len, n)
    k, v, table, cu_q, kv_len = paged([(n, ql)], nkv, hd, ps, dtype, 31)
    q = randn(ql, nh * hd, seed=32, dtype=dtype)
    for h in range(nh):
        q[-1, h * hd:(h + 1) * hd] = q[-1, (h // 2) * 2 * hd:((h // 2) * 2 + 1) * hd]     # one query per group
    first = 3 * chunk
    for j, boost in ((first, 25.0), (first - 1, 50.0)):
        page, off = int(table[0, j // ps]), j % ps
        for g in range(nkv):
            k[page, g, off] = (q[-1, g * 2 * hd:(g * 2 + 1) * hd].float() * boost).to(dtype)
    got = o.attention(q, k, v, table, cu_q, kv_len, 0, 1 / math.sqrt(hd), nh, nkv, hd, ql, n, 1 if ql == 1 else 0,
                      chunk=chunk, sinks=None)
    o.check_errors()
    page, off = int(table[0, first // ps]), first % ps
    for h in range(nh):
        assert torch.allclose(got[-1, h * hd:(h + 1) * hd].float(), v[page, h // 2, off].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("fast", [False, True])
@pytest.mark.parametrize("q_len", [1, 9])
def test_sink_takes_its_share_of_the_weight(ops, slow_ops, fast, q_len):
    """A chunk's first position sees only itself: with a sink s the output is v * e^x / (e^x + e^s), x its own score;
    a very large sink leaves nothing, a very negative one changes nothing.  The sink is not multiplied by the scale."""
    o = ops if fast else slow_ops
    nh, nkv, hd, ps, chunk = 2, 1, 32, 16, 9
    n = 3 * chunk + 1                                   # the last position opens the fourth chunk
    for dtype in (torch.float32, torch.bfloat16):
        k, v, table, cu_q, kv_len = paged([(n, q_len)], nkv, hd, ps, dtype, 51)
        q = randn(q_len, nh * hd, seed=52, dtype=dtype)
        page, off = int(table[0, (n - 1) // ps]), (n - 1) % ps
        scale = 0.2
        x = torch.stack([(q[-1, h * hd:(h + 1) * hd].float() @ k[page, 0, off].float()) * scale for h in range(nh)])
        for sinks in (torch.tensor([0.5, -1.0]), torch.tensor([80.0, -80.0])):
            sinks = sinks.to(DEV)
            got = o.attention(q, k, v, table, cu_q, kv_len, 0, scale, nh, nkv, hd, q_len, n, 1 if q_len == 1 else 0,
                              chunk=chunk, sinks=sinks)
            w = torch.exp(x) / (torch.exp(x) + torch.exp(sinks))
            for h in range(nh):
                want = w[h] * v[page, 0, off].float()
                assert torch.allclose(got[-1, h * hd:(h + 1) * hd].float(), want, rtol=2e-2, atol=1e-2 if dtype == torch.bfloat16 else 1e-5)
    o.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_with_direct_queries_and_neighbour_pairs(ops, dtype):
    """The latent attention's preparation without a query latent and with the rotation on pairs (2i, 2i + 1): cache
    rows and the split query against their plain statement."""
    ref = PlainOps()
    H, dn, dr, rank = 3, 20, 12, 40
    T, ps = 21, 16
    b = batch_of([T], [0], starts=[5])
    width = H * (dn + dr) + rank + dr
    proj = randn(T, width, seed=1)
    kvn = randn(rank, seed=2, std=0.2) + 1.5
    inv_freq = (1000.0 ** (-torch.arange(0, dr, 2).float() / dr)).to(DEV)
    slots = torch.tensor([2 * ps + 5 + i if i < 11 else i - 11 for i in range(T)], dtype=torch.int32, device=DEV)
    cache = torch.zeros(3, 1, ps, rank + dr, device=DEV, dtype=dtype)
    want_cache = cache.clone().cpu()
    off_kv = H * (dn + dr)
    for interleaved in (True, False):
        cq_w = ref.latent_prep(proj.cpu(), 0, 0, None, off_kv, rank, kvn.cpu(), dr, inv_freq.cpu(), dr, b.positions.cpu(),
                               slots.cpu(), 1e-5, want_cache, dtype, interleaved=interleaved)
        cq = ops.latent_prep(proj, 0, 0, None, off_kv, rank, kvn, dr, inv_freq, dr, b.positions, slots, 1e-5, cache, dtype,
                             interleaved=interleaved)
        assert cq is None and cq_w is None
        tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
        assert torch.allclose(cache.float().cpu(), want_cache.float(), **tol)
        qn_w, qr_w = ref.latent_q_split(proj.cpu()[:, :off_kv], b.positions.cpu(), inv_freq.cpu(), dr, H, dn, dr, dtype,
                                        interleaved=interleaved)
        qn, qr = ops.latent_q_split(proj[:, :off_kv], b.positions, inv_freq, dr, H, dn, dr, dtype, interleaved=interleaved)
        assert torch.allclose(qn.float().cpu(), qn_w.float(), **tol) and torch.allclose(qr.cpu(), qr_w, atol=2e-5, rtol=2e-5)
    ops.check_errors()


# ============================================================== the engine against the plain model
def gpu_engine(folder, dtype, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype=dtype, device=DEV, page_size=16, num_pages=64, max_requests=4)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


def worst_error(got, ref):
    return max(float(row_error(row, ref[rid][p])) for (rid, p), row in got.items())


LAYERS = {
    "delta": delta(4, 2, 12, 20, 3),
    "delta_one_tap": delta(2, 2, 16, 8, 1),
    "latent": latent(3, 20, 12, 28, 40, 0.15, 1000.0),
    "pair": parallel(left(6, 3, 24, 40, 0.2, 13, 5000.0, 16), right(3, 10, 14, 8.0), 0.7, 1.4),
    "pair_no_rotation": parallel(left(2, 1, 12, 20, 0.25, 7, 100.0, 0), right(1, 46, 38, 1.0), 1.0, 0.5),
}


@pytest.mark.parametrize("kind", list(LAYERS))
@pytest.mark.parametrize("mlp", [None, dense(56)])
@pytest.mark.parametrize("loop", [None, {"start": 0, "stop": 1, "times": 2}])
def test_each_mixer_alone(kind, mlp, loop, tmp_path):
    """A model of one layer: the mixer (and the feed-forward) alone, whole, token by token and in portions of two;
    also run twice as a repeated pass, each pass with a cache and state of its own."""
    cfg = one_layer(dict(LAYERS[kind], mlp=mlp), width=72, loop=loop)
    tensors = write_model(cfg, str(tmp_path / "m"), seed=11)
    oracle = plain.PlainSalolorn(cfg, tensors)
    reqs = {"a": tokens(1, 45, cfg["vocab"])}
    ref = {"a": oracle.forward(reqs["a"])}
    eng = gpu_engine(str(tmp_path / "m"), "float32")
    for steps in (cuttings.whole(reqs), cuttings.tail_decode(reqs, 44), cuttings.portions(reqs, sizes=(2,))):
        assert worst_error(cuttings.run_trace(eng, steps), ref) < TOL["float32"]


def test_residual_after_every_layer_run(folders):
    folder, oracle = folders["A"]
    toks = tokens(3, 50, CONFIGS["A"]["vocab"])
    _, after = oracle.forward(toks, trace=True)
    eng = gpu_engine(folder, "float32")
    seen = []
    eng.model.after_layer = lambda call, x: seen.append(x.detach().double().cpu())
    slot = eng.cache.open()
    eng.step([(slot, toks, [])])
    eng.cache.close(slot)
    assert len(seen) == after.shape[0]
    for i, x in enumerate(seen):
        assert float((x - after[i]).abs().max() / after[i].abs().max()) < 1e-4, i


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_matches_the_plain_model(name, dtype, folders):
    """Prefill against decoding token by token, portions down to two tokens, unequal requests batched against each
    alone, requests long enough for chunks to end at and inside pages in prompts and in decoding."""
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": tokens(i, n, V) for i, n in enumerate([1, 2, 23, 150, 310])}
    ref, lim = references(oracle, reqs, dtype)
    page = 64 if name == "C" else 16
    eng = gpu_engine(folder, dtype, page_size=page, num_pages=1024 // page)
    mixed, _ = cuttings.mixed(reqs, max_live=4, seed=1, decode_tail=70 if name == "A" else 24)
    for what, steps in (("whole", cuttings.whole(reqs)), ("decode", cuttings.tail_decode(reqs, 140)),
                        ("portions", cuttings.portions(reqs)), ("mixed", mixed)):
        got = cuttings.run_trace(eng, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        worst = worst_error(got, ref)
        print(f"{name} {dtype} {what}: worst relative error {worst:.2e}, worst error / limit {worst_ratio(got, ref, lim):.2f}")
        assert within_limits(got, ref, lim) and (dtype == "bfloat16" or worst_ratio(got, ref, lim) < 1.0), (what, worst)
    assert all(p.used_pages == 0 for p in eng.cache.stats())


def test_cuttings_agree_to_the_last_bit_in_32_bit(folders):
    """In 32-bit every kernel adds in an order of its own that does not depend on the cut: logits are equal bit for
    bit whether a request came whole, token by token, or beside others."""
    folder, _ = folders["A"]
    V = CONFIGS["A"]["vocab"]
    reqs = {f"r{i}": tokens(30 + i, n, V) for i, n in enumerate([5, 60, 33])}
    eng = gpu_engine(folder, "float32")
    base = cuttings.run_trace(eng, cuttings.whole(reqs))
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=4)
    for steps in (cuttings.tail_decode(reqs, 30), cuttings.portions(reqs, sizes=(2, 3)), mixed):
        got = cuttings.run_trace(eng, steps)
        assert all(torch.equal(got[k], base[k]) for k in base)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype, folders):
    folder, oracle = folders["A"]
    V = CONFIGS["A"]["vocab"]
    reqs = {f"q{i}": tokens(20 + i, n, V) for i, n in enumerate([70, 33, 129, 16, 90, 7, 64, 65])}
    steps, _ = cuttings.mixed(reqs, max_live=3, seed=2)
    eng = gpu_engine(folder, dtype, num_pages=cuttings.peak_tokens(steps) // 16, max_requests=3)
    got = cuttings.run_trace(eng, steps)
    ref, lim = references(oracle, reqs, dtype)
    assert within_limits(got, ref, lim)
    assert all(s.used_pages == 0 for s in eng.cache.stats())


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("A", "bfloat16"), ("C", "bfloat16")])
def test_long_greedy_generation_through_scheduler_and_graphs(name, dtype, folders):
    """Engine.generate: prompts in portions under a token budget, then 200 decode steps replayed from graphs, state
    carried in the slots all the way and chunks passing under the decoded tokens.  Every produced token is the plain
    model's choice wherever that is clear, and the logits of the last step agree."""
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    prompts = [tokens(60, 70, V), tokens(61, 3, V), tokens(62, 129, V)]
    page = 64 if name == "C" else 16
    eng = gpu_engine(folder, dtype, page_size=page, num_pages=2048 // page, max_step_tokens=48, max_context=512)
    assert eng.use_graphs
    news = [200, 40, 90]
    ids = [eng.submit(p, max_new_tokens=n) for p, n in zip(prompts, news)]
    last = {}
    while eng.scheduler.has_work():
        produced = eng.run_step()
        if len(produced) == 1 and eng.last_logits.shape[0] == 1:
            last["row"] = eng.last_logits[0].float().cpu().clone()
    outs = [eng.result(i) for i in ids]
    assert eng.graphs_recorded > 0 and [len(o) for o in outs] == news
    seqs = {str(i): p + out[:-1] for i, (p, out) in enumerate(zip(prompts, outs))}
    ref, lim = references(oracle, seqs, dtype)
    clear = 0
    for i, (p, out) in enumerate(zip(prompts, outs)):
        for j, tok in enumerate(out):
            at = len(p) - 1 + j
            row = ref[str(i)][at]
            top2 = torch.topk(row, 2).values
            spread = float((row - row.mean()).pow(2).mean().sqrt())
            if float(top2[0] - top2[1]) > 4 * float(lim[str(i)][at]) * spread:      # the plain model's choice is clear
                assert int(torch.argmax(row)) == tok, (name, dtype, i, j)
                clear += 1
    print(f"{name} {dtype}: {clear} of {sum(news)} tokens were clear choices")
    assert clear >= sum(news) // 8
    assert float(row_error(last["row"], ref["0"][-1]) / lim["0"][-1]) < 1.0


def test_command_line_with_random_weights(tmp_path):
    """`dlm-b200 generate --random CONFIG.json --save-random DIR`: the architecture is found through the registry, the
    weights are drawn and written, and the ids printed are the plain model's greedy choices on that folder."""
    import ast
    import json
    import os
    import subprocess
    import sys
    from plain_zesapel import read_safetensors            # the file format alone, nothing of the package
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_path, folder = str(tmp_path / "config.json"), str(tmp_path / "model")
    with open(cfg_path, "w") as f:
        json.dump(CONFIGS["A"], f)
    prompts = [[5, 6, 7, 100, 3], [9]]
    cmd = [sys.executable, os.path.join(root, "bin", "dlm-b200"), "generate", "--random", cfg_path, "--seed", "3",
           "--save-random", folder, "--max-new-tokens", "6", "--dtype", "float32"]
    for p in prompts:
        cmd += ["--prompt", ",".join(str(t) for t in p)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("generated ids:")]
    assert len(lines) == len(prompts)
    oracle = plain.PlainSalolorn(CONFIGS["A"], read_safetensors(os.path.join(folder, "model.safetensors")))
    for p, ln in zip(prompts, lines):
        ids = ast.literal_eval(ln.split(":", 1)[1].strip())
        assert len(ids) == 6
        seq = list(p)
        for tok in ids:
            row = oracle.forward(seq)[-1]
            top2 = torch.topk(row, 2).values
            spread = float((row - row.mean()).pow(2).mean().sqrt())
            if float(top2[0] - top2[1]) > 1e-3 * spread:
                assert int(torch.argmax(row)) == tok
            seq.append(tok)


MID = {"architecture": "Salolorn", "vocab": 1000, "width": 320, "norm": {"eps": 1e-6}, "logit_scale": 0.8,
       "loop": {"start": 1, "stop": 3, "times": 2},
       "layers": [latent(5, 48, 16, 40, 96, 0.12, 1e4, dense(448)), delta(6, 3, 48, 80, 4, dense(512)),
                  parallel(left(10, 5, 80, 48, 0.11, 100, 1e4, 40), right(5, 24, 72, 6.0), 0.9, 1.1, dense(384)),
                  delta(4, 4, 96, 32, 2)]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_a_long_request(dtype, tmp_path):
    """Sizes between the tiny configurations and a real model's (products large enough for the tensor-core kernels,
    head sizes that are no power of two, chunks of 100 positions over pages of 64), a request of 700 tokens beside
    short ones: whole, decoded, in portions and mixed."""
    tensors = write_model(MID, str(tmp_path / "m"), seed=5)
    oracle = plain.PlainSalolorn(MID, tensors)
    reqs = {f"r{i}": tokens(i, n, MID["vocab"]) for i, n in enumerate([37, 130, 700])}
    ref, lim = references(oracle, reqs, dtype)
    eng = gpu_engine(str(tmp_path / "m"), dtype, page_size=64, num_pages=32)
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=2, decode_tail=40)
    for what, steps in (("whole", cuttings.whole(reqs)), ("decode", cuttings.tail_decode(reqs, 110)),
                        ("portions", cuttings.portions(reqs)), ("mixed", mixed)):
        got = cuttings.run_trace(eng, steps)
        eng.rt.ops.check_errors()
        assert worst_ratio(got, ref, lim) < 1.0, (what, worst_ratio(got, ref, lim))
