"""Faguzen on the GPU.  Kernels alone against their plain PyTorch statements, with inputs made so that a fault shows
(scores far above the cap that must count alike, one key far back or at a page's border that must be found, something
written into the memory hundreds of tokens ago, a gate that lifts the running maximum, identity experts that must
hand the input through); then the engine against the plain model: single layers with every kind of feed-forward,
four configurations of unlike sizes under every cutting in both precisions, slots and pages that are used again, long
greedy decoding through the scheduler and the replayed graphs, the command line."""
import math
from types import SimpleNamespace

import pytest
import torch

import cuttings
import plain_faguzen as plain
from plain_ops import PlainOps
from faguzen_models import (CONFIGS, TOL, layer, left, moe, mostly_within_limits, one_layer, ratios, references, right,
                            row_error, tokens, within_limits, write_model)

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
    base = tmp_path_factory.mktemp("faguzen_gpu")
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(base / name)
        tensors = write_model(cfg, folder, seed=len(name) + ord(name))
        out[name] = (folder, plain.PlainFaguzen(cfg, tensors))
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
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W", [(1, 48), (37, 62), (300, 1024), (5, 2051)])
def test_norm_without_statistics_alone_and_in_pairs(ops, dtype, T, W):
    ref = PlainOps()
    x = randn(T, W, seed=1, std=3.0)
    wa, ba, wb, bb = (randn(W, seed=s, std=0.3) + m for s, m in ((2, 1.0), (3, 0.0), (4, 0.8), (5, 0.1)))
    tol = dict(atol=1e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=1e-2, rtol=1e-2)
    got = ops.dyt_norm(x, wa, ba, 0.6, dtype)
    assert got.dtype == dtype and torch.allclose(got.float().cpu(), ref.dyt_norm(x.cpu(), wa.cpu(), ba.cpu(), 0.6, dtype).float(), **tol)
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    got = ops.dyt_norm(x, wa, ba, 1.7, dtype, rows)
    assert torch.allclose(got.float().cpu(), ref.dyt_norm(x.cpu(), wa.cpu(), ba.cpu(), 1.7, dtype, rows.cpu()).float(), **tol)
    a, b, b32 = ops.dyt_norm_pair(x, wa, ba, 0.6, wb, bb, 1.3, dtype, want_f32=True)
    assert torch.allclose(a.float().cpu(), ref.dyt_norm(x.cpu(), wa.cpu(), ba.cpu(), 0.6, dtype).float(), **tol)
    assert torch.allclose(b.float().cpu(), ref.dyt_norm(x.cpu(), wb.cpu(), bb.cpu(), 1.3, dtype).float(), **tol)
    assert b32.dtype == torch.float32
    assert torch.allclose(b32.cpu(), ref.dyt_norm(x.cpu(), wb.cpu(), bb.cpu(), 1.3, torch.float32), atol=1e-6, rtol=1e-5)
    # a saturated entry is the weight plus the bias, with the sign of the input
    big = torch.full((1, W), 1e4, device=DEV)
    assert torch.allclose(ops.dyt_norm(big, wa, ba, 0.5, torch.float32)[0], wa + ba)
    assert torch.allclose(ops.dyt_norm(-big, wa, ba, 0.5, torch.float32)[0], ba - wa)
    ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cap_on_logits_and_gate_per_entry(ops, dtype):
    ref = PlainOps()
    x = randn(7, 333, seed=1, std=20.0)
    want = x.clone().cpu()
    ref.tanh_cap(want, 12.5)
    ops.tanh_cap(x, 12.5)
    assert torch.allclose(x.cpu(), want, atol=1e-5, rtol=1e-5) and float(x.abs().max()) <= 12.5
    for T, nh, dv, D in ((5, 6, 40, 48), (33, 2, 64, 64), (2, 3, 5, 16), (300, 8, 96, 128)):
        o = randn(T, nh * D, seed=2, dtype=dtype)
        wide = randn(T, nh * dv + 9, seed=3, std=2.0)
        gate = wide[:, 4:4 + nh * dv]                                    # a column slice
        want = o.clone().cpu()
        ref.entry_gate(want, gate.cpu(), nh, dv, D, 0.7)
        before = o.clone()
        ops.entry_gate(o, gate, nh, dv, D, 0.7)
        assert torch.allclose(o.float().cpu(), want.float(), atol=1e-6 if dtype == torch.float32 else 2e-2, rtol=1e-2)
        pad = o.reshape(T, nh, D)[:, :, dv:]
        assert torch.equal(pad, before.reshape(T, nh, D)[:, :, dv:])     # the heads' padding is not touched
        # the same launch may add a bias to every token's row of the residual
        o2, resid, bias = before.clone(), randn(T, 70, seed=4), randn(70, seed=5)
        want_resid = resid.cpu() + bias.cpu()
        ops.entry_gate(o2, gate, nh, dv, D, 0.7, resid=resid, bias=bias)
        assert torch.equal(o2, o) and torch.allclose(resid.cpu(), want_resid, atol=1e-6)
    ops.check_errors()


@pytest.mark.parametrize("heads,dk,dv", [(3, 10, 14), (1, 46, 38), (2, 64, 128), (4, 32, 64), (2, 128, 64), (6, 8, 4),
                                         (2, 40, 56), (1, 200, 24)])
def test_memory_scan_against_its_plain_statement(ops, heads, dk, dv):
    """The matrix memory with a running maximum; inputs are column slices of a wider matrix; three requests whose
    states lie in slots of their own and are not zero at the start."""
    ref = PlainOps()
    lens = [9, 1, 37]
    T = sum(lens)
    Q, V = heads * dk, heads * dv
    wide = randn(T, 2 * Q + V + 2 * heads + 3, seed=1)
    q, k, v = wide[:, 1:1 + Q], wide[:, 1 + Q:1 + 2 * Q], wide[:, 1 + 2 * Q:1 + 2 * Q + V]
    ig = wide[:, 2 + 2 * Q + V:2 + 2 * Q + V + heads] * 3.0
    fg = wide[:, 2 + 2 * Q + V + heads:2 + 2 * Q + V + 2 * heads] * 3.0
    ib, fb = randn(heads, seed=2), randn(heads, seed=3) + 1.0
    S, n = randn(5, heads, dk, dv, seed=4, std=0.2), randn(5, heads, dk, seed=5, std=0.2)
    m = (randn(5, heads, 1, seed=6).expand(5, heads, dv + 1)).contiguous()
    b = batch_of(lens, [3, 0, 4])
    wS, wn, wm = S.clone().cpu(), n.clone().cpu(), m.clone().cpu()
    c = lambda t: t.cpu()
    want_o, want_r = ref.memory_scan(c(q), c(k), c(v), c(ig), c(fg), c(ib), c(fb), 5.0, wS, wn, wm, to_cpu(b), heads, dk, dv,
                                     q_scale=dk ** -0.5, den_eps=1e-6)
    got_o, got_r = ops.memory_scan(q, k, v, ig, fg, ib, fb, 5.0, S, n, m, b, heads, dk, dv, q_scale=dk ** -0.5, den_eps=1e-6)
    ops.check_errors()
    assert torch.allclose(got_o.cpu(), want_o, atol=3e-4, rtol=3e-4)
    assert torch.allclose(got_r.cpu(), want_r, atol=1e-5, rtol=3e-4)
    for got, want in ((S, wS), (n, wn), (m, wm)):
        assert torch.allclose(got.cpu(), want, atol=3e-4, rtol=3e-4)
        assert torch.equal(got[1].cpu(), want[1]) and torch.equal(got[2].cpu(), want[2])       # slots not named
    assert torch.equal(m[..., :1].expand_as(m), m)                                            # the copies stay equal


def test_memory_scan_remembers_a_far_key_and_follows_the_maximum(ops):
    """Forget gates of one (a large raw value) and one loud write at token 0: q = e_5 at token 300 reads it back through
    three steps, with (S, n, m) carried.  The input gate of token 0 is the cap itself, so m jumps there and every
    later, quieter write counts exp(i - m) only; the denominator is |n . q| while that is above exp(-m), else
    exp(-m).  Cutting the tokens anywhere gives the same bits."""
    heads, dk, dv, T, cap = 1, 24, 20, 301, 8.0
    q, k, v = torch.zeros(T, dk, device=DEV), torch.zeros(T, dk, device=DEV), torch.zeros(T, dv, device=DEV)
    q[:, 7] = 1.0                                      # most tokens ask for a direction that nothing is written to
    k[:, 9] = 1.0                                      # ... and write v = 0 somewhere else, quietly
    v0 = torch.arange(1, dv + 1, device=DEV).float()
    k[0] = 0
    k[0, 5], v[0] = 1.0, v0
    q[0] = 0
    q[0, 5] = 1.0
    q[T - 1] = 0
    q[T - 1, 5] = 2.0
    ig = torch.full((T, 1), -3.0, device=DEV)
    ig[0] = 100.0                                      # capped: i = 8
    fg = torch.full((T, 1), 100.0, device=DEV)         # capped to 8: f = log sigmoid(8), about -3.4e-4 a token
    zero = torch.zeros(1, device=DEV)
    S, n = torch.zeros(2, heads, dk, dv, device=DEV), torch.zeros(2, heads, dk, device=DEV)
    m = torch.zeros(2, heads, dv + 1, device=DEV)

    def run(cuts):
        S.zero_(); n.zero_(); m.zero_()
        outs, dens, at = [], [], 0
        for c in cuts:
            s = slice(at, at + c)
            o, r = ops.memory_scan(q[s], k[s], v[s], ig[s], fg[s], zero, zero, cap, S, n, m, batch_of([c], [1]), heads, dk,
                                   dv, q_scale=1.0, den_eps=1e-6)
            outs.append(o); dens.append(r); at += c
        return torch.cat(outs), torch.cat(dens)

    o, r = run([T])
    f = math.log(1 / (1 + math.exp(-cap)))
    # token 0: m = 8, S = k v^T, n = k: o = v0, den = max(1, e^-8) + 1e-6
    assert torch.allclose(o[0], v0, rtol=1e-5) and float(r[0]) == pytest.approx(1 / (1 + 1e-6), rel=1e-5)
    # the last token: m has sunk by 300 f, the write has decayed as much relative to it: S = k v^T exactly still
    m_last = cap + 300 * f
    assert float(m[1, 0, 0]) == pytest.approx(m_last, rel=1e-5)
    assert torch.allclose(o[T - 1], 2.0 * v0, rtol=1e-4)
    assert float(r[T - 1]) == pytest.approx(1 / (2.0 + 1e-6), rel=1e-4)
    # tokens in between read a direction that holds nothing: o = 0 and the denominator is exp(-m)
    assert float(o[150].abs().max()) == 0.0
    assert float(r[150]) == pytest.approx(1 / (math.exp(-(cap + 150 * f)) + 1e-6), rel=1e-4)
    assert torch.equal(S[0], torch.zeros_like(S[0]))                                          # the other slot
    for cuts in ([1, 299, 1], [100, 100, 101], [2] * 150 + [1], [37, 264]):
        o2, r2 = run(cuts)
        assert torch.equal(o2, o) and torch.equal(r2, r)
    ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_a_factor_per_row(ops, dtype):
    ref = PlainOps()
    T, groups, gs = 23, 3, 14
    y, gate = randn(T, groups * gs, seed=1, std=4.0), randn(T, groups * gs, seed=2, std=2.0)
    w = randn(groups * gs, seed=3, std=0.2) + 1.0
    scale = randn(T, groups, seed=4).abs() * 1e-3                      # small factors: the eps must meet the scaled values
    for mode in ("sigmoid_after", "silu_after"):
        got = ops.gated_rmsnorm(y, gate, w, groups, 1e-5, mode, dtype, row_scale=scale)
        want = ref.gated_rmsnorm(y.cpu(), gate.cpu(), w.cpu(), groups, 1e-5, mode, dtype, row_scale=scale.cpu())
        plain_norm = ref.gated_rmsnorm(y.cpu(), gate.cpu(), w.cpu(), groups, 1e-5, mode, dtype)
        assert torch.allclose(got.float().cpu(), want.float(), atol=1e-5 if dtype == torch.float32 else 2e-2, rtol=1e-2)
        assert not torch.allclose(want.float(), plain_norm.float(), atol=1e-2)
    ops.check_errors()


def paged(reqs, nkv, hd, ps, dtype, seed):
    """reqs: [(kv_len, q_len)].  Pages scattered over the pool.  Returns k, v, table, cu_q, kv_len."""
    total = sum(-(-n // ps) for n, _ in reqs) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    k, v = randn(total, nkv, ps, hd, seed=seed + 1, dtype=dtype), randn(total, nkv, ps, hd, seed=seed + 2, dtype=dtype)
    table = torch.full((len(reqs), max(-(-n // ps) for n, _ in reqs) + 1), -1, dtype=torch.int32)
    cu, it = [0], iter(perm)
    for r, (n, ql) in enumerate(reqs):
        for i in range(-(-n // ps)):
            table[r, i] = next(it)
        cu.append(cu[-1] + ql)
    i32 = dict(dtype=torch.int32, device=DEV)
    return k, v, table.to(DEV), torch.tensor(cu, **i32), torch.tensor([n for n, _ in reqs], **i32)


CAP_CASES = [
    # nh, nkv, hd, page, [(kv_len, q_len)]
    (6, 3, 48, 16, [(100, 100), (75, 1), (38, 2), (112, 40)]),
    (4, 4, 16, 16, [(33, 33), (11, 1), (26, 7)]),
    (8, 2, 64, 64, [(300, 300), (129, 1), (128, 1), (193, 66)]),
    (4, 1, 128, 64, [(700, 700), (401, 1), (601, 203)]),
    (6, 2, 96, 64, [(500, 260), (121, 1), (1, 1)]),
    (3, 1, 40, 16, [(90, 90), (77, 1)]),                                                    # no tensor-core kernel
    (12, 2, 64, 64, [(25, 1), (24, 1), (500, 1), (97, 1)]),                                  # single tokens only
    (8, 8, 128, 64, [(1000, 1), (64, 1), (65, 1)]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,ps,reqs", CAP_CASES)
@pytest.mark.parametrize("fast", [False, True])
@pytest.mark.parametrize("cap", [2.0, 25.0])
def test_attention_with_capped_scores(ops, slow_ops, dtype, nh, nkv, hd, ps, reqs, fast, cap):
    """Every attention kernel (FMA, warp-level prefill, both decode kernels) with squashed scores: a small cap that
    bends most scores and a large one that bends few."""
    o, ref = (ops if fast else slow_ops), PlainOps()
    k, v, table, cu_q, kv_len = paged(reqs, nkv, hd, ps, dtype, 21)
    T = int(cu_q[-1])
    q = randn(T, nh * hd, seed=22, dtype=dtype)
    scale = 3.0 / math.sqrt(hd)
    mq, mk = max(ql for _, ql in reqs), max(n for n, _ in reqs)
    ns = sum(1 for _, ql in reqs if ql == 1)
    got = o.attention(q, k, v, table, cu_q, kv_len, 0, scale, nh, nkv, hd, mq, mk, ns, softcap=cap)
    want = ref.attention(q.cpu(), k.cpu(), v.cpu(), table.cpu(), cu_q.cpu(), kv_len.cpu(), 0, scale, nh, nkv, hd, mq, mk,
                         softcap=cap)
    uncapped = ref.attention(q.cpu(), k.cpu(), v.cpu(), table.cpu(), cu_q.cpu(), kv_len.cpu(), 0, scale, nh, nkv, hd, mq, mk)
    o.check_errors()
    tol = dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=1.5e-2)
    assert torch.allclose(got.float().cpu(), want.float(), **tol)
    if cap == 2.0:
        assert not torch.allclose(want.float(), uncapped.float(), rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fast", [False, True])
@pytest.mark.parametrize("hd,ps", [(64, 64), (128, 64), (48, 16), (40, 16)])
@pytest.mark.parametrize("q_len", [1, 2, 70])
def test_two_loud_keys_count_alike_under_the_cap(ops, slow_ops, dtype, fast, hd, ps, q_len):
    """The very first key of a long request and the last key of a page in its middle both stand far above the cap (one
    twice as far as the other): the last query must find both and weigh them alike, so its output is the mean of their
    values.  Without the cap only the louder one would count."""
    o = ops if fast else slow_ops
    nh, nkv = 4, 2
    n = 5 * ps + 3
    k, v, table, cu_q, kv_len = paged([(n, q_len)], nkv, hd, ps, dtype, 31)
    q = randn(q_len, nh * hd, seed=32, dtype=dtype)
    for h in range(nh):
        q[-1, h * hd:(h + 1) * hd] = q[-1, (h // 2) * 2 * hd:((h // 2) * 2 + 1) * hd]     # one query per group
    k *= 0.01                                           # every other key is quiet
    spots = ((0, 40.0), (3 * ps - 1, 80.0))
    for j, boost in spots:
        page, off = int(table[0, j // ps]), j % ps
        for g in range(nkv):
            k[page, g, off] = (q[-1, g * 2 * hd:(g * 2 + 1) * hd].float() * boost).to(dtype)
    cap = 20.0
    got = o.attention(q, k, v, table, cu_q, kv_len, 0, 1 / math.sqrt(hd), nh, nkv, hd, q_len, n, 1 if q_len == 1 else 0,
                      softcap=cap)
    o.check_errors()
    vals = [v[int(table[0, j // ps]), :, j % ps].float() for j, _ in spots]                  # [nkv, hd] each
    for h in range(nh):
        want = 0.5 * (vals[0][h // 2] + vals[1][h // 2])
        assert torch.allclose(got[-1, h * hd:(h + 1) * hd].float(), want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 7, 40, 300])
def test_choice_on_corrected_scores_and_identity_experts(ops, dtype, T):
    """The router's choice is made on score + correction, the weights are the scores over their sum times a factor;
    in the weighted sum an identity expert reads the token's own row; the shared expert counts with the same factor."""
    ref = PlainOps()
    W, E, ident, k = 64, 5, 3, 3
    x = randn(T, W, seed=1)
    w_r = randn(E + ident, W, seed=2, std=0.5, dtype=dtype)
    corr = randn(E + ident, seed=3, std=0.3)
    ids, wts, _, offsets, rows, dest = ops.route(x, w_r, E + ident, k, 2, False, select_bias=corr, scale=0.7)
    wi, ww, _ = ref.router_topk(x.cpu(), w_r.cpu(), E + ident, k, 2, False, select_bias=corr.cpu(), scale=0.7)
    logits = x.cpu() @ w_r.float().cpu().T
    s = torch.softmax(logits, -1)
    pick = torch.sort(s + corr.cpu(), -1, descending=True).values
    clear = (pick[:, k - 1] - pick[:, k]) > 1e-4
    assert torch.equal(ids.cpu()[clear], wi[clear]) and torch.allclose(wts.cpu()[clear], ww[clear], atol=1e-5, rtol=1e-4)
    assert torch.allclose(wts.sum(-1).cpu(), torch.full((T,), 0.7), atol=1e-5)
    assert bool((ids >= E).any()) and not torch.equal(ids.cpu(), torch.topk(s, k).indices.to(torch.int32))
    y = randn(T * k, W, seed=4)
    y[dest.reshape(-1).long()[(ids.reshape(-1) >= E)]] = float("nan")      # rows of identity pairs are never read
    shared = randn(T, W, seed=5)
    resid = randn(T, W, seed=6)
    want = resid.clone().cpu()
    ref.moe_combine(torch.nan_to_num(y).cpu(), dest.cpu(), wts.cpu(), shared.cpu(), None, want, ids=ids.cpu(), num_real=E,
                    passthrough=x.cpu(), shared_scale=0.7)
    ops.moe_combine(y, dest, wts, shared, None, resid, ids=ids, num_real=E, passthrough=x, shared_scale=0.7)
    ops.check_errors()
    assert torch.allclose(resid.cpu(), want, atol=1e-5, rtol=1e-5)
    # only identity experts: nothing but the token's own row and the shared expert
    ids0 = torch.zeros_like(ids)
    resid2 = torch.zeros(T, W, device=DEV)
    ops.moe_combine(None, dest, wts, shared, None, resid2, ids=ids0, num_real=0, passthrough=x, shared_scale=0.7)
    assert torch.allclose(resid2, 0.7 * (x + shared), atol=1e-5, rtol=1e-5)


# ============================================================== the engine against the plain model
def gpu_engine(folder, dtype, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype=dtype, device=DEV, page_size=16, num_pages=64, max_requests=4)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


def worst_error(got, ref):
    return max(float(row_error(row, ref[rid][p])) for (rid, p), row in got.items())


@pytest.mark.parametrize("mlp", [None, moe(3, 0, 3, 10), moe(0, 3, 2, 1), moe(4, 2, 1, 12, 20)])
@pytest.mark.parametrize("loop", [None, {"start": 0, "stop": 1, "times": 2}])
@pytest.mark.parametrize("rot", [False, True])
def test_a_single_layer(mlp, loop, rot, tmp_path):
    """One layer alone in 32-bit: no feed-forward, every expert chosen, identity experts only, one expert of several
    beside a shared one; with and without a rotation and a cap; whole, token by token and in portions of two."""
    lf = left(6, 3, 24, 40, 0.2, 6.0, 5000.0, 16, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}) if rot \
        else left(2, 1, 12, 20, 0.25)
    cfg = one_layer(layer(lf, right(3, 10, 14, 8.0), 0.7, 1.4, mlp), loop=loop, cap=5.0 if rot else 0.0)
    tensors = write_model(cfg, str(tmp_path / "m"), seed=4)
    oracle = plain.PlainFaguzen(cfg, tensors)
    reqs = {"a": tokens(1, 45, cfg["vocab"])}
    ref = {"a": oracle.forward(reqs["a"])}
    eng = gpu_engine(str(tmp_path / "m"), "float32")
    for steps in (cuttings.whole(reqs), cuttings.tail_decode(reqs, 44), cuttings.portions(reqs, sizes=(2,))):
        assert worst_error(cuttings.run_trace(eng, steps), ref) < TOL["float32"]


def test_steps_take_ordinary_launches_and_leave_the_setting_as_it_was(folders):
    """The design's spec asks for ordinary launches: inside a step the library's switch is off, after it the switch
    is what it was, whichever that was; another model's steps do not touch it."""
    folder, _ = folders["B"]
    eng = gpu_engine(folder, "float32")
    k = eng.rt.ops.k
    before = bool(k.dep_launch_enabled())
    seen = []
    eng.model.after_layer = lambda call, x: seen.append(bool(k.dep_launch_enabled()))
    try:
        for setting in (True, False):
            k.set_dep_launch(setting)
            seen.clear()
            slot = eng.cache.open()
            eng.step([(slot, tokens(1, 9, CONFIGS["B"]["vocab"]), [8])])
            eng.cache.close(slot)
            assert seen and not any(seen)
            assert bool(k.dep_launch_enabled()) is setting
    finally:
        k.set_dep_launch(before)
        eng.model.after_layer = None


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
    alone, requests long enough to span many pages in prompts and in decoding.  Positions whose choice of experts is
    a close call are not compared (and in bfloat16 the few behind them)."""
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": tokens(i, n, V) for i, n in enumerate([1, 2, 23, 150, 310])}
    ref, lim, ok = references(oracle, reqs, dtype)
    page = 64 if name == "C" else 16
    eng = gpu_engine(folder, dtype, page_size=page, num_pages=1024 // page)
    mixed, _ = cuttings.mixed(reqs, max_live=4, seed=1, decode_tail=70 if name == "A" else 24)
    for what, steps in (("whole", cuttings.whole(reqs)), ("decode", cuttings.tail_decode(reqs, 140)),
                        ("portions", cuttings.portions(reqs)), ("mixed", mixed)):
        got = cuttings.run_trace(eng, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        r = ratios(got, ref, lim, ok)
        print(f"{name} {dtype} {what}: {len(r)} of {len(got)} rows compared, worst error / limit {max(r):.2f}, "
              f"{sum(x > 1 for x in r)} over")
        if dtype == "float32":
            assert len(r) == len(got) and max(r) < 1.0, (what, max(r))
        else:
            assert len(r) > len(got) // 3 and within_limits(got, ref, lim, ok), (what, max(r))
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
    ref, lim, ok = references(oracle, reqs, dtype)
    assert within_limits(got, ref, lim, ok)
    assert all(s.used_pages == 0 for s in eng.cache.stats())


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("A", "float32"), ("C", "bfloat16")])
def test_long_greedy_generation_through_scheduler_and_graphs(name, dtype, folders):
    """Engine.generate: prompts in portions under a token budget, then 200 decode steps replayed from graphs, memory,
    normaliser and maximum carried in the slots all the way.  Every produced token is the plain model's choice wherever
    that is clear, and in 32-bit the logits of the last step agree."""
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
    ref, lim, ok = references(oracle, seqs, dtype)
    clear = 0
    for i, (p, out) in enumerate(zip(prompts, outs)):
        for j, tok in enumerate(out):
            at = len(p) - 1 + j
            row = ref[str(i)][at]
            top2 = torch.topk(row, 2).values
            spread = float((row - row.mean()).pow(2).mean().sqrt())
            if bool(ok[str(i)][at]) and float(top2[0] - top2[1]) > 4 * float(lim[str(i)][at]) * spread:
                assert int(torch.argmax(row)) == tok, (name, dtype, i, j)
                clear += 1
    print(f"{name} {dtype}: {clear} of {sum(news)} tokens were clear choices")
    assert clear >= sum(news) // 8
    if dtype == "float32":
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
    oracle = plain.PlainFaguzen(CONFIGS["A"], read_safetensors(os.path.join(folder, "model.safetensors")))
    for p, ln in zip(prompts, lines):
        ids = ast.literal_eval(ln.split(":", 1)[1].strip())
        assert len(ids) == 6
        seq = list(p)
        for tok in ids:
            row = oracle.forward(seq)[-1]
            top2 = torch.topk(row, 2).values
            spread = float((row - row.mean()).pow(2).mean().sqrt())
            if float(top2[0] - top2[1]) > 1e-3 * spread and float(oracle.last_gaps.min()) > 1e-4:
                assert int(torch.argmax(row)) == tok
            seq.append(tok)


MID = {"architecture": "Faguzen", "vocab": 1000, "width": 320, "norm": {"eps": 1e-6}, "residual_mult": 0.75,
       "logit_softcap": 12.0, "loop": {"start": 1, "stop": 3, "times": 2},
       "layers": [layer(left(10, 5, 80, 48, 0.11, 25.0, 1e4, 40, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}),
                        right(5, 24, 72, 10.0), 0.9, 1.1, moe(6, 2, 2, 192, 256)),
                  layer(left(5, 1, 64, 64, 0.125, 15.0, 1e4, 64), right(2, 96, 64, 6.0), 0.6, 1.2, moe(10, 0, 3, 96)),
                  layer(left(4, 4, 96, 128, 0.1, None, 500.0, 32), right(4, 48, 40, 14.0), 1.1, 0.7),
                  layer(left(6, 2, 48, 96, 0.14, 8.0), right(1, 128, 128, 9.0), 0.8, 0.9, moe(3, 3, 2, 320, 128))]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_a_long_request(dtype, tmp_path):
    """Sizes between the tiny configurations and a real model's (products large enough for the tensor-core kernels,
    head sizes that are no power of two, pages of 64), a request of 700 tokens beside short ones: whole, decoded, in
    portions and mixed."""
    tensors = write_model(MID, str(tmp_path / "m"), seed=5)
    oracle = plain.PlainFaguzen(MID, tensors)
    reqs = {f"r{i}": tokens(i, n, MID["vocab"]) for i, n in enumerate([37, 130, 700])}
    ref, lim, ok = references(oracle, reqs, dtype, carry=12 if dtype == "bfloat16" else None)
    eng = gpu_engine(str(tmp_path / "m"), dtype, page_size=64, num_pages=32)
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=2, decode_tail=40)
    for what, steps in (("whole", cuttings.whole(reqs)), ("decode", cuttings.tail_decode(reqs, 110)),
                        ("portions", cuttings.portions(reqs)), ("mixed", mixed)):
        got = cuttings.run_trace(eng, steps)
        eng.rt.ops.check_errors()
        r = ratios(got, ref, lim, ok)
        print(f"wider {dtype} {what}: {len(r)} of {len(got)} rows compared, worst error / limit {max(r):.2f}, "
              f"{sum(x > 1 for x in r)} over, median {sorted(r)[len(r) // 2]:.2f}")
        if dtype == "float32":
            assert max(r) < 1.0, (what, max(r))
        else:
            assert mostly_within_limits(got, ref, lim, ok), (what, max(r))


ODD = {"architecture": "Faguzen", "vocab": 1001, "width": 200, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
       "logit_softcap": 7.0, "loop": {"start": 1, "stop": 3, "times": 2},
       "layers": [layer(left(2, 2, 160, 72, 0.08, 11.0, 1e4, 160, {"factor": 2.0, "low": 2.0, "high": 16.0, "original": 512}),
                        right(1, 200, 300, 3.0), 0.3, 2.0, moe(33, 7, 6, 24, 88)),
                  layer(left(12, 4, 16, 8, 0.25, 1.5, 20.0, 2), right(5, 4, 3, 30.0), 1.5, 0.2, moe(1, 1, 1, 40)),
                  layer(left(3, 3, 80, 48, 0.1, 40.0), right(2, 72, 40, 8.0), 1.0, 1.0)]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unusual_sizes(dtype, tmp_path):
    """Heads wider than any tensor-core kernel takes (160) and tiny ones (16 x 8, 4 x 3), a memory of 200 x 300, a single
    memory head, more experts than a warp has lanes with six a token, one expert beside one identity expert, a loop
    that ends with the last layer, a rotation over two entries, a vocabulary that is no multiple of anything."""
    tensors = write_model(ODD, str(tmp_path / "m"), seed=11)
    oracle = plain.PlainFaguzen(ODD, tensors)
    reqs = {f"r{i}": tokens(i, n, ODD["vocab"]) for i, n in enumerate([3, 70, 260])}
    ref, lim, ok = references(oracle, reqs, dtype, carry=12 if dtype == "bfloat16" else None)
    eng = gpu_engine(str(tmp_path / "m"), dtype, page_size=64, num_pages=24)
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=2, decode_tail=30)
    for what, steps in (("whole", cuttings.whole(reqs)), ("decode", cuttings.tail_decode(reqs, 60)),
                        ("portions", cuttings.portions(reqs)), ("mixed", mixed)):
        got = cuttings.run_trace(eng, steps)
        eng.rt.ops.check_errors()
        r = ratios(got, ref, lim, ok)
        assert (max(r) < 1.0) if dtype == "float32" else mostly_within_limits(got, ref, lim, ok), (what, max(r))
