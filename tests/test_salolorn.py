"""Salolorn without a GPU: the config reader and registry, the order of layer calls with repeated passes, tensor
names and shapes, the plain implementation's own hand-made cases (one per mechanism), and the engine's host side
(cache, state slots, step function, scheduler, replay) with the plain PyTorch statement of the kernels standing in
for them."""
import copy
import io
import json
import math
import os
import sys

import numpy as np
import pytest
import torch

import cuttings
import plain_salolorn as plain
from plain_ops import PlainOps
from salolorn_models import (CONFIGS, TOL, delta, dense, latent, left, make_weights, one_layer, parallel, right,
                             row_error, tokens, write_model)

F64 = torch.float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("salolorn")
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(base / name)
        tensors = write_model(cfg, folder, seed=len(name) + ord(name))
        out[name] = (folder, plain.PlainSalolorn(cfg, tensors))
    return out


def cpu_engine(folder, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=40, max_requests=4)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


# ------------------------------------------------------------------ config, registry, tensors
def test_registry_resolves_the_architecture_and_round_trips_the_config():
    from dlm_b200.config import SalolornConfig
    from dlm_b200.registry import architectures, resolve
    assert "Salolorn" in architectures()
    for cfg in CONFIGS.values():
        name, typed, spec = resolve(copy.deepcopy(cfg))
        assert name == "Salolorn" and isinstance(typed, SalolornConfig)
        assert len(spec.layers) == len(cfg["layers"]) and spec.vocab_size == cfg["vocab"]
        assert spec.tie_word_embeddings and (spec.pass_entry is not None) == ("loop" in cfg)
        runs = len(cfg["layers"])
        if "loop" in cfg:
            runs += (cfg["loop"]["stop"] - cfg["loop"]["start"]) * (cfg["loop"]["times"] - 1)
        assert len(spec.order) == runs
        assert SalolornConfig.from_dict(typed.to_dict()) == typed
        assert typed.to_dict()["layers"] == cfg["layers"]


@pytest.mark.parametrize("edit,what", [
    (lambda c: c.pop("layers"), "layers"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].update(type="window_attention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("mask"), "mask"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][1]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=4), "rot"),
    (lambda c: c["layers"][1]["mlp"].update(kind="experts"), "mlp"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_refusals(edit, what):
    from dlm_b200.config import ConfigError
    from dlm_b200.registry import resolve
    cfg = copy.deepcopy(CONFIGS["A"])
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        resolve(cfg)
    assert what.split(".")[0] in str(e.value)


def test_tensor_names_and_shapes_are_the_checkpoints():
    from dlm_b200.parts import DecoderModel, Runtime, WeightError
    from dlm_b200.registry import resolve
    for name, cfg in CONFIGS.items():
        _, _, spec = resolve(copy.deepcopy(cfg))
        model = DecoderModel(spec, Runtime("cpu", torch.float32, None))
        tensors = make_weights(cfg)
        model.check({n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()})      # nothing missing, nothing extra
        for i, L in enumerate(cfg["layers"]):
            if L["mlp"] is None:
                assert not any(n.startswith(f"l{i}.mlp") or n.startswith(f"l{i}.norm2") for n in model.param_specs())
        assert ("loop.step" in model.param_specs()) == ("loop" in cfg)
        assert "head" not in model.param_specs()              # the embedding is the output matrix
    cfg = CONFIGS["A"]
    _, _, spec = resolve(copy.deepcopy(cfg))
    model = DecoderModel(spec, Runtime("cpu", torch.float32, None))
    bad = make_weights(cfg)
    bad.pop("l0.mix.q.conv")
    bad.pop("l1.mix.right.a2.b")
    bad["loop.step"] = torch.zeros(5, cfg["width"])
    bad["l1.mix.left.sink"] = torch.zeros(4)
    bad["l2.mix.dkv.norm"] = torch.zeros(7)
    with pytest.raises(WeightError) as e:
        model.check({n: (t.dtype, tuple(t.shape)) for n, t in bad.items()})
    for n in ("l0.mix.q.conv", "l1.mix.right.a2.b", "loop.step", "l1.mix.left.sink", "l2.mix.dkv.norm"):
        assert n in str(e.value)


def test_random_weights_for_a_config_build_and_load(tmp_path):
    from dlm_b200.config import SalolornConfig
    from dlm_b200.engine import Engine
    from dlm_b200.weights import write_random_model
    cfg = SalolornConfig.from_dict(copy.deepcopy(CONFIGS["D"]))
    folder = write_random_model(cfg, 5, str(tmp_path / "m"))
    toks = tokens(1, 20, cfg.vocab)
    a = cpu_engine(folder)
    b = Engine.from_random(cfg, 5, dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=8, max_requests=2)
    sa, sb = a.cache.open(), b.cache.open()
    la, lb = a.step([(sa, toks, [19])]), b.step([(sb, toks, [19])])
    assert torch.allclose(la, lb, atol=1e-5)
    assert torch.isfinite(la).all() and float(la.std()) > 0


# ------------------------------------------------- the plain implementation's own hand-made cases
def _mix_tensors(cfg, seed=3):
    t = {k: v.to(F64) for k, v in make_weights(cfg, seed).items()}
    return t, (lambda n: t["l0.mix." + n])


def test_plain_delta_rule_two_tokens_written_out():
    """Two tokens of the gated delta rule by hand: S1 = k1 (b1 v1)^T; S2 = g2 S1 + k2 (b2 (v2 - g2 S1^T k2))^T; the
    read-out sees the write of its own token.  Convolution, silu, unit vectors and the factor on q are spelled out."""
    m = {"heads": 2, "kv_heads": 1, "dim": 3, "vdim": 4, "conv": 2}
    cfg = one_layer({"type": "delta", "mixer": m, "mlp": None}, width=8)
    t, p = _mix_tensors(cfg)
    eps = 1e-5
    h = torch.randn(2, 8, dtype=F64, generator=torch.Generator().manual_seed(1))
    got = plain.delta_mixer(h, p, m, eps)

    def conv_silu(name):
        x, w = h @ p(name).T, p(name + ".conv")
        y = torch.stack([x[0] * w[:, 1], x[0] * w[:, 0] + x[1] * w[:, 1]])
        return y / (1 + torch.exp(-y))
    q, k, v = conv_silu("q"), conv_silu("k"), conv_silu("v").reshape(2, 2, 4)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(3)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = 1 / (1 + torch.exp(-(h @ p("b").T)))
    g = torch.exp(-torch.exp(p("A_log")) * torch.log1p(torch.exp(h @ p("a").T + p("dt_bias"))))
    gate = h @ p("g").T
    gate = (gate / (1 + torch.exp(-gate))).reshape(2, 2, 4)
    rows = []
    for n in range(2):
        S1 = torch.outer(k[0], beta[0, n] * v[0, n])
        o1 = S1.T @ q[0]
        S2 = g[1, n] * S1
        S2 = S2 + torch.outer(k[1], beta[1, n] * (v[1, n] - S2.T @ k[1]))
        rows.append(torch.stack([o1, S2.T @ q[1]]))
    o = torch.stack(rows, dim=1)                                             # [T, H, dv]
    y = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * p("norm") * gate
    assert torch.allclose(got, y.reshape(2, 8) @ p("o").T, rtol=1e-10, atol=1e-12)
    # a token's write is read back by the same token: with S = 0 before, o1 = (k1 . q1) b1 v1, not 0
    assert float(o[0].abs().max()) > 0


def test_plain_linear_attention_is_the_decayed_sum_over_the_past():
    """o_t = sum_j<=t (q_t * prod_{j<i<=t} alpha_i) . k_j  v_j, per head, with a decay per key channel."""
    m = right(2, 3, 5, 4.0)
    cfg = one_layer(parallel(left(2, 1, 4, 4, 0.5, 8, 100.0, 4), m, 1.0, 1.0), width=12)
    t, p0 = _mix_tensors(cfg)
    p = lambda n: p0("right." + n)
    T = 6
    h = torch.randn(T, 12, dtype=F64, generator=torch.Generator().manual_seed(2))
    got = plain.gated_linear_attention(h, p, m, 1e-5)
    q = (h @ p("q").T).reshape(T, 2, 3) / math.sqrt(3)
    k, v = (h @ p("k").T).reshape(T, 2, 3), (h @ p("v").T).reshape(T, 2, 5)
    z = (h @ p("a1").T) @ p("a2").T + p("a2.b")
    alpha = ((1 / (1 + torch.exp(-z))) ** 0.25).reshape(T, 2, 3)
    o = torch.zeros(T, 2, 5, dtype=F64)
    for i in range(T):
        for j in range(i + 1):
            w = alpha[j + 1:i + 1].prod(0)                                   # [H, d]; the key's own step does not decay it
            o[i] += ((q[i] * w * k[j]).sum(-1))[:, None] * v[j]
    y = (o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5) * p("norm")).reshape(T, 10)
    gate = h @ p("g").T
    y = y * gate / (1 + torch.exp(-gate))
    assert torch.allclose(got, y @ p("o").T, rtol=1e-9, atol=1e-12)


def test_plain_chunked_attention_edges_sink_and_gate():
    """A chunk's first position sees only itself: its output is gate * v * e^s / (e^s + e^sink).  A key in the chunk
    before is invisible however loud it is; the chunk's own first key is visible from the chunk's last position."""
    size = 5
    m = left(2, 1, 4, 3, 0.5, size, 100.0, 4)
    cfg = one_layer(parallel(m, right(1, 2, 2, 2.0), 1.0, 1.0), width=10)
    t, p0 = _mix_tensors(cfg)
    p = lambda n: p0("left." + n)
    T = 12
    h = torch.randn(T, 10, dtype=F64, generator=torch.Generator().manual_seed(3))
    out = plain.chunked_sink_attention(h, p, m, 1e-5)
    for i in (0, size, 2 * size):
        hi = h[i]
        q = plain.rms_norm((hi @ p("q").T).reshape(2, 4), p("q.norm"), 1e-5)
        k = plain.rms_norm((hi @ p("k").T).reshape(1, 4), p("k.norm"), 1e-5)
        s = (q * k).sum(-1) * 0.5                       # the rotation of q and k at the same position cancels
        w = torch.exp(s) / (torch.exp(s) + torch.exp(p("sink")))
        g = 1 / (1 + torch.exp(-(hi @ p("g").T)))
        v = (hi @ p("v").T).reshape(1, 3)
        assert torch.allclose(out[i], ((w * g)[:, None] * v).reshape(6) @ p("o").T, rtol=1e-9, atol=1e-12)
    # rows of the second chunk do not move when a row of the first does; rows of the first chunk after it do
    h2 = h.clone()
    h2[size - 1] *= 9.0
    out2 = plain.chunked_sink_attention(h2, p, m, 1e-5)
    assert torch.equal(out2[size:], out[size:]) and not torch.allclose(out2[size - 1], out[size - 1])
    h3 = h.clone()
    h3[size] *= 9.0                                     # the second chunk's first key: seen up to the chunk's end
    out3 = plain.chunked_sink_attention(h3, p, m, 1e-5)
    assert not torch.allclose(out3[2 * size - 1], out[2 * size - 1]) and torch.equal(out3[2 * size:], out[2 * size:])


def test_plain_latent_attention_keys_and_values_per_head():
    """Keys and values are built per head from the cached latent; neighbouring pairs are rotated, so a score depends
    on the distance only; the shared rotated key part is not normed."""
    m = latent(2, 3, 4, 5, 6, 0.3, 50.0)["mixer"]
    cfg = one_layer({"type": "latent_attention", "mixer": m, "mlp": None}, width=10)
    t, p = _mix_tensors(cfg)
    T = 4
    h = torch.randn(T, 10, dtype=F64, generator=torch.Generator().manual_seed(4))
    got = plain.latent_attention(h, p, m, 1e-5)
    low = h @ p("dkv").T
    c = low[:, :6] / torch.sqrt((low[:, :6] ** 2).mean(-1, keepdim=True) + 1e-5) * p("dkv.norm")
    f = torch.tensor([1.0, 50.0 ** -0.5], dtype=F64)

    def turn(x, pos):                                   # pairs (0, 1) and (2, 3)
        a = pos * f
        u, v = x[..., 0::2], x[..., 1::2]
        return torch.stack([u * torch.cos(a) - v * torch.sin(a), v * torch.cos(a) + u * torch.sin(a)], -1).flatten(-2)
    q = (h @ p("q").T).reshape(T, 2, 7)
    outs = torch.zeros(T, 2, 5, dtype=F64)
    for n in range(2):
        kn, vn = c @ p("uk")[3 * n:3 * n + 3].T, c @ p("uv")[5 * n:5 * n + 5].T
        for i in range(T):
            s = torch.stack([(q[i, n, :3] @ kn[j] + turn(q[i, n, 3:], i) @ turn(low[j, 6:], j)) * 0.3 for j in range(i + 1)])
            outs[i, n] = torch.softmax(s, 0) @ vn[:i + 1]
    assert torch.allclose(got, outs.reshape(T, 10) @ p("o").T, rtol=1e-9, atol=1e-12)


def test_plain_model_passes_add_the_embedding_and_a_vector():
    """Layer runs, in order, of a model whose middle is repeated; before pass t > 0 the embedded tokens are added, and
    before every pass its own vector."""
    cfg = CONFIGS["A"]
    tensors = make_weights(cfg, 9)
    model = plain.PlainSalolorn(cfg, tensors)
    toks = tokens(2, 7, cfg["vocab"])
    logits, after = model.forward(toks, trace=True)
    assert after.shape[0] == 1 + 2 * 2 + 1
    x0 = tensors["embed"].to(F64)[toks]
    x = model.layer(0, x0)
    assert torch.equal(x, after[0])
    x = model.layer(1, x + tensors["loop.step"][0].to(F64))
    assert torch.equal(x, after[1])
    x = model.layer(2, x)
    x = model.layer(1, x + x0 + tensors["loop.step"][1].to(F64))
    assert torch.equal(x, after[3])
    y = plain.rms_norm(after[-1], tensors["final.norm"].to(F64), cfg["norm"]["eps"])
    assert torch.allclose(logits, 0.5 * (y @ tensors["embed"].to(F64).T))


# ----------------------------------------------------------------- engine host side on the CPU
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_every_cutting_matches_the_plain_model(name, folders):
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": tokens(i, n, V) for i, n in enumerate([1, 17, 41, 80])}
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    eng = cpu_engine(folder)
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=1)
    worst = 0.0
    for steps in (cuttings.whole(reqs), cuttings.tail_decode(reqs, 20), cuttings.portions(reqs), mixed):
        got = cuttings.run_trace(eng, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        for (rid, p), row in got.items():
            worst = max(worst, float(row_error(row, ref[rid][p])))
    print(f"{name}: worst relative error {worst:.2e}")
    assert worst < TOL["float32"]
    assert all(p.used_pages == 0 for p in eng.cache.stats())


def test_residual_after_every_layer_run(folders):
    """The residual stream after each layer run of the engine against the plain model's (a repeated layer counts
    each time)."""
    folder, oracle = folders["A"]
    toks = tokens(3, 23, CONFIGS["A"]["vocab"])
    _, after = oracle.forward(toks, trace=True)
    eng = cpu_engine(folder)
    seen = []
    eng.model.after_layer = lambda call, x: seen.append(x.detach().to(torch.float64).clone())
    slot = eng.cache.open()
    eng.step([(slot, toks, [])])
    eng.cache.close(slot)
    assert len(seen) == after.shape[0]
    for i, x in enumerate(seen):
        err = float((x - after[i]).abs().max() / after[i].abs().max())
        assert err < 2e-5, (i, err)


def test_slots_and_pages_are_used_again_with_fresh_state(folders):
    """Six requests through three slots and a pool that holds only what is live: a request that takes a used slot
    starts from zero state (both recurrences and the convolution's carried inputs) in every pass."""
    folder, oracle = folders["A"]
    V = CONFIGS["A"]["vocab"]
    reqs = {f"q{i}": tokens(20 + i, n, V) for i, n in enumerate([70, 33, 129, 16, 90, 7])}
    steps, _ = cuttings.mixed(reqs, max_live=3, seed=2)
    peak = cuttings.peak_tokens(steps)
    eng = cpu_engine(folder, num_pages=peak // 16, max_requests=3)
    got = cuttings.run_trace(eng, steps)
    worst = max(float(row_error(row, oracle.forward(reqs[rid][:p + 1])[-1])) for (rid, p), row in got.items()
                if p in (0, 1, 2, len(reqs[rid]) - 1))
    assert worst < TOL["float32"]
    assert all(s.used_pages == 0 for s in eng.cache.stats())


def test_greedy_generation_through_the_scheduler(folders):
    """Engine.generate (scheduler, portions under a token budget, sampling, commit) against greedy decoding with the
    plain model; batched prompts give what each gives alone."""
    folder, oracle = folders["B"]
    V = CONFIGS["B"]["vocab"]
    prompts = [tokens(40, 5, V), tokens(41, 37, V), tokens(42, 1, V)]
    eng = cpu_engine(folder, max_step_tokens=16)
    outs = eng.generate(prompts, max_new_tokens=8)
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:
            row = oracle.forward(seq)[-1]
            top2 = torch.topk(row, 2).values
            if float(top2[0] - top2[1]) > 1e-3:
                assert int(torch.argmax(row)) == tok
            seq.append(tok)
    alone = [cpu_engine(folder).generate(p, max_new_tokens=8) for p in prompts]
    assert alone == outs


def test_replay_program_on_the_stand_in(folders, tmp_path, monkeypatch):
    from dlm_b200.engine import replay, Engine
    folder, oracle = folders["A"]
    V = CONFIGS["A"]["vocab"]
    reqs = {"a": tokens(50, 45, V), "b": tokens(51, 9, V)}
    steps, _ = cuttings.mixed(reqs, max_live=2, seed=3)
    real = Engine.from_pretrained
    monkeypatch.setattr(Engine, "from_pretrained", classmethod(
        lambda cls, path, **kw: real(path, **dict(kw, device="cpu", ops=PlainOps()))))
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    out_dir = str(tmp_path / "out")
    assert replay.main(["--model", folder, "--dtype", "float32", "--out", out_dir, "--max-tokens", "128",
                        "--page-size", "16", "--device", "cpu"]) == 0
    fed = {r: 0 for r in reqs}
    for st in steps:
        rows = np.fromfile(os.path.join(out_dir, f"{st['step']}.f32"), dtype="<f4").reshape(-1, V)
        k = 0
        for e in st["entries"]:
            ref = oracle.forward(reqs[e["id"]][:fed[e["id"]] + len(e["tokens"])])
            for w in e["want"]:
                assert float(row_error(torch.from_numpy(rows[k].copy()), ref[fed[e["id"]] + w])) < TOL["float32"]
                k += 1
            fed[e["id"]] += len(e["tokens"])


_ALONE = {
    "delta": delta(3, 1, 10, 6, 3),
    "delta_one_tap": delta(2, 2, 8, 12, 1),
    "latent": latent(2, 8, 4, 12, 16, 0.3, 100.0),
    "pair": parallel(left(4, 2, 8, 12, 0.3, 9, 100.0, 4), right(2, 6, 10, 3.0), 0.6, 1.7),
}


@pytest.mark.parametrize("kinds", [("delta", "delta_one_tap"), ("latent", "latent"), ("pair",), ("pair", "delta")])
@pytest.mark.parametrize("loop", [None, {"start": 0, "stop": 1, "times": 3}])
def test_models_of_one_kind_of_mixer(kinds, loop, tmp_path):
    """A model without any paged cache (recurrent layers only: tokens are still counted against the pool), one without
    any recurrent state, and a single layer; with and without a repeated run; with and without feed-forward."""
    cfg = one_layer(dict(_ALONE[kinds[0]], mlp=dense(24)), width=32, vocab=41, loop=loop)
    cfg["layers"] += [dict(_ALONE[k], mlp=None) for k in kinds[1:]]
    folder = str(tmp_path / "m")
    oracle = plain.PlainSalolorn(cfg, write_model(cfg, folder, seed=5))
    reqs = {"a": tokens(1, 40, 41), "b": tokens(2, 7, 41)}
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    eng = cpu_engine(folder)
    mixed, _ = cuttings.mixed(reqs, max_live=2, seed=6)
    for steps in (cuttings.whole(reqs), cuttings.portions(reqs, sizes=(2, 5)), mixed):
        got = cuttings.run_trace(eng, steps)
        assert max(float(row_error(row, ref[rid][p])) for (rid, p), row in got.items()) < TOL["float32"]
