"""Faguzen without a GPU: the config reader and registry, the order of layer calls with repeated passes, tensor
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
import plain_faguzen as plain
from plain_ops import PlainOps
from faguzen_models import (CONFIGS, SCALING, TOL, layer, left, make_weights, moe, one_layer, right, row_error, tokens,
                            write_model)

F64 = torch.float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("faguzen")
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(base / name)
        tensors = write_model(cfg, folder, seed=len(name) + ord(name))
        out[name] = (folder, plain.PlainFaguzen(cfg, tensors))
    return out


def cpu_engine(folder, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=40, max_requests=4)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


def runs_of(cfg):
    n = len(cfg["layers"])
    if "loop" in cfg:
        n += (cfg["loop"]["stop"] - cfg["loop"]["start"]) * (cfg["loop"]["times"] - 1)
    return n


# ------------------------------------------------------------------ config, registry, tensors
def test_registry_resolves_the_architecture_and_round_trips_the_config():
    from dlm_b200.config import FaguzenConfig
    from dlm_b200.registry import architectures, resolve
    assert "Faguzen" in architectures()
    for cfg in CONFIGS.values():
        name, typed, spec = resolve(copy.deepcopy(cfg))
        assert name == "Faguzen" and isinstance(typed, FaguzenConfig)
        assert len(spec.layers) == len(cfg["layers"]) and spec.vocab_size == cfg["vocab"]
        assert not spec.tie_word_embeddings and (spec.pass_entry is not None) == ("loop" in cfg)
        assert spec.logit_softcap == cfg.get("logit_softcap", 0.0)
        assert spec.dependent_launch is False          # this design's steps take ordinary launches
        assert len(spec.order) == runs_of(cfg)
        assert FaguzenConfig.from_dict(typed.to_dict()) == typed
        assert typed.to_dict()["layers"] == cfg["layers"]


@pytest.mark.parametrize("edit,what", [
    (lambda c: c.pop("layers"), "layers"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].update(type="window_attention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("left"), "left"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("factor"), "factor"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(high=0.5), "high"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "mlp"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("ff"), "ff"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(logit_softcap=-2.0), "logit_softcap"),
])
def test_config_refusals(edit, what):
    from dlm_b200.config import ConfigError
    from dlm_b200.registry import resolve
    cfg = copy.deepcopy(CONFIGS["A"])
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        resolve(cfg)
    assert what in str(e.value)


def test_tensor_names_and_shapes_are_the_checkpoints_own():
    from dlm_b200.parts import DecoderModel, Runtime, WeightError
    from dlm_b200.registry import resolve
    for cfg in CONFIGS.values():
        _, _, spec = resolve(copy.deepcopy(cfg))
        model = DecoderModel(spec, Runtime("cpu", torch.float32, None))
        tensors = make_weights(cfg)
        model.check({n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()})
        assert set(model.param_specs()) == set(tensors)
        assert ("loop.step" in model.param_specs()) == ("loop" in cfg)
    cfg = CONFIGS["A"]
    _, _, spec = resolve(copy.deepcopy(cfg))
    model = DecoderModel(spec, Runtime("cpu", torch.float32, None))
    bad = make_weights(cfg)
    bad.pop("l0.norm1.alpha")
    bad.pop("l0.mix.left.o.b")
    bad.pop("l2.mlp.correction")
    bad["loop.step"] = torch.zeros(5, cfg["width"])
    bad["l0.mlp.router"] = torch.zeros(5, cfg["width"])          # the identity experts' rows are missing
    bad["l1.mix.right.i.b"] = torch.zeros(7)
    bad["l0.mlp.e5.up"] = torch.zeros(30, cfg["width"])          # an identity expert has no tensors
    with pytest.raises(WeightError) as e:
        model.check({n: (t.dtype, tuple(t.shape)) for n, t in bad.items()})
    for n in ("l0.norm1.alpha", "l0.mix.left.o.b", "l2.mlp.correction", "loop.step", "l0.mlp.router", "l1.mix.right.i.b",
              "l0.mlp.e5.up"):
        assert n in str(e.value)


def test_random_weights_for_a_config_build_and_load(tmp_path):
    from dlm_b200.config import FaguzenConfig
    from dlm_b200.engine import Engine
    from dlm_b200.weights import write_random_model
    cfg = FaguzenConfig.from_dict(copy.deepcopy(CONFIGS["D"]))
    folder = write_random_model(cfg, 5, str(tmp_path / "m"))
    toks = tokens(1, 20, cfg.vocab)
    a = cpu_engine(folder)
    b = Engine.from_random(cfg, 5, dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=8, max_requests=2)
    sa, sb = a.cache.open(), b.cache.open()
    la, lb = a.step([(sa, toks, [19])]), b.step([(sb, toks, [19])])
    assert torch.allclose(la, lb, atol=1e-5)
    assert torch.isfinite(la).all() and float(la.std()) > 0


def test_rotary_table_with_slowed_long_waves():
    """The package's table against the plain statement, and the three regimes by hand: with original 64, high 4 and
    low 1, waves shorter than 16 keep their frequency, waves longer than 64 are slowed by the factor, and one in
    between is blended."""
    from dlm_b200.parts import PartSpec, Runtime
    from dlm_b200.registry import build_part
    rt = Runtime("cpu", torch.float32, None)
    for base, dims, sc in ((5000.0, 16, SCALING), (300.0, 20, SCALING), (1e4, 8, None), (1e6, 32, dict(SCALING, original=128))):
        part = build_part("position", PartSpec("rope_scaled_neox", {"head_dim": 40, "theta": base, "rotary_dim": dims,
                                                                    "scaling": sc}))
        table, n = part.rotary(rt)
        assert n == dims and torch.allclose(table.double(), plain.scaled_frequencies(base, dims, sc), rtol=1e-7)
    f = plain.scaled_frequencies(5000.0, 16, SCALING)
    plainf = torch.tensor([5000.0 ** (-2.0 * i / 16) for i in range(8)], dtype=F64)
    wave = 2 * math.pi / plainf
    assert bool((wave < 16).any()) and bool((wave > 64).any()) and bool(((wave > 16) & (wave < 64)).any())
    for i in range(8):
        if wave[i] < 16:
            assert f[i] == plainf[i]
        elif wave[i] > 64:
            assert float(f[i]) == pytest.approx(float(plainf[i]) / 8.0, rel=1e-12)
        else:
            s = (64 / float(wave[i]) - 1.0) / 3.0
            assert float(f[i]) == pytest.approx((1 - s) * float(plainf[i]) / 8.0 + s * float(plainf[i]), rel=1e-12)
            assert float(plainf[i]) / 8.0 < float(f[i]) < float(plainf[i])


# ------------------------------------------------- the plain implementation's own hand-made cases
def _mix_tensors(cfg, seed=3):
    t = {k: v.to(F64) for k, v in make_weights(cfg, seed).items()}
    return t, (lambda n: t["l0.mix." + n])


def test_plain_attention_first_token_cap_and_gate():
    """The first position sees only itself, so its output is gate * (v + bias) whatever the score; a score far above
    the cap counts as the cap: with two keys whose raw scores are 50 and 80 and a cap of 2, the weights are those of
    2 tanh(25) and 2 tanh(40), that is equal."""
    m = left(2, 1, 4, 3, 0.5, 2.0, 100.0, 2)
    cfg = one_layer(layer(m, right(1, 2, 2, 2.0), 1.0, 1.0), width=10)
    t, p0 = _mix_tensors(cfg)
    p = lambda n: p0("left." + n)
    h = torch.randn(5, 10, dtype=F64, generator=torch.Generator().manual_seed(3))
    out = plain.capped_gated_attention(h, p, m)
    v0 = (h[0] @ p("v").T + p("v.b")).reshape(1, 3).expand(2, 3).reshape(6)
    g0 = 1 / (1 + torch.exp(-(h[0] @ p("g").T)))
    assert torch.allclose(out[0], (g0 * v0) @ p("o").T + p("o.b"), rtol=1e-10, atol=1e-12)
    s = torch.tensor([[50.0, 80.0]], dtype=F64)
    w = torch.softmax(plain.tanh_cap(s, 2.0), -1)
    assert torch.allclose(w, torch.tensor([[0.5, 0.5]], dtype=F64), atol=1e-12)
    assert not torch.allclose(torch.softmax(s, -1), w)


def test_plain_attention_scores_depend_on_the_distance_only_where_rotated():
    """Rotating q at i and k at j by their own positions leaves the rotated part's product a function of i - j."""
    f = plain.scaled_frequencies(100.0, 4, None)
    g = torch.Generator().manual_seed(5)
    q, k = torch.randn(1, 1, 6, dtype=F64, generator=g), torch.randn(1, 1, 6, dtype=F64, generator=g)
    def score(i, j):
        a = plain.rotate_halves(q, torch.tensor([i]), f, 4)
        b = plain.rotate_halves(k, torch.tensor([j]), f, 4)
        return float((a * b).sum())
    assert score(9, 4) == pytest.approx(score(105, 100), rel=1e-9)
    assert score(9, 4) != pytest.approx(score(9, 5), rel=1e-3)
    # entries from dims on pass unchanged
    assert torch.equal(plain.rotate_halves(q, torch.tensor([7]), f, 4)[..., 4:], q[..., 4:])


def test_plain_matrix_memory_is_the_gated_sum_over_the_past():
    """Without the running maximum, in 64-bit: S_T = sum_j (prod_{j<i<=T} F_i) I_j k_j v_j^T with F = sigmoid(capped
    forget) and I = exp(capped input); the stabilised recurrence keeps exp(-m) times that.  Carrying (S, n, m) over a
    cut changes nothing, and the first token is written out by hand."""
    m = right(2, 3, 5, 6.0)
    cfg = one_layer(layer(left(2, 1, 4, 4, 0.5), m, 1.0, 1.0), width=12)
    t, p0 = _mix_tensors(cfg)
    p = lambda n: p0("right." + n)
    T = 7
    h = torch.randn(T, 12, dtype=F64, generator=torch.Generator().manual_seed(2))
    got, (S_, n_, m_) = plain.matrix_memory(h, p, m, 1e-5)
    q = (h @ p("q").T).reshape(T, 2, 3) / math.sqrt(3)
    k, v = (h @ p("k").T).reshape(T, 2, 3), (h @ p("v").T).reshape(T, 2, 5)
    I = torch.exp(6.0 * torch.tanh((h @ p("i").T + p("i.b")) / 6.0))
    F = 1 / (1 + torch.exp(-6.0 * torch.tanh((h @ p("f").T + p("f.b")) / 6.0)))
    S_true, n_true = torch.zeros(2, 3, 5, dtype=F64), torch.zeros(2, 3, dtype=F64)
    for j in range(T):
        w = F[j + 1:].prod(0) * I[j]                                        # the key's own step does not decay it
        S_true += w[:, None, None] * k[j][:, :, None] * v[j][:, None, :]
        n_true += w[:, None] * k[j]
    assert torch.allclose(S_ * torch.exp(m_)[:, None, None], S_true, rtol=1e-9)
    assert torch.allclose(n_ * torch.exp(m_)[:, None], n_true, rtol=1e-9)
    a, sa = plain.matrix_memory(h[:3], p, m, 1e-5)
    b, _ = plain.matrix_memory(h[3:], p, m, 1e-5, state=sa)
    assert torch.allclose(torch.cat([a, b]), got, rtol=1e-12, atol=1e-14)
    # the first token by hand: m1 = max(f1 + 0, i1); S1 = exp(i1 - m1) k v^T; den = max(|n . q|, exp(-m1)) + 1e-6
    li, lf = torch.log(I[0]), torch.log(F[0])
    m1 = torch.maximum(lf, li)
    nq = torch.exp(li - m1) * (k[0] * q[0]).sum(-1)
    o1 = nq[:, None] * v[0] / (torch.maximum(nq.abs(), torch.exp(-m1)) + 1e-6)[:, None]
    y1 = (o1 / torch.sqrt((o1 * o1).mean(-1, keepdim=True) + 1e-5)).reshape(10) * p("norm")
    y1 = y1 / (1 + torch.exp(-(h[0] @ p("g").T)))
    assert torch.allclose(got[0], y1 @ p("o").T, rtol=1e-9, atol=1e-12)


def test_plain_router_correction_identity_and_weights():
    """The correction changes who is chosen but not the weights; an identity expert returns the input itself; the
    weights of the chosen add up to one; the shared expert is added unweighted."""
    mlp = moe(3, 2, 2, 6, 5)
    cfg = one_layer(layer(left(1, 1, 2, 2, 0.5), right(1, 2, 2, 2.0), 1.0, 1.0, mlp), width=8)
    t = {k: v.to(F64) for k, v in make_weights(cfg, 4).items()}
    p = lambda n: t["l0.mlp." + n]
    h = torch.randn(9, 8, dtype=F64, generator=torch.Generator().manual_seed(1))
    ids, w, _ = plain.route(h, p, mlp)
    s = torch.softmax(h @ p("router").T, -1)
    assert torch.allclose(w.sum(-1), torch.ones(9, dtype=F64))
    assert torch.allclose(w, torch.gather(s, 1, ids) / torch.gather(s, 1, ids).sum(-1, keepdim=True))
    t2 = dict(t)
    t2["l0.mlp.correction"] = torch.tensor([0.0, 0.0, 0.0, 5.0, 4.0], dtype=F64)      # the identity experts always win
    p2 = lambda n: t2["l0.mlp." + n]
    ids2, w2, _ = plain.route(h, p2, mlp)
    assert ids2.tolist() == [[3, 4]] * 9
    out = plain.expert_mixture(h, p2, mlp)
    shared = plain.gelu_erf(h @ p("shared.up").T) @ p("shared.down").T
    assert torch.allclose(out, h + shared, rtol=1e-12, atol=1e-14)                      # weights add up to one
    t2["l0.mlp.correction"] = torch.tensor([5.0, 0.0, 4.0, 0.0, 0.0], dtype=F64)
    ids3, w3, _ = plain.route(h, p2, mlp)
    e0 = plain.gelu_erf(h @ p("e0.up").T) @ p("e0.down").T
    e2 = plain.gelu_erf(h @ p("e2.up").T) @ p("e2.down").T
    assert torch.allclose(plain.expert_mixture(h, p2, mlp), w3[:, :1] * e0 + w3[:, 1:] * e2 + shared, rtol=1e-10)


def test_plain_norm_layer_and_passes():
    """Layer runs, in order, of a model whose middle is repeated; before every pass its own vector is added (and
    nothing else); a layer adds residual_mult times the sum of both sublayers of the same input; the norm takes no
    statistics; the logits are capped."""
    cfg = CONFIGS["A"]
    tensors = make_weights(cfg, 9)
    model = plain.PlainFaguzen(cfg, tensors)
    toks = tokens(2, 7, cfg["vocab"])
    logits, after = model.forward(toks, trace=True)
    assert after.shape[0] == 1 + 2 * 2 + 1
    t = {k: v.to(F64) for k, v in tensors.items()}
    x0 = t["embed"][toks]
    x = model.layer(0, x0)
    assert torch.equal(x, after[0])
    x = model.layer(1, x + t["loop.step"][0])
    assert torch.equal(x, after[1])
    x = model.layer(2, x)
    x = model.layer(1, x + t["loop.step"][1])
    assert torch.equal(x, after[3])
    # layer 1 has no feed-forward: x + mult * mixer(norm1 x)
    xin = after[0] + t["loop.step"][0]
    h = torch.tanh(t["l1.norm1.alpha"] * xin) * t["l1.norm1"] + t["l1.norm1.b"]
    mix = plain.parallel_mixer(h, lambda n: t["l1.mix." + n], cfg["layers"][1]["mixer"], cfg["norm"]["eps"])
    assert torch.allclose(after[1], xin + 0.8 * mix, rtol=1e-12)
    y = torch.tanh(t["final.norm.alpha"] * after[-1]) * t["final.norm"] + t["final.norm.b"]
    assert torch.allclose(logits, 9.0 * torch.tanh((y @ t["head"].T) / 9.0))
    assert float(logits.abs().max()) < 9.0


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
    starts from zero memory, normaliser and maximum in every pass."""
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


@pytest.mark.parametrize("mlp", [None, moe(3, 0, 3, 10), moe(0, 3, 2, 1), moe(4, 2, 1, 12, 20)])
@pytest.mark.parametrize("loop", [None, {"start": 0, "stop": 1, "times": 3}])
def test_a_single_layer_with_every_kind_of_feed_forward(mlp, loop, tmp_path):
    """One layer, with and without a repeated run; no feed-forward, every expert chosen, identity experts only, one
    expert of several beside a shared one; neither a rotation nor a cap."""
    cfg = one_layer(layer(left(4, 2, 8, 12, 0.3), right(2, 6, 10, 3.0), 0.6, 1.7, mlp), width=32, vocab=41, loop=loop,
                    cap=0.0)
    folder = str(tmp_path / "m")
    oracle = plain.PlainFaguzen(cfg, write_model(cfg, folder, seed=5))
    reqs = {"a": tokens(1, 40, 41), "b": tokens(2, 7, 41)}
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    eng = cpu_engine(folder)
    mixed, _ = cuttings.mixed(reqs, max_live=2, seed=6)
    for steps in (cuttings.whole(reqs), cuttings.portions(reqs, sizes=(2, 5)), mixed):
        got = cuttings.run_trace(eng, steps)
        assert max(float(row_error(row, ref[rid][p])) for (rid, p), row in got.items()) < TOL["float32"]
