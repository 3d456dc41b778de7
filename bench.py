"""Serving benchmark: decode tokens per second of the Qwen1.5-MoE-A2.7B-sized model with
random weights (bfloat16) on one B200, plus prefill, roofline and end-to-end figures; in the same
line, the same measurements at the layer sizes of Qwen2-57B-A14B (`sizes_57b`) and a
continuous-batching workload on the windowed variant of the model (`serving`).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --no-extras             # the headline model only
    python bench.py --workload serving      # the continuous-batching workload alone, a line of its own
    python bench.py --sizes 57b             # the larger model alone as the headline
    python bench.py --workload sweep        # decode at 1k-32k tokens of context, prompts of 8k and 16k
    python bench.py --workload kernels      # the weight-streaming product alone, by shape and row length
    python bench.py --workload zesapel      # the Zesapel design beside Qwen2-MoE at equal sizes, and its kernels alone
    python bench.py --workload zasazen      # the Zasazen design beside Qwen2-MoE at equal sizes, and its kernels alone
    python bench.py --workload salolorn     # the Salolorn design beside a dense Qwen2 at equal sizes, and its kernels alone
    python bench.py --workload faguzen      # the Faguzen design beside Qwen2-MoE at equal sizes, and its kernels alone

A step is one decode step of the whole batch.  One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Layer sizes of the model the benchmark is quoted on (Qwen1.5-MoE-A2.7B).
MODEL = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=24, hidden_size=2048, num_attention_heads=16, num_key_value_heads=16, head_dim=128,
    num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
    norm_topk_prob=False, decoder_sparse_step=1, intermediate_size=5632, vocab_size=151936, rope_theta=1000000.0,
    rms_norm_eps=1e-6, use_sliding_window=False, tie_word_embeddings=False, max_position_embeddings=4096)
MODEL_A = dict(MODEL)
FULL_LAYERS = MODEL["num_hidden_layers"]
MODEL_NAME = "Qwen1.5-MoE-A2.7B"
# The larger model of the same family (--sizes 57b; about 114 GB of weights with all 28 layers).
SIZES_57B = dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                 num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560,
                 shared_expert_intermediate_size=20480, intermediate_size=20480)


def peaks():
    """Measured peaks if the driver wrote them, else this pool's earlier measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p.get("bf16_tflops_sustained") or p["bf16_tflops"]),
                        source="measured")
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not (t0 - 0.05 <= t <= t1 + 0.15):
                continue
            parts = [x.strip() for x in line.split(",")]
            try:
                mhz.append(int(float(parts[0])))
                mx = max(mx, int(float(parts[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def weight_bytes_per_decode_step(cfg, batch, layers, esz=2, distinct=None):
    """Bytes a decode step has to read: every weight it uses once.  Routed experts: `distinct` experts
    with rows per layer (the mean over the layers of what the step's own routing gave); without it, the
    expected number of distinct experts a batch of `batch` tokens touches."""
    H, Q, KV = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    E, k, I, Is = cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
    attn = ((Q + 2 * KV) * H + H * Q) * esz
    if distinct is None:
        distinct = E * (1.0 - (1.0 - k / E) ** batch)
    moe = (E + 1) * H * esz + distinct * 3 * I * H * esz + 3 * Is * H * esz
    head = cfg.vocab_size * H * esz
    return layers * (attn + moe) + head


def prefill_flops(cfg, T, layers):
    H, Q, KV = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    E, k, I, Is = cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
    per_tok = 2 * H * (Q + 2 * KV) + 2 * Q * H + 2 * H * (E + 1) + k * 6 * H * I + 6 * H * Is
    attn = 4 * Q * T * (T + 1) / 2          # QK^T and PV over the causal half
    return layers * (per_tok * T + attn) + 2 * H * cfg.vocab_size


def run_reference():
    print(json.dumps({"impl": "reference", "unavailable":
                      "vedantnimbarte/dlm is a Rust crate (Cargo.toml, no setup.py/pyproject.toml): pip cannot "
                      "install it offline and no Rust toolchain is present"}))
    return 0


def run_serving(args) -> dict:
    """Continuous batching on the windowed variant of the model: 64 requests, prompt lengths uniform in
    [256, 16384], output lengths uniform in [64, 512], seeded uniform token ids; a request arrives every
    second step, so portions of prompts (2,048-token portions) run beside decoded tokens in the same step.
    Everything goes through the scheduler and the Python entry point; one JSON line."""
    import torch

    from dlm_b200.config import Qwen2MoeConfig
    from dlm_b200.engine import Engine

    raw = dict(MODEL_A)
    raw.update(num_hidden_layers=args.layers, use_sliding_window=True, sliding_window=4096,
               max_window_layers=min(21, max(args.layers - 3, 0)), max_position_embeddings=32768)
    cfg = Qwen2MoeConfig.from_dict(raw)
    torch.cuda.set_device(0)
    p_lo, p_hi = args.serving_prompts
    n_req, pool_tokens, max_context = args.serving_requests, 262144, max(p_hi, 4096) + 512 + 64
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", page_size=64, max_tokens=pool_tokens,
                             max_requests=n_req, max_step_tokens=2048, max_context=max_context)
    gen = torch.Generator().manual_seed(4)
    plen = torch.randint(p_lo, p_hi + 1, (n_req,), generator=gen).tolist()
    olen = torch.randint(64, 513, (n_req,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in plen]
    # warm-up: one short request end to end (kernels loaded, graphs of its shapes captured)
    eng.generate([prompts[0][:300]], max_new_tokens=4)
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    submitted, produced, steps = 0, 0, 0
    # per step: time between two events around it, wall time, and whether it carried prompt tokens (the events
    # enclose the host's work inside the step too; what the host costs is in the scheduler's counters below)
    records, prompt_seen = [], eng.scheduler.stats().prompt_tokens
    while submitted < n_req or eng.scheduler.has_work():
        if submitted < n_req and steps % 2 == 0:
            eng.submit(prompts[submitted], max_new_tokens=olen[submitted])
            submitted += 1
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        e0.record()
        out = eng.run_step()
        e1.record()
        e1.synchronize()
        w1 = time.perf_counter()
        now = eng.scheduler.stats().prompt_tokens
        records.append((e0, e1, w1 - w0, now - prompt_seen, len(out)))
        prompt_seen = now
        produced += len(out)
        steps += 1
    torch.cuda.synchronize()
    t1 = time.time()
    kinds = {"decode_only": [], "with_prompt_le_256": [], "with_prompt_gt_256": []}
    for e0, e1, wall, ptoks, rows in records:
        kind = "decode_only" if ptoks == 0 else ("with_prompt_le_256" if ptoks <= 256 else "with_prompt_gt_256")
        kinds[kind].append((e0.elapsed_time(e1), 1e3 * wall))
    step_kinds = {k: {"steps": len(v), "device_ms_mean": round(sum(a for a, _ in v) / len(v), 3),
                      "wall_ms_mean": round(sum(b for _, b in v) / len(v), 3)} for k, v in kinds.items() if v}
    time.sleep(0.2)
    sampler.stop()
    clocks = sampler.summary(t0, t1)
    st = eng.stats()
    ok = st["finished"] >= n_req and produced == sum(olen)
    line = {
        "metric": f"serving: generated tok/s, {n_req} requests, prompts {p_lo}-{p_hi}, outputs 64-512, continuous batching "
                  "(Qwen1.5-MoE-A2.7B sizes, layers 21-23 windowed at 4096, bf16, random weights)",
        "value": round(produced / (t1 - t0), 2), "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)", "impl": "ours",
        "seconds": round(t1 - t0, 3), "generated_tokens": produced, "prompt_tokens": sum(plen),
        "prompt_tok_s": round(sum(plen) / (t1 - t0), 1), "steps": steps, "complete": ok,
        "config": {"model": "Qwen1.5-MoE-A2.7B sizes, window", "requests": n_req, "layers": args.layers,
                   "layers_full": MODEL_A["num_hidden_layers"], "pool_tokens": pool_tokens, "portion": 2048, "page_size": 64,
                   "arrivals": "one request every second step"},
        "scheduler": {k: st[k] for k in ("steps", "prompt_tokens", "decode_tokens", "preemptions", "finished",
                                         "graphs_recorded", "graph_record_seconds", "eager_steps",
                                         "eager_launch_seconds")},
        "pages": st["pages"], "clocks": clocks,
        # the steps by kind; the host's share: seconds spent recording decode graphs (the device idles) and
        # launching the steps that are not replayed (the device works meanwhile)
        "step_kinds": step_kinds,
        "host": {"graphs_recorded": st["graphs_recorded"], "graph_record_s": st["graph_record_seconds"],
                 "eager_steps": st["eager_steps"], "eager_launch_s": st["eager_launch_seconds"]},
    }
    del eng
    return line


class Measurement:
    """One model on the device and the measurements taken on it: decode steps at several batch sizes
    (device time of the replayed step, and end to end through run_step) and one 2,048-token prefill."""

    def __init__(self, raw, layers, prompt_len, context, max_batch, pk, page=64):
        import torch

        from dlm_b200.config import Qwen2MoeConfig
        from dlm_b200.engine import Engine
        self.torch = torch
        raw = dict(raw)
        raw["num_hidden_layers"] = layers
        self.cfg = Qwen2MoeConfig.from_dict(raw)
        self.layers, self.prompt_len, self.pk = layers, prompt_len, pk
        torch.cuda.set_device(0)
        self.page = page
        pool_tokens = max_batch * (prompt_len + 256) + 4096
        t_load = time.time()
        self.eng = Engine.from_random(self.cfg, seed=0, dtype="bfloat16", page_size=self.page, max_tokens=pool_tokens,
                                      max_requests=max_batch, max_step_tokens=2048, max_context=context)
        torch.cuda.synchronize()
        self.load_s = time.time() - t_load
        self.gen = torch.Generator().manual_seed(0)
        # the routing of every captured step: the permutation's offsets stay in the graph's memory
        self.offsets = []
        ops = self.eng.rt.ops
        route = ops.route

        def recording_route(*a, **kw):
            out = route(*a, **kw)
            self.offsets.append(out[3])          # (ids, wts, gate, offsets, rows, dest)
            return out
        ops.route = recording_route

    def close(self):
        import gc
        self.eng._graphs.clear()
        self.eng = None
        self.offsets = []
        gc.collect()
        self.torch.cuda.empty_cache()

    def prompts(self, n, length):
        return [self.torch.randint(0, self.cfg.vocab_size, (length,), generator=self.gen).tolist() for _ in range(n)]

    def decode(self, batch, steps, warmup, sample_clocks=False):
        """Prefills `batch` prompts through the scheduler, then times `steps` decode steps of the step
        function (device time) and the same number through run_step (end to end)."""
        torch, eng = self.torch, self.eng
        ids = [eng.submit(p, max_new_tokens=10 ** 6) for p in self.prompts(batch, self.prompt_len)]
        started = set()
        while len(started) < batch:                   # admit and prefill everything
            started.update(rid for rid, _ in eng.run_step())
        # every request now decodes one token per step
        self.offsets = []
        for _ in range(max(warmup, 3)):
            eng.run_step()
        torch.cuda.synchronize()
        # device time of the decode step itself: `steps` replays of the captured step (the step function
        # and the arg-max over its logits, all kernels of one decode step), no host work in between
        key = next(k for k in eng._graphs if k[0] == batch and k[1] >= self.prompt_len)
        ent = eng._graphs[key]
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
            time.sleep(0.3)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.time()
        e0.record()
        for _ in range(steps):
            ent["graph"].replay()
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        dev_ms = e0.elapsed_time(e1)
        clocks = None
        if sample_clocks:
            time.sleep(0.2)
            sampler.stop()
            clocks = sampler.summary(t0, t1)
        # the experts that had rows in the replayed step, per layer (the last capture's offsets)
        distinct = None
        sparse = sum(1 for i in range(self.layers) if self.cfg.layer_is_sparse(i))
        if sparse and len(self.offsets) >= sparse:
            offs = torch.stack(self.offsets[-sparse:]).cpu()
            distinct = float(((offs[:, 1:] - offs[:, :-1]) > 0).sum(dim=1).double().mean())
        # end to end: wall clock around the public loop, host tokens in and out every step
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += len(eng.run_step())
        torch.cuda.synchronize()
        w1 = time.perf_counter()
        ctx = eng.cache.manager.length(0) if eng.cache.manager.is_open(0) else self.prompt_len
        for i in ids:
            eng.abort(i)
        eng.scheduler.drain_finished()
        ms = dev_ms / steps
        kv_bytes = batch * (self.prompt_len + max(warmup, 3) + 2 + steps // 2) * eng.cache.bytes_per_token()
        step_bytes = weight_bytes_per_decode_step(self.cfg, batch, self.layers, distinct=distinct) + kv_bytes
        achieved = step_bytes / (ms / 1e3) / 1e9
        return dict(ms=ms, tok_s=batch * steps / (dev_ms / 1e3), e2e_tok_s=produced / (w1 - w0),
                    launches=ent["launches"] * steps, clocks=clocks, ctx=ctx, distinct=distinct,
                    step_bytes=step_bytes, achieved=achieved, frac=achieved / self.pk["hbm_gbs"],
                    h2d=int(eng.cache.last_h2d_bytes))

    def decode_sampled(self, batch, steps, temperature=0.8):
        """Tokens a second end to end through run_step with seeded temperature sampling (the sampling kernel
        and its host side on top of the replayed step)."""
        from dlm_b200.sampling import SamplingParams
        torch, eng = self.torch, self.eng
        ids = [eng.submit(p, SamplingParams(temperature=temperature, seed=i), max_new_tokens=10 ** 6)
               for i, p in enumerate(self.prompts(batch, self.prompt_len))]
        started = set()
        while len(started) < batch:
            started.update(rid for rid, _ in eng.run_step())
        for _ in range(3):
            eng.run_step()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += len(eng.run_step())
        torch.cuda.synchronize()
        w1 = time.perf_counter()
        for i in ids:
            eng.abort(i)
        eng.scheduler.drain_finished()
        return produced / (w1 - w0)

    def prefill(self, T=2048, repeats=4):
        torch, eng = self.torch, self.eng
        times = []
        for _ in range(repeats):
            s = eng.cache.open()
            toks = self.prompts(1, T)[0]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step([(s, toks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            eng.cache.close(s)
        pms = min(times[1:]) if len(times) > 1 else times[0]
        flops = prefill_flops(self.cfg, T, self.layers)
        return {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                "frac": round(flops / (pms / 1e3) / (self.pk["bf16_tflops"] * 1e12), 4),
                "peak_tflops": self.pk["bf16_tflops"], "all_ms": [round(t, 3) for t in times]}


def run_sweep(args, pk) -> dict:
    """Further contexts: decode steps at batch 1 / 8 / 64 with 1k to 32k tokens of context each (as far as the
    pool holds them), and prompts of 8k and 16k tokens prefilled in portions of 2,048, each with its fraction of
    the measured peak."""
    out = {"metric": "sweep over contexts (%s sizes, bf16, random weights)" % MODEL_NAME, "layers": args.layers,
           "layers_full": FULL_LAYERS, "decode": {}, "prefill": {}}
    for ctx in (1024, 4096, 8192, 16384, 32768):
        for b in (1, 8, 64):
            if b * ctx > 600_000:          # 64 x 16k and 64 x 32k would not fit beside the weights
                continue
            m = Measurement(MODEL, args.layers, ctx, ctx + 512, b, pk)
            r = m.decode(b, 8, 3)
            out["decode"][f"b{b}_ctx{ctx}"] = {"tok_s": round(r["tok_s"], 1), "ms": round(r["ms"], 3),
                                                "frac": round(r["frac"], 4)}
            m.close()
    import torch
    for plen in (8192, 16384):
        m = Measurement(MODEL, args.layers, plen, plen + 512, 1, pk)
        eng, times = m.eng, []
        for _ in range(2):
            s = eng.cache.open()
            toks = m.prompts(1, plen)[0]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(0, plen, 2048):
                eng.step([(s, toks[i:i + 2048], [2047] if i + 2048 >= plen else [])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            eng.cache.close(s)
        ms = min(times)
        flops = prefill_flops(m.cfg, plen, args.layers)
        out["prefill"][f"prompt{plen}"] = {"tok_s": round(plen / (ms / 1e3), 1), "ms": round(ms, 2),
                                           "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        m.eng.rt.ops.check_errors()
        m.close()
    return out


def run_kernels(pk) -> dict:
    """The decode step's products alone, timed with CUDA events inside a captured graph, the weights rotated
    over several copies so that L2 does not hold them: the dense shapes (8 rows, the weight-streaming kernel), the
    routed experts' products at 1 / 8 / 64 tokens (whichever kernel the rule chooses: the weight-streaming one at
    1 and 8, the tcgen05 one at 64), and 8 rows against 256 MB of weights with rows of 512 to 4,096 elements."""
    import torch

    from dlm_b200.ops import native_ops
    ops = native_ops(fast=True)
    dev = "cuda"
    bf = torch.bfloat16

    def timed(fn, copies, reps=3):
        for c in range(copies):
            fn(c)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                for c in range(copies):
                    fn(c)
        g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1000 / (5 * reps * copies)

    out = {"metric": "the decode step's products alone: us and TB/s", "peak_gbs": pk["hbm_gbs"], "dense": {},
           "grouped": {}, "row_length": {}}
    for (N, K, kind) in [(6144, 2048, "store"), (2048, 2048, "add"), (11264, 2048, "swiglu"), (2048, 5632, "store"),
                         (151936, 2048, "store")]:
        copies = max(2, min(12, int(300e6 // (N * K * 2)) + 1))
        ws = [torch.randn(N, K, device=dev).to(bf) * 0.05 for _ in range(copies)]
        a = torch.randn(8, K, device=dev).to(bf)
        resid = torch.zeros(8, N, device=dev)
        fn = {"store": lambda c: ops.linear(a, ws[c], None, torch.float32),
              "add": lambda c: ops.linear_add(a, ws[c], resid),
              "swiglu": lambda c: ops.linear_swiglu(a, ws[c])}[kind]
        us = timed(fn, copies)
        out["dense"][f"{N}x{K}_{kind}"] = {"us": round(us, 2), "tb_s": round(N * K * 2 / us / 1e6, 2)}
        del ws
    E, k, H, I = MODEL_A["num_experts"], MODEL_A["num_experts_per_tok"], MODEL_A["hidden_size"], MODEL_A["moe_intermediate_size"]
    for T in (1, 8, 64):
        g = torch.Generator().manual_seed(T)
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
        offsets, rows, _ = ops.moe_permute(ids, E)
        active = int(((offsets[1:] - offsets[:-1]) > 0).sum())
        wgu = [torch.randn(E, 2 * I, H, device=dev).to(bf) * 0.05 for _ in range(3)]
        wd = [torch.randn(E, H, I, device=dev).to(bf) * 0.05 for _ in range(3)]
        h = torch.randn(T, H, device=dev).to(bf)
        act = ops.grouped_swiglu(h, wgu[0], offsets, rows)
        u1 = timed(lambda c: ops.grouped_swiglu(h, wgu[c], offsets, rows), 3)
        u2 = timed(lambda c: ops.grouped_linear(act, wd[c], offsets), 3)
        out["grouped"][f"tokens{T}"] = {"experts_with_rows": active,
                                        "gate_up_us": round(u1, 2), "gate_up_tb_s": round(active * 2 * I * H * 2 / u1 / 1e6, 2),
                                        "down_us": round(u2, 2), "down_tb_s": round(active * I * H * 2 / u2 / 1e6, 2)}
        del wgu, wd
    for K in (512, 1024, 1408, 1536, 2048, 2816, 4096):
        N = (256 * 1024 * 1024 // 2) // K // 16 * 16
        ws = [torch.randn(N, K, device=dev).to(bf) for _ in range(2)]
        a = torch.randn(8, K, device=dev).to(bf)
        us = timed(lambda c: ops.linear(a, ws[c], None, torch.float32), 2)
        out["row_length"][f"K{K}"] = {"us": round(us, 1), "tb_s": round(N * K * 2 / us / 1e6, 2)}
        del ws
    ops.check_errors()
    return out


# ------------------------------------------------------------------ the Zesapel design beside Qwen2-MoE
def zesapel_config(width, repeats=2, window=1024, vocab=32768, streams=4):
    """Layer sizes that resemble a real model's: 64-wide recurrent heads, a 512-wide latent with 128 + 64-wide
    query heads, a state of 128 per state-space head, experts as wide as the model."""
    experts, top, ff = width // 64, 2, width
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    delta = {"type": "general_delta", "mixer": {"heads": width // 64, "dim": 64}, "mlp": mlp}
    ssm = {"type": "mamba2", "mixer": {"heads": width // 32, "vdim": 64, "state": 128, "groups": 1, "conv": 4,
                                       "norm_groups": 1}, "mlp": mlp}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": width // 128, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": 768,
                     "mask": {"size": window}, "rot": {"base": 10000.0, "dims": 64}, "scale": 192 ** -0.5}}
    return {"architecture": "Zesapel", "vocab": vocab, "width": width, "streams": streams, "max_positions": 8192,
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "layers": [delta, ssm, lat] * repeats}


def qwen_config_like(z):
    """Qwen2-MoE with the same width, depth, vocabulary and number of experts; as many attention heads of 128 as the
    latent attention has; SwiGLU experts with the same number of weights as the two-matrix experts (3 I' = 2 ff)."""
    width, layers = z["width"], len(z["layers"])
    mlp = z["layers"][0]["mlp"]
    inter = max(64, (2 * mlp["expert"]["ff"] // 3) // 64 * 64)
    return dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=layers, hidden_size=width,
                num_attention_heads=width // 128, num_key_value_heads=width // 128, head_dim=128,
                num_experts=mlp["router"]["experts"], num_experts_per_tok=mlp["router"]["top"], moe_intermediate_size=inter,
                norm_topk_prob=False, decoder_sparse_step=1, intermediate_size=4 * width, vocab_size=z["vocab"],
                rope_theta=10000.0, rms_norm_eps=1e-5, use_sliding_window=False, tie_word_embeddings=False,
                max_position_embeddings=8192)


def _flush(torch, buf):
    buf.zero_()                      # larger than L2: what the step before left there is gone


def measure_engine(raw, batch, prompt_len, steps, prefill_tokens):
    """Prefill tok/s of one prompt (device time of the step function) and decode tok/s of `batch` requests at
    `prompt_len` tokens of context (device time of the replayed step), random weights, bfloat16."""
    import torch

    from dlm_b200.engine import Engine
    from dlm_b200.registry import resolve
    _, cfg, _ = resolve(dict(raw))
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", page_size=64, max_tokens=batch * (prompt_len + 512) + 8192,
                             max_requests=batch, max_step_tokens=2048, max_context=8192)
    gen = torch.Generator().manual_seed(0)
    V = eng.model.spec.vocab_size
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    times = []
    for _ in range(4):
        s = eng.cache.open()
        toks = torch.randint(0, V, (prefill_tokens,), generator=gen).tolist()
        _flush(torch, flush)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([(s, toks, [prefill_tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        eng.cache.close(s)
    eng.rt.ops.check_errors()
    pre_ms = min(times[1:])
    ids = [eng.submit(torch.randint(0, V, (prompt_len,), generator=gen).tolist(), max_new_tokens=10 ** 6) for _ in range(batch)]
    started = set()
    while len(started) < batch:
        started.update(rid for rid, _ in eng.run_step())
    for _ in range(4):
        eng.run_step()
    torch.cuda.synchronize()
    ent = eng._graphs[next(k for k in eng._graphs if k[0] == batch)]
    per = []
    for _ in range(steps):
        _flush(torch, flush)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ent["graph"].replay()
        e1.record()
        torch.cuda.synchronize()
        per.append(e0.elapsed_time(e1))
    w0 = time.perf_counter()
    produced = sum(len(eng.run_step()) for _ in range(steps))
    torch.cuda.synchronize()
    w1 = time.perf_counter()
    for i in ids:
        eng.abort(i)
    eng.scheduler.drain_finished()
    dec_ms = statistics.median(per)
    out = {"prefill_tokens": prefill_tokens, "prefill_ms": round(pre_ms, 3), "prefill_tok_s": round(prefill_tokens / pre_ms * 1e3),
           "decode_batch": batch, "decode_context": prompt_len, "decode_ms": round(dec_ms, 4),
           "decode_tok_s": round(batch / dec_ms * 1e3), "decode_e2e_tok_s": round(produced / (w1 - w0)),
           "launches_per_decode_step": ent["launches"]}
    eng._graphs.clear()
    del eng
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


def zesapel_kernels(z, pk, batch, context, prefill_tokens):
    """Each kernel of the design alone at the layer sizes of `z`: a prompt portion of `prefill_tokens` tokens of one
    request, and a decode step of `batch` requests at `context` tokens.  Microseconds (median of 5, the cache
    flushed before each), the bytes the kernel has to move at least, and that over time over the measured copy
    bandwidth."""
    import math
    from types import SimpleNamespace

    import torch

    from dlm_b200.ops import native_ops
    ops = native_ops(fast=True)
    dev = "cuda"
    W, S = z["width"], z["streams"]
    md = next(L["mixer"] for L in z["layers"] if L["type"] == "general_delta")
    ms = next(L["mixer"] for L in z["layers"] if L["type"] == "mamba2")
    ml = next(L["mixer"] for L in z["layers"] if L["type"] == "latent_attention")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    rows = {}

    def timed(name, case, fn, nbytes):
        ts = []
        for _ in range(6):
            _flush(torch, flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        us = statistics.median(ts[1:]) * 1e3
        rows.setdefault(name, {})[case] = {"us": round(us, 1), "mbytes": round(nbytes / 1e6, 2),
                                           "frac_of_copy": round(nbytes / (us * 1e-6) / 1e9 / pk["hbm_gbs"], 3)}

    for case, lens, start in (("prefill", [prefill_tokens], 0), ("decode", [1] * batch, context)):
        T, R = sum(lens), len(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        b = SimpleNamespace(num_requests=R, cu_q=torch.tensor(cu, **i32), state_slot=torch.arange(R, **i32),
                            token_req=torch.tensor([r for r, n in enumerate(lens) for _ in range(n)], **i32),
                            positions=torch.tensor([start + i for n in lens for i in range(n)], **i32))
        xs = torch.randn(T, S, W, device=dev)
        a, nw, y = torch.randn(S, device=dev), torch.randn(W, device=dev), torch.randn(T, W, device=dev)
        mix = torch.randn(S, S, device=dev)
        timed("streams_reduce+norm", case, lambda: ops.streams_reduce(xs, a, nw, 1e-5, torch.bfloat16), T * W * (4 * S + 2))
        timed("streams_update", case, lambda: ops.streams_update(xs, mix, a, y), T * W * 4 * (2 * S + 1))
        taps = z["canon"]["taps"]
        cw, cst = torch.randn(W, taps, device=dev), torch.zeros(R + 1, taps - 1, W, device=dev)
        timed("causal_conv (mixer input)", case, lambda: ops.causal_conv(y, cw, None, cst, b, True, False, torch.bfloat16),
              T * W * 6 + 2 * R * (taps - 1) * W * 4)
        # state-space scan
        H, P, N, G = ms["heads"], ms["vdim"], ms["state"], ms["groups"]
        C = H * P + 2 * G * N
        xbc, dt = torch.randn(T, C, device=dev), torch.randn(T, H, device=dev)
        hb = torch.randn(H, device=dev) * 0.1
        sst = torch.zeros(R + 1, H, N, P, device=dev)
        timed("ssm_scan", case, lambda: ops.ssm_scan(xbc, dt, hb, hb, hb, sst, b, H, P, N, G),
              T * (C + H + H * P) * 4 + 2 * R * H * N * P * 4)
        z_ = torch.randn(T, H * P, device=dev)
        nw2 = torch.randn(H * P, device=dev)
        timed("gated_rmsnorm", case, lambda: ops.gated_rmsnorm(z_, z_, nw2, ms["norm_groups"], 1e-5, "silu_before", torch.bfloat16),
              T * H * P * 10)
        # delta-rule scan
        Hd, d = md["heads"], md["dim"]
        HD = Hd * d
        proj, lw = torch.randn(T, 5 * HD + 16, device=dev), torch.randn(T, HD, device=dev)
        ab = torch.zeros(HD, device=dev)
        dst = torch.zeros(R + 1, Hd, d, d, device=dev)
        timed("delta_scan", case, lambda: ops.delta_scan(proj, (0, HD, 2 * HD, 3 * HD), lw, ab, dst, b, Hd, d, 1e-6, math.exp(-0.5)),
              T * HD * 6 * 4 + 2 * R * Hd * d * d * 4)
        # latent attention over a filled cache
        Hl, dn, dr, dv, rank, win = ml["heads"], ml["dim"], ml["rot_dim"], ml["vdim"], ml["kv_rank"], ml["mask"]["size"]
        held = start + max(lens)
        pages_each = -(-held // 64)
        cache = (torch.randn(R * pages_each + 1, 1, 64, rank + dr, device=dev) * 0.3).to(torch.bfloat16)
        table = torch.arange(R * pages_each, **i32).reshape(R, pages_each)
        q, gate = torch.randn(T, Hl * (dn + dr), device=dev), torch.randn(T, Hl, device=dev)
        wukT = (torch.randn(Hl, rank, dn, device=dev) * 0.05).to(torch.bfloat16)
        wuv = (torch.randn(Hl, dv, rank, device=dev) * 0.05).to(torch.bfloat16)
        sink = torch.zeros(Hl, device=dev)
        freq = torch.tensor([10000.0 ** (-2.0 * i / dr) for i in range(dr // 2)], device=dev)
        b.max_kv_len = held
        offs = ops.head_offsets(Hl, T, dev)
        qn, q_rot = ops.latent_q_split(q, b.positions, freq, dr, Hl, dn, dr, torch.bfloat16)
        q_lat = ops.grouped_linear(qn.reshape(Hl * T, dn), wukT, offs).reshape(Hl, T, rank)
        lat = ops.latent_attention(q_lat, q_rot, sink, cache, table, b, Hl, dr, rank, win, 0.07)
        val = ops.grouped_linear(lat.reshape(Hl * T, rank), wuv, offs)
        timed("latent_q_split", case, lambda: ops.latent_q_split(q, b.positions, freq, dr, Hl, dn, dr, torch.bfloat16),
              T * Hl * ((dn + dr) * 4 + dn * 2 + dr * 4))
        timed("queries through W_uk (grouped product)", case,
              lambda: ops.grouped_linear(qn.reshape(Hl * T, dn), wukT, offs), Hl * (T * dn * 2 + rank * dn * 2 + T * rank * 4))
        lat_bytes = (R * min(win, held) if case == "decode" else held) * (rank + dr) * 2 + T * Hl * (rank * 6 + dr * 4)
        timed("latent_attention", case, lambda: ops.latent_attention(q_lat, q_rot, sink, cache, table, b, Hl, dr, rank, win, 0.07),
              lat_bytes)
        keys = sum(min(win, start + i + 1) for n in lens for i in range(n))
        flop = 2.0 * keys * Hl * (2 * rank + dr)
        rows["latent_attention"][case]["gflop"] = round(flop / 1e9, 2)
        rows["latent_attention"][case]["frac_of_bf16_peak"] = round(
            flop / (rows["latent_attention"][case]["us"] * 1e-6) / (pk["bf16_tflops"] * 1e12), 4)
        timed("latents through W_uv (grouped product)", case,
              lambda: ops.grouped_linear(lat.reshape(Hl * T, rank), wuv, offs), Hl * (T * rank * 2 + rank * dv * 2 + T * dv * 4))
        timed("latent_gate_out", case, lambda: ops.latent_gate_out(val, gate, Hl, dv, torch.bfloat16), T * Hl * dv * 6)
    ops.check_errors()
    return rows


def run_zesapel(args, pk) -> dict:
    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    out = {"workload": "zesapel", "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)",
           "peaks": pk, "sizes": {}, "l2": "a buffer larger than L2 is written before every timed step"}
    for width in (1024, 2048):
        z = zesapel_config(width)
        q = qwen_config_like(z)
        out["sizes"][str(width)] = {
            "layers": len(z["layers"]), "zesapel": measure_engine(z, args.batch, args.prompt_len, args.steps, 2048),
            "qwen2_moe": measure_engine(q, args.batch, args.prompt_len, args.steps, 2048)}
    out["kernels_width_2048"] = zesapel_kernels(zesapel_config(2048), pk, args.batch, args.prompt_len, 2048)
    t1 = time.time()
    time.sleep(0.2)
    sampler.stop()
    out["clocks"] = sampler.summary(t0, t1)
    return out


# ------------------------------------------------------------------ the Zasazen design beside Qwen2-MoE
def zasazen_config(width, vocab=32768):
    """Layer sizes that resemble a real model's: 64-wide attention heads with four query heads a key/value head,
    retention heads of 64 x 128, a selective scan twice as wide as the model with 16 states a channel, a gelu
    feed-forward four times the width, 16 gated experts of half the width with a shared one of the width; the two
    middle layers run twice (8 layer runs)."""
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": width // 2}, "shared": {"ff": width}}
    dense = {"kind": "dense", "ff": 4 * width}
    hr = width // 128
    pair = {"type": "parallel", "mixer": {
        "left": {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64, "scale": 0.125,
                 "q_temp": {"coef": 0.5, "every": 512}},
        "right": {"heads": hr, "dim": 64, "vdim": 128, "decay": [1.0 - 2.0 ** (-5 - 5 * i / max(hr - 1, 1)) for i in range(hr)],
                  "rot": {"base": 1e6, "dims": 64}}}}
    scan = {"type": "mamba1", "mixer": {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}}
    layers = [dict(pair, mlp=dense), dict(pair, mlp=moe), dict(scan, mlp=moe), dict(pair, mlp=dense), dict(scan, mlp=dense),
              dict(pair, mlp=moe)]
    return {"architecture": "Zasazen", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "loop": {"start": 1, "stop": 3, "times": 2}, "layers": layers}


def qwen_config_like_zasazen(z):
    """Qwen2-MoE with the same width, vocabulary and as many layers as the design has layer runs; attention heads of
    the same number and size; routed layers where the design's runs have experts (same experts, same shared one),
    dense SwiGLU layers with as many weights as the gelu feed-forward (3 I' = 2 ff) elsewhere."""
    from dlm_b200.models.zasazen import layer_order
    width = z["width"]
    runs = [z["layers"][c.layer] for c in layer_order(len(z["layers"]), z.get("loop"))]
    left = z["layers"][0]["mixer"]["left"]
    moe = next(L["mlp"] for L in z["layers"] if L["mlp"]["kind"] == "moe")
    dense = next(L["mlp"] for L in z["layers"] if L["mlp"]["kind"] == "dense")
    return dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=len(runs), hidden_size=width,
                num_attention_heads=left["heads"], num_key_value_heads=left["kv_heads"], head_dim=left["dim"],
                num_experts=moe["router"]["experts"], num_experts_per_tok=moe["router"]["top"],
                moe_intermediate_size=moe["expert"]["ff"], shared_expert_intermediate_size=moe["shared"]["ff"],
                norm_topk_prob=True, decoder_sparse_step=1,
                mlp_only_layers=[i for i, L in enumerate(runs) if L["mlp"]["kind"] == "dense"],
                intermediate_size=(2 * dense["ff"] // 3) // 64 * 64, vocab_size=z["vocab"], rope_theta=10000.0,
                rms_norm_eps=1e-5, use_sliding_window=False, tie_word_embeddings=False, max_position_embeddings=8192)


def zasazen_kernels(z, pk, batch, context, prefill_tokens):
    """Each kernel of the design alone at the layer sizes of `z`: a prompt of `prefill_tokens` tokens of one request,
    and a decode step of `batch` requests at `context` tokens.  Microseconds (median of 5, the cache flushed before
    each), the bytes the kernel has to move at least, and that over time over the measured copy bandwidth; the
    attention also without its distance penalty (the closest model's kernel at the same sizes) and with its flops."""
    from types import SimpleNamespace

    import torch

    from dlm_b200.ops import native_ops
    ops = native_ops(fast=True)
    dev = "cuda"
    W = z["width"]
    pair = next(L["mixer"] for L in z["layers"] if L["type"] == "parallel")
    ms = next(L["mixer"] for L in z["layers"] if L["type"] == "mamba1")
    lf, rt = pair["left"], pair["right"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    rows = {}

    def timed(name, case, fn, nbytes, flop=None):
        ts = []
        for _ in range(6):
            _flush(torch, flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        us = statistics.median(ts[1:]) * 1e3
        row = {"us": round(us, 1), "mbytes": round(nbytes / 1e6, 2),
               "frac_of_copy": round(nbytes / (us * 1e-6) / 1e9 / pk["hbm_gbs"], 3)}
        if flop is not None:
            row["gflop"] = round(flop / 1e9, 2)
            row["frac_of_bf16_peak"] = round(flop / (us * 1e-6) / (pk["bf16_tflops"] * 1e12), 4)
        rows.setdefault(name, {})[case] = row

    for case, lens, start in (("prefill", [prefill_tokens], 0), ("decode", [1] * batch, context)):
        T, R = sum(lens), len(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        b = SimpleNamespace(num_requests=R, cu_q=torch.tensor(cu, **i32), state_slot=torch.arange(R, **i32),
                            token_req=torch.tensor([r for r, n in enumerate(lens) for _ in range(n)], **i32),
                            positions=torch.tensor([start + i for n in lens for i in range(n)], **i32))
        # selective scan and its convolution
        inner, N, taps = ms["inner"], ms["state"], ms["conv"]
        xz = torch.randn(T, 2 * inner, device=dev)
        cw, cb = torch.randn(inner, taps, device=dev), torch.randn(inner, device=dev)
        cst = torch.zeros(R + 1, taps - 1, inner, device=dev)
        timed("causal_conv + silu (scan input)", case,
              lambda: ops.causal_conv(xz[:, :inner], cw, cb, cst, b, False, True, torch.float32),
              T * inner * 8 + 2 * R * (taps - 1) * inner * 4)
        x, dt, bc = torch.randn(T, inner, device=dev), torch.randn(T, inner, device=dev), torch.randn(T, 2 * N, device=dev)
        A_log, vec = torch.rand(inner, N, device=dev), torch.randn(inner, device=dev) * 0.1
        sst = torch.zeros(R + 1, inner, N, device=dev)
        timed("selective_scan", case, lambda: ops.selective_scan(x, dt, bc, xz[:, inner:], vec, A_log, vec, sst, b, torch.bfloat16),
              T * (inner * 14 + 2 * N * 4) + 2 * R * inner * N * 4 + inner * N * 4)
        # retention: rotation, scan with constant decays, head norm and gate
        H2, d2, dv2 = rt["heads"], rt["dim"], rt["vdim"]
        proj = torch.randn(T, 2 * H2 * dv2 + 2 * H2 * d2, device=dev)
        freq = torch.tensor([1e6 ** (-2.0 * i / d2) for i in range(d2 // 2)], device=dev)
        decay = torch.tensor(rt["decay"], device=dev)
        rst = torch.zeros(R + 1, H2, d2, dv2, device=dev)
        timed("rotate_heads (q, k in place)", case,
              lambda: ops.rotate_heads(proj, b.positions, freq, d2, H2, d2, H2 * dv2, d2 ** -0.5, H2 * dv2 + H2 * d2, 1.0),
              T * 2 * H2 * d2 * 8)
        timed("ssm_scan with constant decays (retention)", case,
              lambda: ops.ssm_scan(proj[:, :H2 * dv2 + 2 * H2 * d2], None, None, None, None, rst, b, H2, dv2, d2, H2,
                                   fixed_decay=decay),
              T * (H2 * dv2 * 2 + 2 * H2 * d2) * 4 + 2 * R * H2 * d2 * dv2 * 4)
        o_ = torch.randn(T, H2 * dv2, device=dev)
        timed("gated_rmsnorm (per head, silu gate)", case,
              lambda: ops.gated_rmsnorm(o_, proj[:, H2 * dv2 + 2 * H2 * d2:], None, H2, 1e-5, "silu_after", torch.bfloat16),
              T * H2 * dv2 * 10)
        # attention: norms, temperature and cache write; then the attention with and without the distance penalty
        H, G, d, dv = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
        D = max(d, dv)
        held = start + max(lens)
        pages_each = -(-held // 64)
        k_cache = (torch.randn(R * pages_each + 1, G, 64, D, device=dev) * 0.3).to(torch.bfloat16)
        v_cache = (torch.randn(R * pages_each + 1, G, 64, D, device=dev) * 0.3).to(torch.bfloat16)
        table = torch.arange(R * pages_each, **i32).reshape(R, pages_each)
        slots = torch.cat([table[r, (start + torch.arange(n, device=dev)) // 64] * 64 + (start + torch.arange(n, device=dev)) % 64
                           for r, n in enumerate(lens)]).to(torch.int32)
        qkv = torch.randn(T, (H + G) * d + G * dv, device=dev)
        qn, kn = torch.randn(H * d, device=dev), torch.randn(G * d, device=dev)
        timed("qk_norm_write", case,
              lambda: ops.qk_norm_write(qkv, b.positions, qn, kn, 1e-5, 0.5, 512, slots, k_cache, v_cache, H, G, d, dv, D,
                                        torch.bfloat16), T * ((H + G) * d + G * dv) * 4 + T * (H + 2 * G) * D * 2)
        q = ops.qk_norm_write(qkv, b.positions, qn, kn, 1e-5, 0.5, 512, slots, k_cache, v_cache, H, G, d, dv, D, torch.bfloat16)
        kv_len = torch.tensor([start + n for n in lens], **i32)
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
        single = sum(1 for n in lens if n == 1)
        keys = sum(start + i + 1 for n in lens for i in range(n))
        att_bytes = R * held * G * D * 4 + T * H * D * 4 if case == "decode" else held * G * D * 4 + T * H * D * 4
        for name, sl in (("attention with distance penalty", slopes), ("attention without it (Qwen2-MoE's)", None)):
            timed(name, case, lambda: ops.attention(q, k_cache, v_cache, table, b.cu_q, kv_len, 0, 0.125, H, G, D, max(lens),
                                                    held, single, slopes=sl), att_bytes, flop=4.0 * keys * H * D)
        # the pair's sum and the pass entry
        ya, yb, resid = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
        wv = torch.randn(W, device=dev)
        timed("branch_norm_add", case, lambda: ops.branch_norm_add(resid, ya, wv, yb, wv, 1e-5, 0.5), T * W * 16)
        timed("concat_rows (pass entry)", case, lambda: ops.concat_rows(ya, yb, torch.bfloat16), T * W * 12)
        up = torch.randn(T, 4 * W, device=dev)
        timed("activation gelu (tanh form)", case, lambda: ops.activation(up, "gelu_tanh", torch.bfloat16), T * 4 * W * 6)
    ops.check_errors()
    return rows


def run_zasazen(args, pk) -> dict:
    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    out = {"workload": "zasazen", "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)",
           "peaks": pk, "sizes": {}, "l2": "a buffer larger than L2 is written before every timed step"}
    for width in (1024, 2048):
        z = zasazen_config(width)
        q = qwen_config_like_zasazen(z)
        out["sizes"][str(width)] = {
            "layer_runs": q["num_hidden_layers"], "zasazen": measure_engine(z, args.batch, args.prompt_len, args.steps, 2048),
            "qwen2_moe": measure_engine(q, args.batch, args.prompt_len, args.steps, 2048)}
    out["kernels_width_2048"] = zasazen_kernels(zasazen_config(2048), pk, args.batch, args.prompt_len, 2048)
    t1 = time.time()
    time.sleep(0.2)
    sampler.stop()
    out["clocks"] = sampler.summary(t0, t1)
    return out


def salolorn_config(width, vocab=32768, chunk=2048):
    """Layer sizes that resemble a real model's: delta-rule heads of 128 x 128 with two value heads a query/key head
    behind convolutions of four taps, a 512-wide latent with 128 + 64-wide query heads, 64-wide attention heads with
    four query heads a key/value head inside chunks of `chunk` positions, linear-attention heads of 64 x 128 whose
    decay comes through a bottleneck of 16, a gated feed-forward three times the width; the last three layers run
    twice (7 layer runs)."""
    dense = {"kind": "dense", "ff": 3 * width}
    delta = {"type": "delta", "mlp": dense,
             "mixer": {"heads": width // 128, "kv_heads": width // 256, "dim": 128, "vdim": 128, "conv": 4}}
    lat = {"type": "latent_attention", "mlp": dense,
           "mixer": {"heads": width // 128, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
                     "rot": {"base": 10000.0, "dims": 64}}}
    pair = {"type": "parallel", "mlp": dense, "mixer": {
        "left": {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64, "scale": 0.125,
                 "mask": {"size": chunk}, "rot": {"base": 1e6, "dims": 64}},
        "right": {"heads": width // 128, "dim": 64, "vdim": 128, "tau": 16.0}, "left_scale": 1.0, "right_scale": 1.0}}
    return {"architecture": "Salolorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "max_positions": 8192, "loop": {"start": 1, "stop": 4, "times": 2}, "layers": [delta, dict(delta), lat, pair]}


def qwen_config_like_salolorn(z):
    """A dense Qwen2 (the Qwen2-MoE class with no experts) with the same width, vocabulary and feed-forward and as
    many layers as the design has layer runs; attention heads of the same number and size as the chunked attention."""
    from dlm_b200.models.zasazen import layer_order
    runs = len(layer_order(len(z["layers"]), z.get("loop")))
    left = z["layers"][-1]["mixer"]["left"]
    return dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=runs, hidden_size=z["width"],
                num_attention_heads=left["heads"], num_key_value_heads=left["kv_heads"], head_dim=left["dim"],
                num_experts=0, intermediate_size=z["layers"][0]["mlp"]["ff"], vocab_size=z["vocab"], rope_theta=1e6,
                rms_norm_eps=1e-6, use_sliding_window=False, tie_word_embeddings=True, max_position_embeddings=8192)


def salolorn_kernels(z, pk, batch, context, prefill_tokens):
    """Each kernel of the design alone at the layer sizes of `z`, beside the like kernel of an existing model at the
    same sizes: a prompt of `prefill_tokens` tokens of one request, and a decode step of `batch` requests at `context`
    tokens.  Microseconds (median of 5, the cache flushed before each), the bytes the kernel has to move at least,
    and that over time over the measured copy bandwidth; the attentions also with their flops."""
    import math
    from types import SimpleNamespace

    import torch

    from dlm_b200.ops import native_ops
    ops = native_ops(fast=True)
    dev = "cuda"
    W = z["width"]
    md = next(L["mixer"] for L in z["layers"] if L["type"] == "delta")
    ml = next(L["mixer"] for L in z["layers"] if L["type"] == "latent_attention")
    pair = next(L["mixer"] for L in z["layers"] if L["type"] == "parallel")
    lf, rt = pair["left"], pair["right"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    bf = torch.bfloat16
    rows = {}

    def timed(name, case, fn, nbytes, flop=None):
        ts = []
        for _ in range(6):
            _flush(torch, flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        us = statistics.median(ts[1:]) * 1e3
        row = {"us": round(us, 1), "mbytes": round(nbytes / 1e6, 2),
               "frac_of_copy": round(nbytes / (us * 1e-6) / 1e9 / pk["hbm_gbs"], 3)}
        if flop is not None:
            row["gflop"] = round(flop / 1e9, 2)
            row["frac_of_bf16_peak"] = round(flop / (us * 1e-6) / (pk["bf16_tflops"] * 1e12), 4)
        rows.setdefault(name, {})[case] = row

    for case, lens, start in (("prefill", [prefill_tokens], 0), ("decode", [1] * batch, context)):
        T, R = sum(lens), len(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        b = SimpleNamespace(num_requests=R, cu_q=torch.tensor(cu, **i32), state_slot=torch.arange(R, **i32),
                            token_req=torch.tensor([r for r, n in enumerate(lens) for _ in range(n)], **i32),
                            positions=torch.tensor([start + i for n in lens for i in range(n)], **i32))
        held = start + max(lens)
        b.max_kv_len = held
        pages_each = -(-held // 64)
        table = torch.arange(R * pages_each, **i32).reshape(R, pages_each)
        slots = torch.cat([table[r, (start + torch.arange(n, device=dev)) // 64] * 64 + (start + torch.arange(n, device=dev)) % 64
                           for r, n in enumerate(lens)]).to(torch.int32)
        kv_len = torch.tensor([start + n for n in lens], **i32)
        single = sum(1 for n in lens if n == 1)
        # ---- delta rule: convolutions, the recurrence, the norm per head with its gate
        H, G, d, dv, taps = md["heads"], md["kv_heads"], md["dim"], md["vdim"], md["conv"]
        C = 2 * G * d + H * dv
        proj = torch.randn(T, C + 2 * H + H * dv, device=dev)
        cw = torch.randn(C, taps, device=dev) * 0.5
        cst = torch.zeros(R + 1, taps - 1, C, device=dev)
        timed("causal_conv + silu (q, k, v of the delta rule)", case,
              lambda: ops.causal_conv(proj[:, :C], cw, None, cst, b, False, True, torch.float32),
              T * C * 8 + 2 * R * (taps - 1) * C * 4)
        qkv = ops.causal_conv(proj[:, :C], cw, None, cst, b, False, True, torch.float32)
        A_log, dtb = torch.rand(H, device=dev) - 1.0, torch.randn(H, device=dev)
        dst = torch.zeros(R + 1, H, d, dv, device=dev)
        timed("gated_scan, delta rule with a decay per head", case,
              lambda: ops.gated_scan(qkv[:, :G * d], qkv[:, G * d:2 * G * d], qkv[:, 2 * G * d:], proj[:, C + H:C + 2 * H],
                                     proj[:, C:C + H], dst, b, H, G, d, dv, unit_eps=1e-6, q_scale=d ** -0.5, A_log=A_log,
                                     decay_bias=dtb),
              T * (2 * G * d + 2 * H * dv + 2 * H) * 4 + 2 * R * H * d * dv * 4)
        Hz, dz = W // 64, 64                                       # Zesapel's delta rule at the same width
        HD = Hz * dz
        zproj, lw, ab = torch.randn(T, 5 * HD + 16, device=dev), torch.randn(T, HD, device=dev), torch.zeros(HD, device=dev)
        zst = torch.zeros(R + 1, Hz, dz, dz, device=dev)
        timed("delta_scan (Zesapel's delta rule, 64 x 64 heads)", case,
              lambda: ops.delta_scan(zproj, (0, HD, 2 * HD, 3 * HD), lw, ab, zst, b, Hz, dz, 1e-6, math.exp(-0.5)),
              T * HD * 6 * 4 + 2 * R * Hz * dz * dz * 4)
        o_ = torch.randn(T, H * dv, device=dev)
        nw = torch.randn(H * dv, device=dev)
        timed("gated_rmsnorm (per head, silu gate)", case,
              lambda: ops.gated_rmsnorm(o_, proj[:, C + 2 * H:], nw, H, 1e-6, "silu_after", bf), T * H * dv * 10)
        # ---- linear attention with a decay per key channel, beside the recurrence with constant decays
        H2, d2, dv2 = rt["heads"], rt["dim"], rt["vdim"]
        gp = torch.randn(T, 3 * H2 * d2 + H2 * dv2, device=dev)
        gst = torch.zeros(R + 1, H2, d2, dv2, device=dev)
        timed("gated_scan, decay per key channel", case,
              lambda: ops.gated_scan(gp[:, :H2 * d2], gp[:, H2 * d2:2 * H2 * d2], gp[:, 3 * H2 * d2:], gp[:, 2 * H2 * d2:3 * H2 * d2],
                                     None, gst, b, H2, H2, d2, dv2, q_scale=d2 ** -0.5, tau=rt["tau"]),
              T * (3 * H2 * d2 + 2 * H2 * dv2) * 4 + 2 * R * H2 * d2 * dv2 * 4)
        rp = torch.randn(T, H2 * dv2 + 2 * H2 * d2, device=dev)
        decay = torch.tensor([1.0 - 2.0 ** (-5 - 5 * i / max(H2 - 1, 1)) for i in range(H2)], device=dev)
        rst = torch.zeros(R + 1, H2, d2, dv2, device=dev)
        timed("ssm_scan with constant decays (Zasazen's retention)", case,
              lambda: ops.ssm_scan(rp, None, None, None, None, rst, b, H2, dv2, d2, H2, fixed_decay=decay),
              T * (H2 * dv2 * 2 + 2 * H2 * d2) * 4 + 2 * R * H2 * d2 * dv2 * 4)
        # ---- attention inside chunks with a sink and a gate, beside the plain causal attention
        Ha, Ga, da, dva = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
        D = max(da, dva)
        chunk = lf["mask"]["size"]
        k_cache = (torch.randn(R * pages_each + 1, Ga, 64, D, device=dev) * 0.3).to(bf)
        v_cache = (torch.randn(R * pages_each + 1, Ga, 64, D, device=dev) * 0.3).to(bf)
        aq = torch.randn(T, (Ha + Ga) * da + Ga * dva + Ha, device=dev)
        qn, kn = torch.randn(da, device=dev), torch.randn(da, device=dev)
        freq = torch.tensor([1e6 ** (-2.0 * i / da) for i in range(da // 2)], device=dev)
        io = T * ((Ha + Ga) * da + Ga * dva) * 4 + T * (Ha + 2 * Ga) * D * 2
        timed("head_norm_rope_write", case,
              lambda: ops.head_norm_rope_write(aq, b.positions, qn, kn, 1e-6, freq, da, False, slots, k_cache, v_cache, Ha,
                                               Ga, da, dva, D, bf), io)
        pq = torch.randn(T, (Ha + 2 * Ga) * D, device=dev)
        timed("rope_kv_write (Qwen2's)", case,
              lambda: ops.rope_kv_write(pq, b.positions, freq, D, slots, k_cache, v_cache, Ha, Ga, D, bf), io)
        q = ops.head_norm_rope_write(aq, b.positions, qn, kn, 1e-6, freq, da, False, slots, k_cache, v_cache, Ha, Ga, da,
                                     dva, D, bf)
        sinks = torch.randn(Ha, device=dev)
        seen = [(start + i) % chunk + 1 for n in lens for i in range(n)]       # keys a query meets inside its chunk
        for name, ch, sk, keys, span in (
                ("attention inside chunks with a sink", chunk, sinks, sum(seen), min(chunk, held)),
                ("attention, causal (Qwen2's)", 0, None, sum(start + i + 1 for n in lens for i in range(n)), held)):
            nbytes = (R * max(seen) if (case == "decode" and ch) else (R if case == "decode" else 1) * span) * Ga * D * 4 \
                + T * Ha * D * 4
            timed(name, case, lambda: ops.attention(q, k_cache, v_cache, table, b.cu_q, kv_len, 0, 0.125, Ha, Ga, D, max(lens),
                                                    held, single, chunk=ch, sinks=sk), nbytes, flop=4.0 * keys * Ha * D)
        o2 = torch.randn(T, Ha * D, device=dev).to(bf)
        timed("head_gate", case, lambda: ops.head_gate(o2, aq[:, (Ha + Ga) * da + Ga * dva:], Ha, D, 1.0), T * Ha * D * 4)
        # ---- latent attention: direct queries, neighbour pairs, no window and no sink
        Hl, dn, dr, dvl, rank = ml["heads"], ml["dim"], ml["rot_dim"], ml["vdim"], ml["kv_rank"]
        cache = (torch.randn(R * pages_each + 1, 1, 64, rank + dr, device=dev) * 0.3).to(bf)
        lp = torch.randn(T, Hl * (dn + dr) + rank + dr, device=dev)
        kvn = torch.randn(rank, device=dev)
        lfreq = torch.tensor([10000.0 ** (-2.0 * i / dr) for i in range(dr // 2)], device=dev)
        qc = Hl * (dn + dr)
        timed("latent_prep (norm, rotation, cache write)", case,
              lambda: ops.latent_prep(lp, 0, 0, None, qc, rank, kvn, dr, lfreq, dr, b.positions, slots, 1e-6, cache, bf,
                                      interleaved=True), T * (rank + dr) * 6)
        wukT = (torch.randn(Hl, rank, dn, device=dev) * 0.05).to(bf)
        wuv = (torch.randn(Hl, dvl, rank, device=dev) * 0.05).to(bf)
        offs = ops.head_offsets(Hl, T, dev)
        lq = lp[:, :qc]
        qpl, q_rot = ops.latent_q_split(lq, b.positions, lfreq, dr, Hl, dn, dr, bf, interleaved=True)
        q_lat = ops.grouped_linear(qpl.reshape(Hl * T, dn), wukT, offs).reshape(Hl, T, rank)
        lat = ops.latent_attention(q_lat, q_rot, None, cache, table, b, Hl, dr, rank, 0, 0.07)
        val = ops.grouped_linear(lat.reshape(Hl * T, rank), wuv, offs)
        timed("latent_q_split (neighbour pairs)", case,
              lambda: ops.latent_q_split(lq, b.positions, lfreq, dr, Hl, dn, dr, bf, interleaved=True),
              T * Hl * ((dn + dr) * 4 + dn * 2 + dr * 4))
        timed("queries through W_uk (grouped product)", case,
              lambda: ops.grouped_linear(qpl.reshape(Hl * T, dn), wukT, offs), Hl * (T * dn * 2 + rank * dn * 2 + T * rank * 4))
        zero_sink = torch.zeros(Hl, device=dev)
        for name, win, sk in (("latent_attention, all keys, no sink", 0, None),
                              ("latent_attention, window 1024 and a sink (Zesapel's)", 1024, zero_sink)):
            keys = sum(min(win or 10 ** 9, start + i + 1) for n in lens for i in range(n))
            span = min(win or held, held)
            timed(name, case, lambda: ops.latent_attention(q_lat, q_rot, sk, cache, table, b, Hl, dr, rank, win, 0.07),
                  (R * span if case == "decode" else held) * (rank + dr) * 2 + T * Hl * (rank * 6 + dr * 4),
                  flop=2.0 * keys * Hl * (2 * rank + dr))
        timed("latents through W_uv (grouped product)", case,
              lambda: ops.grouped_linear(lat.reshape(Hl * T, rank), wuv, offs), Hl * (T * rank * 2 + rank * dvl * 2 + T * dvl * 4))
        timed("latent_gate_out (no gate)", case, lambda: ops.latent_gate_out(val, None, Hl, dvl, bf), T * Hl * dvl * 6)
        # ---- norms on both sides of a sublayer, the pass entry
        resid, y, x0 = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
        wv = torch.randn(W, device=dev)
        timed("norm_add_norm (closing norm, add, opening norm)", case,
              lambda: ops.norm_add_norm(resid, y, wv, wv, 1e-6, bf), T * W * 14)
        timed("rmsnorm (Qwen2's opening norm)", case, lambda: ops.rmsnorm(resid, wv, 1e-6, bf), T * W * 6)
        timed("add_vec_rows (pass entry)", case, lambda: ops.add_vec_rows(resid, x0, wv), T * W * 12)
    ops.check_errors()
    return rows


def run_salolorn(args, pk) -> dict:
    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    out = {"workload": "salolorn", "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)",
           "peaks": pk, "sizes": {}, "l2": "a buffer larger than L2 is written before every timed step"}
    for width in (1024, 2048, 4096):
        z = salolorn_config(width)
        q = qwen_config_like_salolorn(z)
        out["sizes"][str(width)] = {
            "layer_runs": q["num_hidden_layers"], "salolorn": measure_engine(z, args.batch, args.prompt_len, args.steps, 2048),
            "qwen2_dense": measure_engine(q, args.batch, args.prompt_len, args.steps, 2048)}
    out["kernels_width_2048"] = salolorn_kernels(salolorn_config(2048), pk, args.batch, args.prompt_len, 2048)
    t1 = time.time()
    time.sleep(0.2)
    sampler.stop()
    out["clocks"] = sampler.summary(t0, t1)
    return out


def faguzen_config(width, vocab=32768):
    """Four layers of the design at a real model's layer sizes, the middle two run twice (6 layer runs): attention
    heads of 128 (four query heads a key/value head, half of each head rotated), a matrix memory with heads of 64 x 128,
    16 experts of `width / 2` of which each token takes 2 out of 16 + 2 (two identity experts), a shared expert of
    `width`; the last layer has no feed-forward."""
    heads = width // 128
    mixer = {"left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                      "softcap": 50.0, "rot": {"base": 1e6, "dims": 64,
                                               "scaling": {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 8192}}},
             "right": {"heads": width // 128, "dim": 64, "vdim": 128, "gate_cap": 15.0}, "left_scale": 1.0, "right_scale": 1.0}
    mlp = {"kind": "moe", "router": {"experts": 16, "identity": 2, "top": 2}, "expert": {"ff": width // 2},
           "shared": {"ff": width}}
    layers = [{"type": "parallel", "mixer": mixer, "mlp": mlp} for _ in range(3)] + [{"type": "parallel", "mixer": mixer, "mlp": None}]
    return {"architecture": "Faguzen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.8,
            "logit_softcap": 25.0, "max_positions": 8192, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": layers}


def qwen_config_like_faguzen(z):
    """Qwen2-MoE with the same width and vocabulary and as many layers as the design has layer runs; attention heads
    of the same number and size; the same experts (count, size, two a token) and shared expert in every layer."""
    from dlm_b200.models.zasazen import layer_order
    runs = len(layer_order(len(z["layers"]), z.get("loop")))
    left, mlp = z["layers"][0]["mixer"]["left"], z["layers"][0]["mlp"]
    return dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=runs, hidden_size=z["width"],
                num_attention_heads=left["heads"], num_key_value_heads=left["kv_heads"], head_dim=left["dim"],
                num_experts=mlp["router"]["experts"], num_experts_per_tok=mlp["router"]["top"],
                moe_intermediate_size=mlp["expert"]["ff"], shared_expert_intermediate_size=mlp["shared"]["ff"],
                norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], intermediate_size=z["width"],
                vocab_size=z["vocab"], rope_theta=10000.0, rms_norm_eps=1e-6, use_sliding_window=False,
                tie_word_embeddings=False, max_position_embeddings=8192)


def faguzen_kernels(z, pk, batch, context, prefill_tokens):
    """Each kernel of the design alone at the layer sizes of `z`, beside the like kernel of an existing model at the
    same sizes: a prompt of `prefill_tokens` tokens of one request, and a decode step of `batch` requests at `context`
    tokens.  Microseconds (median of 5, the cache flushed before each), the bytes the kernel has to move at least,
    and that over time over the measured copy bandwidth; the attentions also with their flops."""
    from types import SimpleNamespace

    import torch

    from dlm_b200.ops import native_ops
    ops = native_ops(fast=True)
    dev = "cuda"
    W = z["width"]
    mixer, mlp = z["layers"][0]["mixer"], z["layers"][0]["mlp"]
    lf, rt = mixer["left"], mixer["right"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    bf = torch.bfloat16
    rows = {}

    def timed(name, case, fn, nbytes, flop=None):
        ts = []
        for _ in range(6):
            _flush(torch, flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        us = statistics.median(ts[1:]) * 1e3
        row = {"us": round(us, 1), "mbytes": round(nbytes / 1e6, 2),
               "frac_of_copy": round(nbytes / (us * 1e-6) / 1e9 / pk["hbm_gbs"], 3)}
        if flop is not None:
            row["gflop"] = round(flop / 1e9, 2)
            row["frac_of_bf16_peak"] = round(flop / (us * 1e-6) / (pk["bf16_tflops"] * 1e12), 4)
        rows.setdefault(name, {})[case] = row

    for case, lens, start in (("prefill", [prefill_tokens], 0), ("decode", [1] * batch, context)):
        T, R = sum(lens), len(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        b = SimpleNamespace(num_requests=R, cu_q=torch.tensor(cu, **i32), state_slot=torch.arange(R, **i32),
                            token_req=torch.tensor([r for r, n in enumerate(lens) for _ in range(n)], **i32),
                            positions=torch.tensor([start + i for n in lens for i in range(n)], **i32))
        held = start + max(lens)
        pages_each = -(-held // 64)
        table = torch.arange(R * pages_each, **i32).reshape(R, pages_each)
        slots = torch.cat([table[r, (start + torch.arange(n, device=dev)) // 64] * 64 + (start + torch.arange(n, device=dev)) % 64
                           for r, n in enumerate(lens)]).to(torch.int32)
        kv_len = torch.tensor([start + n for n in lens], **i32)
        single = sum(1 for n in lens if n == 1)
        # ---- the norm without statistics beside the RMS norm, alone and in pairs
        resid = torch.randn(T, W, device=dev)
        wv, bv = torch.randn(W, device=dev), torch.randn(W, device=dev)
        timed("dyt_norm", case, lambda: ops.dyt_norm(resid, wv, bv, 0.7, bf), T * W * 6)
        timed("rmsnorm (Qwen2's)", case, lambda: ops.rmsnorm(resid, wv, 1e-6, bf), T * W * 6)
        timed("dyt_norm_pair (two norms and the router's 32-bit input)", case,
              lambda: ops.dyt_norm_pair(resid, wv, bv, 0.7, wv, bv, 0.9, bf, want_f32=True), T * W * 12)
        timed("rmsnorm_pair (Zasazen's)", case, lambda: ops.rmsnorm_pair(resid, wv, wv, 1e-6, bf), T * W * 8)
        # ---- matrix memory with a running maximum, beside the recurrences with one decay per head
        H2, d2, dv2 = rt["heads"], rt["dim"], rt["vdim"]
        mp = torch.randn(T, 2 * H2 * d2 + 2 * H2 * dv2 + 2 * H2, device=dev)
        q_, k_, v_ = mp[:, :H2 * d2], mp[:, H2 * d2:2 * H2 * d2], mp[:, 2 * H2 * d2:2 * H2 * d2 + H2 * dv2]
        g_ = mp[:, 2 * H2 * d2 + H2 * dv2:2 * H2 * d2 + 2 * H2 * dv2]
        ig, fg = mp[:, -2 * H2:-H2], mp[:, -H2:]
        ib, fb = torch.zeros(H2, device=dev), torch.ones(H2, device=dev)
        S, nst, mst = (torch.zeros(R + 1, H2, d2, dv2, device=dev), torch.zeros(R + 1, H2, d2, device=dev),
                       torch.zeros(R + 1, H2, dv2 + 1, device=dev))
        scan_bytes = T * (2 * H2 * d2 + 2 * H2 * dv2 + 2 * H2) * 4 + 2 * R * H2 * d2 * dv2 * 4
        timed("memory_scan (exponential gates, running maximum, normaliser)", case,
              lambda: ops.memory_scan(q_, k_, v_, ig, fg, ib, fb, rt["gate_cap"], S, nst, mst, b, H2, d2, dv2,
                                      q_scale=d2 ** -0.5), scan_bytes + T * H2 * 4)
        A_log, dtb = torch.rand(H2, device=dev) - 1.0, torch.randn(H2, device=dev)
        gst = torch.zeros(R + 1, H2, d2, dv2, device=dev)
        timed("gated_scan, delta rule with a decay per head (Salolorn's)", case,
              lambda: ops.gated_scan(q_, k_, v_, fg, ig, gst, b, H2, H2, d2, dv2, unit_eps=1e-6, q_scale=d2 ** -0.5,
                                     A_log=A_log, decay_bias=dtb), scan_bytes)
        rp = torch.randn(T, H2 * dv2 + 2 * H2 * d2, device=dev)
        decay = torch.tensor([1.0 - 2.0 ** (-5 - 5 * i / max(H2 - 1, 1)) for i in range(H2)], device=dev)
        timed("ssm_scan with constant decays (Zasazen's retention)", case,
              lambda: ops.ssm_scan(rp, None, None, None, None, gst, b, H2, dv2, d2, H2, fixed_decay=decay),
              T * (H2 * dv2 * 2 + 2 * H2 * d2) * 4 + 2 * R * H2 * d2 * dv2 * 4)
        o_, rden = ops.memory_scan(q_, k_, v_, ig, fg, ib, fb, rt["gate_cap"], S, nst, mst, b, H2, d2, dv2, q_scale=d2 ** -0.5)
        nw = torch.randn(H2 * dv2, device=dev)
        timed("gated_rmsnorm (per head, a factor per row, sigmoid gate)", case,
              lambda: ops.gated_rmsnorm(o_, g_, nw, H2, 1e-6, "sigmoid_after", bf, row_scale=rden), T * H2 * dv2 * 10)
        timed("gated_rmsnorm (per head, silu gate; Salolorn's)", case,
              lambda: ops.gated_rmsnorm(o_, g_, nw, H2, 1e-6, "silu_after", bf), T * H2 * dv2 * 10)
        # ---- attention with capped scores and a gate per entry, beside the plain causal attention
        Ha, Ga, da, dva = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
        D = max(da, dva)
        k_cache = (torch.randn(R * pages_each + 1, Ga, 64, D, device=dev) * 0.3).to(bf)
        v_cache = (torch.randn(R * pages_each + 1, Ga, 64, D, device=dev) * 0.3).to(bf)
        aq = torch.randn(T, (Ha + Ga) * da + Ga * dva + Ha * dva, device=dev)
        rd = lf["rot"]["dims"]
        freq = torch.tensor([lf["rot"]["base"] ** (-2.0 * i / rd) for i in range(rd // 2)], device=dev)
        io = T * ((Ha + Ga) * da + Ga * dva) * 4 + T * (Ha + 2 * Ga) * D * 2
        timed("head_norm_rope_write (no norms, half of each head rotated)", case,
              lambda: ops.head_norm_rope_write(aq, b.positions, None, None, 1e-6, freq, rd, False, slots, k_cache, v_cache,
                                               Ha, Ga, da, dva, D, bf), io)
        pq = torch.randn(T, (Ha + 2 * Ga) * D, device=dev)
        ffreq = torch.tensor([1e4 ** (-2.0 * i / D) for i in range(D // 2)], device=dev)
        timed("rope_kv_write (Qwen2's)", case,
              lambda: ops.rope_kv_write(pq, b.positions, ffreq, D, slots, k_cache, v_cache, Ha, Ga, D, bf), io)
        q = ops.head_norm_rope_write(aq, b.positions, None, None, 1e-6, freq, rd, False, slots, k_cache, v_cache, Ha, Ga,
                                     da, dva, D, bf)
        keys = sum(start + i + 1 for n in lens for i in range(n))
        nbytes = (R if case == "decode" else 1) * held * Ga * D * 4 + T * Ha * D * 4
        for name, cap in (("attention, causal, scores capped", lf["softcap"]), ("attention, causal (Qwen2's)", 0.0)):
            timed(name, case, lambda: ops.attention(q, k_cache, v_cache, table, b.cu_q, kv_len, 0, lf["scale"], Ha, Ga, D,
                                                    max(lens), held, single, softcap=cap), nbytes, flop=4.0 * keys * Ha * D)
        o2 = torch.randn(T, Ha * D, device=dev).to(bf)
        gate = aq[:, (Ha + Ga) * da + Ga * dva:]
        timed("entry_gate (with the output bias)", case,
              lambda: ops.entry_gate(o2, gate, Ha, dva, D, 1.0, resid=resid, bias=wv), T * Ha * D * 8 + T * W * 8)
        timed("head_gate (Salolorn's)", case, lambda: ops.head_gate(o2, gate[:, :Ha], Ha, D, 1.0), T * Ha * D * 4)
        # ---- the router with a correction and identity experts, beside Qwen2-MoE's
        E, ident, top = mlp["router"]["experts"], mlp["router"]["identity"], mlp["router"]["top"]
        x32 = torch.randn(T, W, device=dev)
        w_r = (torch.randn(E + ident, W, device=dev) * 0.05).to(bf)
        corr = torch.randn(E + ident, device=dev) * 0.1
        timed("route (softmax, choice on score + correction, 16 + 2 experts)", case,
              lambda: ops.route(x32, w_r, E + ident, top, 2, False, select_bias=corr, scale=0.8), T * W * 4 + (E + ident) * W * 2)
        w_q = (torch.randn(E + 1, W, device=dev) * 0.05).to(bf)
        timed("route (Qwen2-MoE's, norm inside, shared gate)", case,
              lambda: ops.route(x32, w_q, E, top, True, True, norm_weight=wv, eps=1e-6), T * W * 4 + (E + 1) * W * 2)
        ids, wts, _, offsets, rws, dest = ops.route(x32, w_r, E + ident, top, 2, False, select_bias=corr, scale=0.8)
        y = torch.randn(T * top, W, device=dev)
        shared = torch.randn(T, W, device=dev)
        timed("moe_combine (identity experts, shared expert with a factor)", case,
              lambda: ops.moe_combine(y, dest, wts, shared, None, resid, ids=ids, num_real=E, passthrough=x32, shared_scale=0.8),
              T * W * 4 * (top + 3))
        gq = torch.rand(T, device=dev)
        timed("moe_combine (Qwen2-MoE's)", case, lambda: ops.moe_combine(y, dest, wts, shared, gq, resid), T * W * 4 * (top + 3))
        # ---- the cap on the logits
        N = 1 if case == "prefill" else R
        logits = torch.randn(N, z["vocab"], device=dev) * 10
        timed("tanh_cap (logits)", case, lambda: ops.tanh_cap(logits, z["logit_softcap"]), N * z["vocab"] * 8)
    ops.check_errors()
    return rows


def run_faguzen(args, pk) -> dict:
    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    out = {"workload": "faguzen", "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)",
           "peaks": pk, "sizes": {}, "l2": "a buffer larger than L2 is written before every timed step"}
    for width in (1024, 2048, 4096):
        z = faguzen_config(width)
        q = qwen_config_like_faguzen(z)
        out["sizes"][str(width)] = {
            "layer_runs": q["num_hidden_layers"], "faguzen": measure_engine(z, args.batch, args.prompt_len, args.steps, 2048),
            "qwen2_moe": measure_engine(q, args.batch, args.prompt_len, args.steps, 2048)}
    out["kernels_width_2048"] = faguzen_kernels(faguzen_config(2048), pk, args.batch, args.prompt_len, 2048)
    t1 = time.time()
    time.sleep(0.2)
    sampler.stop()
    out["clocks"] = sampler.summary(t0, t1)
    return out


def layers_that_fit(raw, want, reserve_gb=40.0):
    """As many layers of `raw` (at most `want`) as the free device memory holds beside `reserve_gb` for
    the cache pool, the head, graphs and activations."""
    import torch
    H, I, Is, E = raw["hidden_size"], raw["moe_intermediate_size"], raw["shared_expert_intermediate_size"], raw["num_experts"]
    Q = raw["num_attention_heads"] * raw["head_dim"]
    KV = raw["num_key_value_heads"] * raw["head_dim"]
    per_layer = 2 * ((Q + 2 * KV) * H + H * Q + (E + 1) * H + E * 3 * I * H + 3 * Is * H)
    free, _ = torch.cuda.mem_get_info(0)
    fit = int((free - reserve_gb * 1e9) // per_layer)
    return max(1, min(want, fit))


def measure_57b(args, pk) -> dict:
    """The layer sizes of Qwen2-57B-A14B: decode at batch 1 / 8 / 64 (context 2,048) and a 2,048-token
    prefill, each with its fraction of the measured peak."""
    raw = dict(MODEL_A)
    raw.update(SIZES_57B)
    raw["max_position_embeddings"] = 4096
    full = SIZES_57B["num_hidden_layers"]
    layers = layers_that_fit(raw, full if args.layers_57b is None else args.layers_57b)
    m = Measurement(raw, layers, 2048, 4096, 64, pk)
    out = {"model": "Qwen2-57B-A14B sizes", "layers": layers, "layers_full": full, "prompt_len": 2048,
           "load_s": round(m.load_s, 1)}
    for b in (8, 1, 64):
        r = m.decode(b, max(4, args.steps // 4), 3, sample_clocks=(b == 8))
        out[f"decode_b{b}"] = round(r["tok_s"], 2)
        out[f"decode_b{b}_ms"] = round(r["ms"], 4)
        out[f"decode_b{b}_frac"] = round(r["frac"], 4)
        out[f"decode_b{b}_experts"] = r["distinct"]
        if b == 8:
            out["clocks"] = r["clocks"]
    out["prefill"] = m.prefill(2048, repeats=3)
    m.eng.rt.ops.check_errors()
    m.close()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--page-size", type=int, default=64, help="tokens per page of the cache (16, 32, 64, 128, ...)")
    ap.add_argument("--serving-prompts", type=int, nargs=2, default=[256, 16384], metavar=("MIN", "MAX"),
                    help="prompt lengths of the serving workload (uniform in MIN..MAX)")
    ap.add_argument("--serving-requests", type=int, default=64, help="requests of the serving workload")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (reported)")
    ap.add_argument("--layers-57b", type=int, default=None, help="layers of the larger model in `sizes_57b` (default: all "
                    "28 if they fit)")
    ap.add_argument("--sizes", default="a2.7b", choices=["a2.7b", "57b"],
                    help="57b: the layer sizes of Qwen2-57B-A14B as the headline (no extras)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    ap.add_argument("--no-extras", action="store_true", help="skip `sizes_57b` and `serving`")
    ap.add_argument("--only-prefill", action="store_true", help="measure the 2,048-token prefill alone (for profiles)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving", "sweep", "kernels", "zesapel", "zasazen", "salolorn", "faguzen"],
                    help="serving: the continuous-batching workload on the windowed model, instead of the default line; "
                         "sweep: decode at contexts of 1k to 32k and prefill of longer prompts, a line of its own; "
                         "kernels: the weight-streaming product alone")
    args = ap.parse_args()
    global FULL_LAYERS, MODEL_NAME
    if args.sizes == "57b":
        MODEL.update(SIZES_57B)
        FULL_LAYERS, MODEL_NAME = SIZES_57B["num_hidden_layers"], "Qwen2-57B-A14B"
        args.no_extras = True
    if args.impl == "reference":
        return run_reference()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload == "serving":
        if args.layers is None:
            args.layers = MODEL_A["num_hidden_layers"]
        line = run_serving(args)
        print(json.dumps(line))
        return 0 if line["complete"] else 1
    if args.layers is None:
        args.layers = FULL_LAYERS
    args.warmup = max(args.warmup, 3)
    pk = peaks()
    if args.workload == "sweep":
        print(json.dumps(run_sweep(args, pk)))
        return 0
    if args.workload == "kernels":
        print(json.dumps(run_kernels(pk)))
        return 0
    if args.workload == "zesapel":
        print(json.dumps(run_zesapel(args, pk)))
        return 0
    if args.workload == "zasazen":
        print(json.dumps(run_zasazen(args, pk)))
        return 0
    if args.workload == "salolorn":
        print(json.dumps(run_salolorn(args, pk)))
        return 0
    if args.workload == "faguzen":
        print(json.dumps(run_faguzen(args, pk)))
        return 0
    max_batch = 64 if not args.no_points else args.batch
    m = Measurement(MODEL, args.layers, args.prompt_len, args.context, max_batch, pk, page=args.page_size)
    cfg = m.cfg
    if args.only_prefill:
        pre = m.prefill(2048, repeats=3)
        print(json.dumps({"prefill_ms": pre["all_ms"], "tokens": 2048, "layers": args.layers}))
        return 0
    main_run = m.decode(args.batch, args.steps, args.warmup, sample_clocks=True)
    out = {
        "metric": "decode tok/s @ batch %d (%s sizes, bf16, random weights)" % (args.batch, MODEL_NAME),
        "value": round(main_run["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)", "impl": "ours",
        "config": {
            "model": MODEL_NAME + " sizes", "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "1 GPU", "prompt_len": args.prompt_len, "layers": args.layers, "layers_full": FULL_LAYERS,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "experts": cfg.num_experts, "top_k": cfg.num_experts_per_tok,
            "moe_inter": cfg.moe_intermediate_size, "shared_inter": cfg.shared_expert_intermediate_size,
            "vocab": cfg.vocab_size, "page_size": m.page,
            "l2": "inputs larger than L2: a step reads %.1f GB" % (main_run["step_bytes"] / 1e9),
            "timed": "K replays of the captured decode step (CUDA graph), CUDA events",
            "peaks": pk["source"]},
        "e2e": {"value": round(main_run["e2e_tok_s"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": int(main_run["launches"]),
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(main_run["achieved"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_run["frac"], 4), "experts_with_rows": main_run["distinct"]},
        "load_s": round(m.load_s, 1),
    }
    if not args.no_points:
        pts, fracs, e2e = {}, {f"decode_b{args.batch}": round(main_run["frac"], 4)}, {}
        for b in (1, 64):
            r = m.decode(b, max(8, args.steps // 2), 3)
            pts[f"decode_b{b}"] = round(r["tok_s"], 2)
            fracs[f"decode_b{b}"] = round(r["frac"], 4)
            e2e[f"decode_b{b}"] = round(r["e2e_tok_s"], 2)
        out["points"] = pts
        out["points_frac"] = fracs          # of the HBM peak, bytes from the experts each step really used
        out["points_e2e"] = e2e             # the same points through run_step, host tokens in and out
        out["e2e_sampled"] = {"value": round(m.decode_sampled(args.batch, args.steps), 2), "unit": "tokens/s",
                              "temperature": 0.8, "batch": args.batch}
        out["prefill"] = m.prefill(2048, repeats=4)
        out["prefill"].pop("all_ms")
    m.eng.rt.ops.check_errors()
    m.close()
    if not args.no_extras and not args.no_points:
        sv_args = argparse.Namespace(layers=MODEL_A["num_hidden_layers"], serving_prompts=args.serving_prompts,
                                     serving_requests=args.serving_requests)
        sv = run_serving(sv_args)
        out["serving"] = {"generated_tok_s": sv["value"], "prompt_tok_s": sv["prompt_tok_s"], "seconds": sv["seconds"],
                          "steps": sv["steps"], "mean_step_ms": round(1e3 * sv["seconds"] / max(sv["steps"], 1), 3),
                          "requests": sv["config"]["requests"], "layers": sv["config"]["layers"],
                          "prompt_tokens": sv["prompt_tokens"], "generated_tokens": sv["generated_tokens"],
                          "preemptions": sv["scheduler"]["preemptions"],
                          "high_water_pages": [p["high_water"] for p in sv["pages"]],
                          "pool_pages": [p["total"] for p in sv["pages"]], "complete": sv["complete"],
                          "host": sv["host"], "step_kinds": sv["step_kinds"],
                          "clocks": sv["clocks"]}
        import gc

        import torch
        gc.collect()
        torch.cuda.empty_cache()
        out["sizes_57b"] = measure_57b(args, pk)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
