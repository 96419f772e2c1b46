#!/usr/bin/env python3
"""Decode and prefill throughput of the Gemma 2 engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--size 2b|9b|27b] [--layers L] [--batch B] [--context C] [--only-headline]
    python bench.py --micro attention|prompt-attention|gemm|products|reference
                    (kernels alone, JSON lines; for the summaries in profiles/)

A "step" is one decode step: every live request gets one token.  Default: the layer sizes of Gemma 2 2B, random
bfloat16 weights, 8 requests at a context of 8192 tokens.  `value` is decoded tokens per second timed with CUDA events
around K steps of the step function (the mean of `reps` such runs, `sd` beside it); `e2e` is the same through the
Python entry point (`Engine.step()`: host scheduling, the step's integers copied from pinned host memory, tokens drawn
on the device and read back).  `prefill` is one step of 2,048 prompt tokens; `roofline` is the bytes a decode step must
read (every weight once, the cache of the live requests) over its time; `points` holds decode at batch 1 and 64.
Beyond the headline the line carries: `mixed` (a step of 8 decode rows beside a 512-token prompt portion at context
8192, and that portion alone: GPU time by events and wall time through `Engine.step()`), `fp32` (the true 32-bit path at
the same sizes) and `sizes` (the same figures at Gemma 2 9B and 27B layer sizes; where 64 requests of 8192 tokens do not
fit beside the weights the context of that point is named).
Method after the reference's `kungfu bench` (crates/kungfu/src/main.rs:544-608): synthetic token ids, every shape run
before timing, mean and standard deviation over repetitions.  Caches are filled with random keys and values instead of
running the long prompts.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SIZES = {
    # the layer sizes of Gemma 2 2B, 9B and 27B
    "2b": dict(num_hidden_layers=26, hidden_size=2304, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
               intermediate_size=9216, query_pre_attn_scalar=256),
    "9b": dict(num_hidden_layers=42, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8, head_dim=256,
               intermediate_size=14336, query_pre_attn_scalar=256),
    "27b": dict(num_hidden_layers=46, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                intermediate_size=36864, query_pre_attn_scalar=144),
}
COMMON = dict(architectures=["Gemma2ForCausalLM"], vocab_size=256000, rope_theta=10000.0, sliding_window=4096,
              attn_logit_softcapping=50.0, final_logit_softcapping=30.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=8192 + 512, hidden_activation="gelu_pytorch_tanh")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            raw = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(raw.get(k), (int, float)):
                out[k] = float(raw[k])
        return out, "measured"
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().split("\n"):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, n_layers: int):
    """Weight bytes a decode step reads (bf16) and matrix parameters per token for the flop count."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.q_size + 2 * cfg.kv_size) * H + H * cfg.q_size + 3 * H * I
    norms = 4 * H * n_layers + H
    weight_bytes = 2 * (per_layer * n_layers + V * H + norms)
    return per_layer, weight_bytes


def kv_bytes_read(cfg, n_layers: int, length: int) -> int:
    """Bytes of keys and values one decode step reads for one request at `length` tokens (bf16)."""
    n = 0
    for l in range(n_layers):
        w = cfg.window_of(l)
        n += 2 * cfg.kv_size * 2 * (min(length, w) if w else length)
    return n


def prefill_flops(cfg, n_layers: int, T: int) -> float:
    per_layer, _ = model_numbers(cfg, n_layers)
    gemm = 2.0 * T * per_layer * n_layers + 2.0 * cfg.vocab_size * cfg.hidden_size
    attn = 0.0
    for l in range(n_layers):
        w = cfg.window_of(l)
        pairs = sum(min(p + 1, w) if w else p + 1 for p in range(T))
        attn += 4.0 * cfg.num_attention_heads * cfg.head_dim * pairs
    return gemm + attn


def fill_cache(runner, rid, n_tokens: int) -> None:
    """Make request `rid` hold `n_tokens` tokens (of whatever the pages contain) without running them; in portions, so
    that a windowed group gives pages back as it would while a prompt is fed."""
    runner.cache.add_request(rid)
    at = 0
    while at < n_tokens:
        n = min(512, n_tokens - at)
        runner.cache.reserve(rid, n)
        runner.cache.commit(rid, n)
        at += n


def randomize_pages(runner, torch) -> None:
    g = torch.Generator(device=runner.device)
    g.manual_seed(1)
    for s, t in runner.cache.storage.items():
        if t.dim() == 5:
            flat = t.view(-1)
            step = 1 << 28
            for i in range(0, flat.numel(), step):
                flat[i:i + step].normal_(0.0, 0.5, generator=g)


def mean_sd(xs) -> tuple[float, float]:
    xs = list(xs)
    return statistics.fmean(xs), (statistics.stdev(xs) if len(xs) > 1 else 0.0)


def time_decode(torch, runner, rids, steps: int, warmup: int, vocab: int, reps: int):
    """`reps` timed runs of `steps` decode steps each (CUDA events around each run, a synchronize on both sides), after
    `warmup` steps.  Returns the ms per step of every run and the kernels launched in the last one."""
    from kungfu_b200 import ops
    from kungfu_b200.engine import StepEntry
    tok = 17
    i = 0

    def one():
        nonlocal i
        entries = [StepEntry(r, [(tok + 31 * i + 7 * k) % vocab], [0]) for k, r in enumerate(rids)]
        i += 1
        return runner.step(entries)

    for _ in range(warmup):
        one()
    out, launches = [], 0
    for _ in range(reps):
        torch.cuda.synchronize()
        l0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / steps)
        launches = ops.launch_count() - l0
    return out, launches


def build(torch, size: str, n_layers: int, dtype: str, *, parallel: int, ctx_len: int, margin: int):
    """Model with random weights, and a runner whose pools hold `parallel` requests of `ctx_len` tokens or what fits."""
    from kungfu_b200 import api
    raw = dict(COMMON, **SIZES[size])
    raw["num_hidden_layers"] = n_layers
    device = torch.device("cuda:0")
    cfg, model = api.random_model(raw, seed=0, dtype=dtype, device=device)
    free, total = torch.cuda.mem_get_info(device)
    budget = int(free) - max(6 << 30, int(total) // 16)
    runner = api.make_runner(cfg, model, dtype=dtype, device=device, page_size=api.DEFAULT_PAGE_SIZE,
                             max_requests=parallel, max_context=ctx_len + margin, batch=512, budget_bytes=budget)
    randomize_pages(runner, torch)
    return cfg, model, runner


def context_that_fits(runner, batch: int, ctx_len: int) -> int:
    """The longest context (a multiple of 1,024, at most `ctx_len`) at which `batch` requests fit the pools."""
    page = runner.cache.page_size
    c = ctx_len
    while c > 1024:
        ok = True
        for g in runner.cache.groups:
            per = c + 64 if g.window is None else min(c + 64, g.window + 512 + page)
            ok = ok and batch * -(-per // page) <= g.pool.n_pages
        if ok:
            return c
        c -= 1024
    return c


def measure_size(torch, args, size: str, dtype: str, pk: dict, *, headline: bool) -> dict:
    """Decode at batch 8 / 1 / 64 and a 2,048-token prompt at one model size and precision."""
    from kungfu_b200 import ops
    from kungfu_b200.engine import StepEntry
    full_layers = SIZES[size]["num_hidden_layers"]
    n_layers = args.layers if (headline and args.layers) else full_layers
    ctx_len = args.context
    reps = args.reps
    steps = args.steps if headline else min(args.steps, 32 if dtype == "bfloat16" else 8)
    warmup = args.warmup
    margin = (reps * steps + warmup) + 128
    batches = [args.batch] if (args.only_headline or dtype != "bfloat16") else sorted({args.batch, 1, 64})
    cfg, model, runner = build(torch, size, n_layers, dtype, parallel=max(batches) + 2, ctx_len=ctx_len, margin=margin)
    vocab = cfg.vocab_size
    elt = 2 if dtype == "bfloat16" else 4
    per_layer, weight_bytes = model_numbers(cfg, n_layers)
    weight_bytes = weight_bytes * elt // 2
    out = {"layers": n_layers, "layers_full": full_layers, "pool_pages": [g.pool.n_pages for g in runner.cache.groups]}

    # ---- a prompt of 2,048 tokens in one step ---------------------------------------------------------------------------
    T = args.prefill_tokens
    toks = [(i * 7919 + 13) % vocab for i in range(T)]
    pf_ms = []
    for rep in range(reps + 1):
        runner.cache.add_request("pf")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("pf", toks, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        pf_ms.append(e0.elapsed_time(e1))
        runner.cache.release("pf")
    m, sd = mean_sd(pf_ms[1:])
    flops = prefill_flops(cfg, n_layers, T)
    peak_flops = pk["bf16_tflops"] * 1e12
    out["prefill"] = {"value": round(T / m * 1e3, 1), "tokens": T, "ms": round(m, 3), "sd_ms": round(sd, 3),
                      "frac": round(flops / (m * 1e-3) / peak_flops, 4) if dtype == "bfloat16" else None}

    # ---- decode ------------------------------------------------------------------------------------------------------------
    out["decode"] = {}
    for b in batches:
        c_len = context_that_fits(runner, b, ctx_len)
        rids = [f"d{b}_{k}" for k in range(b)]
        for r in rids:
            fill_cache(runner, r, c_len - warmup)
        clocks = None
        sampler = ClockSampler()
        if headline and b == args.batch:
            sampler.start()
            time.sleep(0.3)
        ms_runs, launches = time_decode(torch, runner, rids, steps, warmup, vocab, reps)
        if headline and b == args.batch:
            clocks = sampler.stop()
        for r in rids:
            runner.cache.release(r)
        m, sd = mean_sd(ms_runs)
        tps = [b / x * 1e3 for x in ms_runs]
        bytes_step = weight_bytes + b * kv_bytes_read(cfg, n_layers, c_len) * elt // 2
        achieved = bytes_step / (m * 1e-3) / 1e9
        out["decode"][f"b{b}"] = {"value": round(mean_sd(tps)[0], 1), "sd": round(mean_sd(tps)[1], 1), "ms_per_step": round(m, 4),
                                  "sd_ms": round(sd, 4), "context": c_len, "hbm_gbs": round(achieved, 1),
                                  "frac": round(achieved / pk["hbm_gbs"], 4), "launches": int(launches), "clocks": clocks}
    out["_live"] = (cfg, model, runner)
    return out


def measure_mixed(torch, args, cfg, runner) -> dict:
    """A step of `batch` decode rows beside one 512-token prompt portion at the headline context, and that portion
    alone: GPU time by CUDA events around `Runner.step` (tokens drawn on the device) and wall time of `Engine.step()`
    (planning, the step's integers, the launch or graph replay, the tokens read back)."""
    import numpy as np
    from kungfu_b200.engine import StepEntry
    from kungfu_b200.engine.engine import Engine
    from kungfu_b200.engine.scheduler import Request
    from kungfu_b200.sampling import STATE_WORDS, Sampling, pack_state
    B, ctx_len, vocab = args.batch, args.context, cfg.vocab_size
    out = {}
    states = torch.zeros((runner.cache.max_requests, STATE_WORDS), dtype=torch.int32, device=runner.device)
    states[:] = torch.from_numpy(pack_state(Sampling(temperature=0.0), 1)).to(runner.device)
    # the scheduler's budget counts decode rows, so with a budget of 512 a mixed step has 512 rows in all (the second case:
    # two whole 256-token tiles); the first case is 520 rows, a third tile for eight of them
    for name, n_dec, portion in ((f"decode{B}_portion512", B, 512), (f"decode{B}_portion{512 - B}", B, 512 - B), ("portion512", 0, 512)):
        rids = [f"m{k}" for k in range(n_dec)]
        for r in rids:
            fill_cache(runner, r, ctx_len - 16)
        gpu_ms = []
        for rep in range(args.reps + 2):                       # the first runs eagerly, the second is captured
            fill_cache(runner, "mp", ctx_len - portion)
            entries = [StepEntry(r, [(5 + 3 * rep + k) % vocab], [0]) for k, r in enumerate(rids)]
            entries.append(StepEntry("mp", [(i * 31 + rep) % vocab for i in range(portion)], [portion - 1]))
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step(entries, sample=(states, False))
            e1.record()
            torch.cuda.synchronize()
            gpu_ms.append(e0.elapsed_time(e1))
            runner.cache.release("mp")
        for r in rids:
            runner.cache.release(r)
        # the same step through the engine: requests adopted at their long context, one Engine.step() each repetition
        eng = Engine(runner=runner, batch=portion + n_dec, parallel=n_dec + 1, pipeline=False)
        eng.cfg = cfg
        for k in range(n_dec):
            rid = f"e{k}"
            req = Request(rid, [(k * 131 + i) % vocab for i in range(ctx_len - 16)], Sampling(temperature=0.0), max_tokens=10 ** 9,
                          eos=(), ignore_eos=True)
            fill_cache(runner, rid, ctx_len - 17)
            req.n_cached = ctx_len - 17
            eng.requests[rid] = req
            eng.scheduler.adopt(req)
        if n_dec:
            eng.step()                                         # every decoding request has produced a token
        wall_ms = []
        for rep in range(args.reps + 2):
            rid = f"p{rep}"
            req = Request(rid, [(rep + i * 7) % vocab for i in range(ctx_len)], Sampling(temperature=0.0), max_tokens=1, eos=(),
                          ignore_eos=True)
            fill_cache(runner, rid, ctx_len - portion)
            req.n_cached = ctx_len - portion
            eng.requests[rid] = req
            eng.scheduler.adopt(req)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ev = eng.step()
            torch.cuda.synchronize()
            wall_ms.append((time.perf_counter() - t0) * 1e3)
            assert any(r == rid and reason == "length" for r, _t, reason in ev), ev
        for k in range(n_dec):
            eng.cancel(f"e{k}")
        g, gs = mean_sd(gpu_ms[2:])
        w, ws = mean_sd(wall_ms[2:])
        out[name] = {"gpu_ms": round(g, 3), "gpu_sd_ms": round(gs, 3), "engine_wall_ms": round(w, 3), "engine_wall_sd_ms": round(ws, 3),
                     "eager_first_ms": round(gpu_ms[0], 3), "rows": n_dec + portion, "context": ctx_len}
    return out


def measure_e2e(torch, args, cfg, runner) -> dict:
    """Decode through the Python entry point: `Engine.step()` with host token ids in and out."""
    from kungfu_b200.engine.engine import Engine
    from kungfu_b200.engine.scheduler import Request
    from kungfu_b200.sampling import Sampling
    B, ctx_len, vocab = args.batch, args.context, cfg.vocab_size
    eng = Engine(runner=runner, batch=max(512, B), parallel=B)
    eng.cfg = cfg
    start = ctx_len - args.warmup
    for k in range(B):
        rid = f"e{k}"
        prompt = [(k * 131 + i * 7919 + 13) % vocab for i in range(start)]
        req = Request(rid, prompt, Sampling(temperature=0.0), max_tokens=10 ** 9, eos=(), ignore_eos=True)
        fill_cache(runner, rid, start - 1)               # all but the last prompt token are "already run"
        req.n_cached = start - 1
        eng.requests[rid] = req
        eng.scheduler.adopt(req)
    for _ in range(args.warmup):
        eng.step()
    rates, per_step = [], []
    for _ in range(args.reps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(args.steps):
            n_tok += sum(1 for _id, tok, _r in eng.step() if tok is not None)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        rates.append(n_tok / dt)
        per_step.append(dt / args.steps * 1e3)
    meta_ints = runner.last_meta_ints
    for k in range(B):
        eng.cancel(f"e{k}")
    return {"value": round(mean_sd(rates)[0], 1), "sd": round(mean_sd(rates)[1], 1), "unit": "tokens/s",
            "h2d_bytes_per_step": int(meta_ints * 4), "d2h_bytes_per_step": int(B * 4),
            "ms_per_step": round(mean_sd(per_step)[0], 3),
            "reads": "ids of step n read on the host while step n+1 runs" if eng.pipeline else "every step before the next"}


def run_ours(args) -> dict:
    import torch
    from kungfu_b200 import api, ops

    pk, pk_src = peaks()
    api.require_cuda("cuda:0")
    ops.library()
    head = measure_size(torch, args, args.size, "bfloat16", pk, headline=True)
    cfg, model, runner = head.pop("_live")
    B, ctx_len = args.batch, args.context
    hd = head["decode"][f"b{B}"]
    e2e = measure_e2e(torch, args, cfg, runner)
    mixed = None if args.only_headline else measure_mixed(torch, args, cfg, runner)
    n_layers, full_layers = head["layers"], head["layers_full"]
    config = {"model": f"gemma2-{args.size}", "layers": n_layers, "layers_full": full_layers,
              "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
              "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
              "sliding_window": cfg.sliding_window, "global_batch": B, "seq_len": ctx_len, "page_size": runner.cache.page_size,
              "parallelism": "single", "weights": "random bf16", "cache": "bf16 random fill", "l2": "inputs larger than L2",
              "cuda_graphs": bool(getattr(runner, "cuda_graphs", False)), "reps": args.reps}
    del model, runner
    gc.collect()
    torch.cuda.empty_cache()

    fp32, sizes = None, {}
    if not args.only_headline:
        r = measure_size(torch, args, args.size, "float32", pk, headline=False)
        r.pop("_live")
        gc.collect()
        torch.cuda.empty_cache()
        fp32 = {"decode": r["decode"], "prefill": r["prefill"], "layers": r["layers"]}
        for other in [s for s in ("9b", "27b") if s != args.size]:
            r = measure_size(torch, args, other, "bfloat16", pk, headline=False)
            r.pop("_live")
            gc.collect()
            torch.cuda.empty_cache()
            sizes[other] = r
    points = {k: v["value"] for k, v in head["decode"].items() if k != f"b{B}"}
    return {"metric": "decode tokens/s (batch 8, context 8192, Gemma 2 2B sizes, 1 B200)" if (args.size, B, ctx_len) == ("2b", 8, 8192)
            else f"decode tokens/s (batch {B}, context {ctx_len}, Gemma 2 {args.size} sizes, 1 B200)",
            "value": hd["value"], "sd": hd["sd"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": hd["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic token ids, random-init weights, random-filled cache",
            "config": config, "clocks": hd["clocks"], "e2e": e2e, "gpu_launches": hd["launches"], "prefill": head["prefill"],
            "roofline": {"bound": "hbm", "achieved": hd["hbm_gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": hd["frac"],
                         "peaks": pk_src},
            "points": {f"decode_{k}": v for k, v in points.items()},
            "decode": {k: {kk: vv for kk, vv in v.items() if kk != "clocks"} for k, v in head["decode"].items()},
            "mixed": mixed, "fp32": fp32, "sizes": sizes, "slow_kernel_fallbacks": ops.fallbacks(), "impl": "ours"}


def micro_attention() -> int:
    """Decode attention alone: eight launches over distinct pages replayed from a CUDA graph, per batch size; one JSON
    line each with microseconds per launch and bytes of keys and values over that time."""
    import torch
    from kungfu_b200 import api, ops

    class View:
        def __init__(self, pages, page_size):
            self.pages, self.page_size, self.group, self.writes = pages, page_size, 0, False

    class Ctx:
        pass

    device = api.require_cuda("cuda:0")
    ops.library()
    nh, nkv, d, page, ctx_len, launches = 8, 4, 256, 64, 8192, 8
    for batch in (1, 2, 4, 8, 16, 64):
        per_req = ctx_len // page
        pages = torch.randn(launches * batch * per_req + 1, 2, nkv, page, d, device=device, dtype=torch.bfloat16)
        ctxs = []
        for l in range(launches):
            c = Ctx()
            c.positions = torch.full((batch,), ctx_len - 1, dtype=torch.int32, device=device)
            c.row_req = torch.arange(batch, dtype=torch.int32, device=device)
            c.block_tables = [(torch.arange(batch * per_req, dtype=torch.int32, device=device) + l * batch * per_req)
                              .view(batch, per_req).contiguous()]
            c.n_rows = c.n_dec_rows = batch
            c.n_pre_rows = c.n_tiles = c.n_wide = 0
            c.dec_rows = c.pre_rows = None
            c.max_kv_len = ctx_len
            ctxs.append(c)
        q = torch.randn(batch, nh * d, device=device, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        view = View(pages, page)
        for window in (None, 4096):
            def run():
                for c in ctxs:
                    ops.paged_attention(q, out, c, view, nh, nkv, d, 1.0 / 16.0, 50.0, window)
            run()
            torch.cuda.synchronize()
            graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
            with torch.cuda.stream(side):
                run()
                with torch.cuda.graph(graph, stream=side):
                    run()
            torch.cuda.synchronize()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 10 / launches * 1e3
            n_bytes = batch * min(ctx_len, window or ctx_len) * nkv * d * 2 * 2
            print(json.dumps({"micro": "decode attention", "batch": batch, "keys": min(ctx_len, window or ctx_len),
                              "us_per_launch": round(us, 1), "gb_per_s": round(n_bytes / us / 1e3, 1)}))
        del pages
    return 0


def micro_prompt_attention() -> int:
    """Prompt attention alone (8 heads / 4 kv heads of 256, softcap 50, page 64): whole prompts of 512 to 4,096 rows and a
    512-row portion at context 8,192, each replayed from a CUDA graph of three launches over distinct pages; one JSON line
    each with microseconds per launch and TFLOP/s."""
    import math
    import torch
    from kungfu_b200 import api, ops

    class View:
        def __init__(self, pages, page_size):
            self.pages, self.page_size, self.group, self.writes = pages, page_size, 0, False

    class Ctx:
        pass

    device = api.require_cuda("cuda:0")
    ops.library()
    gen = torch.Generator(device=device)
    gen.manual_seed(0)
    nh, nkv, d, page, copies = 8, 4, 256, 64, 3
    scale = 1.0 / math.sqrt(d)
    for T, past in ((512, 0), (1024, 0), (2048, 0), (4096, 0), (512, 7680)):
        total = T + past
        per_req = total // page
        pages = torch.empty(copies * per_req, 2, nkv, page, d, device=device, dtype=torch.bfloat16).normal_(0.0, 0.5, generator=gen)
        ctxs = []
        for k in range(copies):
            c = Ctx()
            c.positions = torch.arange(past, total, dtype=torch.int32, device=device)
            c.row_req = torch.zeros(T, dtype=torch.int32, device=device)
            c.block_tables = [(torch.arange(per_req, dtype=torch.int32, device=device) + k * per_req).view(1, per_req).contiguous()]
            c.n_rows = c.n_pre_rows = T
            c.n_dec_rows = 0
            c.dec_rows = None
            c.pre_rows = torch.arange(T, dtype=torch.int32, device=device)
            c.n_tiles, c.n_wide = T // 64, T // 128
            c.tile_row0 = torch.arange(0, T, 64, dtype=torch.int32, device=device)
            c.tile_nrows = torch.full((T // 64,), 64, dtype=torch.int32, device=device)
            c.wide_row0 = torch.arange(0, T, 128, dtype=torch.int32, device=device)
            c.wide_nrows = torch.full((T // 128,), 128, dtype=torch.int32, device=device)
            c.max_kv_len = total
            ctxs.append(c)
        q = torch.randn(T, nh * d, device=device, generator=gen).to(torch.bfloat16)
        out = torch.empty_like(q)
        view = View(pages, page)
        us = _graph_us(torch, lambda: [ops.paged_attention(q, out, c, view, nh, nkv, d, scale, 50.0, None) for c in ctxs], copies)
        flops = 4.0 * nh * d * (T * (T + 1) / 2 + T * past)
        print(json.dumps({"micro": "prompt attention", "rows": T, "keys_before": past, "us_per_launch": round(us, 1),
                          "tflops": round(flops / us / 1e6, 1)}), flush=True)
        del pages
    ops.raise_on_device_error()
    return 0


def micro_gemm() -> int:
    """One square bfloat16 product (8192 cubed) on the tensor-core kernel, timed with CUDA events; one JSON line."""
    import torch
    from kungfu_b200 import api, ops
    device = api.require_cuda("cuda:0")
    n = 8192
    x = torch.randn(n, n, device=device).bfloat16()
    w = torch.randn(n, n, device=device).bfloat16()
    out = torch.empty(n, n, device=device)
    for _ in range(3):
        ops.linear(x, w, out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        ops.linear(x, w, out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 5
    ops.raise_on_device_error()
    print(json.dumps({"micro": "product 8192^3 bf16", "ms": round(ms, 4), "tflops": round(2.0 * n ** 3 / ms / 1e9, 1)}))
    return 0


def micro_products(size: str = "2b") -> int:
    """The four products of a Gemma 2 layer (`--size`) over 8 to 2,048 rows, each replayed from a CUDA graph of six
    launches over distinct weights; one JSON line per (rows, product) with microseconds per launch."""
    import torch
    from kungfu_b200 import api, ops
    device = api.require_cuda("cuda:0")
    ops.library()
    sz = SIZES[size]
    H, inner, n_w = sz["hidden_size"], sz["intermediate_size"], 6
    Q = sz["num_attention_heads"] * sz["head_dim"]
    qkv = Q + 2 * sz["num_key_value_heads"] * sz["head_dim"]
    gen = torch.Generator(device=device)
    gen.manual_seed(0)
    shapes = {"q,k,v": (qkv, H, False), "o": (H, Q, False), "gate+up": (inner, H, True), "down": (H, inner, False)}
    for rows in (8, 64, 128, 256, 384, 512, 768, 1024, 2048):
        for name, (n_out, k, gated) in shapes.items():
            ws = [(torch.randn(2 * n_out if gated else n_out, k, device=device, generator=gen) * 0.02).to(torch.bfloat16)
                  for _ in range(n_w)]
            x = torch.randn(rows, k, device=device).to(torch.bfloat16)
            out = torch.empty(rows, n_out, device=device, dtype=torch.bfloat16 if gated else torch.float32)

            def run():
                for w in ws:
                    if gated:
                        ops.linear_gated(x, w, out, "gelu_tanh", None)
                    else:
                        ops.linear(x, w, out)
            run()
            torch.cuda.synchronize()
            graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
            with torch.cuda.stream(side):
                run()
                with torch.cuda.graph(graph, stream=side):
                    run()
            torch.cuda.synchronize()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 10 / n_w * 1e3
            flops = 2.0 * rows * n_out * k * (2 if gated else 1)
            print(json.dumps({"micro": "product", "size": size, "rows": rows, "product": name, "us": round(us, 1),
                              "tflops": round(flops / us / 1e6, 1)}))
            del ws
    ops.raise_on_device_error()
    return 0


def micro_qkv_rope(size: str = "2b") -> int:
    """The q,k,v product of a prompt with rotation and cache append: the product that files its own result
    (`ops.linear_rope_kv_append`) beside the product that leaves 32-bit rows plus the kernel that rotates and files them;
    four launches over distinct weights and pages replayed from a CUDA graph, one JSON line per row count."""
    import torch
    from kungfu_b200 import api, ops
    device = api.require_cuda("cuda:0")
    ops.library()
    sz = SIZES[size]
    nh, nkv, d, K, P, n_w = sz["num_attention_heads"], sz["num_key_value_heads"], sz["head_dim"], sz["hidden_size"], 64, 4
    N = (nh + 2 * nkv) * d

    class View:
        def __init__(self, pages):
            self.pages, self.page_size, self.group, self.writes = pages, P, 0, True

    class Ctx:
        pass
    for rows in (768, 1024, 2048, 4096):
        ws = [(torch.randn(N, K, device=device) * 0.02).to(torch.bfloat16) for _ in range(n_w)]
        x = torch.randn(rows, K, device=device).to(torch.bfloat16)
        n_pages = -(-rows // P)
        ctx = Ctx()
        ctx.positions = torch.arange(rows, dtype=torch.int32, device=device)
        ctx.row_req = torch.zeros(rows, dtype=torch.int32, device=device)
        ctx.block_tables = [torch.arange(n_pages, dtype=torch.int32, device=device)[None, :].contiguous()]
        views = [View(torch.zeros(n_pages, 2, nkv, P, d, dtype=torch.bfloat16, device=device)) for _ in range(n_w)]
        inv = (10000.0 ** (-2.0 * torch.arange(d // 2, dtype=torch.float64) / d)).float().to(device)
        ang = ctx.positions.float()[:, None] * inv[None, :]
        cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
        q = torch.empty(rows, nh * d, dtype=torch.bfloat16, device=device)
        qkv = torch.empty(rows, N, device=device)
        line = {"micro": "qkv-rope", "size": size, "rows": rows}

        def two():
            for w, v in zip(ws, views):
                ops.linear(x, w, qkv)
                ops.rope_kv_append(qkv, cos, sin, d, nh, nkv, d, ctx, v, q)

        def fused():
            for w, v in zip(ws, views):
                if not ops.linear_rope_kv_append(x, w, cos, sin, d, nh, nkv, d, ctx, v, q):
                    raise RuntimeError("declined")
        line["two_kernels_us"] = round(_graph_us(torch, two, n_w), 1)
        try:
            line["fused_us"] = round(_graph_us(torch, fused, n_w), 1)
        except RuntimeError:
            line["fused_us"] = None                       # this shape keeps the two-kernel path (head size 128)
        print(json.dumps(line))
        del ws, views
    ops.raise_on_device_error()
    return 0


def _graph_us(torch, run, n_launches: int, reps: int = 10) -> float:
    """Microseconds per launch of `run()` (which issues `n_launches` kernels) replayed from a CUDA graph."""
    run()
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        run()
        with torch.cuda.graph(graph, stream=side):
            run()
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps / n_launches * 1e3


def micro_reference() -> int:
    """The reference's own kernels (compiled unchanged, kungfu_b200/measure/reference_kernels.py) beside this engine's
    kernels on the same device and shapes: prompt attention over 2,048 rows, decode attention over 8 x 8,192 keys, the
    products of a Gemma 2 2B layer at 8 and 2,048 rows, the norm with residual.  Every case is replayed from a CUDA graph
    over several copies of its operands (more than the L2 holds), timed with CUDA events; one JSON line per case with
    microseconds per launch for both and their ratio.  The reference's kernels read 32-bit activations and a
    half-precision ring cache; this engine's read bfloat16 activations and pages."""
    import math
    import torch
    from kungfu_b200 import api, ops
    from kungfu_b200.measure import reference_kernels as rk
    device = api.require_cuda("cuda:0")
    ops.library()
    ref = rk.Reference()
    gen = torch.Generator(device=device)
    gen.manual_seed(0)

    class View:
        def __init__(self, pages, page_size):
            self.pages, self.page_size, self.group, self.writes = pages, page_size, 0, False

    class Ctx:
        pass

    def emit(case, us_ref, us_ours, note=""):
        print(json.dumps({"micro": "reference", "case": case, "reference_us": round(us_ref, 1), "ours_us": round(us_ours, 1),
                          "speedup": round(us_ref / us_ours, 2), "note": note}), flush=True)

    # ---- products: one row block against n_w copies of the weight -------------------------------------------------------
    H, Q, inner = 2304, 2048, 9216
    for rows in (8, 2048):
        for name, n_out, k in (("q,k,v", 4096, H), ("o", H, Q), ("gate or up", inner, H), ("down", H, inner)):
            n_w = max(2, int(300e6 // (n_out * k * 2)))
            ws = [(torch.randn(n_out, k, device=device, generator=gen) * 0.02).to(torch.bfloat16) for _ in range(n_w)]
            x32 = torch.randn(rows, k, device=device, generator=gen).to(torch.bfloat16).float()
            x16 = x32.to(torch.bfloat16)
            out = torch.empty(rows, n_out, device=device)
            us_ref = _graph_us(torch, lambda: [ref.linear_bf16(w, x32) for w in ws], n_w, reps=3 if rows > 8 else 10)
            us_ours = _graph_us(torch, lambda: [ops.linear(x16, w, out) for w in ws], n_w)
            emit(f"product {name} [{n_out} x {k}] x {rows} rows", us_ref, us_ours,
                 "reference: matvec (one warp per output)" if rows <= 8 else "reference: 32 x 64 x 64 tiles of 32-bit FMA")
            del ws
    # ---- norm with residual ------------------------------------------------------------------------------------------------
    for rows in (8, 2048):
        n_c = 16 if rows > 8 else 2
        xs = [torch.randn(rows, H, device=device, generator=gen) for _ in range(n_c)]
        res = [torch.randn(rows, H, device=device, generator=gen) for _ in range(n_c)]
        w32 = torch.randn(H, device=device, generator=gen) * 0.1
        w16 = w32.to(torch.bfloat16)
        us_ref = _graph_us(torch, lambda: [ref.rms_norm_add(x, w32, r, 1e-6) for x, r in zip(xs, res)], n_c)
        us_ours = _graph_us(torch, lambda: [ops.add_rmsnorm(x, w16, 1e-6, True, r) for x, r in zip(xs, res)], n_c)
        emit(f"norm + residual, {rows} rows x {H}", us_ref, us_ours)
    # ---- decode attention: 8 requests x 8,192 keys, heads 8/4 x 256 (Gemma 2 2B) and 32/16 x 128 (27B) -----------------------
    for nh, nkv, d in ((8, 4, 256), (32, 16, 128)):
        batch, keys, page, copies = 8, 8192, 64, 3
        scale = 1.0 / math.sqrt(d)
        caches = [ref.make_cache(batch, keys, nkv * d, device) for _ in range(copies)]
        for kc, vc in caches:
            kc.normal_(0.0, 0.5, generator=gen)
            vc.normal_(0.0, 0.5, generator=gen)
        q32 = torch.randn(batch, nh * d, device=device, generator=gen)
        pos = torch.full((batch,), keys - 1, dtype=torch.int32, device=device)
        seq = torch.arange(batch, dtype=torch.int32, device=device)
        us_ref = _graph_us(torch, lambda: [ref.attention_decode(q32, kc, vc, pos, seq, nh, nkv, d, scale, None, 50.0) for kc, vc in caches], copies)
        per_req = keys // page
        pages = torch.empty(copies * batch * per_req, 2, nkv, page, d, device=device, dtype=torch.bfloat16).normal_(0.0, 0.5, generator=gen)
        ctxs = []
        for c_i in range(copies):
            c = Ctx()
            c.positions, c.row_req = pos, seq
            c.block_tables = [(torch.arange(batch * per_req, dtype=torch.int32, device=device) + c_i * batch * per_req).view(batch, per_req).contiguous()]
            c.n_rows = c.n_dec_rows = batch
            c.n_pre_rows = c.n_tiles = c.n_wide = 0
            c.dec_rows = c.pre_rows = None
            c.max_kv_len = keys
            ctxs.append(c)
        q16 = q32.to(torch.bfloat16)
        o16 = torch.empty_like(q16)
        view = View(pages, page)
        us_ours = _graph_us(torch, lambda: [ops.paged_attention(q16, o16, c, view, nh, nkv, d, scale, 50.0, None) for c in ctxs], copies)
        n_bytes = batch * keys * nkv * d * 2 * 2
        emit(f"decode attention, {batch} x {keys} keys, heads {nh}/{nkv} x {d}", us_ref, us_ours,
             f"keys and values {n_bytes / 1e6:.0f} MB: reference {n_bytes / us_ref / 1e3:.0f} GB/s, ours {n_bytes / us_ours / 1e3:.0f} GB/s")
        del caches, pages
    # ---- prompt attention: one prompt of 2,048 rows ---------------------------------------------------------------------------
    for nh, nkv, d in ((8, 4, 256), (32, 16, 128)):
        T, page, copies = 2048, 64, 4
        scale = 1.0 / math.sqrt(d)
        pos = torch.arange(T, dtype=torch.int32, device=device)
        seq0 = torch.zeros(T, dtype=torch.int32, device=device)
        caches = [ref.make_cache(1, T, nkv * d, device) for _ in range(copies)]
        for kc, vc in caches:
            kc.normal_(0.0, 0.5, generator=gen)
            vc.normal_(0.0, 0.5, generator=gen)
        q32 = torch.randn(T, nh * d, device=device, generator=gen)
        tiles = ref.flash_tiles(pos, [(0, 0, T)], device)
        us_ref = _graph_us(torch, lambda: [ref.flash_prefill(q32, kc, vc, pos, seq0, [(0, 0, T)], nh, nkv, d, scale, None, 50.0, tiles=tiles)
                                           for kc, vc in caches], copies, reps=5)
        per_req = T // page
        pages = torch.empty(copies * per_req, 2, nkv, page, d, device=device, dtype=torch.bfloat16).normal_(0.0, 0.5, generator=gen)
        ctxs = []
        for c_i in range(copies):
            c = Ctx()
            c.positions, c.row_req = pos, seq0
            c.block_tables = [(torch.arange(per_req, dtype=torch.int32, device=device) + c_i * per_req).view(1, per_req).contiguous()]
            c.n_rows = c.n_pre_rows = T
            c.n_dec_rows = 0
            c.dec_rows = None
            c.pre_rows = torch.arange(T, dtype=torch.int32, device=device)
            c.n_tiles, c.n_wide = T // 64, T // 128
            c.tile_row0 = torch.arange(0, T, 64, dtype=torch.int32, device=device)
            c.tile_nrows = torch.full((T // 64,), 64, dtype=torch.int32, device=device)
            c.wide_row0 = torch.arange(0, T, 128, dtype=torch.int32, device=device)
            c.wide_nrows = torch.full((T // 128,), 128, dtype=torch.int32, device=device)
            c.max_kv_len = T
            ctxs.append(c)
        q16 = q32.to(torch.bfloat16)
        o16 = torch.empty_like(q16)
        view = View(pages, page)
        us_ours = _graph_us(torch, lambda: [ops.paged_attention(q16, o16, c, view, nh, nkv, d, scale, 50.0, None) for c in ctxs], copies)
        flops = 4.0 * nh * d * T * (T + 1) / 2
        emit(f"prompt attention, {T} rows, heads {nh}/{nkv} x {d}", us_ref, us_ours,
             f"reference {flops / us_ref / 1e6:.0f} TFLOP/s, ours {flops / us_ours / 1e6:.0f} TFLOP/s")
        del caches, pages
    ops.raise_on_device_error()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--reps", type=int, default=3, help="timed runs of --steps steps each; mean and sd are reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="2b", choices=sorted(SIZES))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the size has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--only-headline", action="store_true", help="skip the other batch sizes, the mixed steps, 32-bit and the other model sizes")
    ap.add_argument("--micro", choices=["attention", "prompt-attention", "gemm", "products", "qkv-rope", "reference"],
                    help="time kernels alone instead of the model step")
    args = ap.parse_args()
    if args.micro:
        return {"attention": micro_attention, "prompt-attention": micro_prompt_attention, "gemm": micro_gemm,
                "products": lambda: micro_products(args.size), "qkv-rope": lambda: micro_qkv_rope(args.size),
                "reference": micro_reference}[args.micro]()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "nickheyer/kungfu is a Rust workspace (no setup.py or "
                          "pyproject.toml; pip: 'not installable') and this image has no cargo/rustc and no network, so it cannot be built "
                          "(its CUDA kernels alone are timed by --micro reference)"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    args.reps = max(args.reps, 1)
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
