#!/usr/bin/env python3
"""Decode and prefill throughput of the Gemma 2 engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--layers L] [--batch B] [--context C] [--size 2b|9b|27b]
    python bench.py --micro attention|gemm|products   (one kernel alone, JSON lines; used for the summaries in profiles/)

A "step" is one decode step: every live request gets one token.  Default: the layer sizes of Gemma 2 2B,
random bfloat16 weights, 8 requests at a context of 8192 tokens.  `value` is decoded tokens per second timed
with CUDA events around K steps of the step function; `e2e` is the same through the Python entry point
(`Engine.step()`: host scheduling, the step's integers copied from pinned host memory, tokens read back).
`prefill` is one step of 2,048 prompt tokens; `roofline` is the bytes a decode step must read (every weight
once, the cache of the live requests) over its time; `points` holds decode at batch 1 and 64.
Method after the reference's `kungfu bench` (crates/kungfu/src/main.rs:544-608): synthetic token ids, every
shape run before timing.  Caches are filled with random keys and values instead of running the long prompts.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SIZES = {
    # BASELINE.json configs[2..4]
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


def fill_cache(runner, rid, n_tokens: int, gen) -> None:
    """Make request `rid` hold `n_tokens` tokens of random keys and values without running them."""
    runner.cache.add_request(rid)
    runner.cache.reserve(rid, n_tokens)
    runner.cache.commit(rid, n_tokens)


def randomize_pages(runner, torch) -> None:
    g = torch.Generator(device=runner.device)
    g.manual_seed(1)
    for s, t in runner.cache.storage.items():
        if t.dim() == 5:
            flat = t.view(-1)
            step = 1 << 28
            for i in range(0, flat.numel(), step):
                flat[i:i + step].normal_(0.0, 0.5, generator=g)


def time_decode(torch, runner, rids, steps: int, warmup: int, vocab: int):
    from kungfu_b200 import ops
    from kungfu_b200.engine import StepEntry
    tok = 17

    def one(i):
        entries = [StepEntry(r, [(tok + 31 * i + 7 * k) % vocab], [0]) for k, r in enumerate(rids)]
        return runner.step(entries)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    l0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        one(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    return ms / steps, ops.launch_count() - l0


def run_ours(args) -> dict:
    import torch
    from kungfu_b200 import api, ops
    from kungfu_b200.engine import StepEntry
    from kungfu_b200.engine.engine import Engine
    from kungfu_b200.engine.scheduler import Request
    from kungfu_b200.sampling import Sampling

    pk, pk_src = peaks()
    device = api.require_cuda("cuda:0")
    ops.library()
    raw = dict(COMMON, **SIZES[args.size])
    full_layers = raw["num_hidden_layers"]
    n_layers = args.layers or full_layers
    raw["num_hidden_layers"] = n_layers
    cfg, model = api.random_model(raw, seed=0, dtype="bfloat16", device=device)
    ctx_len, B = args.context, args.batch
    page = api.DEFAULT_PAGE_SIZE
    margin = 2 * (args.steps + args.warmup) + 64
    big_b = max(B, 64 if not args.no_points else B)
    per_req = -(-(ctx_len + margin) // page) * page
    runner = api.make_runner(cfg, model, dtype="bfloat16", device=device, page_size=page,
                             max_tokens=big_b * per_req + 4096, max_requests=big_b + 2,
                             max_context=ctx_len + margin)
    randomize_pages(runner, torch)
    vocab = cfg.vocab_size
    per_layer, weight_bytes = model_numbers(cfg, n_layers)

    # ---- prefill: one step of 2,048 prompt tokens -----------------------------------------------------------
    T = args.prefill_tokens
    toks = [(i * 7919 + 13) % vocab for i in range(T)]
    pf_ms = []
    for rep in range(3):
        runner.cache.add_request("pf")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("pf", toks, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        pf_ms.append(e0.elapsed_time(e1))
        runner.cache.release("pf")
    pf = min(pf_ms[1:])
    flops = prefill_flops(cfg, n_layers, T)
    prefill = {"value": round(T / pf * 1e3, 1), "tokens": T, "ms": round(pf, 3),
               "frac": round(flops / (pf * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode at the headline batch, with clocks sampled ----------------------------------------------------
    def decode_at(batch: int, steps: int, warmup: int, sample_clocks: bool):
        rids = [f"d{batch}_{k}" for k in range(batch)]
        start = ctx_len - warmup                      # the timed steps run at positions ctx_len, ctx_len+1, ...
        for r in rids:
            fill_cache(runner, r, start, None)
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
            time.sleep(0.3)
        ms, launches = time_decode(torch, runner, rids, steps, warmup, vocab)
        clocks = sampler.stop() if sample_clocks else None
        for r in rids:
            runner.cache.release(r)
        return ms, launches, clocks

    ms_step, launches, clocks = decode_at(B, args.steps, args.warmup, True)
    value = B / ms_step * 1e3
    bytes_step = weight_bytes + B * kv_bytes_read(cfg, n_layers, ctx_len)
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_src}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            ms_b, _, _ = decode_at(b, max(8, args.steps // 2), args.warmup, False)
            points[f"decode_b{b}"] = round(b / ms_b * 1e3, 1)

    # ---- end to end through the Python entry point ---------------------------------------------------------------
    eng = Engine(runner=runner, batch=max(512, B), parallel=B)
    eng.cfg = cfg
    start = ctx_len - args.warmup
    for k in range(B):
        rid = f"e{k}"
        prompt = [(k * 131 + i * 7919 + 13) % vocab for i in range(start)]
        req = Request(rid, prompt, Sampling(temperature=0.0), max_tokens=10 ** 9, eos=(), ignore_eos=True)
        fill_cache(runner, rid, start - 1, None)      # all but the last prompt token are "already run"
        req.n_cached = start - 1
        eng.requests[rid] = req
        eng.scheduler.adopt(req)
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(args.steps):
        n_tok += sum(1 for _id, tok, _r in eng.step() if tok is not None)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    meta_ints = runner.last_meta_ints
    e2e = {"value": round(n_tok / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(meta_ints * 4),
           "d2h_bytes_per_step": int(B * 4), "ms_per_step": round(dt / args.steps * 1e3, 3)}

    config = {"model": f"gemma2-{args.size}", "layers": n_layers, "layers_full": full_layers,
              "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
              "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
              "sliding_window": cfg.sliding_window, "global_batch": B, "seq_len": ctx_len, "page_size": page,
              "parallelism": "single", "weights": "random bf16", "cache": "bf16 random fill", "l2": "inputs larger than L2",
              "cuda_graphs": bool(getattr(runner, "cuda_graphs", False)),
              "e2e_reads": "ids of step n read on the host while step n+1 runs" if eng.pipeline else "every step before the next"}
    return {"metric": "decode tokens/s (batch 8, context 8192, Gemma 2 2B sizes, 1 B200)" if (args.size, B, ctx_len) == ("2b", 8, 8192)
            else f"decode tokens/s (batch {B}, context {ctx_len}, Gemma 2 {args.size} sizes, 1 B200)",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic token ids, random-init weights, random-filled cache",
            "config": config, "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "prefill": prefill,
            "roofline": roofline, "points": points, "impl": "ours"}


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


def micro_products() -> int:
    """The four products of a Gemma 2 2B layer over 8 to 2,048 rows, each replayed from a CUDA graph of six launches over
    distinct weights; one JSON line per (rows, product) with microseconds per launch."""
    import torch
    from kungfu_b200 import api, ops
    device = api.require_cuda("cuda:0")
    ops.library()
    H, Q, inner, n_w = 2304, 2048, 9216, 6
    gen = torch.Generator(device=device)
    gen.manual_seed(0)
    shapes = {"q,k,v": (4096, H, False), "o": (H, Q, False), "gate+up": (inner, H, True), "down": (H, inner, False)}
    for rows in (8, 64, 128, 256, 512, 1024, 2048):
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
            print(json.dumps({"micro": "product", "rows": rows, "product": name, "us": round(us, 1),
                              "tflops": round(flops / us / 1e6, 1)}))
            del ws
    ops.raise_on_device_error()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="2b", choices=sorted(SIZES))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the size has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--micro", choices=["attention", "gemm", "products"], help="time one kernel alone instead of the model step")
    args = ap.parse_args()
    if args.micro == "attention":
        return micro_attention()
    if args.micro == "gemm":
        return micro_gemm()
    if args.micro == "products":
        return micro_products()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "nickheyer/kungfu is a Rust workspace (no setup.py or "
                          "pyproject.toml; pip: 'not installable') and this image has no cargo/rustc and no network, so it cannot be built"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
