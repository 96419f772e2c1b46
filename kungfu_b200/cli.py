"""The command line, in the manner of the reference's `kungfu` binary (crates/kungfu/src/main.rs:17-137).

Subcommands and option names follow it where it has them:
  inspect <model> [--json]      what the folder is, its tensors and what each layer keeps       (:19,213-311)
  describe                      capabilities and parameters of this build as JSON               (:21,149-152)
  generate --model --ids ...    complete a prompt given as token ids                            (:107-136,611-645)
  score --model --ids --prefix  greedy prediction (or top-k ids) at every position              (:30-55,173-197)
  bench --model --pp --tg --reps  prompt and generation throughput                              (:82-105,544-608)
  random-weights                write a model folder from a config.json and a seed (ours; the reference has no such mode)
There is no tokenizer here: prompts are token ids (`--ids`), and output is always ids.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time


def _common(p: argparse.ArgumentParser) -> None:
    p.add_argument("--backend", default="auto", choices=["auto", "cuda", "cpu"], help="cuda when a device is visible; cpu is refused")
    p.add_argument("--device", type=int, default=0, help="ordinal among the visible devices")
    p.add_argument("--ctx", default="4096", help="tokens of context per sequence, or auto for the trained length")
    p.add_argument("--batch", type=int, default=512, help="most tokens one pass feeds")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="compute precision")
    p.add_argument("--page-size", type=int, default=None, help="tokens per cache page")


def _device(args) -> str:
    if args.backend == "cpu":
        raise SystemExit("error: this build has no cpu backend; kernels run on sm_100a only")
    return f"cuda:{args.device}"


def _engine(args, parallel: int = 1):
    from .engine.engine import Engine
    common = dict(dtype=args.dtype, device=_device(args), ctx=args.ctx if args.ctx == "auto" else int(args.ctx),
                  batch=args.batch, parallel=parallel, page_size=args.page_size, events=getattr(args, "events", False))
    if getattr(args, "random_weights", False):
        # no file: weights are drawn on the device from the configuration and the seed (the same values that
        # `random-weights` would write into a model folder)
        if not getattr(args, "config", None):
            raise SystemExit("error: --random-weights needs --config (a config.json)")
        return Engine(config=args.config, seed=args.weights_seed, **common)
    if not args.model:
        raise SystemExit("error: give --model DIR, or --config FILE --random-weights")
    return Engine(args.model, **common)


# ---- inspect ------------------------------------------------------------------------------------------------

def cmd_inspect(args) -> int:
    from . import registry
    from .api import load_config
    from .weights.safetensors_io import open_model_tensors
    from .config.base import ConfigError
    from .registry import UnknownArchitecture
    try:
        cfg = load_config(args.model)
    except (ConfigError, UnknownArchitecture) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    arch = registry.find(cfg.architecture)
    tensors = open_model_tensors(args.model)
    specs = {s.name: s for s in arch.tensor_specs(cfg)}
    missing = sorted(n for n in specs if n not in tensors)
    unexpected = sorted(n for n in tensors if n not in specs)
    wrong = sorted((n, list(specs[n].shape), list(tensors[n][1].shape)) for n in specs
                   if n in tensors and tuple(tensors[n][1].shape) != tuple(specs[n].shape))
    hist: dict = {}
    groups: dict = {}
    total_bytes = total_params = 0
    for n, (_sf, info) in tensors.items():
        hist[info.dtype] = hist.get(info.dtype, 0) + 1
        total_bytes += info.nbytes
        total_params += info.numel
        parts = n.split(".")
        gid = f"layer.{parts[2]}" if n.startswith("model.layers.") else ("embedding" if "embed" in n else "output")
        g = groups.setdefault(gid, {"id": gid, "bytes": 0, "elements": 0, "count": 0})
        g["bytes"] += info.nbytes
        g["elements"] += info.numel
        g["count"] += 1
    elt = 2
    states = [{"layer": l, "kind": "kv_cache", "bytes_per_token": 2 * cfg.num_key_value_heads * cfg.head_dim * elt,
               "window": cfg.window_of(l), "fixed_bytes": 0} for l in range(cfg.num_hidden_layers)]
    doc = {"architecture": cfg.architecture, "tensors": len(tensors), "bytes": total_bytes, "params": total_params,
           "dtypes": hist, "hparams": cfg.to_dict(), "layers": cfg.num_hidden_layers,
           "context_train": cfg.max_position_embeddings, "groups": list(groups.values()), "states": states,
           "missing": missing, "unexpected": unexpected, "wrong_shape": wrong}
    if args.json:
        print(json.dumps(doc))
    else:
        print(f"architecture  {doc['architecture']}")
        print(f"tensors       {doc['tensors']}  ({total_bytes / 1e6:.1f} MB, {total_params / 1e6:.2f} M parameters)")
        print(f"dtypes        {hist}")
        print(f"layers        {doc['layers']}  context_train {doc['context_train']}")
        for k, v in doc["hparams"].items():
            if k != "layer_types":
                print(f"  {k:32s} {v}")
        for g in doc["groups"]:
            print(f"group {g['id']:12s} tensors {g['count']:3d}  bytes {g['bytes']}")
        for s in states:
            print(f"state layer {s['layer']:3d} kv_cache bytes_per_token {s['bytes_per_token']} window {s['window']}")
    if missing or unexpected or wrong:
        print(f"error: weights do not match the configuration: missing {missing}, unexpected {unexpected}, "
              f"wrong shapes {wrong}", file=sys.stderr)
        return 1
    return 0


# ---- describe -----------------------------------------------------------------------------------------------

PARAMS = [
    # name, type, default, flag, description   (reference: the PARAMS table, crates/kf-serve/src/params.rs:50-87)
    ("model", "path", "", "--model", "folder with config.json and model.safetensors"),
    ("n_ctx", "int", "4096", "--ctx", "tokens of context per sequence, auto for the trained length"),
    ("n_batch", "int", "512", "--batch", "most tokens one pass feeds"),
    ("n_parallel", "int", "1", "--parallel", "sequences decoded together"),
    ("backend", "string", "auto", "--backend", "cuda when a device is visible; there is no cpu backend"),
    ("device", "int", "0", "--device", "ordinal among the visible devices"),
    ("dtype", "string", "bfloat16", "--dtype", "bfloat16 or float32 (true 32-bit, no reduced-precision products)"),
    ("page_size", "int", "64", "--page-size", "tokens per cache page"),
    ("temperature", "float", "0.7", "--temperature", "zero for greedy"),
    ("top_k", "int", "40", "--top-k", "zero disables"),
    ("top_p", "float", "0.95", "--top-p", "one disables"),
    ("min_p", "float", "0", "--min-p", "zero disables"),
    ("repeat_penalty", "float", "1", "--repeat-penalty", "one disables"),
    ("max_tokens", "int", "64", "--max-tokens", "tokens generated per request"),
]


def cmd_describe(args) -> int:
    import torch
    from . import __version__, ops, registry
    from .parts import base
    devices = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            devices.append({"index": i, "name": p.name, "memory": p.total_memory, "sm": f"{p.major}{p.minor}", "sms": p.multi_processor_count})
    doc = {"name": "kungfu_b200", "version": __version__, "protocol": 1,
           "architectures": registry.names(), "formats": ["safetensors"], "dtypes": ["bfloat16", "float32"],
           "backends": [{"name": "cuda", "arch": "sm_100a", "devices": devices}],
           "parts": {k: base.known(k) for k in ("mixer", "feed_forward", "norm", "position", "block")},
           "params": [{"name": n, "type": t, "default": d, "flag": f, "description": desc} for n, t, d, f, desc in PARAMS],
           "events": ["plan", "alloc", "ready", "request", "error"], "finish_reasons": ["eos", "length", "context", "cancelled", "no_fit"],
           "errors": ["config", "unknown_arch", "weights", "model_open", "no_fit"],
           "kernel_library": ops.library_path(),
           # how often bfloat16 work of this process left the tensor-core kernels for a generic one, by reason
           "slow_kernel_fallbacks": ops.fallbacks()}
    print(json.dumps(doc, indent=2))
    return 0


# ---- generate -----------------------------------------------------------------------------------------------

def cmd_generate(args) -> int:
    from .sampling import Sampling
    if args.ids is None:
        raise SystemExit("error: this build has no tokenizer; give the prompt as --ids '[1, 2, 3]'")
    ids = json.loads(args.ids)
    eng = _engine(args)
    sampling = Sampling(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                        repeat_penalty=args.repeat_penalty)
    out = eng.generate([ids], sampling, max_tokens=args.max_tokens, ignore_eos=args.ignore_eos, seed=args.seed)[0]
    eos = set(getattr(eng.cfg, "eos_token_id", ()) or ())
    if out and out[-1] in eos and not args.ignore_eos and not args.emit_ids:
        out = out[:-1]
    print(json.dumps({"prompt": ids, "generated": out}))
    return 0


# ---- score --------------------------------------------------------------------------------------------------

def cmd_score(args) -> int:
    import torch
    from .engine.step import StepEntry
    ids = json.loads(args.ids)
    eng = _engine(args)
    runner = eng.runner
    prefix = len(ids) if args.prefix is None else max(1, min(args.prefix, len(ids)))
    runner.cache.add_request("score")
    rows = []
    head = ids[:prefix]
    chunks = [head[i:i + args.batch] for i in range(0, prefix, args.batch)] + [[t] for t in ids[prefix:]]
    eos = set(getattr(eng.cfg, "eos_token_id", ()) or ())
    from . import ops
    if args.topk > 64:
        raise SystemExit("error: --topk is at most 64 (the candidates the device ranks per row)")
    for chunk in chunks:
        logits = runner.step([StepEntry("score", chunk, list(range(len(chunk))))]).clone()
        if args.ignore_eos and eos:
            logits[:, sorted(eos)] = float("-inf")
        n = logits.shape[0]
        if args.topk > 0:
            best = torch.empty((n, args.topk), dtype=torch.int32, device=logits.device)
            vals = torch.empty((n, args.topk), dtype=torch.float32, device=logits.device)
            lse = torch.empty((n,), dtype=torch.float32, device=logits.device)
            ops.topk_lse(logits, args.topk, best, vals, lse)
            rows += best.cpu().tolist()
        else:
            best = torch.empty((n,), dtype=torch.int32, device=logits.device)
            ops.argmax(logits, best)
            rows += best.cpu().tolist()
    runner.cache.release("score")
    print(json.dumps({"ids": ids, "predictions": rows}))
    return 0


# ---- bench --------------------------------------------------------------------------------------------------

def cmd_bench(args) -> int:
    import torch
    from .engine.step import StepEntry
    eng = _engine(args)
    runner = eng.runner
    vocab = runner.vocab
    toks = [(i * 7919 + 13) % vocab for i in range(args.pp + args.tg)]       # reference: main.rs:549

    def prefill(rid):
        runner.cache.add_request(rid)
        for i in range(0, args.pp, args.batch):
            chunk = toks[i:i + args.batch]
            runner.step([StepEntry(rid, chunk, [len(chunk) - 1] if i + args.batch >= args.pp else [])])

    def timed(fn):
        torch.cuda.synchronize()
        t = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        return time.perf_counter() - t

    prefill("warm")
    for t in toks[args.pp:args.pp + 2]:
        runner.step([StepEntry("warm", [t], [0])])
    runner.cache.release("warm")
    pp_rates, tg_rates = [], []
    for r in range(args.reps):
        pp_rates.append(args.pp / timed(lambda: prefill(f"b{r}")))
        dt = timed(lambda: [runner.step([StepEntry(f"b{r}", [t], [0])]) for t in toks[args.pp:]])
        tg_rates.append(args.tg / dt)
        runner.cache.release(f"b{r}")

    def stats(x):
        m = sum(x) / len(x)
        return m, math.sqrt(sum((v - m) ** 2 for v in x) / len(x))

    if args.trace:
        # one more prompt pass and one more decode step with every kernel timed (CUDA events, launches serialised)
        from . import ops
        runner.cache.add_request("trace")
        ops.trace_begin()
        runner.step([StepEntry("trace", toks[:min(args.pp, args.batch)], [0])])
        pp_trace = ops.trace_end()
        ops.trace_begin()
        runner.step([StepEntry("trace", [toks[0]], [0])])
        tg_trace = ops.trace_end()
        runner.cache.release("trace")
        for title, rec in (("prompt pass", pp_trace), ("decode step", tg_trace)):
            agg: dict = {}
            for name, ms in rec:
                n, t = agg.get(name, (0, 0.0))
                agg[name] = (n + 1, t + ms)
            total = sum(t for _, t in agg.values())
            print(f"kernel times, {title} ({len(rec)} operations, {total:.3f} ms):", file=sys.stderr)
            for name, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
                print(f"  {name:18s} x{n:<4d} {t * 1e3:10.1f} us  {100 * t / total:5.1f} %", file=sys.stderr)
    print("| model | dtype | test | t/s |")
    print("|---|---|---|---|")
    for name, rates in ((f"pp{args.pp}", pp_rates), (f"tg{args.tg}", tg_rates)):
        m, sd = stats(rates)
        print(f"| {eng.cfg.architecture} | {args.dtype} | {name} | {m:.2f} ± {sd:.2f} |")
    return 0


def cmd_random_weights(args) -> int:
    import torch
    from .api import load_config
    from .weights import write_random_model
    cfg = load_config(args.config)
    write_random_model(args.out, cfg, args.seed, dtype=torch.float32 if args.dtype == "float32" else torch.bfloat16,
                       device="cuda:0" if torch.cuda.is_available() else None)
    print(args.out)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kungfu", description="Gemma 2 on B200: inspect, describe, generate, score, bench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("inspect", help="what the folder is, how its tensors group, what state each layer keeps")
    p.add_argument("model")
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_inspect)
    p = sub.add_parser("describe", help="capabilities and parameters of this build as JSON")
    p.set_defaults(fn=cmd_describe)
    p = sub.add_parser("generate", help="complete a prompt of token ids")
    p.add_argument("--model", default=None, help="folder with config.json and model.safetensors")
    p.add_argument("--prompt", default="", help="text prompts need a tokenizer, which this build lacks: use --ids")
    p.add_argument("--ids", default=None, help="prompt as a JSON array of token ids")
    p.add_argument("--config", default=None, help="with --random-weights: the config.json to build from")
    p.add_argument("--random-weights", action="store_true", help="no model folder: draw weights from --config and --weights-seed")
    p.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
    p.add_argument("--emit-ids", action="store_true", help="print prompt and generated ids as JSON (always so here)")
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=40)
    p.add_argument("--top-p", type=float, default=0.95)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--repeat-penalty", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--events", action="store_true", help="print `kungfu event=` lines on stderr")
    _common(p)
    p.set_defaults(fn=cmd_generate)
    p = sub.add_parser("score", help="greedy prediction at every position of a token sequence")
    p.add_argument("--model", required=True)
    p.add_argument("--ids", required=True)
    p.add_argument("--prefix", type=int, default=None, help="tokens fed as one batch before the rest go one at a time")
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--topk", type=int, default=0)
    _common(p)
    p.set_defaults(fn=cmd_score)
    p = sub.add_parser("bench", help="prompt and generation throughput")
    p.add_argument("--model", required=True)
    p.add_argument("--pp", type=int, default=512)
    p.add_argument("--tg", type=int, default=128)
    p.add_argument("--reps", type=int, default=3)
    p.add_argument("--trace", action="store_true", help="also print per-kernel times of one prompt pass and one decode step")
    _common(p)
    p.set_defaults(fn=cmd_bench)
    p = sub.add_parser("random-weights", help="write a model folder from a config.json and a seed")
    p.add_argument("--config", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.set_defaults(fn=cmd_random_weights)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
