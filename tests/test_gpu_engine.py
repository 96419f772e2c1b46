"""The engine on the GPU against the plain implementation: every way of cutting the work, in 32-bit and bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_gemma2

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# rel = max|got - ref| / max|ref| over all wanted rows, always against float64.  32-bit: rounding of sums only.
# bfloat16: activations, cached keys/values and softmax weights are rounded to 8 bits of mantissa at every product
# (the reference's own bound for half-precision caches is 2e-2, crates/kf-backend-cuda/tests/common/mod.rs:181-187).
# Draws of the weights (helpers.sharpen_tensors): 'plain' for both precisions; 'sharp' (scores at the attention cap,
# logits beyond the final cap) for 32-bit; 'loud' (logits at the final cap) for bfloat16.
# tests/test_oracle_sensitivity.py shows which constant of the architecture each combination would notice.
TOL = {"float32": 2e-4, "bfloat16": 2e-2}
DRAWS = [("plain", "float32"), ("plain", "bfloat16"), ("sharp", "float32"), ("loud", "bfloat16")]

# six requests each, at most four live in the mixed traces: what the first ones give back the last ones take
CASES = {"A": (helpers.TINY_A, [5, 17, 23, 40, 11, 30], 4), "B": (helpers.TINY_B, [1, 31, 40, 70, 9, 50], 8),
         "C": (helpers.TINY_C, [3, 50, 64, 29, 120, 77], 16), "D": (helpers.TINY_D, [2, 40, 17, 90, 33, 8], 4)}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, lengths, page) in CASES.items():
        for draw in ("plain", "loud", "sharp"):
            folder = helpers.write_model(str(tmp_path_factory.mktemp(name) / "m"), cfg, seed=21, dtype=torch.bfloat16, draw=draw)
            vocab = cfg["vocab_size"] if draw == "plain" else helpers.quiet_vocab(cfg)
            reqs = {f"r{i}": helpers.random_tokens(n, vocab, 300 + i) for i, n in enumerate(lengths)}
            tensors = helpers.read_tensors(folder)
            ref = {rid: plain_gemma2.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
            out[(name, draw)] = (folder, cfg, reqs, ref, page)
        out[name] = out[(name, "plain")]
    return out


def _check(got, ref, tol):
    scale = max(float(r.abs().max()) for r in ref.values())
    worst, wrong_top = 0.0, 0
    for (rid, pos), row in got.items():
        worst = max(worst, float((row - ref[rid][pos]).abs().max()))
        wrong_top += int(torch.argmax(row) != torch.argmax(ref[rid][pos]))
    assert worst / scale < tol, f"rel err {worst / scale:.3e} (first wrong top-1 count {wrong_top}/{len(got)})"
    return wrong_top


def _steps(mode, reqs):
    return {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_decode_tail(r, 32),
            "chunks": helpers.trace_chunks, "mixed": lambda r: helpers.trace_mixed(r, seed=5)}[mode](reqs)


@pytest.mark.parametrize("draw,dtype", DRAWS)
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_modes_match_plain(models, name, mode, draw, dtype):
    from kungfu_b200 import api
    folder, cfg, reqs, ref, page = models[(name, draw)]
    steps = _steps(mode, reqs)
    c, model = api.load_model(folder, dtype=dtype, device=DEV)
    runner = api.make_runner(c, model, dtype=dtype, device=DEV, page_size=page,
                             max_tokens=helpers.trace_max_tokens(steps, page), max_requests=8,
                             max_context=cfg["max_position_embeddings"])
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    _check(got, ref, TOL[dtype])
    assert runner.cache.n_live == 0
    if mode == "mixed":                                # the pool is smaller than what the trace hands out: pages came back
        assert all(n > g.pool.n_pages for n, g in zip(runner.cache.pages_handed_out(), runner.cache.groups)), \
            (runner.cache.pages_handed_out(), [g.pool.n_pages for g in runner.cache.groups])


@pytest.mark.parametrize("draw,dtype", DRAWS)
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_fast_kernel_sizes_match_plain(tmp_path_factory, mode, draw, dtype):
    """Configuration E: sizes at which the tcgen05 products (pairs included), the tcgen05 prompt attention and the
    tensor-core decode attention all run, with pages of 64, prompts longer than the window and than a CTA tile, and a
    pool small enough that pages come back and are used again."""
    from kungfu_b200 import api
    cfg = helpers.TINY_E
    cache = test_fast_kernel_sizes_match_plain.__dict__.setdefault("cache", {})
    if draw not in cache:
        folder = helpers.write_model(str(tmp_path_factory.mktemp("E") / "m"), cfg, seed=31, dtype=torch.bfloat16, draw=draw)
        vocab = cfg["vocab_size"] if draw == "plain" else helpers.quiet_vocab(cfg)
        reqs = {f"r{i}": helpers.random_tokens(n, vocab, 700 + i) for i, n in enumerate([300, 70, 513, 129, 2])}
        tensors = helpers.read_tensors(folder)
        cache[draw] = (folder, reqs, {rid: plain_gemma2.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()})
    folder, reqs, ref = cache[draw]
    steps = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_decode_tail(r, 32),
             "chunks": lambda r: helpers.trace_chunks(r, sizes=(150, 2, 64, 131, 7, 300, 3)),
             "mixed": lambda r: helpers.trace_mixed(r, seed=8)}[mode](reqs)
    c, model = api.load_model(folder, dtype=dtype, device=DEV)
    runner = api.make_runner(c, model, dtype=dtype, device=DEV, page_size=64,
                             max_tokens=helpers.trace_max_tokens(steps, 64), max_requests=8, max_context=1024)
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    _check(got, ref, TOL[dtype])
    from kungfu_b200 import ops
    ops.raise_on_device_error()
    if mode == "mixed":
        assert all(n > g.pool.n_pages for n, g in zip(runner.cache.pages_handed_out(), runner.cache.groups))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_stored_in_32_bit_stay_so(tmp_path, dtype):
    """A file whose tensors are 32-bit floats: the bfloat16 engine keeps them 32-bit (and multiplies them with the
    generic product), the 32-bit engine uses them as they are."""
    from kungfu_b200 import api
    cfg = helpers.TINY_A
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=23, dtype=torch.float32)
    reqs = {"r0": helpers.random_tokens(30, cfg["vocab_size"], 1), "r1": helpers.random_tokens(11, cfg["vocab_size"], 2)}
    tensors = helpers.read_tensors(folder)
    ref = {rid: plain_gemma2.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    c, model = api.load_model(folder, dtype=dtype, device=DEV)
    assert model.layers[0].ffn.w_down.dtype == torch.float32 and model.embedding.table.dtype == torch.float32
    steps = helpers.trace_mixed(reqs, seed=1)
    runner = api.make_runner(c, model, dtype=dtype, device=DEV, page_size=8, max_tokens=helpers.trace_max_tokens(steps, 8),
                             max_requests=4, max_context=64)
    _check(helpers.run_trace_with_runner(runner, steps), ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    """bin/trace_run as a user runs it: steps on standard input, logits files out, `done` after every step."""
    folder, cfg, reqs, ref, _ = models[("B", "sharp" if dtype == "float32" else "loud")]
    steps = helpers.trace_mixed(reqs, seed=9)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(helpers.trace_max_tokens(steps, 64))],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l] == [f"done {s['step']}" for s in steps]
    V = cfg["vocab_size"]
    got, fed = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        arr = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n_want, V)
        k = 0
        for e in s["entries"]:
            start = fed.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], start + w)] = torch.from_numpy(arr[k].copy())
                k += 1
            fed[e["id"]] = start + len(e["tokens"])
    _check(got, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decode_and_first_tokens(models, dtype):
    """A request decoded token by token from its very first token, far past the window and over many pages."""
    from kungfu_b200 import api
    folder, cfg, _, _, _ = models["A"]
    toks = helpers.random_tokens(64, cfg["vocab_size"], 77)
    ref = plain_gemma2.forward(cfg, helpers.read_tensors(folder), toks).float()
    c, model = api.load_model(folder, dtype=dtype, device=DEV)
    runner = api.make_runner(c, model, dtype=dtype, device=DEV, page_size=4, max_tokens=64, max_requests=2, max_context=64)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    steps[-1]["end"] = ["x"]
    got = helpers.run_trace_with_runner(runner, steps)
    _check(got, {"x": ref}, TOL[dtype])
