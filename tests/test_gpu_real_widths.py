"""The engine at the layer sizes of Gemma 2 2B, 9B and 27B against the plain implementation.

Two layers (one sliding, one global) of the real widths, head counts, head sizes and attention scales (27B:
1/sqrt(144) with heads of 128), with the vocabulary cut to 4,096 and, in all but one case, the window cut to 100 so
that short prompts cross it.  Weights come from the framework's random-weights generator on the device and are
sharpened (`helpers.sharpen_tensors`: the 'sharp' draw for 32-bit, the 'loud' draw for bfloat16), so that the
constants of the architecture matter; the plain model runs in float64 on the same device (torch arithmetic, no code
of the engine).  Every way of cutting the work, in 32-bit and in bfloat16, against float64.
One case keeps the real window of 4,096 at 2B widths with a prompt of 4,200 tokens.
"""
import gc

import pytest
import torch

import helpers
import plain_gemma2

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": 2e-4, "bfloat16": 2e-2}
DRAW = {"float32": "sharp", "bfloat16": "loud"}


def _config(hidden, heads, kv_heads, head_dim, inner, scalar, window, max_pos):
    return {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "num_hidden_layers": 2, "hidden_size": hidden,
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inner,
            "vocab_size": 4096, "rope_theta": 10000.0, "sliding_window": window, "attn_logit_softcapping": 50.0,
            "final_logit_softcapping": 30.0, "query_pre_attn_scalar": scalar, "rms_norm_eps": 1e-6,
            "tie_word_embeddings": True, "max_position_embeddings": max_pos, "hidden_activation": "gelu_pytorch_tanh"}


# layer sizes of the three models; "v4096" and "w100" say what was cut
SIZES = {"2b-widths-2layers-v4096-w100": _config(2304, 8, 4, 256, 9216, 256, 100, 1024),
         "9b-widths-2layers-v4096-w100": _config(3584, 16, 8, 256, 14336, 256, 100, 1024),
         "27b-widths-2layers-v4096-w100": _config(4608, 32, 16, 128, 36864, 144, 100, 1024)}
LONG = _config(2304, 8, 4, 256, 9216, 256, 4096, 8192)          # 2B widths with the real window
LENGTHS = [150, 40, 333, 70, 2]


def _weights(cfg, seed, draw):
    """Random weights for `cfg`, sharpened as `draw` says, as {file name: bfloat16 tensor on the device}."""
    from kungfu_b200 import api, registry
    from kungfu_b200.weights.store import random_tensor_device
    typed = api.load_config(dict(cfg))
    arch = registry.find(typed.architecture)
    tensors = {s.name: random_tensor_device(s, seed, torch.bfloat16, torch.device(DEV)) for s in arch.tensor_specs(typed)}
    helpers.sharpen_tensors(cfg, tensors, seed, device=DEV, **helpers.DRAWS[draw])
    return typed, arch, tensors


def _model(typed, arch, tensors, dtype):
    from kungfu_b200 import api
    from kungfu_b200.weights.store import WeightStore
    store = WeightStore.from_tensors(tensors, device=DEV, compute_dtype=api.parse_dtype(dtype))
    return arch.build(typed, store)


def _check(got, ref, tol):
    scale = max(float(r.abs().max()) for r in ref.values())
    worst = max(float((row - ref[rid][pos]).abs().max()) for (rid, pos), row in got.items())
    assert worst / scale < tol, f"rel err {worst / scale:.3e}"


@pytest.fixture(scope="module")
def cases():
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made.clear()                                    # one model on the device at a time
            gc.collect()
            torch.cuda.empty_cache()
            cfg = SIZES[name]
            typed, arch, tensors = _weights(cfg, 41, DRAW[dtype])
            reqs = {f"r{i}": helpers.random_tokens(n, helpers.quiet_vocab(cfg), 900 + i) for i, n in enumerate(LENGTHS)}
            ref = {r: plain_gemma2.forward(cfg, tensors, t, device=DEV).float() for r, t in reqs.items()}
            made[(name, dtype)] = (cfg, typed, arch, tensors, reqs, ref)
        return made[(name, dtype)]
    yield get
    made.clear()
    gc.collect()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SIZES))
def test_real_widths_match_plain(cases, name, dtype, mode):
    from kungfu_b200 import api, ops
    cfg, typed, arch, tensors, reqs, ref = cases(name, dtype)
    steps = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_decode_tail(r, 32),
             "chunks": lambda r: helpers.trace_chunks(r, sizes=(150, 2, 64, 131, 7, 300, 3)),
             "mixed": lambda r: helpers.trace_mixed(r, seed=8, max_live=3)}[mode](reqs)
    model = _model(typed, arch, tensors, dtype)
    runner = api.make_runner(typed, model, dtype=dtype, device=DEV, page_size=64,
                             max_tokens=helpers.trace_max_tokens(steps, 64), max_requests=8, max_context=1024)
    slow_before = ops.fallback_count()
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(LENGTHS)
    _check(got, ref, TOL[dtype])
    ops.raise_on_device_error()
    if dtype == "bfloat16":                                   # everything ran on the tensor-core kernels
        assert ops.fallback_count() == slow_before, ops.fallbacks()
    if mode == "mixed":
        assert all(n > g.pool.n_pages for n, g in zip(runner.cache.pages_handed_out(), runner.cache.groups))


@pytest.mark.parametrize("name", list(SIZES))
def test_a_prompt_whose_qkv_product_rotates_and_files_its_result(cases, name):
    """700 and 50 tokens of two requests in one step at head sizes 256 and 128: so many rows that the q,k,v product runs as whole
    tiles on CTA pairs and writes rotated q rows and the pages itself (checked by its launch count); then eight tokens
    one by one, which read those pages.  Every logit against the plain implementation."""
    from kungfu_b200 import api, ops
    cfg, typed, arch, tensors, _, _ = cases(name, "bfloat16")
    toks = {"a": helpers.random_tokens(708, helpers.quiet_vocab(cfg), 31), "b": helpers.random_tokens(50, helpers.quiet_vocab(cfg), 32)}
    ref = {r: plain_gemma2.forward(cfg, tensors, t, device=DEV).float() for r, t in toks.items()}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks["a"][:700], "want": list(range(700))},
                                     {"id": "b", "tokens": toks["b"], "want": list(range(50))}], "end": ["b"]}]
    for i in range(8):
        steps.append({"step": 1 + i, "entries": [{"id": "a", "tokens": [toks["a"][700 + i]], "want": [0]}], "end": ["a"] if i == 7 else []})
    model = _model(typed, arch, tensors, "bfloat16")
    runner = api.make_runner(typed, model, dtype="bfloat16", device=DEV, page_size=64, max_tokens=1024, max_requests=2,
                             max_context=1024, batch=768)
    fused_before = ops.fused_qkv_rope_launches
    got = helpers.run_trace_with_runner(runner, steps)
    assert ops.fused_qkv_rope_launches == fused_before + cfg["num_hidden_layers"]
    assert len(got) == 758
    _check(got, ref, TOL["bfloat16"])
    ops.raise_on_device_error()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_real_window_with_a_prompt_that_crosses_it(dtype):
    """2B widths, window 4,096, 4,200 tokens: whole, and in portions of 512 with the last 8 tokens one by one; the
    windowed group's pool holds window + portion + page tokens, so its pages come back while the prompt is fed."""
    from kungfu_b200 import api, ops
    gc.collect()
    torch.cuda.empty_cache()
    cfg = LONG
    typed, arch, tensors = _weights(cfg, 43, DRAW[dtype])
    toks = helpers.random_tokens(4200, helpers.quiet_vocab(cfg), 77)
    want = list(range(4000, 4200))                          # positions whose keys 0..103 have slid out on layer 0
    ref = plain_gemma2.forward(cfg, tensors, toks, device=DEV).float()
    model = _model(typed, arch, tensors, dtype)
    whole = [{"step": 0, "entries": [{"id": "x", "tokens": toks, "want": want}], "end": ["x"]}]
    cut, at, k = [], 0, 0
    while at < 4192:
        n = min(512, 4192 - at)
        cut.append({"step": k, "entries": [{"id": "x", "tokens": toks[at:at + n], "want": [w - at for w in want if at <= w < at + n]}], "end": []})
        at, k = at + n, k + 1
    for i in range(4192, 4200):
        cut.append({"step": k, "entries": [{"id": "x", "tokens": [toks[i]], "want": [0]}], "end": []})
        k += 1
    cut[-1]["end"] = ["x"]
    for steps, batch in ((whole, 4200), (cut, 512)):
        runner = api.make_runner(typed, model, dtype=dtype, device=DEV, page_size=64, max_requests=1, max_context=8192, batch=batch)
        got = helpers.run_trace_with_runner(runner, steps)
        assert sorted(p for _, p in got) == want
        _check(got, {"x": ref}, TOL[dtype])
        ops.raise_on_device_error()
    pools = {g.window: g.pool.n_pages for g in runner.cache.groups}
    assert pools == {4096: (4096 + 512 + 64) // 64, None: 8192 // 64}
