"""Each part alone, on the GPU, against the plain function of the same part, in 32-bit and in bfloat16;
and greedy generation through the Python entry point."""
import math

import pytest
import torch

import helpers
import plain_gemma2 as pg

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


def rel(a, b):
    a, b = a.detach().float().cpu().double(), b.detach().cpu().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request, tmp_path_factory):
    """A tiny model (configuration B), a runner, and a step context holding two requests: a whole prompt of 21
    tokens and a portion (positions 9..13) of a second request whose first 9 tokens went in an earlier step."""
    from kungfu_b200 import api
    from kungfu_b200.engine import StepEntry
    dtype = request.param
    cfg = helpers.TINY_B
    folder = helpers.write_model(str(tmp_path_factory.mktemp("parts") / "m"), cfg, seed=8, dtype=torch.bfloat16, draw="sharp")
    c, model = api.load_model(folder, dtype=dtype, device=DEV)
    runner = api.make_runner(c, model, dtype=dtype, device=DEV, page_size=8, max_tokens=128, max_requests=4, max_context=128)
    toks_a = helpers.random_tokens(21, helpers.quiet_vocab(cfg), 1)
    toks_b = helpers.random_tokens(14, helpers.quiet_vocab(cfg), 2)
    runner.cache.add_request("a")
    runner.cache.add_request("b")
    runner.step([StepEntry("b", toks_b[:9], [])])
    entries = [StepEntry("a", toks_a, [20]), StepEntry("b", toks_b[9:], [0, 4])]
    for e in entries:
        runner.cache.reserve(e.request, len(e.tokens))
    tensors = helpers.read_tensors(folder)

    class Fresh(dict):
        """`s["ctx"]` rebuilds the step's integer block: a context is valid only until the runner fills the next one."""
        def __getitem__(self, k):
            return runner._fill(entries) if k == "ctx" else dict.__getitem__(self, k)
    return Fresh(dtype=dtype, cfg=cfg, c=c, model=model, runner=runner, tensors=tensors, toks_a=toks_a, toks_b=toks_b,
                 act=torch.float32 if dtype == "float32" else torch.bfloat16)


def test_embedding(setup):
    s = setup
    x = s["model"].embedding.forward(s["ctx"])
    ref = pg.embed(s["tensors"]["model.embed_tokens.weight"], torch.tensor(s["toks_a"] + s["toks_b"][9:]), s["cfg"]["hidden_size"], torch.float64)
    assert x.shape == (26, 96) and rel(x, ref) < 1e-6


def test_norm_and_fused_add(setup):
    s = setup
    norm = s["model"].layers[1].pre_mixer
    post, nxt = s["model"].layers[1].post_mixer, s["model"].layers[1].pre_ffn
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(26, 96, generator=g) * 2).to(DEV)
    w = s["tensors"]["model.layers.1.input_layernorm.weight"]
    eps = s["cfg"]["rms_norm_eps"]
    assert rel(norm.forward(x, s["ctx"], s["act"]), pg.rms_norm(x.cpu().double(), w, eps)) < max(TOL[s["dtype"]] / 3, 1e-6)
    branch = torch.randn(26, 96, generator=g).to(DEV)
    resid = x.clone()
    n = post.add_into(branch, resid, s["ctx"], then=nxt, out_dtype=s["act"])
    r_ref = x.cpu().double() + pg.rms_norm(branch.cpu().double(), s["tensors"]["model.layers.1.post_attention_layernorm.weight"], eps)
    assert rel(resid, r_ref) < 1e-6                                      # the residual stream is 32-bit in both paths
    assert rel(n, pg.rms_norm(r_ref, s["tensors"]["model.layers.1.pre_feedforward_layernorm.weight"], eps)) < max(TOL[s["dtype"]] / 3, 1e-6)


def test_rope_table(setup):
    s = setup
    cos, sin = s["model"].layers[0].mixer.position.rotation(s["ctx"])
    pos = torch.tensor(list(range(21)) + list(range(9, 14)))
    c_ref, s_ref = pg.rope_angles(pos, s["cfg"]["head_dim"], s["cfg"]["rope_theta"], torch.float64)
    assert float((cos.cpu().double() - c_ref).abs().max()) < 1e-5 and float((sin.cpu().double() - s_ref).abs().max()) < 1e-5


@pytest.mark.parametrize("layer", [0, 1])
def test_attention_mixer(setup, layer):
    """The mixer on a windowed (layer 0) and a global (layer 1) layer: request a whole, request b continuing from
    its cache, compared with whole-sequence attention of the plain implementation.  Sharp query and key matrices and
    input rows of spread 2 put the scores at and beyond the softcap of 20, so that the cap, the scale and the rotation
    base all move the result by far more than the tolerance (tests/test_oracle_sensitivity.py)."""
    s = setup
    cfg, t = s["cfg"], s["tensors"]
    mixer = s["model"].layers[layer].mixer
    g = torch.Generator().manual_seed(4 + layer)
    xa = torch.randn(21, 96, generator=g) * 2
    xb = torch.randn(14, 96, generator=g) * 2
    if s["dtype"] == "bfloat16":
        xa, xb = xa.bfloat16().float(), xb.bfloat16().float()
    p = f"model.layers.{layer}.self_attn."
    kw = dict(n_heads=6, n_kv_heads=2, head_dim=32, scale=1 / math.sqrt(24), cap=20.0, window=16 if layer == 0 else None, base=1e6)
    ref_a = pg.attention(xa.double(), t[p + "q_proj.weight"], t[p + "k_proj.weight"], t[p + "v_proj.weight"], t[p + "o_proj.weight"], **kw)
    ref_b = pg.attention(xb.double(), t[p + "q_proj.weight"], t[p + "k_proj.weight"], t[p + "v_proj.weight"], t[p + "o_proj.weight"], **kw)
    runner = s["runner"]
    # fill request b's first 9 positions of this layer's cache with this test's inputs, through the mixer itself
    from kungfu_b200.engine import StepEntry
    runner.cache.add_request("tmp")
    runner.cache.reserve("tmp", 9)
    ctx0 = runner._fill([StepEntry("tmp", [0] * 9, [])])
    view = runner.cache.view(layer, True)
    mixer.forward(xb[:9].to(DEV).to(s["act"]), ctx0, view)
    # copy tmp's pages over b's (same positions 0..8): page ids differ, contents are what matter
    g_idx = runner.cache.group_of(layer)
    for pt, pb in zip(runner.cache.block_table(g_idx, "tmp"), runner.cache.block_table(g_idx, "b")):
        if pt >= 0 and pb >= 0:
            view.pages[pb] = view.pages[pt]
    runner.cache.cancel_reservation("tmp")
    runner.cache.release("tmp")
    x = torch.cat([xa, xb[9:]]).to(DEV).to(s["act"])
    y = mixer.forward(x, s["ctx"], view)
    assert y.dtype == torch.float32 and y.shape == (26, 96)
    assert rel(y[:21], ref_a) < TOL[s["dtype"]]
    assert rel(y[21:], ref_b[9:]) < TOL[s["dtype"]]


def test_feed_forward(setup):
    s = setup
    ffn = s["model"].layers[2].ffn
    g = torch.Generator().manual_seed(6)
    x = torch.randn(26, 96, generator=g)
    if s["dtype"] == "bfloat16":
        x = x.bfloat16().float()
    t = s["tensors"]
    ref = pg.feed_forward(x.double(), t["model.layers.2.mlp.gate_proj.weight"], t["model.layers.2.mlp.up_proj.weight"],
                          t["model.layers.2.mlp.down_proj.weight"], "gelu_pytorch_tanh")
    y = ffn.forward(x.to(DEV).to(s["act"]), s["ctx"])
    assert y.dtype == torch.float32 and rel(y, ref) < TOL[s["dtype"]]


def test_head_only_scores_wanted_rows(setup):
    s = setup
    g = torch.Generator().manual_seed(7)
    x = torch.randn(26, 96, generator=g)
    t = s["tensors"]
    logits = s["model"].head.forward(x.to(DEV), s["ctx"])
    n = pg.rms_norm(x.double()[[20, 21, 25]], t["model.norm.weight"], s["cfg"]["rms_norm_eps"])
    ref = pg.softcap(n @ t["model.embed_tokens.weight"].double().T, 15.0)
    assert logits.shape == (3, 1000) and rel(logits, ref) < TOL[s["dtype"]]


@pytest.mark.parametrize("name", ["A", "B"])
def test_generate_through_the_entry_point(tmp_path, name):
    """Greedy ids from `Engine.generate` (host ids in, host ids out): identical to the plain implementation in 32-bit;
    in bfloat16 every chosen token must be the plain implementation's best or within the bfloat16 bound of it."""
    from kungfu_b200 import Engine
    from kungfu_b200.sampling import Sampling
    cfg = {"A": helpers.TINY_A, "B": helpers.TINY_B}[name]
    lengths = {"A": (5, 17, 23), "B": (1, 31, 40)}[name]
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=12, dtype=torch.bfloat16)
    tensors = helpers.read_tensors(folder)
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 40 + n) for n in lengths]
    want = [pg.greedy(cfg, tensors, p, 8) for p in prompts]
    eng = Engine(folder, dtype="float32", device=DEV, ctx=cfg["max_position_embeddings"], batch=16, parallel=4, page_size=8)
    assert eng.generate(prompts, Sampling(temperature=0.0), max_tokens=8) == want
    eng16 = Engine(folder, dtype="bfloat16", device=DEV, ctx=cfg["max_position_embeddings"], batch=16, parallel=4, page_size=8)
    got = eng16.generate(prompts, Sampling(temperature=0.0), max_tokens=8)
    for p, out in zip(prompts, got):
        logits = pg.forward(cfg, tensors, p + out).float()
        scale = float(logits.abs().max())
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) <= 2 * 2e-2 * scale
    # decode steps launched before the step before them was read (the ids stay on the device) against steps read at once,
    # with an end-of-sequence id that ends one request early and enough steps for the replayed graphs to be in use
    long = [pg.greedy(cfg, tensors, p, 20) for p in prompts]
    eos = long[1][9]
    cut = [seq[:seq.index(eos) + 1] if eos in seq else seq for seq in long]
    for pipeline in (True, False):
        e = Engine(folder, dtype="float32", device=DEV, ctx=cfg["max_position_embeddings"], batch=16, parallel=4, page_size=8,
                   pipeline=pipeline)
        assert e.generate(prompts, Sampling(temperature=0.0), max_tokens=20, eos=[eos]) == cut
        assert [e.finish_reason(i) for i in range(len(prompts))] == ["eos" if eos in seq else "length" for seq in long]
        assert e.runner.cache.n_live == 0 and e.idle
    # temperature sampling in 32-bit: the ids of the plain sampler applied to the plain model's logits, same seeds
    import plain_sampler
    for rules in (dict(temperature=0.8, top_k=0, top_p=1.0), dict(temperature=1.2, top_k=40, top_p=0.9, repeat_penalty=1.3)):
        want_s = []
        for i, p in enumerate(prompts):
            rng, out = plain_sampler.Rng(5 + i), []
            for _ in range(10):
                row = pg.forward(cfg, tensors, p + out)[-1].float().numpy()
                out.append(plain_sampler.sample(row, recent=out, rng=rng, **rules)[0])
            want_s.append(out)
        e = Engine(folder, dtype="float32", device=DEV, ctx=cfg["max_position_embeddings"], parallel=4, page_size=8)
        assert e.generate(prompts, Sampling(**rules), max_tokens=10, seed=5) == want_s, rules
    # temperature sampling with a fixed seed is reproducible and differs between seeds
    s = Sampling(temperature=0.8, top_k=0, top_p=1.0)
    a = Engine(folder, dtype="float32", device=DEV, ctx=cfg["max_position_embeddings"], parallel=4, page_size=8).generate(prompts, s, max_tokens=12, seed=5)
    b = Engine(folder, dtype="float32", device=DEV, ctx=cfg["max_position_embeddings"], parallel=4, page_size=8).generate(prompts, s, max_tokens=12, seed=5)
    c = Engine(folder, dtype="float32", device=DEV, ctx=cfg["max_position_embeddings"], parallel=4, page_size=8).generate(prompts, s, max_tokens=12, seed=6)
    assert a == b and a != c


def test_mixed_steps_replayed_from_graphs_give_the_plain_tokens(tmp_path):
    """Long prompts fed under a small token budget while other requests decode: the scheduler's steps (decode rows
    beside a prompt portion) repeat in shape and are replayed from CUDA graphs under a padded layout.  Greedy ids in
    32-bit equal the plain implementation's, and equal the engine that launches every step eagerly."""
    from kungfu_b200 import Engine, ops
    from kungfu_b200.sampling import Sampling
    cfg = helpers.TINY_E
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=14, dtype=torch.bfloat16)
    tensors = helpers.read_tensors(folder)
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 60 + n) for n in (40, 700, 2, 513, 330)]
    want = [pg.greedy(cfg, tensors, p, 6) for p in prompts]
    outs = {}
    for graphs in (True, False):
        e = Engine(folder, dtype="float32", device=DEV, ctx=1024, batch=96, parallel=4, page_size=64, cuda_graphs=graphs)
        outs[graphs] = e.generate(prompts, Sampling(temperature=0.0), max_tokens=6, ignore_eos=True)
        ops.raise_on_device_error()
        mixed = [k for k, st in e.runner._graphs.items() if isinstance(k, tuple) and isinstance(k[1], tuple) and st["graph"] is not None]
        assert bool(mixed) == graphs, list(e.runner._graphs)
        assert e.runner.cache.n_live == 0
    assert outs[True] == want and outs[False] == want
    # bfloat16 through the same path: every token within the bfloat16 bound of the plain model's best, given the engine's own tokens
    e = Engine(folder, dtype="bfloat16", device=DEV, ctx=1024, batch=96, parallel=4, page_size=64)
    got = e.generate(prompts, Sampling(temperature=0.0), max_tokens=6, ignore_eos=True)
    for p, out in zip(prompts, got):
        logits = pg.forward(cfg, tensors, p + out).float()
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) <= 2 * 2e-2 * float(logits.abs().max())


def test_warm_up_captures_the_decode_graphs(tmp_path):
    """After `Engine.warm_up()` the decode steps of every batch bucket replay from graphs; what a request generates
    afterwards is what the plain implementation gives, and the warm-up leaves no request, page or state behind."""
    from kungfu_b200 import Engine
    from kungfu_b200.sampling import Sampling
    cfg = helpers.TINY_A
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=6, dtype=torch.bfloat16)
    tensors = helpers.read_tensors(folder)
    e = Engine(folder, dtype="float32", device=DEV, ctx=64, batch=32, parallel=4, page_size=4)
    e.warm_up()
    assert e.idle and e.runner.cache.n_live == 0
    assert e.runner.cache.free_pages() == [g.pool.n_pages for g in e.runner.cache.groups]
    captured = {k[1] for k, st in e.runner._graphs.items() if isinstance(k, tuple) and k[0] == "sample" and st["graph"] is not None}
    assert {1, 2, 4} <= captured
    prompt = helpers.random_tokens(9, cfg["vocab_size"], 5)
    assert e.generate([prompt], Sampling(temperature=0.0), max_tokens=6, ignore_eos=True) == [pg.greedy(cfg, tensors, prompt, 6)]


def test_many_requests_of_random_lengths_under_a_tight_cache(tmp_path):
    """Two dozen requests of random prompt lengths through one engine with six state slots, a budget of 96 rows and a
    cache of forty pages of 16 tokens: admission in waves, prompts fed in portions beside decoding
    requests (steps replayed from graphs, decode rows padded in the budget), pages given back and used again, requests
    preempted and recomputed.  Greedy ids in 32-bit equal the plain implementation's for every request, with and
    without graphs, and nothing is left behind."""
    import random
    from kungfu_b200 import Engine, ops
    from kungfu_b200.sampling import Sampling
    cfg = helpers.TINY_E
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=23, dtype=torch.bfloat16)
    tensors = helpers.read_tensors(folder)
    rnd = random.Random(5)
    lengths = [rnd.choice([1, 2, 3, 7, 30, 63, 64, 65, 100, 129, 200, 260]) for _ in range(24)]
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 300 + i) for i, n in enumerate(lengths)]
    want = [pg.greedy(cfg, tensors, p, 20) for p in prompts]
    for graphs in (True, False):
        e = Engine(folder, dtype="float32", device=DEV, ctx=512, batch=96, parallel=6, page_size=16, cuda_graphs=graphs,
                   max_tokens_in_cache=640)
        got = e.generate(prompts, Sampling(temperature=0.0), max_tokens=20, ignore_eos=True)
        ops.raise_on_device_error()
        assert got == want, [i for i, (a, b) in enumerate(zip(got, want)) if a != b]
        assert e.runner.cache.n_live == 0 and e.idle
        assert e.runner.cache.free_pages() == [g.pool.n_pages for g in e.runner.cache.groups]
        handed = e.runner.cache.pages_handed_out()
        assert all(h > g.pool.n_pages for h, g in zip(handed, e.runner.cache.groups)), "pages were used again"
        assert e.scheduler.n_preemptions > 0


def test_preemption_and_recompute_on_the_device(tmp_path):
    """Pages run out while three requests decode: the scheduler preempts the one admitted last, which is recomputed later
    from its prompt and the tokens it had produced.  The engine must read the tokens of the step in flight before it
    plans such a step (a preempted request's tokens become a prompt), and the ids, greedy and sampled, must equal those
    of an engine with room, in 32-bit those of the plain implementation."""
    import plain_sampler
    from kungfu_b200 import Engine, ops
    from kungfu_b200.sampling import Sampling
    cfg = helpers.TINY_A
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=4, dtype=torch.bfloat16)
    tensors = helpers.read_tensors(folder)
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 90 + n) for n in (5, 7, 6)]
    want = [pg.greedy(cfg, tensors, p, 8) for p in prompts]
    rules = dict(temperature=0.9, top_k=30, top_p=0.95, repeat_penalty=1.2)
    want_s = []
    for i, p in enumerate(prompts):
        rng, out = plain_sampler.Rng(7 + i), []
        for _ in range(8):
            row = pg.forward(cfg, tensors, p + out)[-1].float().numpy()
            out.append(plain_sampler.sample(row, recent=out, rng=rng, **rules)[0])
        want_s.append(out)
    for pipeline in (True, False):
        tight = Engine(folder, dtype="float32", device=DEV, ctx=64, batch=16, parallel=4, page_size=4, max_tokens_in_cache=36,
                       pipeline=pipeline)
        assert tight.generate(prompts, Sampling(temperature=0.0), max_tokens=8) == want
        assert tight.scheduler.n_preemptions > 0 and tight.runner.cache.n_live == 0
        tight = Engine(folder, dtype="float32", device=DEV, ctx=64, batch=16, parallel=4, page_size=4, max_tokens_in_cache=36,
                       pipeline=pipeline)
        assert tight.generate(prompts, Sampling(**rules), max_tokens=8, seed=7) == want_s
        assert tight.scheduler.n_preemptions > 0
        assert tight.runner.cache.free_pages() == [g.pool.n_pages for g in tight.runner.cache.groups]
    ops.raise_on_device_error()
