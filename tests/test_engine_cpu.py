"""The engine's host logic against the plain implementation, kernels replaced by the CPU stand-in.

Covers the same four ways of cutting the work that the GPU tests cover: whole, most of it then token
by token, portions of changing size, and mixed batches with so few pages that they are used again."""
import pytest
import torch

import helpers
import plain_gemma2
from kungfu_b200 import api


def _runner(folder, cfg_dict, page_size, max_tokens):
    cfg, model = api.load_model(folder, dtype="float32", device="cpu")
    return api.make_runner(cfg, model, dtype="float32", device="cpu", page_size=page_size, max_tokens=max_tokens,
                           max_requests=8, max_context=cfg_dict["max_position_embeddings"])


def _reference(folder, cfg_dict, reqs):
    tensors = helpers.read_tensors(folder)
    return {rid: plain_gemma2.forward(cfg_dict, tensors, toks).float() for rid, toks in reqs.items()}


def _compare(got, ref, tol):
    assert got, "no logits came back"
    worst = 0.0
    for (rid, pos), row in got.items():
        worst = max(worst, float((row - ref[rid][pos]).abs().max()))
    assert worst < tol, f"max abs logit difference {worst}"


CASES = [(helpers.TINY_A, [5, 17, 23, 40], 4), (helpers.TINY_B, [1, 31, 40, 70], 8), (helpers.TINY_C, [3, 50, 64, 29, 33], 16),
         (helpers.TINY_D, [2, 40, 17, 90], 4)]


@pytest.mark.parametrize("cfg_dict,lengths,page", CASES, ids=["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_cpu_modes_match_plain(tmp_path, cpu_ops, cfg_dict, lengths, page, mode):
    folder = helpers.write_model(str(tmp_path / "m"), cfg_dict, seed=11, dtype=torch.float32)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg_dict["vocab_size"], 100 + i) for i, n in enumerate(lengths)}
    ref = _reference(folder, cfg_dict, reqs)
    steps = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_decode_tail(r, 12),
             "chunks": helpers.trace_chunks, "mixed": lambda r: helpers.trace_mixed(r, seed=3)}[mode](reqs)
    runner = _runner(folder, cfg_dict, page, helpers.trace_max_tokens(steps, page))
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(lengths)
    _compare(got, ref, 2e-4)
    assert runner.cache.n_live == 0
    assert all(f == g.pool.n_pages for f, g in zip(runner.cache.free_pages(), runner.cache.groups))


def _engine(folder, cfg_dict, *, page, pool_tokens, batch, parallel, pipeline=True):
    from kungfu_b200.engine.engine import Engine
    cfg, model = api.load_model(folder, dtype="float32", device="cpu")
    runner = api.make_runner(cfg, model, dtype="float32", device="cpu", page_size=page, max_tokens=pool_tokens,
                             max_requests=parallel, max_context=cfg_dict["max_position_embeddings"])
    return Engine(runner=runner, batch=batch, parallel=parallel, pipeline=pipeline)


def test_generate_matches_plain_greedy_and_survives_preemption(tmp_path, cpu_ops):
    """Greedy ids through the scheduler equal the plain implementation's, also when pages run out and a request
    is preempted and recomputed."""
    from kungfu_b200.sampling import Sampling
    cfg_dict = helpers.TINY_A
    folder = helpers.write_model(str(tmp_path / "m"), cfg_dict, seed=4, dtype=torch.float32)
    tensors = helpers.read_tensors(folder)
    prompts = [helpers.random_tokens(n, cfg_dict["vocab_size"], 50 + n) for n in (5, 17, 23)]
    want = [plain_gemma2.greedy(cfg_dict, tensors, p, 8) for p in prompts]
    roomy = _engine(folder, cfg_dict, page=4, pool_tokens=256, batch=16, parallel=4)
    assert roomy.generate(prompts, Sampling(temperature=0.0), max_tokens=8) == want
    assert roomy.scheduler.n_preemptions == 0
    # all three are admitted (2 pages each) and then outgrow a pool of 9 pages: someone has to be preempted
    short = [helpers.random_tokens(n, cfg_dict["vocab_size"], 90 + n) for n in (5, 7, 6)]
    want_short = [plain_gemma2.greedy(cfg_dict, tensors, p, 8) for p in short]
    tight = _engine(folder, cfg_dict, page=4, pool_tokens=36, batch=16, parallel=4)
    assert tight.generate(short, Sampling(temperature=0.0), max_tokens=8) == want_short
    assert tight.scheduler.n_preemptions > 0
    assert tight.runner.cache.n_live == 0 and tight.runner.cache.free_pages() == [9, 9]


def _plain_generate(cfg_dict, tensors, prompt, n_new, rules, seed):
    """Token by token with the plain model and the plain sampler (whole sequence recomputed each step)."""
    import plain_sampler
    rng = plain_sampler.Rng(seed)
    out = []
    for _ in range(n_new):
        row = plain_gemma2.forward(cfg_dict, tensors, list(prompt) + out)[-1].float().numpy()
        tok, _margin = plain_sampler.sample(row, recent=out, rng=rng, **rules)
        out.append(tok)
    return out


def test_sampled_tokens_equal_the_plain_sampler_on_plain_logits_and_survive_preemption(tmp_path, cpu_ops):
    """Temperature, top-k beyond and within the candidates, top-p and a repeat penalty through the scheduler: the ids
    are those of the plain sampler applied to the plain model's logits with the same seed, request by request, with
    and without the pipeline, and also when a request is preempted and recomputed (its generator goes on where it was)."""
    from kungfu_b200.sampling import Sampling
    cfg_dict = helpers.TINY_A
    folder = helpers.write_model(str(tmp_path / "m"), cfg_dict, seed=4, dtype=torch.float32)
    tensors = helpers.read_tensors(folder)
    prompts = [helpers.random_tokens(n, cfg_dict["vocab_size"], 90 + n) for n in (5, 7, 6)]
    for rules in (dict(temperature=0.8, top_k=0, top_p=1.0), dict(temperature=1.1, top_k=40, top_p=0.9, repeat_penalty=1.3),
                  dict(temperature=0.0, repeat_penalty=1.5, repeat_window=4)):
        want = [_plain_generate(cfg_dict, tensors, p, 8, rules, seed=9 + i) for i, p in enumerate(prompts)]
        for pipeline in (True, False):
            roomy = _engine(folder, cfg_dict, page=4, pool_tokens=256, batch=16, parallel=4, pipeline=pipeline)
            assert roomy.generate(prompts, Sampling(**rules), max_tokens=8, seed=9) == want, (rules, pipeline)
        tight = _engine(folder, cfg_dict, page=4, pool_tokens=36, batch=16, parallel=4)
        assert tight.generate(prompts, Sampling(**rules), max_tokens=8, seed=9) == want, rules
        assert tight.scheduler.n_preemptions > 0


def test_tokens_read_one_step_late_end_requests_where_they_should(tmp_path, cpu_ops):
    """Greedy decode steps are launched before the step before them has been read.  A request that an end-of-sequence id
    ends has then run one step too many: its output must still end with that id, with reason eos, the others go on to
    their length, everything is given back, and the result equals the engine that reads every step at once."""
    from kungfu_b200.sampling import Sampling
    cfg_dict = helpers.TINY_A
    folder = helpers.write_model(str(tmp_path / "m"), cfg_dict, seed=4, dtype=torch.float32)
    tensors = helpers.read_tensors(folder)
    prompts = [helpers.random_tokens(n, cfg_dict["vocab_size"], 50 + n) for n in (5, 17, 23)]
    full = [plain_gemma2.greedy(cfg_dict, tensors, p, 12) for p in prompts]
    eos = full[1][5]                                       # ends the second request at its sixth token at the latest
    want, why = [], []
    for seq in full:
        cut = seq.index(eos) + 1 if eos in seq else len(seq)
        want.append(seq[:cut])
        why.append("eos" if eos in seq else "length")
    assert "eos" in why and len(want[1]) <= 6
    for pipeline in (True, False):
        e = _engine(folder, cfg_dict, page=4, pool_tokens=256, batch=16, parallel=4, pipeline=pipeline)
        ids = [e.add_request(p, Sampling(temperature=0.0), max_tokens=12, eos=[eos]) for p in prompts]
        seen = {i: [] for i in ids}
        ended = {}
        late = 0
        while not e.idle:
            n_running = len(e.scheduler.running)
            ev = e.step()
            late += int(e._inflight is not None)
            for rid, tok, reason in ev:
                assert rid not in ended, "a token after the request's end"
                seen[rid].append(tok)
                if reason is not None:
                    ended[rid] = reason
        assert [seen[i] for i in ids] == want and [ended[i] for i in ids] == why
        assert [e.requests[i].output for i in ids] == want and [e.finish_reason(i) for i in ids] == why
        assert (late > 0) == pipeline
        assert e.runner.cache.n_live == 0 and e.runner.cache.free_pages() == [64, 64]
    # the last token of a request that ends by its length arrives with flush() at the latest
    e = _engine(folder, cfg_dict, page=4, pool_tokens=256, batch=16, parallel=4)
    rid = e.add_request(prompts[0], Sampling(temperature=0.0), max_tokens=3)
    got = []
    for _ in range(3):
        got += [tok for _rid, tok, _r in e.step()]
    assert e.scheduler.idle and not e.idle and len(got) == 2      # counted out, but its last token is still on its way
    got += [tok for _rid, tok, _r in e.flush()]
    assert got == full[0][:3] and e.idle and e.finish_reason(rid) == "length"


def test_requests_that_arrive_or_are_cancelled_while_a_step_is_in_flight(tmp_path, cpu_ops):
    """A request added while decode steps are in flight joins with a prompt portion beside the others' tokens (the
    engine reads what is in flight first); one that is cancelled keeps the tokens it had; the others are not disturbed."""
    from kungfu_b200.sampling import Sampling
    cfg_dict = helpers.TINY_B
    folder = helpers.write_model(str(tmp_path / "m"), cfg_dict, seed=8, dtype=torch.float32)
    tensors = helpers.read_tensors(folder)
    prompts = [helpers.random_tokens(n, cfg_dict["vocab_size"], 20 + n) for n in (9, 30, 14)]
    want = [plain_gemma2.greedy(cfg_dict, tensors, p, 10) for p in prompts]
    e = _engine(folder, cfg_dict, page=8, pool_tokens=512, batch=16, parallel=4)
    a = e.add_request(prompts[0], Sampling(temperature=0.0), max_tokens=10)
    b = e.add_request(prompts[1], Sampling(temperature=0.0), max_tokens=10)
    events = []
    for _ in range(6):
        events += e.step()
    assert e._inflight is not None
    c = e.add_request(prompts[2], Sampling(temperature=0.0), max_tokens=10)      # joins while a step is in flight
    events += e.step()
    events += e.step()
    assert e._inflight is not None
    events += e.cancel(b)                        # hands out the tokens of the step that was in flight, then the cancellation
    kept = list(e.requests[b].output)
    assert e.finish_reason(b) == "cancelled" and 0 < len(kept) < 10 and kept == want[1][:len(kept)]
    while not e.idle:
        events += e.step()
    events += e.flush()
    assert e.requests[a].output == want[0] and e.requests[c].output == want[2] and e.requests[b].output == kept
    assert e.runner.cache.n_live == 0
    # a caller that only reads events sees every token of every request once, in order, and one finish reason each
    for rid in (a, b, c):
        mine = [(tok, reason) for r, tok, reason in events if r == rid]
        assert [tok for tok, _ in mine if tok is not None] == e.requests[rid].output
        reasons = [reason for _, reason in mine if reason is not None]
        assert reasons == [e.finish_reason(rid)], (rid, reasons)


def test_temperature_sampling_is_reproducible(tmp_path, cpu_ops):
    from kungfu_b200.sampling import Sampling
    cfg_dict = helpers.TINY_B
    folder = helpers.write_model(str(tmp_path / "m"), cfg_dict, seed=6, dtype=torch.float32)
    prompts = [helpers.random_tokens(n, cfg_dict["vocab_size"], 70 + n) for n in (1, 31)]
    outs = []
    for _ in range(2):
        e = _engine(folder, cfg_dict, page=8, pool_tokens=256, batch=7, parallel=4)
        outs.append(e.generate(prompts, Sampling(temperature=0.8, top_k=0, top_p=1.0), max_tokens=12, seed=9))
    assert outs[0] == outs[1] and all(len(o) == 12 for o in outs[0])
    e = _engine(folder, cfg_dict, page=8, pool_tokens=256, batch=7, parallel=4)
    other = e.generate(prompts, Sampling(temperature=0.8, top_k=0, top_p=1.0), max_tokens=12, seed=10)
    assert other != outs[0]


def test_a_step_that_fails_gives_its_pages_back(tmp_path, cpu_ops):
    """A step that raises after its pages were reserved (here: a kernel error in the pass) leaves the cache as it was:
    no reservation stays behind, and the same step runs afterwards."""
    from kungfu_b200 import ops
    from kungfu_b200.engine import StepEntry
    cfg_dict = helpers.TINY_A
    folder = helpers.write_model(str(tmp_path / "m"), cfg_dict, seed=3, dtype=torch.float32)
    runner = _runner(folder, cfg_dict, 4, 64)
    toks = helpers.random_tokens(13, cfg_dict["vocab_size"], 5)
    runner.cache.add_request("x")
    free_before = runner.cache.free_pages()
    impl = ops._override
    real_linear = impl.linear

    def broken(*a, **k):
        raise ops.KernelError("injected")
    impl.linear = broken
    try:
        with pytest.raises(ops.KernelError):
            runner.step([StepEntry("x", toks, [12])])
    finally:
        impl.linear = real_linear
    assert runner.cache.free_pages() == free_before and runner.cache.length("x") == 0
    runner.cache.check()
    from kungfu_b200.engine.step import StepError
    with pytest.raises(StepError):                 # refused before anything is reserved
        runner.step([StepEntry("x", toks[:2], [1])], feedback=torch.zeros(1, dtype=torch.int32))
    assert runner.cache.free_pages() == free_before
    logits = runner.step([StepEntry("x", toks, [12])])
    ref = _reference(folder, cfg_dict, {"x": toks})["x"]
    assert float((logits[0].float().cpu() - ref[12]).abs().max()) < 2e-4
    runner.cache.release("x")
    assert runner.cache.free_pages() == [g.pool.n_pages for g in runner.cache.groups]


def test_padded_mixed_layout_gives_the_same_logits_as_the_natural_one(tmp_path, cpu_ops):
    """The layout that mixed steps are replayed under on the GPU (decode rows first, then prompt rows, every count
    rounded up to a bucket, unused rows and tiles empty): its sections are what the kernels expect, and the model run
    over it yields, at the wanted places, the logits of the same step laid out as it is."""
    from kungfu_b200.engine import StepEntry
    cfg_dict = helpers.TINY_B
    folder = helpers.write_model(str(tmp_path / "m"), cfg_dict, seed=6, dtype=torch.float32)
    toks = {r: helpers.random_tokens(n, cfg_dict["vocab_size"], 30 + i) for i, (r, n) in enumerate((("a", 20), ("b", 9), ("c", 100), ("d", 31)))}

    def make():
        runner = _runner(folder, cfg_dict, 8, 512)
        for r in toks:
            runner.cache.add_request(r)
        runner.step([StepEntry("a", toks["a"][:19], []), StepEntry("b", toks["b"][:8], []), StepEntry("c", toks["c"][:30], [])])
        return runner
    entries = [StepEntry("a", [toks["a"][19]], [0]), StepEntry("b", [toks["b"][8]], [0]),
               StepEntry("c", toks["c"][30:], [69]), StepEntry("d", toks["d"], [])]
    natural = make()
    want = natural.step(entries).clone()
    padded = make()
    for e in entries:
        padded.cache.reserve(e.request, len(e.tokens))
    bucket = ("mixed", 4, 128, 2)
    ctx = padded._fill(entries, bucket)
    assert (ctx.n_rows, ctx.n_reqs, ctx.n_logits, ctx.n_dec_rows, ctx.n_pre_rows) == (132, 6, 6, 4, 128)
    assert ctx.n_tiles == 128 // 64 + 2 and ctx.n_wide == 128 // 128 + 2
    assert ctx.row_req.tolist() == [0, 1, -1, -1] + [4] * 70 + [5] * 31 + [-1] * 27
    assert ctx.positions.tolist()[:2] == [19, 8] and ctx.positions.tolist()[4:7] == [30, 31, 32] and ctx.positions.tolist()[74] == 0
    assert ctx.dec_rows.tolist()[:4] == [0, 1, 2, 3] and ctx.pre_rows.tolist()[:128] == list(range(4, 132))
    assert ctx.tile_row0.tolist()[:4] == [4, 68, 74, 4] and ctx.tile_nrows.tolist()[:4] == [64, 6, 31, 0]
    assert ctx.wide_row0.tolist()[:3] == [4, 74, 4] and ctx.wide_nrows.tolist()[:3] == [70, 31, 0]
    assert ctx.logit_rows.tolist() == [0, 1, 0, 0, 73, 0] and ctx.logit_req.tolist() == [0, 1, -1, -1, 4, -1]
    assert ctx.req_n_rows.tolist() == [1, 1, 0, 0, 70, 31] and ctx.req_kv_len.tolist() == [20, 9, 0, 0, 100, 31]
    assert padded._logit_index(entries, bucket) == [0, 1, 4]
    logits = padded.model.forward(ctx)
    got = logits[padded._logit_index(entries, bucket)]
    assert float((got - want).abs().max()) < 1e-5
    # a step that does not fit the layout is refused, not squeezed in
    from kungfu_b200.engine.step import StepError
    for e in entries:
        padded.cache.cancel_reservation(e.request)
    with pytest.raises(StepError, match="does not fit its layout"):
        padded._fill(entries, ("mixed", 1, 128, 2))
    with pytest.raises(StepError, match="does not fit its layout"):
        padded._fill([entries[2], entries[0]], ("mixed", 4, 128, 2))       # a prompt portion before a decode row
