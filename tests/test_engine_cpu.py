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


def _engine(folder, cfg_dict, *, page, pool_tokens, batch, parallel):
    from kungfu_b200.engine.engine import Engine
    cfg, model = api.load_model(folder, dtype="float32", device="cpu")
    runner = api.make_runner(cfg, model, dtype="float32", device="cpu", page_size=page, max_tokens=pool_tokens,
                             max_requests=parallel, max_context=cfg_dict["max_position_embeddings"])
    return Engine(runner=runner, batch=batch, parallel=parallel)


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
