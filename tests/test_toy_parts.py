"""Parts that are not Gemma 2's, defined here, registered, built and stepped without a change to the framework.

* `RunningMean`: a mixer with a state of its own (a fixed-size per-request state: the sum of its inputs and their
  count); token i gets W . mean(x_0..x_i).
* `RoutedFfn`: a feed-forward with routing (two experts, the router's top choice, 32-bit router logits).
* `ClockHands`: another position encoding (only the first half of a head is rotated, hand i turns by position / (i + 2):
  no power law, no base), handed to the framework's attention in place of its rotary embedding.
* a toy architecture that mixes these with the framework's paged attention layer by layer, names one layer twice in
  its schedule and lets one call read the cache another call wrote.
The toy model is compared with a whole-sequence computation written here, for whole prompts, portions and
single tokens, several requests per step.
"""
from dataclasses import dataclass

import pytest
import torch

import helpers

DEV = "cuda:0"


def _define():
    from kungfu_b200 import registry
    from kungfu_b200.config.base import KeyReader
    from kungfu_b200.parts import (DecoderModel, Embedding, FeedForward, FixedState, LayerCall, LmHead, Mixer,
                                   PagedAttention, PositionEncoding, RmsNorm, SandwichBlock, known,
                                   register_feed_forward, register_mixer, register_position)
    from kungfu_b200.weights.store import TensorSpec

    class RunningMean(Mixer):
        graph_safe = False                       # loops over the step's requests on the host

        def __init__(self, w):
            self.w = w                           # [width, width]
            self.width = w.shape[0]

        def state_need(self):
            return FixedState((self.width + 1,), torch.float32)      # running sum and count

        def forward(self, x, ctx, cache):
            out = torch.empty(x.shape[0], self.width, dtype=torch.float32, device=x.device)
            starts, counts, slots = ctx.host["req_row_start"], ctx.host["req_n_rows"], ctx.host["req_state_slot"]
            for r0, n, slot in zip(starts, counts, slots):
                st = cache.state[int(slot)]
                run = torch.cumsum(x[r0:r0 + n].float(), dim=0) + st[:-1]
                cnt = st[-1] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[r0:r0 + n] = (run / cnt[:, None]) @ self.w.float().T
                if cache.writes:
                    st[:-1] = run[-1]
                    st[-1] = cnt[-1]
            return out

    class RoutedFfn(FeedForward):
        graph_safe = False

        def __init__(self, router, w_in, w_out):
            self.router, self.w_in, self.w_out = router, w_in, w_out     # [2, H], [2, I, H], [2, H, I]

        def forward(self, x, ctx):
            xf = x.float()
            choice = torch.argmax(xf @ self.router.float().T, dim=-1)
            y = torch.zeros(x.shape[0], self.w_out.shape[1], dtype=torch.float32, device=x.device)
            for e in range(2):
                sel = choice == e
                y[sel] = torch.relu(xf[sel] @ self.w_in[e].float().T) @ self.w_out[e].float().T
            return y

    class ClockHands(PositionEncoding):
        graph_safe = False

        def __init__(self, head_dim, device):
            self.turn = (1.0 / torch.arange(2, 2 + head_dim // 4, dtype=torch.float32)).to(device)   # rotates head_dim / 2

        def rotation(self, ctx):
            angle = ctx.positions[:ctx.n_rows].to(torch.float32)[:, None] * self.turn[None, :]
            return torch.cos(angle).contiguous(), torch.sin(angle).contiguous()

    if "running_mean" not in known("mixer"):
        register_mixer("running_mean", RunningMean)
        register_feed_forward("routed", RoutedFfn)
        register_position("clock_hands", ClockHands)

    @dataclass(frozen=True)
    class ToyConfig:
        architecture: str
        hidden_size: int
        intermediate_size: int
        vocab_size: int
        num_attention_heads: int
        head_dim: int
        rms_norm_eps: float
        max_position_embeddings: int

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            k = KeyReader(raw, where)
            return cls(k.list("architectures")[0], k.int("hidden_size"), k.int("intermediate_size"), k.int("vocab_size"),
                       k.int("num_attention_heads"), k.int("head_dim"), k.float("rms_norm_eps"),
                       k.int("max_position_embeddings"))

        def to_dict(self):
            return {"architectures": [self.architecture], "hidden_size": self.hidden_size,
                    "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
                    "num_attention_heads": self.num_attention_heads, "head_dim": self.head_dim,
                    "rms_norm_eps": self.rms_norm_eps, "max_position_embeddings": self.max_position_embeddings}

    def specs(c):
        H, I, q = c.hidden_size, c.intermediate_size, c.num_attention_heads * c.head_dim
        out = [TensorSpec("emb", (c.vocab_size, H)), TensorSpec("final_norm", (H,), 0.1, "norm"),
               TensorSpec("l0.mean_w", (H, H), 0.2), TensorSpec("l1.wqkv", (3 * q, H), 0.2), TensorSpec("l1.wo", (H, q), 0.2)]
        for l in range(2):
            out += [TensorSpec(f"l{l}.n1", (H,), 0.1, "norm"), TensorSpec(f"l{l}.n2", (H,), 0.1, "norm"),
                    TensorSpec(f"l{l}.router", (2, H), 0.5), TensorSpec(f"l{l}.w_in", (2, I, H), 0.2),
                    TensorSpec(f"l{l}.w_out", (2, H, I), 0.2)]
        return out

    def build(c, w):
        from kungfu_b200.parts import make
        H, I, nh, d = c.hidden_size, c.intermediate_size, c.num_attention_heads, c.head_dim
        emb = Embedding(w.take("emb", (c.vocab_size, H)))
        rope = make("position", "clock_hands", d, w.device)
        mixers = [make("mixer", "running_mean", w.take("l0.mean_w", (H, H))),
                  PagedAttention(w.take("l1.wqkv", (3 * nh * d, H)), w.take("l1.wo", (H, nh * d)), n_heads=nh,
                                 n_kv_heads=nh, head_dim=d, scale=d ** -0.5, position=rope)]
        layers = []
        for l in range(2):
            ffn = make("feed_forward", "routed", w.take(f"l{l}.router", (2, H)), w.take(f"l{l}.w_in", (2, I, H)),
                       w.take(f"l{l}.w_out", (2, H, I)))
            layers.append(SandwichBlock(RmsNorm(w.take(f"l{l}.n1", (H,)), c.rms_norm_eps, True), mixers[l], None,
                                        RmsNorm(w.take(f"l{l}.n2", (H,)), c.rms_norm_eps, True), ffn, None))
        head = LmHead(RmsNorm(w.take("final_norm", (H,)), c.rms_norm_eps, True), emb.table)
        w.finish()
        # layer 0 (running mean) runs twice, each time with its own state; layer 1 (attention) runs, and then runs
        # again reading the keys and values its first call wrote
        schedule = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(1, 1, writes=False)]
        return DecoderModel(emb, layers, head, schedule, name=c.architecture)

    registry.register("ToyForCausalLM", ToyConfig.from_dict, build, specs, replace=True)
    return ToyConfig


def _plain(cfg, t, tokens):
    """The toy model over a whole sequence, in float64."""
    dt = torch.float64
    T = len(tokens)
    H, nh, d = cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * (1 + w.to(dt))

    def mean_mixer(x):
        run = torch.cumsum(x, 0) / torch.arange(1, T + 1, dtype=dt)[:, None]
        return run @ t["l0.mean_w"].to(dt).T

    kept = {}

    def attn(x):
        import plain_gemma2 as pg
        qkv = x @ t["l1.wqkv"].to(dt).T
        q, k, v = [qkv[:, i * nh * d:(i + 1) * nh * d].view(T, nh, d) for i in range(3)]
        angle = torch.arange(T, dtype=dt)[:, None] / torch.arange(2, 2 + d // 4, dtype=dt)[None, :]

        def turn(x):                             # the first d / 2 elements of a head, element i paired with i + d / 4
            a, b = x[..., :d // 4], x[..., d // 4:d // 2]
            c, s_ = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            return torch.cat([a * c - b * s_, a * s_ + b * c, x[..., d // 2:]], -1)
        q, k = turn(q), turn(k)
        if "kv" in kept:                         # the second call reads what the first call cached
            k, v = kept["kv"]
        else:
            kept["kv"] = (k, v)
        mask = pg.visible(T, None)
        o = torch.empty(T, nh, d, dtype=dt)
        for h in range(nh):
            s = (q[:, h] @ k[:, h].T) * d ** -0.5
            o[:, h] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, h]
        return o.reshape(T, nh * d) @ t["l1.wo"].to(dt).T

    def ffn(x, l):
        choice = torch.argmax(x @ t[f"l{l}.router"].to(dt).T, -1)
        y = torch.zeros(T, H, dtype=dt)
        for e in range(2):
            sel = choice == e
            y[sel] = torch.relu(x[sel] @ t[f"l{l}.w_in"][e].to(dt).T) @ t[f"l{l}.w_out"][e].to(dt).T
        return y

    x = t["emb"].to(dt)[torch.tensor(tokens)]
    for l, mix in ((0, mean_mixer), (1, attn), (0, mean_mixer), (1, attn)):
        x = x + mix(norm(x, t[f"l{l}.n1"]))
        x = x + ffn(norm(x, t[f"l{l}.n2"]), l)
    return (norm(x, t["final_norm"]) @ t["emb"].to(dt).T).float()


@pytest.mark.gpu
def test_toy_model_registers_builds_and_steps(tmp_path):
    _run_toy(tmp_path, DEV)


def test_toy_model_host_logic(tmp_path, cpu_ops):
    """The same toy model with the kernels replaced by the CPU stand-in: state slots, schedule and cache sharing."""
    _run_toy(tmp_path, "cpu")


def _run_toy(tmp_path, DEV):
    ToyConfig = _define()
    from kungfu_b200 import api, registry
    from kungfu_b200.parts import FixedState, PagedKV
    from kungfu_b200.weights import write_random_model
    cfg = ToyConfig("ToyForCausalLM", 48, 80, 200, 3, 16, 1e-5, 96)
    folder = write_random_model(str(tmp_path / "toy"), cfg, seed=3, dtype=torch.float32)
    assert "ToyForCausalLM" in registry.names()
    c, model = api.load_model(folder, dtype="float32", device=DEV)
    needs = model.state_needs()
    assert [type(n) for n in needs] == [FixedState, PagedKV, FixedState]
    tensors = helpers.read_tensors(folder)
    reqs = {f"t{i}": helpers.random_tokens(n, cfg.vocab_size, 500 + i) for i, n in enumerate((33, 7, 50, 1))}
    ref = {rid: _plain(cfg, tensors, toks) for rid, toks in reqs.items()}
    scale = max(float(r.abs().max()) for r in ref.values())
    for mode, steps in (("whole", helpers.trace_whole(reqs)), ("tail", helpers.trace_decode_tail(reqs, 8)),
                        ("chunks", helpers.trace_chunks(reqs)), ("mixed", helpers.trace_mixed(reqs, seed=2))):
        runner = api.make_runner(c, model, dtype="float32", device=DEV, page_size=8,
                                 max_tokens=helpers.trace_max_tokens(steps, 8), max_requests=4, max_context=96)
        got = helpers.run_trace_with_runner(runner, steps)
        worst = max(float((row - ref[rid][pos]).abs().max()) for (rid, pos), row in got.items())
        assert len(got) == sum(len(t) for t in reqs.values()) and worst / scale < 2e-4, (mode, worst / scale)
    registry.unregister("ToyForCausalLM")


# ---- a third kind of state and a second position axis, both defined here --------------------------------------------

def _define_latent():
    """`LatentTrail`: a mixer that keeps, for every token, a latent of 24 numbers in pages of its own layout
    ([page_size, 24], not keys and values), windowed: token i gets W_up . mean(latents of the last `window` tokens).
    `GridHands`: a position encoding that turns by a SECOND integer stream ('column') the requests give with their
    tokens.  Neither the state kind nor the stream is known to the framework before this function runs."""
    from dataclasses import dataclass as dc
    from kungfu_b200.cache.kinds import register_state_kind
    from kungfu_b200.parts import Mixer, PositionEncoding

    @dc(frozen=True)
    class PagedLatent:
        width: int
        window: int | None = None

    class LatentView:
        def __init__(self, pages, page_size, group, writes):
            self.pages, self.page_size, self.group, self.writes = pages, page_size, group, writes

    class LatentKind:
        paged = True

        def window(self, need):
            return need.window

        def page_shape(self, need, page_size):
            return (page_size, need.width)

        def page_bytes(self, need, page_size, elsize):
            return page_size * need.width * 4

        def dtype(self, need, cache_dtype):
            return torch.float32

        def view(self, storage, page_size, group, writes, need):
            return LatentView(storage, page_size, group, writes)

    register_state_kind(PagedLatent, LatentKind())

    class LatentTrail(Mixer):
        graph_safe = False

        def __init__(self, w_down, w_up, window, position=None):
            self.w_down, self.w_up, self.window = w_down, w_up, window          # [24, H], [H, 24]
            self.position = position

        def state_need(self):
            return PagedLatent(self.w_down.shape[0], self.window)

        def forward(self, x, ctx, cache):
            P = cache.page_size
            lat = x.float() @ self.w_down.float().T                              # [rows, 24]
            if self.position is not None:                                        # scaled by the second position axis
                cos, _ = self.position.rotation(ctx)
                lat = lat * cos[:, :1]
            table = ctx.block_tables[cache.group]
            pos = ctx.positions[:ctx.n_rows].long()
            req = ctx.row_req[:ctx.n_rows].long()
            page = table[req, pos // P].long()
            if cache.writes:
                cache.pages[page, pos % P] = lat
            out = torch.empty(x.shape[0], self.w_up.shape[0], dtype=torch.float32, device=x.device)
            for r in range(x.shape[0]):
                p = int(ctx.host["positions"][r])
                q = int(ctx.host["row_req"][r])
                js = torch.arange(max(0, p - self.window + 1), p + 1, device=x.device)
                pj = table[q, js // P].long()
                assert bool((pj >= 0).all()), "a page inside the window was given back"
                out[r] = cache.pages[pj, js % P].mean(0) @ self.w_up.float().T
            return out

    class GridHands(PositionEncoding):
        graph_safe = False
        step_streams = ("column",)

        def rotation(self, ctx):
            col = ctx.streams["column"][:ctx.n_rows].to(torch.float32)
            angle = col[:, None] * 0.37
            return torch.cos(angle).contiguous(), torch.sin(angle).contiguous()

    return PagedLatent, LatentTrail, GridHands


def _run_latent(DEV):
    from kungfu_b200.cache import CacheManager
    from kungfu_b200.cache.plan import plan_cache
    from kungfu_b200.engine import Runner, StepEntry
    from kungfu_b200.parts import DecoderModel, Embedding, FixedState, LayerCall, LmHead, PagedKV, RmsNorm, SandwichBlock
    PagedLatent, LatentTrail, GridHands = _define_latent()
    _define()
    from kungfu_b200.parts import make
    g = torch.Generator().manual_seed(5)
    H, V, W, P = 32, 50, 6, 4

    def rnd(*shape, s=0.3):
        return (torch.randn(*shape, generator=g) * s).to(DEV)
    emb = Embedding(rnd(V, H, s=1.0))
    grid = GridHands()
    ones = torch.zeros(H, device=DEV)
    layers = []
    for l in range(2):
        mixer = LatentTrail(rnd(24, H), rnd(H, 24), W, position=grid if l == 1 else None)
        ffn = make("feed_forward", "routed", rnd(2, H, s=0.5), rnd(2, 40, H), rnd(2, H, 40))
        layers.append(SandwichBlock(RmsNorm(ones, 1e-5, True), mixer, None, RmsNorm(ones, 1e-5, True), ffn, None))
    model = DecoderModel(emb, layers, LmHead(RmsNorm(ones, 1e-5, True), emb.table), [LayerCall(0, 0), LayerCall(1, 1)])
    needs = model.state_needs()
    assert [type(n).__name__ for n in needs] == ["PagedLatent", "PagedLatent"] and model.step_stream_names() == ["column"]
    plan = plan_cache(needs, page_size=P, parallel=2, ctx=40, batch=5, element_size=4)
    assert plan.pages_by_window() == {W: 2 * 4}                    # ceil((6 + 5 + 4) / 4) pages per request
    cache = CacheManager(needs, page_size=P, n_pages=plan.pages_by_window(), max_requests=2, max_context=40,
                         dtype=torch.float32, device=DEV)
    assert cache.storage[0].shape == (8, P, 24)
    runner = Runner(model, cache, act_dtype=torch.float32, device=DEV)
    reqs = {"a": (helpers.random_tokens(23, V, 1), [i % 5 for i in range(23)]), "b": (helpers.random_tokens(9, V, 2), None)}

    def plain(tokens, cols):
        cols = list(range(len(tokens))) if cols is None else cols
        x = emb.table.double().cpu()[torch.tensor(tokens)]
        norm = lambda v: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)
        for l, blk in enumerate(layers):
            lat = norm(x) @ blk.mixer.w_down.double().cpu().T
            if l == 1:
                lat = lat * torch.cos(torch.tensor(cols, dtype=torch.float64) * 0.37)[:, None]
            m = torch.stack([lat[max(0, i - W + 1):i + 1].mean(0) for i in range(len(tokens))])
            x = x + m @ blk.mixer.w_up.double().cpu().T
            n = norm(x)
            choice = torch.argmax(n @ blk.ffn.router.double().cpu().T, -1)
            y = torch.zeros_like(x)
            for e in range(2):
                sel = choice == e
                y[sel] = torch.relu(n[sel] @ blk.ffn.w_in[e].double().cpu().T) @ blk.ffn.w_out[e].double().cpu().T
            x = x + y
        return (norm(x) @ emb.table.double().cpu().T).float()
    ref = {rid: plain(t, c) for rid, (t, c) in reqs.items()}
    for rid in reqs:
        cache.add_request(rid)
    fed = {rid: 0 for rid in reqs}
    sizes = [5, 1, 3, 2, 4, 1, 1, 5]
    k = 0
    worst = 0.0
    while any(fed[r] < len(reqs[r][0]) for r in reqs):
        entries = []
        for rid, (toks, cols) in reqs.items():
            n = min(sizes[k % len(sizes)], len(toks) - fed[rid])
            k += 1
            if n:
                st = None if cols is None else {"column": cols[fed[rid]:fed[rid] + n]}
                entries.append(StepEntry(rid, toks[fed[rid]:fed[rid] + n], list(range(n)), streams=st))
        logits = runner.step(entries).float().cpu()
        row = 0
        for e in entries:
            for w in e.want:
                worst = max(worst, float((logits[row] - ref[e.request][fed[e.request] + w]).abs().max()))
                row += 1
            fed[e.request] += len(e.tokens)
        cache.check()
    scale = max(float(r.abs().max()) for r in ref.values())
    assert worst / scale < 2e-4, worst / scale
    assert max(g.pool.n_pages - g.pool.n_free for g in cache.groups) <= 8
    cache.release("a")
    cache.add_request("c")
    free = cache.free_pages()
    with pytest.raises(Exception, match="stream 'column' has 1 values for 2 tokens"):
        runner.step([StepEntry("c", [1, 2], [], streams={"column": [0]})])
    assert cache.free_pages() == free and cache.length("c") == 0


@pytest.mark.gpu
def test_a_third_state_kind_and_a_second_position_axis_from_a_test_file():
    _run_latent(DEV)


def test_a_third_state_kind_and_a_second_position_axis_host_logic(cpu_ops):
    _run_latent("cpu")
