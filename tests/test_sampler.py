"""The sampler: generator, greedy, the dense pipeline and the sparse shortcut."""
import numpy as np
import pytest

from kungfu_b200.sampling import Candidates, Rng, Sampling, argmax, sample, sample_sparse


def test_rng_is_xorshift64():
    r = Rng(42)
    x = 42
    for _ in range(5):
        x ^= (x << 13) & (2 ** 64 - 1)
        x ^= x >> 7
        x ^= (x << 17) & (2 ** 64 - 1)
        assert r.next_f32() == (x >> 40) / 2 ** 24
    assert Rng(0).state == 1             # seed max(seed, 1)


def test_greedy_takes_the_first_maximum():
    l = np.array([0.5, 2.0, -1.0, 2.0], dtype=np.float32)
    assert argmax(l) == 1
    assert sample(l, Sampling(temperature=0.0), [], Rng(1)) == 1
    assert sample(l, Sampling(temperature=0.0, repeat_penalty=2.0), [1], Rng(1)) == 3     # 2.0 / 2 < 2.0


def test_temperature_follows_the_distribution():
    l = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    s = Sampling(temperature=1.0, top_k=0, top_p=1.0)
    rng = Rng(7)
    counts = np.bincount([sample(l, s, [], rng) for _ in range(8000)], minlength=4) / 8000
    assert np.abs(counts - [0.5, 0.3, 0.15, 0.05]).max() < 0.02
    s = Sampling(temperature=1.0, top_k=2, top_p=1.0)
    assert set(sample(l, s, [], rng) for _ in range(200)) == {0, 1}
    s = Sampling(temperature=1.0, top_k=0, top_p=0.75)                # 0.5 + 0.3 reaches 0.75
    assert set(sample(l, s, [], rng) for _ in range(200)) == {0, 1}
    s = Sampling(temperature=1.0, top_k=0, top_p=1.0, min_p=0.5)      # floor 0.25
    assert set(sample(l, s, [], rng) for _ in range(200)) == {0, 1}


@pytest.mark.parametrize("seed", range(5))
def test_sparse_equals_dense_token_and_generator_state(seed):
    """Whenever the candidates settle the draw, token and generator state equal the dense sampler's
    (the reference's own check, crates/kf-engine/src/sampler.rs:229-321)."""
    g = np.random.default_rng(seed)
    V, K = 300, 64
    agree = 0
    for round_ in range(80):
        l = g.normal(size=V).astype(np.float32) * 3
        order = np.argsort(-l, kind="stable")[:K]
        lse = float(np.log(np.exp(l.astype(np.float64)).sum()))
        c = Candidates(order.astype(np.int32), l[order], lse, V)
        s = Sampling(temperature=float(g.choice([0.0, 0.7, 1.3])), top_k=int(g.choice([0, 1, 40, 64])),
                     top_p=float(g.choice([1.0, 0.9])), min_p=float(g.choice([0.0, 0.1])),
                     repeat_penalty=float(g.choice([1.0, 1.3])))
        recent = [int(t) for t in g.integers(0, V, size=5)]
        a, b = Rng(seed * 100 + round_ + 1), Rng(seed * 100 + round_ + 1)
        sparse = sample_sparse(c, s, recent, a)
        if sparse is None:
            assert a.state == b.state                    # the generator is untouched when nothing comes back
            continue
        assert sparse == sample(l, s, recent, b) and a.state == b.state
        agree += 1
    assert agree > 20
