"""The sampling rules: the plain sampler's own properties, and the state the device draws from."""
import numpy as np
import pytest

import plain_sampler
from kungfu_b200.sampling import RING, STATE_WORDS, Sampling, generator_state, pack_state


def test_rng_is_xorshift64():
    r = plain_sampler.Rng(42)
    x = 42
    for _ in range(5):
        x ^= (x << 13) & (2 ** 64 - 1)
        x ^= x >> 7
        x ^= (x << 17) & (2 ** 64 - 1)
        assert r.next_f32() == (x >> 40) / 2 ** 24
    assert plain_sampler.Rng(0).state == 1             # seed max(seed, 1)


def test_greedy_takes_the_first_maximum():
    l = np.array([0.5, 2.0, -1.0, 2.0], dtype=np.float32)
    assert plain_sampler.sample(l, temperature=0.0, rng=plain_sampler.Rng(1))[0] == 1
    # the penalty applies even at temperature 0: 2.0 / 2 < 2.0
    assert plain_sampler.sample(l, temperature=0.0, repeat_penalty=2.0, recent=[1], rng=plain_sampler.Rng(1))[0] == 3
    # a token that occurs twice in the window is penalised twice; negative logits are multiplied
    l = np.array([4.0, 1.5, -1.0, -0.6], dtype=np.float32)
    tok, _ = plain_sampler.sample(l, temperature=0.0, repeat_penalty=2.0, recent=[0, 0, 9999], rng=plain_sampler.Rng(1))
    assert tok == 1                                     # 4 / 2 / 2 = 1 < 1.5


def test_temperature_follows_the_distribution():
    l = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    rng = plain_sampler.Rng(7)
    draws = [plain_sampler.sample(l, temperature=1.0, rng=rng)[0] for _ in range(8000)]
    counts = np.bincount(draws, minlength=4) / 8000
    assert np.abs(counts - [0.5, 0.3, 0.15, 0.05]).max() < 0.02
    assert set(plain_sampler.sample(l, temperature=1.0, top_k=2, rng=rng)[0] for _ in range(200)) == {0, 1}
    assert set(plain_sampler.sample(l, temperature=1.0, top_p=0.75, rng=rng)[0] for _ in range(200)) == {0, 1}   # 0.5 + 0.3 reaches 0.75
    assert set(plain_sampler.sample(l, temperature=1.0, min_p=0.5, rng=rng)[0] for _ in range(200)) == {0, 1}    # floor 0.25
    # the margin says how close the drawn number came to the next token's share
    tok, margin = plain_sampler.sample(l, temperature=1.0, rng=plain_sampler.Rng(3))
    assert 0.0 <= margin <= 0.25


def test_state_words():
    s = Sampling(temperature=0.8, top_k=7, top_p=0.9, min_p=0.05, repeat_penalty=1.2, repeat_window=32)
    st = pack_state(s, seed=0, recent=list(range(1000, 1300)))
    assert st.shape == (STATE_WORDS,) and st.dtype == np.int32
    assert generator_state(st) == 1
    assert generator_state(pack_state(s, seed=(1 << 40) + 5)) == (1 << 40) + 5
    f = st[2:6].view(np.float32)
    assert [float(v) for v in f] == [np.float32(0.8), np.float32(0.9), np.float32(0.05), np.float32(1.2)]
    assert (int(st[6]), int(st[7]), int(st[8])) == (7, 32, 300)
    for i in range(300 - RING, 300):                    # the last 256 tokens, token i at 16 + i % 256
        assert st[16 + i % RING] == 1000 + i
    assert Sampling(temperature=0.0).greedy and not Sampling(temperature=0.0, repeat_penalty=1.1).greedy
    assert Sampling(temperature=0.7, top_k=0).needs_whole_ranking and Sampling(temperature=0.7, top_k=65).needs_whole_ranking
    assert not Sampling(temperature=0.7, top_k=64).needs_whole_ranking and not Sampling(temperature=0.0, top_k=0).needs_whole_ranking


@pytest.mark.parametrize("bad", [dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=-0.1), dict(repeat_penalty=0.0),
                                 dict(repeat_window=RING + 1)])
def test_rules_are_validated(bad):
    with pytest.raises(ValueError):
        Sampling(**bad)
