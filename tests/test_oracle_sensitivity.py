"""A test of the tests: would the comparisons with the plain implementation notice a wrong constant?

Every constant of the architecture (attention softcap, final softcap, attention scale, rotation base, window length,
which layers slide) is changed, one at a time, in the plain model, and the logits (or, one layer deep, the attention
output) must move by more than ten times the tolerance of the comparison that claims to cover that constant, in the
measure those comparisons use (largest difference over largest value).  The books:

  32-bit engine, 'sharp' draw, tolerance 2e-4 against float64          every constant
  bfloat16 engine, 'loud' draw, tolerance 2e-2 against float64         final softcap, window, sliding layers
  bfloat16 attention part, sharp weights and doubled inputs, 1.5e-2     attention softcap, rotation base
  bfloat16 attention kernels (tests/test_gpu_kernels.py                 attention softcap and scale: the kernel test
    test_softcap_where_it_bends)                                        itself asserts the factor of ten

With plainly drawn weights (spread 0.02) most of these changes move the logits by 1e-7 to 1e-2, below the bfloat16
tolerance and some below the 32-bit one: this file fails if the sharpening is ever lost.  Why bfloat16 cannot be
checked on the 'sharp' draw at engine level is measured in `test_sharp_attention_multiplies_bfloat16_rounding`.
"""
import math

import pytest
import torch

import helpers
import plain_gemma2

TOL_ENGINE = {"float32": 2e-4, "bfloat16": 2e-2}          # tests/test_gpu_engine.py, tests/test_gpu_real_widths.py
TOL_PART_BF16 = 1.5e-2                                    # tests/test_gpu_parts.py

CASES = {"A": (helpers.TINY_A, [5, 17, 23, 40, 11, 30]), "B": (helpers.TINY_B, [1, 31, 40, 70, 9, 50]),
         "C": (helpers.TINY_C, [3, 50, 64, 29, 120, 77]), "D": (helpers.TINY_D, [2, 40, 17, 90, 33, 8]),
         "E": (helpers.TINY_E, [300, 70, 513, 129, 2])}


def _model(cfg, lengths, draw, tmp_path):
    folder = helpers.write_model(str(tmp_path / f"m_{draw}"), cfg, seed=21, draw=draw)
    tensors = helpers.read_tensors(folder)
    reqs = [helpers.random_tokens(n, helpers.quiet_vocab(cfg), 300 + i) for i, n in enumerate(lengths)]
    base = [plain_gemma2.forward(cfg, tensors, r) for r in reqs]
    return tensors, reqs, base, max(float(b.abs().max()) for b in base)


def _effects(cfg, lengths, draw, tmp_path):
    tensors, reqs, base, scale = _model(cfg, lengths, draw, tmp_path)
    out = {}
    for name, changed in helpers.mutations(cfg).items():
        got = [plain_gemma2.forward(changed, tensors, r) for r in reqs]
        out[name] = max(float((a - b).abs().max()) for a, b in zip(base, got)) / scale
    return out


@pytest.mark.parametrize("name", list(CASES))
def test_32_bit_engine_tests_notice_every_constant(tmp_path, name):
    cfg, lengths = CASES[name]
    effects = _effects(cfg, lengths, "sharp", tmp_path)
    expected = {"A": 5, "B": 6, "C": 5, "D": 3, "E": 6}[name]           # constants this configuration has at all
    assert len(effects) == expected, sorted(effects)
    weak = {k: v for k, v in effects.items() if v <= 10 * TOL_ENGINE["float32"]}
    assert not weak, f"changes the 32-bit engine tests would not notice: {weak}"


@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_bfloat16_engine_tests_notice_final_cap_window_and_sliding_layers(tmp_path, name):
    cfg, lengths = CASES[name]
    effects = _effects(cfg, lengths, "loud", tmp_path)
    for constant in ("final softcap off", "window + 1", "sliding on odd layers"):
        assert effects[constant] > 10 * TOL_ENGINE["bfloat16"], (constant, effects[constant])


def test_bfloat16_attention_part_test_notices_cap_and_rotation_base(tmp_path):
    """The inputs of tests/test_gpu_parts.py::test_attention_mixer (configuration B, sharp weights, rows of spread 2)."""
    cfg = helpers.TINY_B
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=8, draw="sharp")
    t = helpers.read_tensors(folder)
    for layer in (0, 1):
        g = torch.Generator().manual_seed(4 + layer)
        xs = [(torch.randn(21, 96, generator=g) * 2).bfloat16().double(), (torch.randn(14, 96, generator=g) * 2).bfloat16().double()]
        p = f"model.layers.{layer}.self_attn."
        w = [t[p + n + ".weight"] for n in ("q_proj", "k_proj", "v_proj", "o_proj")]
        kw = dict(n_heads=6, n_kv_heads=2, head_dim=32, scale=1 / math.sqrt(24), cap=20.0, window=16 if layer == 0 else None, base=1e6)
        for x in xs:
            base = plain_gemma2.attention(x, *w, **kw)
            for constant, change in (("attention softcap off", dict(cap=0.0)), ("rope base x 10", dict(base=1e7))):
                moved = plain_gemma2.attention(x, *w, **{**kw, **change})
                effect = float((base - moved).abs().max() / base.abs().max())
                assert effect > 10 * TOL_PART_BF16, (layer, len(x), constant, effect)


def test_plain_draws_would_hide_them(tmp_path):
    """The reason for the sharpening, kept as a fact: with the plain draw the attention softcap is invisible even in
    32-bit and the attention scale in bfloat16."""
    effects = _effects(helpers.TINY_B, [1, 31, 40, 70], "plain", tmp_path)
    assert effects["attention softcap off"] < TOL_ENGINE["float32"]
    assert effects["scale from head_dim"] < 10 * TOL_ENGINE["bfloat16"]
    assert effects["final softcap off"] < 10 * TOL_ENGINE["bfloat16"]


def test_sharp_attention_multiplies_bfloat16_rounding(tmp_path):
    """Why the bfloat16 engine is not compared on the 'sharp' draw: the plain model rounded to bfloat16 where a
    bfloat16 engine rounds (product inputs, queries, keys, values, softmax weights) differs from float64 by several per
    cent there, against about 1 % on the 'loud' draw and under 1 % on the plain one.  Nothing of the engine runs here."""
    cfg, lengths = CASES["B"]
    noise = {}
    for draw in ("plain", "loud", "sharp"):
        tensors, reqs, base, scale = _model(cfg, lengths, draw, tmp_path)
        rounded = [plain_gemma2.forward(cfg, tensors, r, rounding=torch.bfloat16) for r in reqs]
        noise[draw] = max(float((a - b).abs().max()) for a, b in zip(base, rounded)) / scale
    assert noise["plain"] < 1e-2 and noise["loud"] < 2e-2 < noise["sharp"], noise


def test_rounded_oracle_differs_from_exact_only_by_rounding(tmp_path):
    """`rounding=torch.float64` is the identity; `rounding=torch.bfloat16` moves a plain draw by parts in a thousand."""
    cfg = helpers.TINY_B
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=21)
    tensors = helpers.read_tensors(folder)
    toks = helpers.random_tokens(40, cfg["vocab_size"], 3)
    exact = plain_gemma2.forward(cfg, tensors, toks)
    assert float((plain_gemma2.forward(cfg, tensors, toks, rounding=torch.float64) - exact).abs().max()) < 1e-12
    r = plain_gemma2.forward(cfg, tensors, toks, rounding=torch.bfloat16)
    rel = float((r - exact).abs().max() / exact.abs().max())
    assert 1e-4 < rel < 2e-2
