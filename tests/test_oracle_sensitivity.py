"""A test of the tests: would the comparisons with the plain implementation notice a wrong constant?

For every sharpened test model (`helpers.sharpen_tensors`) and every constant of the architecture (attention
softcap, final softcap, attention scale, rotation base, window length, which layers slide), the plain model with
that one constant changed must move its logits by more than ten times the tolerance of the comparison that claims
to cover it, in the measure those comparisons use (largest difference over largest logit).  With plainly drawn
weights (spread 0.02) most of these changes move the logits by 1e-7 to 1e-2, below the bfloat16 tolerance: this
file fails if the sharpening is ever lost.
"""
import pytest
import torch

import helpers
import plain_gemma2

# the tolerances of tests/test_gpu_engine.py (32-bit against float64; bfloat16 against the plain model rounded at the
# same places)
TOL = {"float32": 2e-4, "bfloat16": 1e-2}

CASES = {"A": (helpers.TINY_A, [5, 17, 23, 40]), "B": (helpers.TINY_B, [1, 31, 40, 70]),
         "C": (helpers.TINY_C, [3, 50, 64, 29, 120]), "D": (helpers.TINY_D, [2, 40, 17, 90]), "E": (helpers.TINY_E, [300, 70])}


def _effects(cfg, lengths, sharp, tmp_path):
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=21, sharp=sharp)
    tensors = helpers.read_tensors(folder)
    reqs = [helpers.random_tokens(n, helpers.quiet_vocab(cfg), 300 + i) for i, n in enumerate(lengths)]
    base = [plain_gemma2.forward(cfg, tensors, r) for r in reqs]
    scale = max(float(b.abs().max()) for b in base)
    out = {}
    for name, changed in helpers.mutations(cfg).items():
        got = [plain_gemma2.forward(changed, tensors, r) for r in reqs]
        out[name] = max(float((a - b).abs().max()) for a, b in zip(base, got)) / scale
    return out


@pytest.mark.parametrize("name", list(CASES))
def test_every_constant_moves_the_sharp_models_logits(tmp_path, name):
    cfg, lengths = CASES[name]
    effects = _effects(cfg, lengths, True, tmp_path)
    expected = {"A": 5, "B": 6, "C": 5, "D": 3, "E": 6}[name]           # constants this configuration has at all
    assert len(effects) == expected, sorted(effects)
    bar = 10 * max(TOL.values())
    weak = {k: v for k, v in effects.items() if v <= bar}
    assert not weak, f"changes the tests would not notice (bar {bar}): {weak}"


def test_plain_draws_would_hide_them(tmp_path):
    """The reason for the sharpening, kept as a fact: with the plain draw the attention softcap is invisible even in
    32-bit and the attention scale in bfloat16."""
    effects = _effects(helpers.TINY_B, [1, 31, 40, 70], False, tmp_path)
    assert effects["attention softcap off"] < TOL["float32"]
    assert effects["scale from head_dim"] < 10 * TOL["bfloat16"]


def test_rounded_oracle_differs_from_exact_only_by_rounding(tmp_path):
    """`rounding=torch.bfloat16` changes nothing but the stored precision: on a plain draw the two agree to a few
    parts in a thousand, and rounding to float64 is the identity."""
    cfg = helpers.TINY_B
    folder = helpers.write_model(str(tmp_path / "m"), cfg, seed=21)
    tensors = helpers.read_tensors(folder)
    toks = helpers.random_tokens(40, cfg["vocab_size"], 3)
    exact = plain_gemma2.forward(cfg, tensors, toks)
    assert torch.equal(plain_gemma2.forward(cfg, tensors, toks, rounding=torch.float64), exact)
    r = plain_gemma2.forward(cfg, tensors, toks, rounding=torch.bfloat16)
    rel = float((r - exact).abs().max() / exact.abs().max())
    assert 1e-4 < rel < 2e-2
