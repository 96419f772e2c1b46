"""Configuration reading, the registry, safetensors round trip and every weight error."""
import json
import os

import pytest
import torch

import helpers
from kungfu_b200 import api, registry
from kungfu_b200.config import ConfigError, Gemma2Config, SLIDING, FULL
from kungfu_b200.weights import (WeightError, WeightFileError, WeightStore, open_model_tensors, write_random_model,
                                 write_safetensors)
from kungfu_b200.models import gemma2


def test_tiny_configs_parse_and_differ():
    a = Gemma2Config.from_dict(helpers.TINY_A)
    b = Gemma2Config.from_dict(helpers.TINY_B)
    for f in ("hidden_size", "num_hidden_layers", "num_attention_heads", "head_dim", "intermediate_size", "vocab_size",
              "rms_norm_eps", "rope_theta", "sliding_window", "attn_logit_softcapping", "final_logit_softcapping",
              "query_pre_attn_scalar", "max_position_embeddings"):
        assert getattr(a, f) != getattr(b, f), f
    assert a.layer_types == (SLIDING, FULL) and b.layer_types == (SLIDING, FULL, SLIDING)
    assert a.window_of(0) == 8 and a.window_of(1) is None
    assert abs(b.attention_scale - 24 ** -0.5) < 1e-12
    assert b.q_size == 192 != b.hidden_size


def test_real_sizes_round_trip():
    for L, H, nh, nkv, d, I, q in ((26, 2304, 8, 4, 256, 9216, 256), (42, 3584, 16, 8, 256, 14336, 256), (46, 4608, 32, 16, 128, 36864, 144)):
        raw = dict(helpers.TINY_A, num_hidden_layers=L, hidden_size=H, num_attention_heads=nh, num_key_value_heads=nkv,
                   head_dim=d, intermediate_size=I, vocab_size=256000, sliding_window=4096, query_pre_attn_scalar=q,
                   max_position_embeddings=8192)
        cfg = Gemma2Config.from_dict(raw)
        again = Gemma2Config.from_dict(cfg.to_dict())
        assert again == cfg
        assert len(gemma2.tensor_specs(cfg)) == 2 + 11 * L


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in helpers.TINY_A.items() if k not in ("sliding_window", "attn_logit_softcapping",
                                                                 "final_logit_softcapping", "rope_theta", "query_pre_attn_scalar")}
    cfg = Gemma2Config.from_dict(raw)
    assert (cfg.sliding_window, cfg.attn_logit_softcapping, cfg.final_logit_softcapping, cfg.rope_theta) == (4096, 50.0, 30.0, 10000.0)
    assert cfg.query_pre_attn_scalar == cfg.head_dim


@pytest.mark.parametrize("change,needle", [
    ({"rms_norm_eps": None}, "rms_norm_eps"), ({"hidden_size": "64"}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"hidden_activation": "relu"}, "hidden_activation"),
    ({"layer_types": ["full_attention"]}, "layer_types"), ({"layer_types": ["x", "y"]}, "layer_types"),
    ({"attention_bias": True}, "attention_bias"), ({"rope_scaling": {"type": "linear"}}, "rope_scaling"),
    ({"attn_logit_softcapping": -1.0}, "softcapping"), ({"num_hidden_layers": 0}, "num_hidden_layers"),
])
def test_bad_configs_are_refused_by_name(change, needle):
    raw = dict(helpers.TINY_A)
    for k, v in change.items():
        if v is None:
            raw.pop(k)
        else:
            raw[k] = v
    with pytest.raises(ConfigError) as e:
        Gemma2Config.from_dict(raw)
    assert needle in str(e.value)


def test_explicit_layer_types_and_zero_caps():
    raw = dict(helpers.TINY_B, layer_types=[FULL, FULL, SLIDING], attn_logit_softcapping=0.0, final_logit_softcapping=0)
    cfg = Gemma2Config.from_dict(raw)
    assert cfg.window_of(0) is None and cfg.window_of(2) == 16 and cfg.final_logit_softcapping == 0.0


def test_null_switches_a_feature_off():
    raw = dict(helpers.TINY_A, attn_logit_softcapping=None, final_logit_softcapping=None, sliding_window=None)
    cfg = Gemma2Config.from_dict(raw)
    assert cfg.attn_logit_softcapping == 0.0 and cfg.final_logit_softcapping == 0.0
    assert cfg.layer_types == (FULL, FULL) and cfg.window_of(0) is None


def test_registry():
    assert "Gemma2ForCausalLM" in registry.names()
    with pytest.raises(registry.UnknownArchitecture) as e:
        registry.find("LlamaForCausalLM")
    assert "Gemma2ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        api.load_config({"hidden_size": 8})
    assert api.load_config(dict(helpers.TINY_A)).architecture == "Gemma2ForCausalLM"


def test_safetensors_round_trip(tmp_path):
    from safetensors.torch import load_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, t, metadata={"k": "v"})
    theirs = load_file(p)                       # the safetensors library reads what we wrote
    ours = open_model_tensors(str(tmp_path))
    for name, ref in t.items():
        assert torch.equal(theirs[name], ref)
        sf, info = ours[name]
        assert info.shape == tuple(ref.shape) and torch.equal(sf.read(name), ref)


def test_random_model_folder_is_deterministic(tmp_path):
    cfg = Gemma2Config.from_dict(helpers.TINY_A)
    a = write_random_model(str(tmp_path / "a"), cfg, seed=3)
    b = write_random_model(str(tmp_path / "b"), cfg, seed=3)
    c = write_random_model(str(tmp_path / "c"), cfg, seed=4)
    ta, tb, tc = helpers.read_tensors(a), helpers.read_tensors(b), helpers.read_tensors(c)
    assert set(ta) == {s.name for s in gemma2.tensor_specs(cfg)}
    assert all(torch.equal(ta[n], tb[n]) for n in ta)
    assert not torch.equal(ta["model.norm.weight"], tc["model.norm.weight"])
    assert ta["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert 0.01 < float(ta["model.embed_tokens.weight"].float().std()) < 0.03
    assert 0.05 < float(ta["model.layers.0.input_layernorm.weight"].float().std()) < 0.15
    assert Gemma2Config.from_dict(json.load(open(os.path.join(a, "config.json")))) == cfg


def test_weight_errors_are_listed_together(tmp_path):
    cfg = Gemma2Config.from_dict(helpers.TINY_A)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=1)
    tensors = dict(helpers.read_tensors(folder))
    tensors.pop("model.layers.1.mlp.up_proj.weight")                         # missing
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(31, 64)   # wrong shape
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)      # unexpected
    tensors["extra.weight"] = torch.zeros(2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        api.load_model(folder, dtype="float32", device="cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight"]
    assert sorted(err.unexpected) == ["extra.weight", "model.layers.0.self_attn.rotary.inv_freq"]
    assert [(n, tuple(x), tuple(f)) for n, x, f in err.wrong_shape] == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (31, 64))]
    msg = str(err)
    assert "missing tensors" in msg and "unexpected tensors" in msg and "wrong shapes" in msg and "expected [32, 64] found [31, 64]" in msg


def test_weight_file_errors(tmp_path):
    with pytest.raises(WeightFileError):
        open_model_tensors(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{not json")
    with pytest.raises(WeightFileError):
        open_model_tensors(str(tmp_path))


def test_dtype_policy():
    t = {"w": torch.randn(4, 4).to(torch.bfloat16), "n": torch.randn(4), "h": torch.randn(4).to(torch.float16),
         "i": torch.arange(4, dtype=torch.int64)}
    s = WeightStore.from_tensors(t, device="cpu", compute_dtype=torch.bfloat16)
    assert s.take("w", (4, 4)).dtype == torch.bfloat16       # bfloat16 stays
    assert s.take("n", (4,)).dtype == torch.float32           # stored in 32-bit stays so
    assert s.take("h", (4,)).dtype == torch.bfloat16
    assert s.take("i", (4,)).dtype == torch.int32             # integer tables as int32
    s.finish()
    s32 = WeightStore.from_tensors(t, device="cpu", compute_dtype=torch.float32)
    w = s32.take("w", (4, 4))
    assert w.dtype == torch.float32 and torch.equal(w, t["w"].float())


def test_tied_and_untied_head(tmp_path):
    raw = dict(helpers.TINY_A, tie_word_embeddings=False)
    cfg = Gemma2Config.from_dict(raw)
    folder = write_random_model(str(tmp_path / "u"), cfg, seed=2)
    _, model = api.load_model(folder, dtype="float32", device="cpu")
    assert model.head.weight.data_ptr() != model.embedding.table.data_ptr()
    tensors = dict(helpers.read_tensors(folder))
    tensors.pop("lm_head.weight")
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        api.load_model(folder, dtype="float32", device="cpu")
    assert e.value.missing == ["lm_head.weight"]


def test_random_generator_is_counter_based():
    """Any part of a tensor can be drawn alone; the first values of one stream are pinned so that a change of the
    generator (which would silently change every test model) shows."""
    from kungfu_b200.weights.store import TensorSpec, _tensor_seed, random_tensor, random_values
    spec = TensorSpec("model.layers.3.mlp.up_proj.weight", (37, 53), 0.02)
    whole = random_tensor(spec, 7, torch.float32).view(-1)
    part = torch.from_numpy(random_values(_tensor_seed(7, spec.name), 1000, 61, 0.02))
    assert torch.equal(part, whole[1000:1061])
    big = random_tensor(TensorSpec("x", (200000,), 1.0), 1, torch.float32)
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01 and float(big.abs().max()) < 6.0
    assert 0.66 < float((big.abs() < 1.0).float().mean()) < 0.70          # bell-shaped: about 68 % within one spread
    first = random_values(0x0123456789ABCDEF, 0, 4, 65536.0).tolist()
    assert first == [float(v) for v in first] and len(set(first)) == 4
    assert [int(v) for v in first] == PINNED_FIRST_VALUES


PINNED_FIRST_VALUES = [-11654, -90132, -84309, 221047]
