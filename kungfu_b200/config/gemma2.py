"""Gemma 2 hyperparameters, read from the model's own config.json keys.

What each field means and its default follow the reference's Gemma 2 reading
(crates/kf-arch/src/archs/gemma2.rs:16-30 and crates/kf-arch/src/hparams.rs:269-488):
window 4096, attention softcap 50, final softcap 30, rope base 10000, sliding
layers every other layer starting with layer 0 (hparams.rs:541-554), norm epsilon
required (hparams.rs:576-581).  The attention scale is 1/sqrt(query_pre_attn_scalar);
the reference derives the same numbers from the layer count (gemma2.rs:28).
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

SLIDING = "sliding_attention"
FULL = "full_attention"

_ACTIVATIONS = {
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_tanh": "gelu_tanh",
    "gelu_new": "gelu_tanh",
    "gelu": "gelu_erf",
    "silu": "silu",
}


@dataclass(frozen=True)
class Gemma2Config:
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    sliding_window: int
    attn_logit_softcapping: float      # 0 switches the cap off
    final_logit_softcapping: float     # 0 switches the cap off
    query_pre_attn_scalar: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    activation: str                    # gelu_tanh | gelu_erf | silu
    layer_types: tuple = field(default_factory=tuple)   # per layer: SLIDING or FULL
    eos_token_id: tuple = field(default_factory=tuple)
    bos_token_id: int | None = None

    # ---- derived -------------------------------------------------------------------------
    @property
    def attention_scale(self) -> float:
        return 1.0 / math.sqrt(self.query_pre_attn_scalar)

    @property
    def embedding_scale(self) -> float:
        """sqrt(hidden) rounded to 32-bit, as the reference computes it (gemma2.rs:34)."""
        import struct
        return struct.unpack("f", struct.pack("f", math.sqrt(self.hidden_size)))[0]

    def window_of(self, layer: int) -> int | None:
        return self.sliding_window if self.layer_types[layer] == SLIDING else None

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "Gemma2Config":
        k = KeyReader(raw, where)
        arch = k.list("architectures")[0]
        hidden = k.int("hidden_size", min=1)
        layers = k.int("num_hidden_layers", min=1)
        heads = k.int("num_attention_heads", min=1)
        kv_heads = k.int("num_key_value_heads", heads, min=1)
        if hidden % heads != 0 and "head_dim" not in raw:
            raise ConfigError(f"{where}: 'head_dim' is missing and hidden_size {hidden} is not a multiple of num_attention_heads {heads}")
        head_dim = k.int("head_dim", hidden // heads, min=2)
        inter = k.int("intermediate_size", min=1)
        vocab = k.int("vocab_size", min=1)
        eps = k.float("rms_norm_eps")
        theta = k.float("rope_theta", 10000.0)
        # a key that is present with the value null switches the feature off (no window, no cap); a key that is
        # absent takes the reference's default (gemma2.rs:22-27)
        no_window = "sliding_window" in raw and raw["sliding_window"] is None
        window = k.int("sliding_window", 4096, min=1)
        attn_cap = 0.0 if ("attn_logit_softcapping" in raw and raw["attn_logit_softcapping"] is None) else k.float("attn_logit_softcapping", 50.0)
        final_cap = 0.0 if ("final_logit_softcapping" in raw and raw["final_logit_softcapping"] is None) else k.float("final_logit_softcapping", 30.0)
        qpas = k.float("query_pre_attn_scalar", float(head_dim))
        max_pos = k.int("max_position_embeddings", 8192, min=1)
        tied = k.bool("tie_word_embeddings", True)
        act_key = "hidden_activation" if raw.get("hidden_activation") is not None else "hidden_act"
        act_name = k.str(act_key, "gelu_pytorch_tanh")
        if act_name not in _ACTIVATIONS:
            raise ConfigError(f"{where}: key '{act_key}' is {act_name!r}, expected one of {sorted(_ACTIVATIONS)}")
        if raw.get("attention_bias"):
            raise ConfigError(f"{where}: 'attention_bias' true is not supported: Gemma 2 projections carry no bias")
        if raw.get("rope_scaling") is not None:
            raise ConfigError(f"{where}: 'rope_scaling' is not supported: Gemma 2 uses unscaled rotary positions")
        types = k.list("layer_types", None)
        if types is None:
            period = k.int("sliding_window_pattern", 2, min=1)
            # reference: swa(l) = (l % n) < n - 1, so with n = 2 even layers slide (hparams.rs:541-554)
            types = [SLIDING if (l % period) < period - 1 else FULL for l in range(layers)]
        if no_window:
            types = [FULL] * layers
        if len(types) != layers:
            raise ConfigError(f"{where}: 'layer_types' has {len(types)} entries for {layers} layers")
        for t in types:
            if t not in (SLIDING, FULL):
                raise ConfigError(f"{where}: 'layer_types' entry {t!r} is neither {SLIDING!r} nor {FULL!r}")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos = ()
        elif isinstance(eos, int):
            eos = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos = tuple(eos)
        else:
            raise ConfigError(f"{where}: key 'eos_token_id' must be an integer or a list of integers")
        bos = raw.get("bos_token_id")
        cfg = cls(arch, hidden, layers, heads, kv_heads, head_dim, inter, vocab, eps, theta, window,
                  attn_cap, final_cap, qpas, max_pos, tied, _ACTIVATIONS[act_name], tuple(types), eos,
                  bos if isinstance(bos, int) else None)
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"{where}: num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"{where}: head_dim {self.head_dim} must be even for rotary pairs")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"{where}: rms_norm_eps must be positive, found {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"{where}: rope_theta must be positive, found {self.rope_theta}")
        if self.attn_logit_softcapping < 0 or self.final_logit_softcapping < 0:
            raise ConfigError(f"{where}: softcapping values must be >= 0 (0 switches the cap off)")
        if not (self.query_pre_attn_scalar > 0):
            raise ConfigError(f"{where}: query_pre_attn_scalar must be positive")

    def to_dict(self) -> dict:
        """A config.json dictionary that `from_dict` reads back to this configuration."""
        act = {"gelu_tanh": "gelu_pytorch_tanh", "gelu_erf": "gelu", "silu": "silu"}[self.activation]
        d = {
            "architectures": [self.architecture],
            "model_type": "gemma2",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "sliding_window": self.sliding_window,
            "attn_logit_softcapping": self.attn_logit_softcapping,
            "final_logit_softcapping": self.final_logit_softcapping,
            "query_pre_attn_scalar": self.query_pre_attn_scalar,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_activation": act,
            "layer_types": list(self.layer_types),
        }
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    def replace(self, **kw) -> "Gemma2Config":
        if "num_hidden_layers" in kw and "layer_types" not in kw:
            n = kw["num_hidden_layers"]
            base = self.layer_types
            kw["layer_types"] = tuple(base[i % len(base)] for i in range(n))
        cfg = dataclasses.replace(self, **kw)
        cfg.validate()
        return cfg
