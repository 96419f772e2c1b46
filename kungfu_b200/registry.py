"""One table from an architecture's name to its configuration class and model builder.

The name is `architectures[0]` of config.json.  The reference keeps the same table as a
static slice of `Architecture {id, hparams, build}` and fails with `UnknownArch` for a
name it does not hold (crates/kf-arch/src/lib.rs:15-28, archs/mod.rs:29-56,
crates/kf-engine/src/loader.rs:96).  Adding an architecture is one `register` call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable


class UnknownArchitecture(KeyError):
    def __str__(self) -> str:
        return self.args[0]


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable          # dict, where -> typed configuration
    build: Callable                 # (configuration, WeightStore) -> DecoderModel
    tensor_specs: Callable          # configuration -> [TensorSpec]


_TABLE: dict[str, Architecture] = {}


def register(name: str, parse_config: Callable, build: Callable, tensor_specs: Callable, *, replace: bool = False) -> Architecture:
    if name in _TABLE and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _TABLE[name] = Architecture(name, parse_config, build, tensor_specs)
    return _TABLE[name]


def unregister(name: str) -> None:
    _TABLE.pop(name, None)


def find(name: str) -> Architecture:
    if name not in _TABLE:
        raise UnknownArchitecture(f"unknown architecture '{name}'; registered: {sorted(_TABLE)}")
    return _TABLE[name]


def names() -> list[str]:
    return sorted(_TABLE)


def _register_builtin() -> None:
    from .config.gemma2 import Gemma2Config
    from .models import gemma2
    register("Gemma2ForCausalLM", Gemma2Config.from_dict, gemma2.build, gemma2.tensor_specs, replace=True)


_register_builtin()
