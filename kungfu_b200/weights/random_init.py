"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

Matrices are drawn from N(0, 0.02) and norm weights from N(0, 0.1), each tensor from its own
stream keyed by (seed, tensor name), so the file does not depend on the order of writing.
The reference has no such mode in the product; its tests synthesise tensors the same way
(crates/kf-backend-cuda/tests/common/mod.rs:71-97,114-147).
"""
from __future__ import annotations

import json
import os

import torch

from .safetensors_io import write_safetensors
from .store import random_tensor


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16,
                       norm_dtype: torch.dtype | None = None) -> str:
    """Write `folder/config.json` and `folder/model.safetensors` for `config` (a typed configuration
    whose architecture is registered).  `dtype` is the stored element type of matrices; norm vectors
    use `norm_dtype` when given.  Returns the folder."""
    from .. import registry
    arch = registry.find(config.architecture)
    os.makedirs(folder, exist_ok=True)
    tensors = {}
    for spec in arch.tensor_specs(config):
        dt = norm_dtype if (norm_dtype is not None and spec.kind == "norm") else dtype
        tensors[spec.name] = random_tensor(spec, seed, dt)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed, "generator": "kungfu_b200 random weights"})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
    return folder
