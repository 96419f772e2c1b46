"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

Matrices are drawn bell-shaped around 0 with spread 0.02 and norm weights with spread 0.1, each tensor from its own
stream keyed by (seed, tensor name) and each element by its index (a counter-based generator, `store.random_values`), so
the file does not depend on the order of writing and the device draws the same bits as the host.
The reference has no such mode in the product; its tests synthesise tensors the same way
(crates/kf-backend-cuda/tests/common/mod.rs:71-97,114-147).
"""
from __future__ import annotations

import json
import os

import torch

from .safetensors_io import write_safetensors
from .store import random_tensor, random_tensor_device


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16,
                       norm_dtype: torch.dtype | None = None, device=None) -> str:
    """Write `folder/config.json` and `folder/model.safetensors` for `config` (a typed configuration
    whose architecture is registered).  `dtype` is the stored element type of matrices; norm vectors
    use `norm_dtype` when given.  With a CUDA `device` the values are drawn there (the same bits, much faster for
    models of real size).  Returns the folder."""
    from .. import registry
    arch = registry.find(config.architecture)
    os.makedirs(folder, exist_ok=True)
    tensors = {}
    for spec in arch.tensor_specs(config):
        dt = norm_dtype if (norm_dtype is not None and spec.kind == "norm") else dtype
        if device is not None and torch.device(device).type == "cuda":
            tensors[spec.name] = random_tensor_device(spec, seed, dt, torch.device(device)).cpu()
        else:
            tensors[spec.name] = random_tensor(spec, seed, dt)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed, "generator": "kungfu_b200 random weights"})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
    return folder
