"""The Python entry point: load a model folder, make an engine, generate.

Shape of the reference's public surface (crates/kf-engine/src/lib.rs:13-19): `load` opens the weight
file, finds the architecture by the name the file gives and builds the model
(crates/kf-engine/src/loader.rs:88-104); a session feeds tokens and steps; `sample` picks tokens.
"""
from __future__ import annotations

import os

import torch

from . import registry
from .cache.manager import CacheManager
from .config.base import architecture_name, read_config_json
from .engine.step import Runner
from .weights.store import WeightStore

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


DEFAULT_PAGE_SIZE = 64


def parse_dtype(dtype) -> torch.dtype:
    if dtype not in _DTYPES:
        raise ValueError(f"dtype {dtype!r} is not one of bfloat16, float32")
    return _DTYPES[dtype]


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("kungfu_b200 runs on a CUDA device only (there is no CPU path)")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is visible; kungfu_b200 has no CPU path")
    torch.cuda.set_device(device)
    return device


def load_config(path_or_dict):
    """The typed configuration of a model folder, config.json file or dictionary, through the registry."""
    raw = path_or_dict if isinstance(path_or_dict, dict) else read_config_json(path_or_dict)
    where = "config" if isinstance(path_or_dict, dict) else str(path_or_dict)
    arch = registry.find(architecture_name(raw, where))
    return arch.parse_config(raw, where)


def load_model(folder: str, *, dtype="bfloat16", device="cuda:0"):
    """(configuration, model) from a folder holding config.json and model.safetensors."""
    dtype = parse_dtype(dtype)
    cfg = load_config(folder)
    arch = registry.find(cfg.architecture)
    store = WeightStore.from_folder(folder, device=device, compute_dtype=dtype)
    model = arch.build(cfg, store)
    return cfg, model


def random_model(config, seed: int = 0, *, dtype="bfloat16", device="cuda:0", on_device: bool = True):
    """(configuration, model) with random weights drawn without a file (for measurements)."""
    dtype = parse_dtype(dtype)
    cfg = config if not isinstance(config, (dict, str)) else load_config(config)
    arch = registry.find(cfg.architecture)
    store = WeightStore.from_random(arch.tensor_specs(cfg), seed, device=device, compute_dtype=dtype,
                                    on_device=on_device)
    return cfg, arch.build(cfg, store)


def make_runner(cfg, model, *, dtype, device, page_size: int = DEFAULT_PAGE_SIZE, max_tokens: int | None = None,
                n_pages: int | None = None, max_requests: int = 64, max_context: int | None = None,
                cuda_graphs: bool = True, batch: int | None = None, budget_bytes: int | None = None) -> Runner:
    """A step runner with its cache.  Every group's pool holds `max_tokens` tokens (rounded up to whole pages; default
    `max_requests * max_context`), except that a windowed group never gets more than its requests can hold when
    `batch` (the most tokens one step feeds of one request) is given: `max_requests * (window + batch + page)`.
    `budget_bytes`: the memory the cache may take; pools are cut to fit it (`cache.plan.NoFit` if one request of
    `max_context` tokens does not fit).  `n_pages` sets every pool to that many pages and skips the sizing."""
    from .cache.plan import plan_cache
    dtype = parse_dtype(dtype)
    if max_context is None:
        max_context = getattr(cfg, "max_position_embeddings", 8192)
    needs = model.state_needs()
    plan = None
    if n_pages is None:
        elsize = torch.empty(0, dtype=dtype).element_size()
        plan = plan_cache(needs, page_size=page_size, parallel=max_requests, ctx=max_context,
                          batch=batch if batch is not None else max_context, element_size=elsize,
                          budget_bytes=budget_bytes, pool_tokens=max_tokens)
        pages = plan.pages_by_window()
    else:
        pages = int(n_pages)
    cache = CacheManager(needs, page_size=page_size, n_pages=pages, max_requests=max_requests,
                         max_context=max_context, dtype=dtype, device=device)
    cache.plan = plan
    runner = Runner(model, cache, act_dtype=dtype, device=device)
    runner.cuda_graphs = bool(cuda_graphs) and torch.device(device).type == "cuda"
    return runner


class Engine:
    """Placeholder; the full engine (scheduler, sampling) is defined in engine/engine.py."""

    def __new__(cls, *a, **k):
        from .engine.engine import Engine as _E
        return _E(*a, **k)
