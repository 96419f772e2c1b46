"""Binding weights to a model by tensor name.

Contract (reference: crates/kf-arch/src/weights.rs:11-51 and compose.rs:726-732):
a builder takes every tensor it needs by name; a name that is absent, a tensor
whose shape is not the one the configuration implies, and a tensor in the file that
no part claimed are all errors.  Here they are gathered while the model is built and
raised together by `finish()` as one `WeightError` listing all three kinds.

Element types: bfloat16 stays bfloat16, a tensor stored in 32-bit floats stays so,
float16 is converted to bfloat16, integer tables become int32.  With
`compute_dtype=torch.float32` every floating tensor is widened (exactly) to 32-bit.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Callable, Iterable

import torch

from .safetensors_io import open_model_tensors


class WeightError(ValueError):
    """Missing, unexpected or wrongly shaped tensors; `.missing`, `.unexpected`, `.wrong_shape` hold the lists."""

    def __init__(self, where: str, missing, unexpected, wrong_shape):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"{where}: weights do not match the configuration"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in self.wrong_shape))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorSpec:
    """One tensor an architecture expects: its file name, shape, and how random weights draw it."""
    name: str
    shape: tuple
    std: float = 0.02
    kind: str = "matrix"          # matrix | norm | table(int)


def _stored_dtype(t: torch.Tensor, compute_dtype: torch.dtype) -> torch.dtype:
    if not t.dtype.is_floating_point:
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if t.dtype in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


class WeightStore:
    """Hands out device tensors by name and keeps the three error lists."""

    def __init__(self, source: dict[str, Callable[[], torch.Tensor]], shapes: dict[str, tuple], *,
                 device, compute_dtype: torch.dtype, where: str):
        self._source = source
        self._shapes = shapes
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        self.where = where
        self.claimed: dict[str, torch.Tensor] = {}
        self.missing: list[str] = []
        self.wrong_shape: list[tuple] = []
        self.bytes_loaded = 0

    # ---- construction ---------------------------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str, *, device, compute_dtype: torch.dtype) -> "WeightStore":
        tensors = open_model_tensors(folder)
        source = {n: (lambda sf=sf, n=n: sf.read(n)) for n, (sf, _info) in tensors.items()}
        shapes = {n: info.shape for n, (_sf, info) in tensors.items()}
        return cls(source, shapes, device=device, compute_dtype=compute_dtype, where=folder)

    @classmethod
    def from_tensors(cls, tensors: dict[str, torch.Tensor], *, device, compute_dtype: torch.dtype,
                     where: str = "<tensors>") -> "WeightStore":
        source = {n: (lambda t=t: t) for n, t in tensors.items()}
        shapes = {n: tuple(t.shape) for n, t in tensors.items()}
        return cls(source, shapes, device=device, compute_dtype=compute_dtype, where=where)

    @classmethod
    def from_random(cls, specs: Iterable[TensorSpec], seed: int, *, device, compute_dtype: torch.dtype,
                    stored_dtype: torch.dtype = torch.bfloat16, on_device: bool = False) -> "WeightStore":
        """Random weights without a file.  With `on_device` the values are drawn by the device's
        generator (fast, for measurements); otherwise they are the ones `write_random_model` stores."""
        specs = list(specs)
        dev = torch.device(device)
        source = {}
        for s in specs:
            if on_device and dev.type == "cuda":
                source[s.name] = (lambda s=s: random_tensor_device(s, seed, stored_dtype, dev))
            else:
                source[s.name] = (lambda s=s: random_tensor(s, seed, stored_dtype))
        shapes = {s.name: tuple(s.shape) for s in specs}
        return cls(source, shapes, device=device, compute_dtype=compute_dtype, where=f"<random seed {seed}>")

    # ---- taking ---------------------------------------------------------------------------
    def has(self, name: str) -> bool:
        return name in self._source

    def take(self, name: str, shape: tuple) -> torch.Tensor:
        """The tensor `name`, which must have `shape`.  A fault is recorded, not raised: `finish()` reports all."""
        shape = tuple(int(s) for s in shape)
        if self.claimed.get(name) is not None:
            return self.claimed[name]
        if name not in self._source:
            self.missing.append(name)
            return torch.empty(0)
        found = tuple(self._shapes[name])
        if found != shape:
            self.wrong_shape.append((name, shape, found))
            self.claimed[name] = torch.empty(0)
            return self.claimed[name]
        host = self._source[name]()
        dtype = _stored_dtype(host, self.compute_dtype)
        t = host.to(device=self.device, dtype=dtype).contiguous()
        if t.data_ptr() == host.data_ptr():        # same device and dtype: do not alias a file mapping
            t = t.clone()
        self.bytes_loaded += t.numel() * t.element_size()
        self.claimed[name] = t
        return t

    def release(self, *names: str) -> None:
        """Drop the store's hold on tensors that were copied into a stacked matrix; they stay claimed."""
        for n in names:
            if n in self.claimed:
                self.claimed[n] = None

    @property
    def faulty(self) -> bool:
        return bool(self.missing or self.wrong_shape)

    def take_optional(self, name: str, shape: tuple) -> torch.Tensor | None:
        return self.take(name, shape) if name in self._source else None

    def finish(self) -> None:
        """Raise one error if anything was missing, unclaimed or wrongly shaped."""
        unexpected = sorted(n for n in self._source if n not in self.claimed)
        if self.missing or unexpected or self.wrong_shape:
            raise WeightError(self.where, self.missing, unexpected, self.wrong_shape)


# ---- random weights ---------------------------------------------------------------------------

def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(spec: TensorSpec, seed: int, stored_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The host tensor random-weights mode stores for `spec`: N(0, std), its own stream per tensor name."""
    g = torch.Generator(device="cpu")
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.kind == "table":
        return torch.randint(0, 2 ** 15, tuple(spec.shape), generator=g, dtype=torch.int32)
    t = torch.empty(tuple(spec.shape), dtype=torch.float32)
    t.normal_(0.0, spec.std, generator=g)
    return t.to(stored_dtype)


def random_tensor_device(spec: TensorSpec, seed: int, stored_dtype: torch.dtype, device) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.kind == "table":
        return torch.randint(0, 2 ** 15, tuple(spec.shape), generator=g, dtype=torch.int32, device=device)
    t = torch.empty(tuple(spec.shape), dtype=stored_dtype, device=device)
    t.normal_(0.0, spec.std, generator=g)
    return t
