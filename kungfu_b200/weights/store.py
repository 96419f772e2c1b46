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


# ---- random weights ---------------------------------------------------------------------------------------------
# A counter-based generator keyed by (seed, tensor name, element index), so that any tensor can be drawn on the host or
# on the device, whole or in part, with the same bits (the kernel is `random_normal_kernel` in csrc/elementwise.cu):
#   w_j = mix(key + (3 i + j) * 0x9E3779B97F4A7C15) for j = 0, 1, 2   (splitmix64's finaliser, arithmetic modulo 2^64)
#   s   = the sum of the twelve 16-bit pieces of w_0, w_1, w_2         (mean 393210, standard deviation 65536)
#   x_i = float32(s - 393210) * float32(std / 65536), then rounded to the stored type
# Only integers, one exact conversion and one correctly rounded product: no library function whose last bit could
# differ between machines.  The reference's tests draw tensors from a small generator of their own in the same spirit
# (crates/kf-backend-cuda/tests/common/mod.rs:71-97).

_GOLDEN = 0x9E3779B97F4A7C15
_M1, _M2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def _mix64(z):
    import numpy as np
    z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
    return z ^ (z >> np.uint64(31))


def random_values(key: int, start: int, count: int, std: float):
    """Elements start..start+count-1 of stream `key` as a float32 numpy array (the host restatement of the kernel)."""
    import numpy as np
    out = np.empty(count, dtype=np.float32)
    step = np.float32(np.float32(std) / np.float32(65536.0))
    chunk = 1 << 22
    with np.errstate(over="ignore"):
        for a in range(0, count, chunk):
            n = min(chunk, count - a)
            i3 = (np.arange(start + a, start + a + n, dtype=np.uint64) * np.uint64(3))
            s = np.zeros(n, dtype=np.int64)
            for j in range(3):
                w = _mix64(np.uint64(key) + (i3 + np.uint64(j)) * np.uint64(_GOLDEN))
                s += ((w & np.uint64(0xFFFF)) + ((w >> np.uint64(16)) & np.uint64(0xFFFF))
                      + ((w >> np.uint64(32)) & np.uint64(0xFFFF)) + (w >> np.uint64(48))).astype(np.int64)
            out[a:a + n] = (s - 393210).astype(np.float32) * step
    return out


def random_table_values(key: int, count: int):
    import numpy as np
    with np.errstate(over="ignore"):
        i3 = np.arange(count, dtype=np.uint64) * np.uint64(3)
        return (_mix64(np.uint64(key) + i3 * np.uint64(_GOLDEN)) & np.uint64(0x7FFF)).astype(np.int32)


def random_tensor(spec: TensorSpec, seed: int, stored_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The host tensor random-weights mode stores for `spec`: bell-shaped around 0 with spread `spec.std`, its own
    stream per tensor name."""
    import math
    key = _tensor_seed(seed, spec.name)
    n = int(math.prod(spec.shape))
    if spec.kind == "table":
        return torch.from_numpy(random_table_values(key, n)).view(tuple(spec.shape))
    return torch.from_numpy(random_values(key, 0, n, spec.std)).view(tuple(spec.shape)).to(stored_dtype)


def random_tensor_device(spec: TensorSpec, seed: int, stored_dtype: torch.dtype, device) -> torch.Tensor:
    """The same values as `random_tensor`, drawn on the device by the library's own kernel."""
    import ctypes
    from .. import ops
    key = _tensor_seed(seed, spec.name)
    if spec.kind == "table":
        t = torch.empty(tuple(spec.shape), dtype=torch.int32, device=device)
        code = -1
    else:
        if stored_dtype not in (torch.float32, torch.bfloat16):
            return random_tensor(spec, seed, stored_dtype).to(device)
        t = torch.empty(tuple(spec.shape), dtype=stored_dtype, device=device)
        code = ops.F32 if stored_dtype == torch.float32 else ops.BF16
    with torch.cuda.device(device):
        rc = ops.library().kf_random_fill(ctypes.c_void_p(t.data_ptr()), code, ctypes.c_long(t.numel()),
                                          ctypes.c_ulonglong(key), ctypes.c_float(spec.std),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise ops.KernelError(f"random weights on the device failed (status {rc})")
    return t
