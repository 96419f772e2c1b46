"""Reading and writing the safetensors container.

File layout: 8 bytes little-endian header length N, N bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}},
then the tensor bytes.  The reference maps its weight file and hands out tensors by
name (crates/kf-gguf/src/lib.rs:171-222); this reader does the same for safetensors:
the file is memory-mapped and a tensor's bytes are touched only when it is taken.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch


class WeightFileError(ValueError):
    """A weight file that cannot be opened or parsed."""


# safetensors dtype tag -> (numpy dtype to map the bytes, torch dtype of the view)
_DTYPES = {
    "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16),
    "F64": (np.float64, torch.float64),
    "I64": (np.int64, torch.int64),
    "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16),
    "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8),
    "BOOL": (np.bool_, torch.bool),
}
_TAG_OF = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64",
           torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
           torch.uint8: "U8", torch.bool: "BOOL"}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str          # safetensors tag
    shape: tuple
    begin: int          # byte offsets inside the data section
    end: int
    file: str

    @property
    def nbytes(self) -> int:
        return self.end - self.begin

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][1]


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightFileError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightFileError(f"{path}: too short for a safetensors header")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise WeightFileError(f"{path}: header length {n} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self.tensors: dict[str, TensorInfo] = {}
        for name, rec in header.items():
            try:
                dtype, shape, (b, e) = rec["dtype"], tuple(int(s) for s in rec["shape"]), rec["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise WeightFileError(f"{path}: malformed header entry for tensor '{name}'") from None
            if dtype not in _DTYPES:
                raise WeightFileError(f"{path}: tensor '{name}' has unsupported dtype {dtype}")
            info = TensorInfo(name, dtype, shape, int(b), int(e), path)
            want = info.numel * np.dtype(_DTYPES[dtype][0]).itemsize
            if info.end - info.begin != want or self._data_start + info.end > size:
                raise WeightFileError(f"{path}: tensor '{name}' spans {info.end - info.begin} bytes, its shape needs {want}")
            self.tensors[name] = info
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def read(self, name: str) -> torch.Tensor:
        """A host tensor that copies nothing until it is used (a view of the mapping)."""
        info = self.tensors[name]
        np_dtype, t_dtype = _DTYPES[info.dtype]
        arr = np.frombuffer(self._mm, dtype=np_dtype, count=info.numel, offset=self._data_start + info.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")           # read-only mapping: the view is never written
            t = torch.from_numpy(arr)
        if t_dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(info.shape)


def open_model_tensors(folder: str) -> dict[str, tuple[SafetensorsFile, TensorInfo]]:
    """All tensors of a model folder: `model.safetensors`, or the shards an index names."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    files: list[str]
    if os.path.exists(single):
        files = [single]
    elif os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        files = sorted({os.path.join(folder, v) for v in weight_map.values()})
        if not files:
            raise WeightFileError(f"{index}: empty weight_map")
    else:
        raise WeightFileError(f"{folder}: neither model.safetensors nor model.safetensors.index.json found")
    out: dict[str, tuple[SafetensorsFile, TensorInfo]] = {}
    for p in files:
        sf = SafetensorsFile(p)
        for name, info in sf.tensors.items():
            if name in out:
                raise WeightFileError(f"{p}: tensor '{name}' also appears in {out[name][1].file}")
            out[name] = (sf, info)
    return out


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write host tensors to one .safetensors file, in the order given."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _TAG_OF:
            raise WeightFileError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).reshape(-1) if t.numel() else torch.empty(0, dtype=torch.uint8)
        if t.dtype == torch.bfloat16:
            raw = t.view(torch.int16).reshape(-1).view(torch.uint8)
        n = raw.numel()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw.numpy().tobytes())
    os.replace(tmp, path)
