"""The reference's own CUDA kernels, compiled unchanged at run time and launched through the driver API.

nickheyer/kungfu compiles its kernels (crates/kf-backend-cuda/src/kernels/*.cu) with NVRTC when it runs and exposes
them as `extern "C"` entry points; its host code is Rust, which cannot be built where this engine is developed.  The
kernels alone can: this module finds the reference's kernel sources, compiles one file at a time with nvcc into a
temporary folder (a cubin that is only ever loaded, never listed), loads it with `cuModuleLoadData` and launches
entry points with the grid, block and shared-memory sizes the reference's executor uses
(crates/kf-backend-cuda/src/exec.rs:2094-2112 products, :2506-2513 norms, :2600-2675 attention, :1817-1848 tensor-core
attention and its tile table).  Nothing of the reference is copied into this repository.

Two uses: tests pin the plain implementation of this repository on what the reference's kernels compute, and
`bench.py --micro reference` times them beside this engine's kernels on the same device.

The sources are looked for in $KUNGFU_REFERENCE_KERNELS, in `baseline/_ref/kernels` under the repository root (a staged
copy that travels with the repository to a machine that has a GPU but not the reference checkout; `stage()` makes it),
and in `../reference/crates/kf-backend-cuda/src/kernels` beside the repository.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
STAGED = os.path.join(ROOT, "baseline", "_ref", "kernels")
FILES = ("norm.cu", "rope.cu", "elementwise.cu", "attention.cu", "flash.cu", "sample.cu", "quant_bf16.cu", "quant_f32.cu")


class ReferenceUnavailable(RuntimeError):
    pass


def find_sources() -> str:
    cands = [os.environ.get("KUNGFU_REFERENCE_KERNELS"), STAGED,
             os.path.join(os.path.dirname(ROOT), "reference", "crates", "kf-backend-cuda", "src", "kernels")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "common.cuh")):
            return c
    raise ReferenceUnavailable("the reference's kernel sources were not found (looked at $KUNGFU_REFERENCE_KERNELS, "
                               f"{STAGED} and ../reference beside the repository)")


def stage() -> str:
    """Copy the reference's kernel folder to `baseline/_ref/kernels` (ignored by git) so that it travels with the
    repository.  Returns the staged folder; does nothing when it is already there."""
    if os.path.isfile(os.path.join(STAGED, "common.cuh")):
        return STAGED
    src = find_sources()
    os.makedirs(os.path.dirname(STAGED), exist_ok=True)
    shutil.copytree(src, STAGED)
    return STAGED


def _nvcc() -> str:
    for cand in (os.environ.get("KUNGFU_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise ReferenceUnavailable("nvcc not found")


def compile_cubin(file: str, out_dir: str) -> str:
    """Compile one of the reference's kernel files for sm_100 into `out_dir`; returns the cubin's path."""
    src_dir = find_sources()
    out = os.path.join(out_dir, file.replace(".cu", ".cubin"))
    cmd = [_nvcc(), "-arch=sm_100", "-cubin", "-O3", "-std=c++17", "-I", src_dir, os.path.join(src_dir, file), "-o", out]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise ReferenceUnavailable(f"nvcc failed on the reference's {file}:\n{r.stderr[-2000:]}")
    return out


# ---- the driver API, as much of it as launching needs ----------------------------------------------------------------

_cuda = None


def _driver():
    global _cuda
    if _cuda is None:
        lib = ctypes.CDLL("libcuda.so.1")
        lib.cuModuleLoadData.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
        lib.cuModuleGetFunction.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_char_p]
        lib.cuFuncSetAttribute.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        lib.cuLaunchKernel.argtypes = [ctypes.c_void_p] + [ctypes.c_uint] * 6 + [ctypes.c_uint, ctypes.c_void_p,
                                                                               ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
        lib.cuModuleUnload.argtypes = [ctypes.c_void_p]
        _cuda = lib
    return _cuda


def _ok(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: CUDA driver error {rc}")


P = ctypes.c_void_p
I = ctypes.c_int
F = ctypes.c_float
L = ctypes.c_longlong


def ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


class Module:
    """One compiled kernel file of the reference, loaded into the current CUDA context."""

    def __init__(self, file: str, tmp_dir: str):
        import torch
        torch.cuda.current_stream()                          # makes torch's context current on this thread
        with open(compile_cubin(file, tmp_dir), "rb") as f:
            self._image = f.read()
        self._mod = ctypes.c_void_p()
        _ok(_driver().cuModuleLoadData(ctypes.byref(self._mod), self._image), f"loading {file}")
        self._fns: dict = {}
        self.file = file

    def function(self, name: str, smem: int = 0):
        fn = self._fns.get(name)
        if fn is None:
            fn = ctypes.c_void_p()
            _ok(_driver().cuModuleGetFunction(ctypes.byref(fn), self._mod, name.encode()), f"{self.file}:{name}")
            self._fns[name] = fn
        if smem > 48 * 1024:
            _ok(_driver().cuFuncSetAttribute(fn, 8, int(smem)), f"{name}: shared memory {smem}")   # MAX_DYNAMIC_SHARED_SIZE_BYTES
        return fn

    def launch(self, name: str, grid, block: int, smem: int, args: list, stream=None) -> None:
        import torch
        fn = self.function(name, smem)
        grid = tuple(grid) + (1,) * (3 - len(grid))
        params = (ctypes.c_void_p * len(args))(*[ctypes.cast(ctypes.pointer(a), ctypes.c_void_p) for a in args])
        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        _ok(_driver().cuLaunchKernel(fn, grid[0], grid[1], grid[2], block, 1, 1, smem, ctypes.c_void_p(s), params, None),
            f"launching {name}")


class Reference:
    """The reference's kernels behind Python functions that take torch tensors (all 32-bit floats unless said)."""

    def __init__(self):
        self._tmp = tempfile.TemporaryDirectory(prefix="kf_reference_")
        self._mods: dict = {}

    def module(self, file: str) -> Module:
        if file not in self._mods:
            self._mods[file] = Module(file, self._tmp.name)
        return self._mods[file]

    @staticmethod
    def _flat(n: int):
        return (max(1, min((n + 255) // 256, 65535)),)

    # norm.cu: one block of 256 threads per row (exec.rs:2506-2513)
    def rms_norm(self, x, w, eps: float):
        import torch
        out = torch.empty_like(x)
        self.module("norm.cu").launch("rms_norm", (x.shape[0],), 256, 0, [ptr(x), ptr(w), P(0), ptr(out), I(x.shape[1]), F(eps)])
        return out

    def rms_norm_add(self, x, w, res, eps: float):
        import torch
        out = torch.empty_like(x)
        self.module("norm.cu").launch("rms_norm_add", (x.shape[0],), 256, 0,
                                      [ptr(x), ptr(w), P(0), ptr(res), ptr(out), I(x.shape[1]), F(eps)])
        return out

    # rope.cu: positions as four streams per row (only stream 0 is read in mode 0), NeoX pairs
    def rope(self, x, positions, freq, n_head: int, head_dim: int):
        import torch
        rows = x.shape[0]
        out = torch.empty_like(x)
        rope4 = torch.zeros(rows, 4, dtype=torch.int32, device=x.device)
        rope4[:, 0] = positions
        half = freq.shape[0]
        n = x.numel()
        self.module("rope.cu").launch("rope", self._flat(n), 256, 0,
                                      [ptr(x), ptr(out), ptr(rope4), ptr(freq), I(rows), I(n_head), I(head_dim), I(half), I(1),
                                       F(1.0), I(0), I(0), I(0), I(0), I(1), I(0), F(1.0)])
        return out

    # elementwise.cu
    def softcap(self, a, cap: float):
        import torch
        out = torch.empty_like(a)
        self.module("elementwise.cu").launch("softcap", self._flat(a.numel()), 256, 0, [ptr(a), F(cap), ptr(out), I(a.numel())])
        return out

    def gated_gelu(self, gate, up):
        import torch
        out = torch.empty_like(gate)
        self.module("elementwise.cu").launch("gated_act", self._flat(gate.numel()), 256, 0,
                                             [ptr(gate), ptr(up), ptr(out), I(gate.numel()), I(1)])
        return out

    # attention.cu: the ring cache of the reference, [n_seq, cap, n_kv * d] half precision for keys and for values
    def make_cache(self, n_seq: int, cap: int, width: int, device):
        import torch
        return (torch.zeros(n_seq, cap, width, dtype=torch.float16, device=device),
                torch.zeros(n_seq, cap, width, dtype=torch.float16, device=device))

    def kv_append(self, k, v, kc, vc, pos, seq):
        rows, kw = k.shape
        cap = kc.shape[1]
        self.module("attention.cu").launch("kv_append", self._flat(rows * 2 * kw), 256, 0,
                                           [ptr(k), ptr(v), ptr(kc), ptr(vc), ptr(pos), ptr(seq), I(rows), I(kw), I(kw), I(cap)])

    def attention_classic(self, q, kc, vc, pos, seq, n_head, n_kv, d, scale, window, softcap):
        """The per-row kernel with one part (exec.rs:2643-2675)."""
        import torch
        rows = q.shape[0]
        out = torch.empty(rows, n_head * d, dtype=torch.float32, device=q.device)
        smem = (d + 8 + 4 * 512) * 4
        self.module("attention.cu").launch("attention", (rows, n_head, 1), 128, smem,
                                           [ptr(q), ptr(kc), ptr(vc), ptr(pos), ptr(seq), ptr(pos), P(0), ptr(out), P(0), I(128),
                                            I(n_head), I(n_kv), I(d), I(d), F(scale), I(window or 0), F(softcap), I(kc.shape[1]), P(0)])
        return out

    def attention_decode(self, q, kc, vc, pos, seq, n_head, n_kv, d, scale, window, softcap, parts: int | None = None, sm_count: int = 148):
        """attention_decode_hd{d}: grid (rows * n_kv, parts, ceil(group / 4)), 256 threads, parts = clamp(ceil(2 SMs /
        (rows * n_kv)), 2, 64) (exec.rs:1805-1815,2600-2629); partials [parts, rows, n_head, 2 + d], zeroed counters."""
        import torch
        rows = q.shape[0]
        if parts is None:
            parts = max(2, min(64, -(-2 * sm_count // (rows * n_kv))))
        nsplit = max(1, -(-(n_head // n_kv) // 4))
        out = torch.empty(rows, n_head * d, dtype=torch.float32, device=q.device)
        key = ("dec_scratch", rows, n_head, n_kv, d, parts)
        if getattr(self, "_scratch_key", None) != key:
            self._parts = torch.empty(parts * rows * n_head * (2 + d), dtype=torch.float32, device=q.device)
            self._counters = torch.zeros(rows * (n_kv * nsplit + 1) + 16, dtype=torch.int32, device=q.device)
            self._scratch_key = key
        args = [ptr(q), ptr(kc), ptr(vc), ptr(pos), ptr(seq), ptr(pos), P(0), ptr(out), ptr(self._parts), I(n_head), I(n_kv), F(scale),
                I(window or 0), F(softcap), I(kc.shape[1]), I(rows), ptr(self._counters), I(0)]
        args += [P(0)] * 5                                                        # no quantised output
        args += [P(0), P(0), P(0), P(0), I(0), I(0), F(0.0)] + [I(0)] * 5         # no rope folded in
        args += [I(0), P(0), P(0), F(0.0), I(0), P(0), P(0), F(0.0)]              # no q / k norms
        args += [P(0)]                                                            # no tree
        self.module("attention.cu").launch(f"attention_decode_hd{d}", (rows * n_kv, parts, nsplit), 256, 0, args)
        return out

    def flash_tiles(self, pos, runs, device):
        """The tile table of flash_prefill: tiles of 64 rows of one slot, heaviest first (exec.rs:1825-1848); `runs` is a
        list of (slot, first row, row count).  Returns (device table, tile count)."""
        import torch
        tiles = []
        pos_h = pos.tolist()
        for slot, r0, n in runs:
            r = r0
            while r < r0 + n:
                m = min(64, r0 + n - r)
                tiles.append((pos_h[r + m - 1], r, m, slot))
                r += m
        tiles.sort(key=lambda t: -t[0])
        table = [len(tiles), 0, 0, 0]
        for _, r, m, slot in tiles:
            table += [r, m, slot, 0]
        return torch.tensor(table, dtype=torch.int32, device=device), len(tiles)

    def flash_prefill(self, q, kc, vc, pos, seq, runs, n_head, n_kv, d, scale, window, softcap, tiles=None):
        """flash_prefill_hd{d} over the rows of `runs` (see flash_tiles; pass its result as `tiles` to keep the call free
        of host reads, e.g. under graph capture)."""
        import torch
        tiles_dev, n_tiles = tiles if tiles is not None else self.flash_tiles(pos, runs, q.device)
        out = torch.empty(q.shape[0], n_head * d, dtype=torch.float32, device=q.device)
        nch = -(-(d // 8) // 8) * 8
        bk = 64 if d <= 128 else 32
        smem = (64 + 4 * bk) * nch * 16
        self._keep = tiles_dev
        self.module("flash.cu").launch(f"flash_prefill_hd{d}", (n_tiles, n_head, 1), 128, smem,
                                       [ptr(q), ptr(kc), ptr(vc), ptr(pos), ptr(seq), ptr(pos), ptr(tiles_dev), P(0), ptr(out),
                                        I(n_head), I(n_kv), F(scale), I(window or 0), F(softcap), I(kc.shape[1])])
        return out

    # quant_bf16.cu: y = x . w^T with bfloat16 weight rows; x must already be rounded to bfloat16 values (exec.rs:2094-2112)
    def linear_bf16(self, w, x):
        import torch
        rows, n = x.shape
        n_out = w.shape[0]
        y = torch.empty(rows, n_out, dtype=torch.float32, device=x.device)
        args = [ptr(w), ptr(x), P(0), P(0), ptr(y), I(rows), I(n), I(n_out), L(n * 2)]
        if rows <= 8:
            self.module("quant_bf16.cu").launch("matvec", (-(-n_out // 4),), 128, 0, args)
        else:
            self.module("quant_bf16.cu").launch("matmul", (-(-n_out // 64), -(-rows // 32)), 256, 0, args)
        return y
