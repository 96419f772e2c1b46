"""The operations parts are written in, each one a hand-written CUDA kernel of `csrc/`.

Every function here checks its arguments on the host and launches on the current CUDA stream.
There is no CPU implementation and no library fallback: a tensor that is not on a CUDA device, a
missing compiler or a failed build raises.  (Tests that have no GPU replace this table of
functions with a slow emulation of their own through `set_override`; the package ships none.)
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

F32, BF16 = 0, 1
_ACT = {"gelu_tanh": 0, "gelu_erf": 1, "silu": 2}
_STATUS = {1: "unsupported combination of element types", 2: "unsupported size", 3: "CUDA launch failed",
           4: "alignment rule broken", 5: "one-time set-up failed"}

MAX_HEAD_DIM = 256


class KernelError(RuntimeError):
    pass


_lib = None
_lib_lock = threading.Lock()
_override = None


def set_override(impl) -> None:
    """Tests without a GPU install an object whose attributes replace the functions of this module."""
    global _override
    _override = impl


def library():
    """The compiled kernel library (built at first use)."""
    global _lib
    if _lib is None:
        with _lib_lock:
            if _lib is None:
                from .csrc import build as _build
                path = _build.build()
                lib = ctypes.CDLL(path)
                lib.kf_last_cuda_error.restype = ctypes.c_char_p
                # kernels may start before their predecessor in the stream has finished (each waits for it before
                # touching dependent memory); KUNGFU_PDL=0 switches that off
                lib.kf_set_pdl(0 if os.environ.get("KUNGFU_PDL", "1") == "0" else 1)
                _lib = lib
    return _lib


def library_path() -> str:
    from .csrc import build as _build
    return os.path.join(_build.build_dir(), _build.LIB_NAME)


_launches = 0
_fallbacks: dict[str, int] = {}


def note_fallback(what: str) -> None:
    """A bfloat16 operation that ran on a slower generic kernel because the fast one refuses its shape."""
    _fallbacks[what] = _fallbacks.get(what, 0) + 1


def fallbacks() -> dict[str, int]:
    """How often, and why, bfloat16 work left the tensor-core kernels (shown by `describe` and the bench)."""
    return dict(_fallbacks)


def fallback_count() -> int:
    return sum(_fallbacks.values())


def launch_count() -> int:
    """Kernels launched through this module so far (graph replays add the kernels they hold)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    _launches += 1
    if status != 0:
        detail = _STATUS.get(status, f"status {status}")
        if status == 3:
            detail += f" ({library().kf_last_cuda_error().decode()})"
        raise KernelError(f"{what}: {detail}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {t.dtype} is not supported (float32 and bfloat16 are)")


def _p(t: torch.Tensor | None):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kungfu_b200 kernels run on CUDA tensors only; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError("kernel arguments must be contiguous")
    return ctypes.c_void_p(t.data_ptr())


_pinned_stream = None


def _stream():
    if _pinned_stream is not None:
        return _pinned_stream
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class pinned_stream:
    """Within this context every launch goes to the stream that is current on entry, looked up once (asking torch for the
    current stream costs as much as a launch).  The step function wraps the model's pass in it."""

    def __enter__(self):
        global _pinned_stream
        self._was = _pinned_stream
        _pinned_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self._was
        return False


def _f(x: float):
    return ctypes.c_float(x)


# ---- per-kernel timing (the reference's KF_TRACE_KERNELS, crates/kf-backend-cuda/src/exec.rs:2836-2853) -----------
_trace: list | None = None


def trace_begin() -> None:
    """Start timing every operation of this module with CUDA events (steps then run eagerly, not from graphs)."""
    global _trace
    _trace = []


def trace_end() -> list[tuple[str, float]]:
    """Stop timing; returns (operation, milliseconds) in launch order."""
    global _trace
    rec, _trace = _trace or [], None
    if rec:
        torch.cuda.synchronize()
    return [(name, e0.elapsed_time(e1)) for name, e0, e1 in rec]


def tracing() -> bool:
    return _trace is not None


# NVTX ranges around every part and operation, for timelines of a profiler (KUNGFU_NVTX=1 or ops.nvtx_ranges = True).
nvtx_ranges = os.environ.get("KUNGFU_NVTX", "0") == "1"


class nvtx_range:
    """`with ops.nvtx_range("layer 3"):` opens an NVTX range when ranges are switched on, and costs a test otherwise."""

    def __init__(self, name: str):
        self.name = name
        self.on = False

    def __enter__(self):
        self.on = nvtx_ranges and _override is None
        if self.on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()
        return False


def _dispatch(name):
    def deco(fn):
        def wrapper(*a, **k):
            if _override is not None:
                return getattr(_override, name)(*a, **k)
            if nvtx_ranges:
                with nvtx_range(name):
                    return fn(*a, **k)
            if _trace is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = fn(*a, **k)
                e1.record()
                _trace.append((name, e0, e1))
                return out
            return fn(*a, **k)
        wrapper.__name__ = name
        wrapper.__wrapped__ = fn
        wrapper.__doc__ = fn.__doc__
        return wrapper
    return deco


# ---- size rules ---------------------------------------------------------------------------------------

def check_attention_sizes(n_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """Head sizes the attention kernels take: 2..256, even.  Anything else is refused here, at build time."""
    if head_dim < 2 or head_dim > MAX_HEAD_DIM or head_dim % 2:
        raise KernelError(f"head_dim {head_dim} is not supported: the attention kernels take even sizes up to {MAX_HEAD_DIM}")
    if n_kv_heads < 1 or n_heads % n_kv_heads:
        raise KernelError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")


# ---- operations -----------------------------------------------------------------------------------------

@_dispatch("embed")
def embed(tokens, table, scale: float, out) -> None:
    """out[t, :] = table[tokens[t], :] * scale (32-bit out).  Token ids are validated by the caller on the host."""
    T, (V, H) = out.shape[0], table.shape
    _check(library().kf_embed(_p(tokens), _p(table), _dt(table), _f(scale), _p(out), T, H, V, ctypes.c_void_p(0), _stream()),
           "embed")


@_dispatch("rmsnorm")
def rmsnorm(x, weight, eps: float, plus_one: bool, out, rows=None) -> None:
    """out[r] = rmsnorm(x[rows[r]] if rows is given else x[r]) * (weight or 1 + weight)."""
    n, H = out.shape
    _check(library().kf_rmsnorm(_p(x), _p(weight), _dt(weight), _f(eps), int(plus_one), _p(out), _dt(out), _p(rows), n, H,
                                _stream()), "rmsnorm")


@_dispatch("add_rmsnorm")
def add_rmsnorm(branch, weight, eps: float, plus_one: bool, residual, *, next_weight=None, next_eps: float = 0.0,
                next_plus_one: bool = False, next_out=None) -> None:
    """residual += rmsnorm(branch) * g; if next_out is given, next_out = rmsnorm(residual) * g_next."""
    T, H = residual.shape
    _check(library().kf_add_rmsnorm(_p(branch), _p(weight), _dt(weight), _f(eps), int(plus_one), _p(residual),
                                    _p(next_weight), _dt(next_weight) if next_weight is not None else F32, _f(next_eps),
                                    int(next_plus_one), _p(next_out), _dt(next_out) if next_out is not None else F32,
                                    T, H, _stream()), "add_rmsnorm")


@_dispatch("add")
def add(a, x) -> None:
    """x += a (32-bit)."""
    _check(library().kf_add(_p(a), _p(x), ctypes.c_long(x.numel()), _stream()), "add")


# ---- scratch memory of the split-K products and the device error word ---------------------------------------

_scratch: dict = {}          # device -> {"partial": tensor, "counters": tensor, "error": tensor, "retired": [tensors]}
use_tensor_cores = True      # tests switch this off to reach the generic product with bfloat16 operands
use_fast_attention = True    # likewise for the generic attention kernel
fused_qkv_rope = True        # False: the q,k,v product of a prompt always leaves 32-bit rows for `rope_kv_append`
fused_qkv_rope_launches = 0  # how often the product that rotates and files its own result has run (tests look at it)
prefill_on_tcgen05 = True       # False: the mma.sync prompt kernel for every head and page size
split_prompt_keys = True        # False: one block per (tile of rows, head) however few blocks that makes
decode_on_tensor_cores = True   # False: the SIMT split-KV decode kernel (kept for groups of more than 16 heads)
prefill_plan_override = None    # (runs per tile, key tiles above which a tile is cut): tests reach every launch shape with it


def _dev_scratch(device) -> dict:
    key = (device.type, device.index)
    sc = _scratch.get(key)
    if sc is None:
        sc = {"partial": torch.empty(1 << 20, dtype=torch.float32, device=device),
              "counters": torch.zeros(8192, dtype=torch.int32, device=device),
              "error": torch.zeros(1, dtype=torch.int32, device=device), "retired": []}
        _scratch[key] = sc
    return sc


def _partial(device, n_floats: int) -> torch.Tensor:
    sc = _dev_scratch(device)
    if sc["partial"].numel() < n_floats:
        sc["retired"].append(sc["partial"])          # a captured graph may still point at it
        sc["partial"] = torch.empty(max(n_floats, 2 * sc["partial"].numel()), dtype=torch.float32, device=device)
    return sc["partial"]


def device_error(device=None) -> int:
    """The error word kernels with bounded waits write (0 = none).  Reading it waits for the device."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    sc = _scratch.get((device.type, device.index))
    return 0 if sc is None else int(sc["error"].item())


def clear_device_error(device=None) -> None:
    """Set the error word back to 0 (after a failure that was looked at)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    sc = _scratch.get((device.type, device.index))
    if sc is not None:
        sc["error"].zero_()


def raise_on_device_error(device=None) -> None:
    code = device_error(device)
    if code:
        raise KernelError(f"a kernel gave up waiting (code {code}: 1 = operands never arrived, 2 = stage never freed, "
                          f"3 = accumulator never completed)")


_rope_plans: dict = {}            # (rows, K, heads, kv heads, head size, rotated) -> whether the fused q,k,v product takes them
_linear_plans: dict = {}          # (rows, features, K, mode) -> (token tile, K splits) as the library plans them


def _linear_tc(x, weight, out, mode: int, N: int, softcap: float, act: int) -> bool:
    """Launch the tcgen05 product if it takes these operands; False if the generic kernel must run."""
    T, K = x.shape
    lib = library()
    if not (use_tensor_cores and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16):
        return False
    if not lib.kf_linear_tc_supported(_p(x), _p(weight), K):
        note_fallback(f"linear: rows of {K} bfloat16 elements are no multiple of 16 bytes (or a base is unaligned)")
        return False
    plan = _linear_plans.get((T, N, K, mode))
    if plan is None:
        bn, splits = ctypes.c_int(0), ctypes.c_int(0)
        lib.kf_linear_tc_plan(T, N, K, int(mode == 2), ctypes.byref(bn), ctypes.byref(splits))
        plan = _linear_plans[(T, N, K, mode)] = (bn.value, splits.value)
    bn, splits = plan
    sc = _dev_scratch(x.device)
    partial = None
    if splits > 1:
        if -(-N // 128) * -(-T // bn) > sc["counters"].numel():
            note_fallback("linear: more output tiles than split counters")
            return False
        partial = _partial(x.device, splits * T * (2 * N if mode == 2 else N))
    _check(lib.kf_linear_tc(_p(x), _p(weight), _p(out), mode, T, N, K, _f(softcap), act, bn, splits,
                            _p(partial), _p(sc["counters"]), _p(sc["error"]), _stream()), "linear (tensor cores)")
    return True


@_dispatch("linear")
def linear(x, weight, out, softcap: float = 0.0) -> None:
    """out[T, N] = x[T, K] . weight[N, K]^T, 32-bit accumulation; softcap > 0 applies cap*tanh(v/cap).
    bfloat16 operands run on the tensor cores (tcgen05) when rows are multiples of 16 bytes; everything else,
    and the whole 32-bit path, runs the generic 32-bit FMA kernel."""
    T, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or tuple(out.shape) != (T, N):
        raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(weight.shape)} out{tuple(out.shape)} do not agree")
    if out.dtype == torch.float32 or softcap == 0.0:
        if _linear_tc(x, weight, out, 0 if out.dtype == torch.float32 else 1, N, softcap, 0):
            return
    _check(library().kf_linear_simt(_p(x), _dt(x), _p(weight), _dt(weight), _p(out), _dt(out), T, N, K, _f(softcap),
                                    _stream()), "linear")


@_dispatch("linear_gated")
def linear_gated(x, w_gate_up, out, activation: str, ctx) -> None:
    """out[T, I] = act(x . Wgate^T) * (x . Wup^T) with w_gate_up = [Wgate; Wup] stacked by rows."""
    T = x.shape[0]
    I = out.shape[1]
    if out.dtype == torch.bfloat16 and _linear_tc(x, w_gate_up, out, 2, I, 0.0, _ACT[activation]):
        return
    gu = ctx.buf("ffn_gate_up", (T, 2 * I), torch.float32)
    linear(x, w_gate_up, gu)
    _check(library().kf_gated_act(_p(gu), _dt(gu), _p(out), _dt(out), T, I, _ACT[activation], _stream()), "gated_act")


@_dispatch("rope_table")
def rope_table(positions, inv_freq, cos, sin) -> None:
    """cos/sin[t, i] of positions[t] * inv_freq[i], 32-bit."""
    T, half = cos.shape
    _check(library().kf_rope_table(_p(positions), _p(inv_freq), _p(cos), _p(sin), T, half, _stream()), "rope_table")


@_dispatch("rope_kv_append")
def rope_kv_append(qkv, cos, sin, rot: int, n_heads: int, n_kv_heads: int, head_dim: int, ctx, cache, q_out) -> None:
    """Rotate q and k (pairs i, i+rot/2), write q to q_out and k, v into the pages of `cache` (if it writes)."""
    T = qkv.shape[0]
    table = ctx.block_tables[cache.group]
    _check(library().kf_rope_kv_append(_p(qkv), _p(cos), _p(sin), rot, n_heads, n_kv_heads, head_dim,
                                       _p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1], cache.page_size,
                                       _p(cache.pages), _dt(cache.pages), _p(q_out), _dt(q_out), int(cache.writes),
                                       T, _stream()), "rope_kv_append")


@_dispatch("linear_rope_kv_append")
def linear_rope_kv_append(x, wqkv, cos, sin, rot: int, n_heads: int, n_kv_heads: int, head_dim: int, ctx, cache, q_out) -> bool:
    """q,k,v = x . wqkv^T, q and k rotated, q to q_out, k and v into the pages of `cache`: one launch whose product files
    its own result (no 32-bit q,k,v rows in memory).  True if it ran; False if this step does not qualify (then the
    caller runs `linear` and `rope_kv_append`): it takes bfloat16 operands, q and pages, head size 256 or 128 rotated in full,
    and so many rows that the product runs as whole tiles on CTA pairs."""
    T, K = x.shape
    if not (use_tensor_cores and fused_qkv_rope and cos is not None and x.dtype == torch.bfloat16
            and wqkv.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16 and cache.pages.dtype == torch.bfloat16):
        return False
    lib = library()
    key = (T, K, n_heads, n_kv_heads, head_dim, rot)
    ok = _rope_plans.get(key)
    if ok is None:
        ok = _rope_plans[key] = bool(lib.kf_linear_rope_append_supported(_p(x), _p(wqkv), T, K, n_heads, n_kv_heads, head_dim, rot))
    if not ok or (x.data_ptr() | wqkv.data_ptr()) & 15:
        return False
    table = ctx.block_tables[cache.group]
    sc = _dev_scratch(x.device)
    global fused_qkv_rope_launches
    fused_qkv_rope_launches += 1
    _check(lib.kf_linear_rope_append(_p(x), _p(wqkv), T, K, n_heads, n_kv_heads, head_dim, _p(cos), _p(sin), _p(ctx.positions),
                                     _p(ctx.row_req), _p(table), table.shape[1], cache.page_size, _p(cache.pages), _p(q_out),
                                     int(cache.writes), _p(sc["error"]), _stream()), "linear_rope_kv_append")
    return True


@_dispatch("paged_attention")
def paged_attention(q, out, ctx, cache, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, softcap: float,
                    window: int | None) -> None:
    """Causal (optionally windowed, softcapped) attention of every row of the step over its request's pages.
    bfloat16: rows of single-row requests run the split-KV decode kernel, the rest the prefill kernel, when the
    head size has an instance of them; the 32-bit path and other head sizes run the generic kernel."""
    T = q.shape[0]
    lib = library()
    table = ctx.block_tables[cache.group]
    pages = cache.pages
    common = (_p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1], cache.page_size, n_heads, n_kv_heads, head_dim,
              _f(scale), _f(softcap), int(window or 0))
    n_dec = getattr(ctx, "n_dec_rows", 0)
    fast = (use_fast_attention and q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16)
    if fast and n_dec > 0 and lib.kf_attention_decode_supported(head_dim):
        ht, splits = ctypes.c_int(0), ctypes.c_int(0)
        max_keys = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        group = n_heads // n_kv_heads
        if decode_on_tensor_cores and group <= 16:
            lib.kf_attention_decode_mma_plan(n_dec, n_heads, n_kv_heads, head_dim, int(max_keys), ctypes.byref(splits))
            n_counters = n_dec * n_kv_heads                      # ht stays 0: the tensor-core variant
        else:
            lib.kf_attention_decode_plan(n_dec, n_heads, n_kv_heads, head_dim, int(max_keys), ctypes.byref(ht), ctypes.byref(splits))
            n_counters = n_dec * n_kv_heads * -(-group // ht.value)
        sc = _dev_scratch(q.device)
        if n_counters > sc["counters"].numel():
            rest, n_rest = None, T
        else:
            partial = _partial(q.device, T * n_heads * splits.value * (head_dim + 4)) if splits.value > 1 else None
            items = None if n_dec == T else ctx.dec_rows
            _check(lib.kf_attention_decode(_p(q), _p(out), _p(pages), _p(items), n_dec, *common[:8], *common[8:], ht.value,
                                           splits.value, _p(partial), _p(sc["counters"]), _stream()), "attention (decode)")
            if n_dec == T:
                return
            rest, n_rest = ctx.pre_rows, ctx.n_pre_rows
    elif fast and n_dec == 0 and getattr(ctx, "n_pre_rows", 0) == T:
        rest, n_rest = ctx.pre_rows, T
    else:
        rest, n_rest = None, T
    prompt_tiles = fast and rest is not None and n_rest == ctx.n_pre_rows and getattr(ctx, "n_tiles", 0) > 0
    if (prompt_tiles and prefill_on_tcgen05 and getattr(ctx, "n_wide", 0) > 0
            and lib.kf_attention_prefill_tc_supported(head_dim, cache.page_size, _p(q), _p(pages))):
        sc = _dev_scratch(q.device)
        max_keys = min(ctx.max_kv_len, window + 128) if window else ctx.max_kv_len
        run_tiles = ctypes.c_int(0)
        if prefill_plan_override is not None:
            parts, run_tiles = int(prefill_plan_override[0]), ctypes.c_int(int(prefill_plan_override[1]))
        else:
            parts = lib.kf_attention_prefill_tc_plan(ctx.n_wide, n_heads, int(max_keys), ctypes.byref(run_tiles)) if split_prompt_keys else 1
        partial = _partial(q.device, T * n_heads * parts * (head_dim + 4)) if parts > 1 else None
        _check(lib.kf_attention_prefill_tc(_p(q), _p(out), _p(pages), ctypes.c_long(pages.shape[0]), T, _p(ctx.wide_row0),
                                           _p(ctx.wide_nrows), ctx.n_wide, *common, _p(sc["error"]), parts, run_tiles.value,
                                           _p(partial), _stream()),
               "attention (prefill, tcgen05)")
        if parts > 1:
            add_launches(1)
        return
    if prompt_tiles and lib.kf_attention_prefill_supported(head_dim):
        _check(lib.kf_attention_prefill(_p(q), _p(out), _p(pages), _p(ctx.tile_row0), _p(ctx.tile_nrows), ctx.n_tiles,
                                        *common, _stream()), "attention (prefill)")
        return
    if fast and use_fast_attention:
        note_fallback(f"attention: head size {head_dim} or page size {cache.page_size} has no tensor-core kernel")
    _check(lib.kf_attention_generic(_p(q), _p(out), _dt(q), _p(pages), _dt(pages), _p(rest), *common, n_rest, _stream()),
           "attention (generic)")


fuse_rope_into_decode = os.environ.get("KUNGFU_FUSE_ROPE", "1") != "0"   # False: rotation and append always run as their own kernel


def decode_attention_takes_qkv(ctx, cache, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether `rope_append_attend` can run this step's attention: every row is the single row of its request (a decode
    step), bfloat16 pages, and the tensor-core decode kernel has an instance for the head size and group."""
    if _override is not None or not (fuse_rope_into_decode and use_fast_attention and decode_on_tensor_cores):
        return False
    T = ctx.n_rows
    if T <= 0 or getattr(ctx, "n_dec_rows", 0) != T or cache is None or cache.pages.dtype != torch.bfloat16:
        return False
    if n_heads // n_kv_heads > 16 or not library().kf_attention_decode_supported(head_dim):
        return False
    return T * n_kv_heads <= _dev_scratch(cache.pages.device)["counters"].numel()


@_dispatch("rope_append_attend")
def rope_append_attend(qkv, cos, sin, rot: int, out, ctx, cache, n_heads: int, n_kv_heads: int, head_dim: int,
                       scale: float, softcap: float, window: int | None) -> None:
    """For a decode step: rotate q and k, append k and v to the pages and attend, in the split-KV decode kernel itself
    (one launch instead of two).  qkv: 32-bit [T, (n_heads + 2 n_kv_heads) * head_dim]; out: bfloat16 [T, n_heads * head_dim]."""
    T = qkv.shape[0]
    lib = library()
    table = ctx.block_tables[cache.group]
    max_keys = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
    splits = ctypes.c_int(0)
    lib.kf_attention_decode_mma_plan(T, n_heads, n_kv_heads, head_dim, int(max_keys), ctypes.byref(splits))
    sc = _dev_scratch(qkv.device)
    partial = _partial(qkv.device, T * n_heads * splits.value * (head_dim + 4)) if splits.value > 1 else None
    _check(lib.kf_attention_decode_fused(_p(qkv), _p(cos), _p(sin), int(rot), int(cache.writes), _p(out), _p(cache.pages),
                                         None, T, _p(ctx.positions), _p(ctx.row_req), _p(table), table.shape[1],
                                         cache.page_size, n_heads, n_kv_heads, head_dim, _f(scale), _f(softcap),
                                         int(window or 0), splits.value, _p(partial), _p(sc["counters"]), _stream()),
           "attention (decode, rotation and append inside)")


@_dispatch("argmax")
def argmax(logits, out) -> None:
    """out[r] = index of the first maximum of logits[r, :] (int32)."""
    rows, V = logits.shape
    sc = _dev_scratch(logits.device)
    if "argmax" not in sc or sc["argmax"].numel() < rows * 128:
        if "argmax" in sc:
            sc["retired"].append(sc["argmax"])
        sc["argmax"] = torch.empty(max(rows, 64) * 128, dtype=torch.float32, device=logits.device)
    _check(library().kf_argmax(_p(logits), _p(out), rows, V, _p(sc["argmax"]), _stream()), "argmax")


def _sample_scratch(device, rows: int, V: int, full: bool) -> dict:
    lib = library()
    sc = _dev_scratch(device)
    n_slices = lib.kf_sample_slices(V)
    need = rows * n_slices
    if sc.get("sample_rows", 0) < need:
        for k in ("sample_keys", "sample_stats", "sample_flags"):
            if k in sc:
                sc["retired"].append(sc[k])
        cap = max(need, 64 * n_slices)
        sc["sample_keys"] = torch.empty(cap * 64, dtype=torch.int64, device=device)
        sc["sample_stats"] = torch.empty(cap * 2, dtype=torch.float32, device=device)
        sc["sample_flags"] = torch.zeros(max(rows, 64) * 2, dtype=torch.int32, device=device)
        sc["sample_rows"] = cap
    if sc["sample_flags"].numel() < rows:
        sc["retired"].append(sc["sample_flags"])
        sc["sample_flags"] = torch.zeros(rows * 2, dtype=torch.int32, device=device)
    if full and sc.get("sample_pen_n", 0) < rows * V:
        if "sample_pen" in sc:
            sc["retired"].append(sc["sample_pen"])
        sc["sample_pen"] = torch.empty(rows * V, dtype=torch.float32, device=device)
        sc["sample_pen_n"] = rows * V
    return sc


@_dispatch("sample")
def sample(logits, states, out_ids, *, logit_rows=None, row_req=None, req_slot=None, whole_ranking: bool = False,
           cand_ids=None, cand_vals=None, cand_lse=None) -> None:
    """The end of a step, on the device: out_ids[i] = the token row i of `logits` yields under the rules, generator and
    recent tokens of its request's state (`states` [requests, STATE_WORDS] int32, see sampling/sampler.py), which the
    kernels update.  The request of row i is req_slot[row_req[logit_rows[i]]] (each map None for the identity; rows of
    a negative request are skipped).  `whole_ranking`: some request's rules reach below the 64th candidate (top_k of 0
    or above 64 at a temperature above 0); one more kernel then runs.  cand_*: also write the ranked candidates."""
    rows, V = logits.shape
    sc = _sample_scratch(logits.device, rows, V, whole_ranking)
    k = 0 if cand_ids is None else cand_ids.shape[1]
    _check(library().kf_sample(_p(logits), rows, V, _p(sc["sample_keys"]), _p(sc["sample_stats"]), _p(cand_ids), _p(cand_vals),
                               _p(cand_lse), k, _p(logit_rows), _p(row_req), _p(req_slot), _p(states), _p(out_ids),
                               _p(sc["sample_flags"]), _p(sc["sample_pen"]) if whole_ranking else None,
                               int(whole_ranking), _stream()), "sample")
    add_launches(2 if whole_ranking else 1)


@_dispatch("topk_lse")
def topk_lse(logits, k: int, out_ids, out_vals, out_lse) -> None:
    """Top-k ids (falling value, lower id first among equals), their values, and the row's log-sum-exp; k <= 64."""
    rows, V = logits.shape
    if k < 1 or k > 64 or k > V:
        raise KernelError(f"topk_lse: k = {k} is not in 1..min(64, {V})")
    sc = _sample_scratch(logits.device, rows, V, False)
    _check(library().kf_sample(_p(logits), rows, V, _p(sc["sample_keys"]), _p(sc["sample_stats"]), _p(out_ids), _p(out_vals),
                               _p(out_lse), k, None, None, None, None, None, None, None, 0, _stream()), "topk_lse")
    add_launches(1)


def device_arch() -> int:
    return int(library().kf_device_arch())
