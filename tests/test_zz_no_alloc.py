"""The allocation-free decode attention entry point, called through its exported C symbol.

Some hosts of the kernel library cannot allocate device memory when they call it (a runtime that only hands out
a fixed arena, code running under stream capture, a real-time loop), so `kf_attention_decode_static` keeps its
scratch (split partials and arrival counters) in arrays that are part of the library.  This test calls it twice in
a row, on different inputs, and checks each result against the ordinary entry point, which gets its scratch from
the caller.  It runs last so that a failure here cannot hide another test's.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _case(seed, lens, nh, nkv, d, P):
    from test_gpu_kernels import _Ctx, _paged_setup
    pages, table, _ks, _vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, lens, seed=seed)
    rows = [(r, n - 1) for r, n in enumerate(lens)]
    g = torch.Generator().manual_seed(seed + 1)
    q = torch.randn(len(rows), nh * d, generator=g).to(torch.bfloat16).to(DEV)
    ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
               torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV),
               dec_rows=list(range(len(rows))), pre_rows=[])
    return q, pages.to(DEV), ctx


@pytest.mark.parametrize("nh,nkv,d,P,window,cap", [(8, 4, 256, 64, None, 50.0), (6, 2, 32, 16, 40, 20.0)])
def test_static_entry_point_matches_the_ordinary_one(nh, nkv, d, P, window, cap):
    from kungfu_b200 import ops
    from test_gpu_kernels import _View
    lib = ops.library()
    fn = lib.kf_attention_decode_static                       # the exported C symbol
    fn.restype = ctypes.c_int
    scale = 1.0 / math.sqrt(d)
    for call, (seed, lens) in enumerate([(31, [5, 2100, 700, 64]), (41, [900, 3, 1500, 65, 129])]):
        q, pages, ctx = _case(seed, lens, nh, nkv, d, P)
        want = torch.empty_like(q)
        ops.paged_attention(q, want, ctx, _View(pages, P), nh, nkv, d, scale, cap, window)
        got = torch.full_like(q, float("nan"))
        table = ctx.block_tables[0]
        max_keys = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = fn(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(got.data_ptr()), ctypes.c_void_p(pages.data_ptr()),
                q.shape[0], ctypes.c_void_p(ctx.positions.data_ptr()), ctypes.c_void_p(ctx.row_req.data_ptr()),
                ctypes.c_void_p(table.data_ptr()), table.shape[1], P, nh, nkv, d, ctypes.c_float(scale),
                ctypes.c_float(cap), int(window or 0), int(max_keys), stream)
        assert rc == 0, f"call {call}: status {rc} ({lib.kf_last_cuda_error().decode()})"
        torch.cuda.synchronize()
        a, b = got.float().cpu(), want.float().cpu()
        assert bool(torch.isfinite(a).all()), f"call {call}"
        rel = float((a - b).abs().max() / b.abs().max())
        assert rel < 1e-2, f"call {call}: rel err {rel}"


def test_static_entry_point_refuses_what_does_not_fit():
    from kungfu_b200 import ops
    lib = ops.library()
    fn = lib.kf_attention_decode_static
    fn.restype = ctypes.c_int
    null = ctypes.c_void_p(0)
    # 3000 rows x 32 heads x (256 + 2) floats per split exceeds the built-in scratch: refused before any launch
    rc = fn(null, null, null, 3000, null, null, null, 4, 64, 32, 16, 256, ctypes.c_float(1.0), ctypes.c_float(0.0), 0,
            100000, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 2
    assert b"scratch" in lib.kf_last_cuda_error()
