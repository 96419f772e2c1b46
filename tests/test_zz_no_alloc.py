"""The allocation-free decode attention entry point, called through its exported C symbol.

Some hosts of the kernel library cannot allocate device memory when they call it (a runtime that only hands out
a fixed arena, code running under stream capture, a real-time loop), so `kf_attention_decode_static` keeps its
scratch (split partials and arrival counters) in arrays that are part of the library.  This test calls it twice in
a row, on different inputs, and checks each result against the ordinary entry point, which gets its scratch from
the caller, and against a float64 restatement of the attention.  It runs last so that a failure here cannot hide
another test's.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _case(seed, lens, nh, nkv, d, P):
    from test_gpu_kernels import _Ctx, _paged_setup
    pages, table, ks, vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, lens, seed=seed)
    rows = [(r, n - 1) for r, n in enumerate(lens)]
    g = torch.Generator().manual_seed(seed + 1)
    q = torch.randn(len(rows), nh * d, generator=g).to(torch.bfloat16).to(DEV)
    ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
               torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV),
               dec_rows=list(range(len(rows))), pre_rows=[])
    return q, pages.to(DEV), ctx, ks, vs


def _call(lib, q, got, pages, ctx, P, nh, nkv, d, scale, cap, window):
    fn = lib.kf_attention_decode_static                       # the exported C symbol
    fn.restype = ctypes.c_int
    table = ctx.block_tables[0]
    max_keys = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return fn(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(got.data_ptr()), ctypes.c_void_p(pages.data_ptr()),
              q.shape[0], ctypes.c_void_p(ctx.positions.data_ptr()), ctypes.c_void_p(ctx.row_req.data_ptr()),
              ctypes.c_void_p(table.data_ptr()), table.shape[1], P, nh, nkv, d, ctypes.c_float(scale),
              ctypes.c_float(cap), int(window or 0), int(max_keys), stream)


@pytest.mark.parametrize("nh,nkv,d,P,window,cap", [(8, 4, 256, 64, None, 50.0), (6, 2, 32, 16, 40, 20.0)])
def test_static_entry_point_matches_the_ordinary_one(nh, nkv, d, P, window, cap):
    from kungfu_b200 import ops
    from test_gpu_kernels import _View, _attn_ref
    lib = ops.library()
    scale = 1.0 / math.sqrt(d)
    for call, (seed, lens) in enumerate([(31, [5, 2100, 700, 64]), (41, [900, 3, 1500, 65, 129])]):
        q, pages, ctx, ks, vs = _case(seed, lens, nh, nkv, d, P)
        want = torch.empty_like(q)
        ops.paged_attention(q, want, ctx, _View(pages, P), nh, nkv, d, scale, cap, window)
        got = torch.full_like(q, float("nan"))
        rc = _call(lib, q, got, pages, ctx, P, nh, nkv, d, scale, cap, window)
        assert rc == 0, f"call {call}: status {rc} ({lib.kf_last_cuda_error().decode()})"
        torch.cuda.synchronize()
        a, b = got.float().cpu(), want.float().cpu()
        assert bool(torch.isfinite(a).all()), f"call {call}"
        rel = float((a - b).abs().max() / b.abs().max())
        assert rel < 1e-2, f"call {call}: rel err {rel} against the ordinary entry point"
        ref = torch.stack([_attn_ref(q[r].view(nh, d).cpu(), ks[r], vs[r], n - 1, nh, nkv, scale, cap, window)
                           for r, n in enumerate(lens)]).view(len(lens), nh * d)
        rel = float((a.double() - ref).abs().max() / ref.abs().max())
        assert rel < 1e-2, f"call {call}: rel err {rel} against float64"


def test_static_entry_point_takes_any_size_when_one_split_suffices():
    """Many rows leave nothing to cut: the plan is one split, which uses neither built-in array, so a launch whose
    rows x heads x (head_dim + 4) is far beyond the arrays is still taken, and is right."""
    from kungfu_b200 import ops
    from test_gpu_kernels import _attn_ref
    lib = ops.library()
    nh, nkv, d, P = 8, 4, 256, 64
    lens = [3 + (i * 7) % 60 for i in range(1200)]            # 1200 rows x 8 heads x 260 floats > 2 Mi floats
    q, pages, ctx, ks, vs = _case(51, lens, nh, nkv, d, P)
    assert lib.kf_attention_decode_static_fits(len(lens), nh, nkv, d, 2, 2) == 2
    got = torch.full_like(q, float("nan"))
    rc = _call(lib, q, got, pages, ctx, P, nh, nkv, d, 1.0 / 16.0, 50.0, None)
    assert rc == 0, lib.kf_last_cuda_error().decode()
    torch.cuda.synchronize()
    pick = list(range(0, len(lens), 97)) + [len(lens) - 1]
    ref = torch.stack([_attn_ref(q[r].view(nh, d).cpu(), ks[r], vs[r], lens[r] - 1, nh, nkv, 1.0 / 16.0, 50.0, None)
                       for r in pick]).view(len(pick), nh * d)
    a = got.float().cpu()
    assert bool(torch.isfinite(a).all())
    assert float((a[pick].double() - ref).abs().max() / ref.abs().max()) < 1e-2


def test_static_entry_point_refuses_what_does_not_fit():
    """The size rule, asked without a launch: several splits whose partial results or counters exceed the built-in
    arrays are refused with status 2 and a message; the same rows with one split are not."""
    from kungfu_b200 import ops
    lib = ops.library()
    fits = lib.kf_attention_decode_static_fits
    assert fits(8, 8, 4, 256, 2, 9) == 0
    assert fits(3000, 32, 16, 256, 2, 2) == 2                 # 3000 x 32 x 2 x 260 floats
    assert b"scratch" in lib.kf_last_cuda_error()
    assert fits(5000, 8, 4, 64, 1, 2) == 2                    # 5000 x 4 x 2 counters
    assert fits(3000, 32, 16, 256, 2, 1) == 0
    assert fits(8, 8, 4, 80, 2, 2) == 2                       # no kernel for this head size
