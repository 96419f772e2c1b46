"""The plain implementation pinned on the reference's own kernels.

nickheyer/kungfu's model code is Rust and cannot be built here, but its CUDA kernels compile unchanged with nvcc and
expose `extern "C"` entry points.  These tests compile them at test time into a temporary folder
(kungfu_b200/measure/reference_kernels.py; nothing is copied into the repository), run them on small inputs in the
reference's own layout (32-bit activations, half-precision ring caches, positions and slots per row) and compare what
they compute with the functions of tests/plain_gemma2.py: the norms, the rotation, the softcap, the gated activation,
and the three attention kernels with window, softcap, grouped heads and two slots of unequal runs in one pass (the
reference's own softcap test: crates/kf-backend-cuda/tests/attention.rs:195-236).  Tolerances are the reference's:
2e-3 for pure 32-bit operations, 2e-2 where the cache is half precision (tests/common/mod.rs:181-187).
"""
import math

import pytest
import torch

import plain_gemma2 as pg

DEV = "cuda:0"


def rel(a, b):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def test_reference_kernels_compile_unchanged(tmp_path):
    """nvcc cross-compiles every kernel file these tests use, as the reference ships it (no GPU needed); this also
    stages the sources where a machine with a GPU finds them."""
    from concurrent.futures import ThreadPoolExecutor
    from kungfu_b200.measure import reference_kernels as rk
    try:
        rk.stage()
    except rk.ReferenceUnavailable as e:
        pytest.skip(str(e))
    with ThreadPoolExecutor(8) as ex:
        outs = list(ex.map(lambda f: rk.compile_cubin(f, str(tmp_path)), rk.FILES))
    assert len(outs) == len(rk.FILES)


@pytest.fixture(scope="module")
def ref():
    from kungfu_b200.measure import reference_kernels as rk
    try:
        rk.find_sources()
    except rk.ReferenceUnavailable as e:
        pytest.skip(str(e))
    return rk.Reference()


@pytest.mark.gpu
def test_norms(ref):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(7, 2304, generator=g) * 3).to(DEV)
    res = torch.randn(7, 2304, generator=g).to(DEV)
    w = (torch.randn(2304, generator=g) * 0.1)
    # the reference multiplies by the stored vector (GGUF files hold 1 + w): give it 1 + w
    stored = (1.0 + w).to(DEV)
    want = pg.rms_norm(x.cpu().double(), w, 1e-6)
    assert rel(ref.rms_norm(x, stored, 1e-6), want) < 2e-3
    assert rel(ref.rms_norm_add(x, stored, res, 1e-6), want + res.cpu().double()) < 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("d,base", [(256, 10000.0), (32, 1e6)])
def test_rotation(ref, d, base):
    g = torch.Generator().manual_seed(2)
    nh, rows = 3, 9
    x = torch.randn(rows, nh, d, generator=g)
    pos = torch.tensor([0, 1, 2, 17, 100, 511, 1000, 3, 4], dtype=torch.int32)
    freq = (base ** (-2.0 * torch.arange(d // 2, dtype=torch.float64) / d)).float()
    got = ref.rope(x.view(rows, nh * d).to(DEV), pos.to(DEV), freq.to(DEV), nh, d)
    cos, sin = pg.rope_angles(pos, d, base, torch.float64)
    assert rel(got.view(rows, nh, d), pg.apply_rope(x.double(), cos, sin)) < 2e-3


@pytest.mark.gpu
def test_softcap_and_gated_activation(ref):
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(5000, generator=g) * 40).to(DEV)
    assert rel(ref.softcap(a, 30.0), pg.softcap(a.cpu().double(), 30.0)) < 2e-3
    gate, up = (torch.randn(5000, generator=g) * 2).to(DEV), torch.randn(5000, generator=g).to(DEV)
    assert rel(ref.gated_gelu(gate, up), pg.gelu_tanh(gate.cpu().double()) * up.cpu().double()) < 2e-3


def _attention_case(ref, nh, nkv, d, runs, cap_rows, seed, spread, past=None):
    """Two slots with earlier tokens in their ring caches and a pass of `runs` = [(slot, new rows)].  Returns the
    pass's rows and the whole sequences' q, k, v (as the cache holds them: half precision)."""
    g = torch.Generator().manual_seed(seed)
    past = past or {0: 70, 1: 5}
    total = {s: past[s] + n for s, n in runs}
    q, k, v = {}, {}, {}
    for s, n in total.items():
        q[s] = (torch.randn(n, nh, d, generator=g) * spread)
        k[s] = torch.randn(n, nkv, d, generator=g).half().float()
        v[s] = torch.randn(n, nkv, d, generator=g).half().float()
    kc, vc = ref.make_cache(2, cap_rows, nkv * d, DEV)
    for s, n in total.items():                              # everything goes through the reference's own append
        pos = torch.arange(n, dtype=torch.int32, device=DEV)
        seq = torch.full((n,), s, dtype=torch.int32, device=DEV)
        ref.kv_append(k[s].view(n, nkv * d).to(DEV), v[s].view(n, nkv * d).to(DEV), kc, vc, pos, seq)
    rows_q, rows_pos, rows_seq, row_runs = [], [], [], []
    at = 0
    for s, n in runs:
        rows_q.append(q[s][past[s]:])
        rows_pos += list(range(past[s], past[s] + n))
        rows_seq += [s] * n
        row_runs.append((s, at, n))
        at += n
    return (torch.cat(rows_q).view(at, nh * d).to(DEV), torch.tensor(rows_pos, dtype=torch.int32, device=DEV),
            torch.tensor(rows_seq, dtype=torch.int32, device=DEV), row_runs, kc, vc, q, k, v, past)


def _plain_rows(q, k, v, past, runs, nh, nkv, scale, cap, window):
    """What plain attention gives for the pass's rows: scores, cap, mask, softmax, weighted sum as in
    plain_gemma2.attention (no projections, no rotation: the kernels get rotated q and cached k, v)."""
    out = []
    for s, n in runs:
        T = q[s].shape[0]
        mask = pg.visible(T, window)
        o = torch.empty(T, nh, q[s].shape[-1], dtype=torch.float64)
        for h in range(nh):
            kh, vh = k[s][:, h // (nh // nkv)].double(), v[s][:, h // (nh // nkv)].double()
            sc = pg.softcap((q[s][:, h].double() @ kh.T) * scale, cap).masked_fill(~mask, float("-inf"))
            o[:, h] = torch.softmax(sc, -1) @ vh
        out.append(o[past[s]:].reshape(n, -1))
    return torch.cat(out)


@pytest.mark.gpu
@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("window", [None, 24])
def test_tensor_core_prompt_attention(ref, d, window):
    """flash_prefill: two slots of unequal runs (40 and 90 rows) in one pass, softcap 20, grouped heads, scores that
    reach the cap."""
    nh, nkv, cap = 4, 2, 20.0
    scale = 1.0 / math.sqrt(d)
    runs = [(1, 40), (0, 90)]
    qd, pos, seq, row_runs, kc, vc, q, k, v, past = _attention_case(ref, nh, nkv, d, runs, 512, 5, spread=10.0)
    got = ref.flash_prefill(qd, kc, vc, pos, seq, row_runs, nh, nkv, d, scale, window, cap)
    want = _plain_rows(q, k, v, past, runs, nh, nkv, scale, cap, window)
    assert rel(got, want) < 2e-2
    nocap = _plain_rows(q, k, v, past, runs, nh, nkv, scale, 0.0, window)
    assert rel(nocap, want) > 0.2                           # the cap matters in this case


@pytest.mark.gpu
@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("window", [None, 24])
def test_decode_attention(ref, d, window):
    """attention_decode: both slots decoded in one pass (one row each), keys split into parts and merged."""
    nh, nkv, cap = 8, 4, 20.0
    scale = 1.0 / math.sqrt(d)
    runs = [(0, 1), (1, 1)]
    qd, pos, seq, row_runs, kc, vc, q, k, v, past = _attention_case(ref, nh, nkv, d, runs, 1024, 6, spread=10.0,
                                                                    past={0: 700, 1: 5})       # 701 keys: six parts to merge
    got = ref.attention_decode(qd, kc, vc, pos, seq, nh, nkv, d, scale, window, cap)
    want = _plain_rows(q, k, v, past, runs, nh, nkv, scale, cap, window)
    assert rel(got, want) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("window", [None, 8])
def test_per_row_attention(ref, window):
    """The per-row kernel the reference runs at head sizes without a tensor-core instance (here 16, as in its own tiny
    attention model, tests/attention.rs:7-42): windowed and not, three query heads per kv head."""
    nh, nkv, d, cap = 6, 2, 16, 50.0
    scale = 1.0 / math.sqrt(24)                             # not 1/sqrt(head size)
    runs = [(0, 7), (1, 3)]
    qd, pos, seq, row_runs, kc, vc, q, k, v, past = _attention_case(ref, nh, nkv, d, runs, 128, 7, spread=12.0)
    got = ref.attention_classic(qd, kc, vc, pos, seq, nh, nkv, d, scale, window, cap)
    want = _plain_rows(q, k, v, past, runs, nh, nkv, scale, cap, window)
    assert rel(got, want) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [3, 40])
def test_bfloat16_products(ref, rows):
    """matvec (up to 8 rows) and matmul of the reference over bfloat16 weight rows, activations rounded to bfloat16."""
    g = torch.Generator().manual_seed(8)
    w = (torch.randn(300, 520, generator=g) * 0.05).bfloat16()
    x = torch.randn(rows, 520, generator=g).bfloat16().float()
    got = ref.linear_bf16(w.to(DEV), x.to(DEV))
    assert rel(got, x.double() @ w.double().T) < 2e-3
