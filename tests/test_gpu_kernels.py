"""Each kernel alone against a plain torch reference of the same operation, at sizes other than the engine's."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def rel_err(a, b):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module")
def ops():
    from kungfu_b200 import ops as o
    o.library()
    return o


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(ops, dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(301, 70, generator=g).to(dtype).to(DEV)
    tokens = torch.randint(0, 301, (37,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(37, 70, device=DEV)
    ops.embed(tokens, table, 8.3666, out)
    ref = table.float()[tokens.long()] * torch.tensor(8.3666, dtype=torch.float32)
    assert torch.equal(out, ref)


@pytest.mark.parametrize("H", [70, 2304, 5000, 9000])
@pytest.mark.parametrize("wdtype,odtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16)])
def test_rmsnorm(ops, H, wdtype, odtype):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(19, H, generator=g) * 3).to(DEV)
    w = (torch.randn(H, generator=g) * 0.1).to(wdtype).to(DEV)
    rows = torch.tensor([3, 0, 18, 3], dtype=torch.int32, device=DEV)
    for r in (None, rows):
        n = 19 if r is None else 4
        out = torch.empty(n, H, dtype=odtype, device=DEV)
        ops.rmsnorm(x, w, 1e-5, True, out, r)
        xs = (x if r is None else x[r.long()]).double()
        ref = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5) * (1 + w.double())
        assert rel_err(out, ref) < (1e-5 if odtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("H", [96, 2304, 3584, 4608, 9000])
@pytest.mark.parametrize("odtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [11, 300])
def test_add_rmsnorm(ops, H, odtype, T):
    g = torch.Generator().manual_seed(2)
    a = torch.randn(T, H, generator=g).to(DEV)
    x = torch.randn(T, H, generator=g).to(DEV)
    w1 = (torch.randn(H, generator=g) * 0.1).to(DEV)
    w2 = (torch.randn(H, generator=g) * 0.1).to(DEV)
    ad, xd = a.double(), x.double()
    x_ref = xd + ad * torch.rsqrt(ad.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + w1.double())
    n_ref = x_ref * torch.rsqrt(x_ref.pow(2).mean(-1, keepdim=True) + 1e-4) * w2.double()
    x1 = x.clone()
    ops.add_rmsnorm(a, w1, 1e-6, True, x1)
    assert rel_err(x1, x_ref) < 1e-5
    x2 = x.clone()
    out = torch.empty(T, H, dtype=odtype, device=DEV)
    ops.add_rmsnorm(a, w1, 1e-6, True, x2, next_weight=w2, next_eps=1e-4, next_plus_one=False, next_out=out)
    assert torch.equal(x1, x2)
    assert rel_err(out, n_ref) < (1e-5 if odtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("T,N,K", [(1, 1000, 96), (7, 130, 200), (65, 777, 123), (130, 64, 2304)])
@pytest.mark.parametrize("xd,wd", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_linear(ops, T, N, K, xd, wd):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, K, generator=g).to(xd).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(wd).to(DEV)
    ref = x.double() @ w.double().T
    out = torch.empty(T, N, device=DEV)
    ops.linear(x, w, out)
    assert rel_err(out, ref) < 2e-6 * math.sqrt(K) + 1e-6
    capped = torch.empty(T, N, device=DEV)
    ops.linear(x, w, capped, softcap=0.7)
    assert rel_err(capped, 0.7 * torch.tanh(ref / 0.7)) < 1e-5
    # a row's result does not depend on the other rows of the launch: to the bit on the generic kernel (the order of
    # the sum over K is fixed per output), to the rounding of a 32-bit sum on the tensor cores (how K is cut across
    # CTAs depends on the number of rows)
    one = torch.empty(1, N, device=DEV)
    ops.linear(x[T - 1:T].contiguous(), w, one)
    if xd == torch.bfloat16 and wd == torch.bfloat16 and K % 8 == 0:
        assert rel_err(one[0], out[T - 1]) < 2e-6 * math.sqrt(K)
    else:
        assert torch.equal(one[0], out[T - 1])


TC_SHAPES = [(1, 256, 64), (8, 2304, 2048), (5, 130, 200), (16, 128, 96), (17, 1000, 120), (40, 4096, 2304), (64, 777, 320),
             (100, 300, 72), (256, 512, 512), (300, 2304, 9216), (700, 136, 64), (2048, 256, 128),
             # a few hundred rows: K cut four and two ways inside a cluster of CTA pairs (ragged N, K and T), whole tiles on pairs
             (256, 2304, 2048), (512, 4096, 2304), (250, 1002, 1032), (700, 130, 2056), (400, 8192, 512)]


def test_linear_plans_for_a_few_hundred_rows(ops):
    """What the planner picks between 65 and about a thousand rows: up to 192 rows 64-token tiles with K cut as far as all
    clusters still run at once; beyond (and below where the clusters cover most of the GPU) (token tile, K splits) = (256, 4) while the tiles of
    256 x 256 fit the clusters of eight that run at once, (256, 2) while they fit the clusters of four, whole tiles on
    CTA pairs beyond that; short K, nearly empty token tiles and gated products keep their earlier plans."""
    import ctypes
    lib = ops.library()

    def plan(T, N, K, gated=0):
        bn, sp = ctypes.c_int(0), ctypes.c_int(0)
        lib.kf_linear_tc_plan(T, N, K, gated, ctypes.byref(bn), ctypes.byref(sp))
        return bn.value, sp.value

    assert plan(256, 2304, 9216) == (256, 4)            # 9 tiles
    assert plan(512, 2304, 9216) == (256, 2)            # 18 tiles
    assert plan(512, 4096, 2304) == (256, 2)            # 32 tiles
    assert plan(512, 8192, 3584) == (256, 1)            # 64 tiles: whole tiles
    assert plan(768, 2304, 2048) == (256, 2)            # 27 tiles
    assert plan(1024, 2304, 2048) == (256, 1)           # 36 tiles
    assert plan(250, 1002, 1032) == (256, 2)            # K too short to cut in four
    assert plan(300, 2304, 9216)[0] == 64               # the second token tile would be a sixth full
    assert plan(200, 2304, 9216) == (256, 4)
    assert plan(160, 2304, 9216) == (64, 4)             # three 64-token tiles; nine clusters of eight would leave half the GPU idle
    assert plan(160, 3584, 14336) == (256, 4)           # fourteen clusters of eight
    assert plan(128, 2304, 9216) == (64, 4)             # 36 tiles: clusters of eight would need a second round
    assert plan(128, 4608, 4096) == (64, 2)             # 72 tiles: so would clusters of four
    assert plan(128, 4096, 2304) == (64, 4)             # 64 tiles
    assert plan(256, 2304, 512)[0] == 64                # K too short to cut
    assert plan(512, 9216, 2304, 1) == (256, 1)         # gated: as before
    assert plan(8, 2304, 9216) == (16, 8)               # decode: as before


@pytest.mark.parametrize("T,N,K", TC_SHAPES)
def test_linear_tensor_cores(ops, T, N, K):
    """bfloat16 product on tcgen05 against float64, ragged in every dimension, with and without split-K."""
    g = torch.Generator().manual_seed(T * 7 + N)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ref = x.double() @ w.double().T
    out = torch.full((T, N), float("nan"), device=DEV)
    ops.linear(x, w, out)
    ops.raise_on_device_error()
    bound = 2e-6 * math.sqrt(K) + 1e-6            # 32-bit accumulation over K terms
    assert rel_err(out, ref) < bound, "32-bit out"
    capped = torch.empty(T, N, device=DEV)
    ops.linear(x, w, capped, softcap=0.9)
    assert rel_err(capped, 0.9 * torch.tanh(ref / 0.9)) < bound
    half = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    ops.linear(x, w, half)
    assert rel_err(half, ref) < 5e-3
    # the generic kernel agrees (same operands, 32-bit FMA)
    ops.use_tensor_cores = False
    try:
        slow = torch.empty(T, N, device=DEV)
        ops.linear(x, w, slow)
    finally:
        ops.use_tensor_cores = True
    assert rel_err(out, slow) < bound
    # twice the same launch gives the same bits (split-K sums in split order)
    again = torch.empty(T, N, device=DEV)
    ops.linear(x, w, again)
    assert torch.equal(out, again)
    ops.raise_on_device_error()


@pytest.mark.parametrize("T,I,K", [(1, 128, 64), (8, 9216, 2304), (33, 200, 120), (64, 320, 96), (300, 1000, 256), (2048, 384, 128)])
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_linear_gated_tensor_cores(ops, T, I, K, act):
    from cpu_ops import _act
    g = torch.Generator().manual_seed(T + I)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    out = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_gated(x, w, out, act, None)
    ops.raise_on_device_error()
    gu = x.double() @ w.double().T
    ref = _act(act, gu[:, :I]) * gu[:, I:]
    assert rel_err(out, ref) < 6e-3


@pytest.mark.parametrize("act", ["gelu_tanh", "gelu_erf", "silu"])
def test_linear_gated(ops, act):
    from cpu_ops import _act

    class Ctx:
        def buf(self, tag, shape, dtype):
            return torch.empty(shape, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(9, 72, generator=g).to(DEV)
    w = (torch.randn(2 * 50, 72, generator=g) * 0.3).to(DEV)
    out = torch.empty(9, 50, device=DEV)
    ops.linear_gated(x, w, out, act, Ctx())
    gu = x.double() @ w.double().T
    ref = _act(act, gu[:, :50]) * gu[:, 50:]
    assert rel_err(out, ref) < 1e-5


def test_rope_table(ops):
    pos = torch.tensor([0, 1, 5, 100, 8191], dtype=torch.int32, device=DEV)
    inv = (10000.0 ** (-2.0 * torch.arange(24, dtype=torch.float64) / 48)).float().to(DEV)
    cos = torch.empty(5, 24, device=DEV)
    sin = torch.empty(5, 24, device=DEV)
    ops.rope_table(pos, inv, cos, sin)
    ang = pos.double()[:, None] * inv.double()[None, :]           # 32-bit frequencies, their product with the position exact
    assert float((cos.double() - torch.cos(ang)).abs().max()) < 1e-6
    assert float((sin.double() - torch.sin(ang)).abs().max()) < 1e-6


class _View:
    def __init__(self, pages, page_size, writes=True):
        self.pages, self.page_size, self.group, self.writes = pages, page_size, 0, writes


class _Ctx:
    def __init__(self, positions, row_req, table, dec_rows=None, pre_rows=None):
        self.positions, self.row_req, self.block_tables = positions, row_req, [table]
        self.n_dec_rows = 0 if dec_rows is None else len(dec_rows)
        self.n_pre_rows = 0 if pre_rows is None else len(pre_rows)
        self.dec_rows = None if dec_rows is None else torch.tensor(dec_rows, dtype=torch.int32, device=DEV)
        self.pre_rows = None if pre_rows is None else torch.tensor(pre_rows or [0], dtype=torch.int32, device=DEV)
        self.max_kv_len = int(positions.max()) + 1
        # tiles of up to 64 consecutive rows of one request, as the step function builds them
        tiles = []
        if pre_rows:
            req, pos = row_req.tolist(), positions.tolist()
            start = pre_rows[0]
            for a, b in zip(pre_rows, pre_rows[1:] + [None]):
                if b is None or b != a + 1 or req[b] != req[a] or a + 1 - start == 64:
                    tiles.append((start, a + 1 - start))
                    start = b
        self.n_tiles = len(tiles)
        self.tile_row0 = torch.tensor([t[0] for t in tiles] or [0], dtype=torch.int32, device=DEV)
        self.tile_nrows = torch.tensor([t[1] for t in tiles] or [0], dtype=torch.int32, device=DEV)
        wide = []
        if pre_rows:
            start = pre_rows[0]
            for a, b in zip(pre_rows, pre_rows[1:] + [None]):
                if b is None or b != a + 1 or req[b] != req[a] or a + 1 - start == 128:
                    wide.append((start, a + 1 - start))
                    start = b
        self.n_wide = len(wide)
        self.wide_row0 = torch.tensor([t[0] for t in wide] or [0], dtype=torch.int32, device=DEV)
        self.wide_nrows = torch.tensor([t[1] for t in wide] or [0], dtype=torch.int32, device=DEV)


def _paged_setup(dtype, nh, nkv, d, P, lens, seed, scramble=True):
    """Random requests of the given lengths with their K/V spread over scrambled pages."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // P) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist() if scramble else list(range(n_pages))
    pages = torch.zeros(n_pages, 2, nkv, P, d, dtype=dtype)
    width = max(-(-n // P) for n in lens)
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    ks, vs = [], []
    nxt = 0
    for r, n in enumerate(lens):
        k = torch.randn(n, nkv, d, generator=g).to(dtype)
        v = torch.randn(n, nkv, d, generator=g).to(dtype)
        ks.append(k)
        vs.append(v)
        for i in range(-(-n // P)):
            pg = perm[nxt]
            nxt += 1
            table[r, i] = pg
            m = min(P, n - i * P)
            pages[pg, 0, :, :m] = k[i * P:i * P + m].transpose(0, 1)
            pages[pg, 1, :, :m] = v[i * P:i * P + m].transpose(0, 1)
    return pages, table, ks, vs


def _attn_ref(q, k, v, pos, nh, nkv, scale, cap, window):
    """q [nh, d] at position pos against keys k, v [n, nkv, d] (double)."""
    lo = max(0, pos - window + 1) if window else 0
    out = []
    for h in range(nh):
        kh, vh = k[lo:pos + 1, h // (nh // nkv)].double(), v[lo:pos + 1, h // (nh // nkv)].double()
        s = (kh @ q[h].double()) * scale
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        out.append(torch.softmax(s, 0) @ vh)
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,P,window,cap", [(4, 2, 16, 4, 8, 50.0), (6, 2, 32, 16, None, 20.0), (9, 3, 48, 8, 24, 0.0),
                                                   (8, 4, 256, 64, 100, 50.0), (5, 5, 112, 32, None, 30.0), (16, 2, 128, 64, 4096, 50.0)])
def test_paged_attention(ops, dtype, nh, nkv, d, P, window, cap):
    lens = [1, 37, 150, 70]
    pages, table, ks, vs = _paged_setup(dtype, nh, nkv, d, P, lens, seed=5)
    # rows: the whole of request 1, the last row of request 2, rows 60..69 of request 3, the only row of request 0
    rows = [(1, p) for p in range(37)] + [(2, 149)] + [(3, p) for p in range(60, 70)] + [(0, 0)]
    g = torch.Generator().manual_seed(6)
    q = torch.randn(len(rows), nh, d, generator=g).to(dtype)
    # make one far key stand out for one row: scale a key and the query that should find it
    scale = 1.0 / math.sqrt(d)
    ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
               torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV))
    out = torch.empty(len(rows), nh * d, dtype=dtype, device=DEV)
    ops.paged_attention(q.view(len(rows), nh * d).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, scale, cap, window)
    ref = torch.stack([_attn_ref(q[i], ks[r], vs[r], p, nh, nkv, scale, cap, window) for i, (r, p) in enumerate(rows)])
    assert rel_err(out.view(len(rows), nh, d), ref) < (2e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("nh,nkv,d,P,window,cap", [(4, 2, 16, 4, 8, 50.0), (6, 2, 32, 16, None, 20.0), (8, 4, 256, 64, 1000, 50.0),
                                                   (5, 5, 64, 32, None, 30.0), (16, 2, 128, 64, 4096, 50.0), (8, 1, 128, 16, None, 0.0)])
@pytest.mark.parametrize("mixed", [False, True])
@pytest.mark.parametrize("tensor_cores", [True, False])
def test_decode_attention(ops, nh, nkv, d, P, window, cap, mixed, tensor_cores):
    """The split-KV decode kernel: single rows of requests of very different lengths (one of them long enough for
    several splits), alone and beside rows of a multi-row request that the other kernel handles."""
    lens = [1, 37, 3000, 700, 64, 65]
    pages, table, ks, vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, lens, seed=11)
    rows = [(r, n - 1) for r, n in enumerate(lens)]          # the last position of every request
    dec, pre = list(range(len(rows))), []
    if mixed:                                               # request 3 brings 5 rows instead of 1
        rows = rows[:3] + [(3, p) for p in range(695, 700)] + rows[4:]
        dec, pre = [0, 1, 2, 8, 9], [3, 4, 5, 6, 7]
    g = torch.Generator().manual_seed(12)
    q = torch.randn(len(rows), nh, d, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
               torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV), dec, pre)
    out = torch.full((len(rows), nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.decode_on_tensor_cores = tensor_cores
    try:
        ops.paged_attention(q.view(len(rows), nh * d).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, scale, cap, window)
    finally:
        ops.decode_on_tensor_cores = True
    ref = torch.stack([_attn_ref(q[i], ks[r], vs[r], p, nh, nkv, scale, cap, window) for i, (r, p) in enumerate(rows)])
    assert bool(torch.isfinite(out.float()).all())
    assert rel_err(out.view(len(rows), nh, d), ref) < 1.5e-2


@pytest.mark.parametrize("nh,nkv,d", [(2, 1, 256), (4, 2, 128), (2, 2, 64)])
@pytest.mark.parametrize("shape", ["rising", "falling", "sawtooth"])
@pytest.mark.parametrize("window", [None, 200])
def test_prompt_attention_when_the_running_maximum_moves(ops, nh, nkv, d, shape, window):
    """The tcgen05 prompt kernel keeps one running maximum per row that its two softmax groups hand to each other tile by
    tile, rescales O only when the maximum grows by more than 2^8, and carries each group's sum along.  Scores that rise
    by about 12 nats per 64-key tile raise the maximum (and rescale O) at every tile of both groups; falling scores never
    raise it after the first tile, so late tiles add weights near 2^-400 (flushed to zero) to a sum made early; a sawtooth
    mixes both.  No cap (a cap would flatten the differences), with and without a window, against float64."""
    P, n = 64, 1100
    g = torch.Generator().manual_seed(77)
    pages, table, ks, vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, [n], seed=78)
    j = torch.arange(n, dtype=torch.float32)
    ramp = {"rising": j * 0.19, "falling": (n - j) * 0.19, "sawtooth": (j % 150) * 0.9}[shape]
    # the first coordinate of every key carries the ramp; queries have 1 there, so the score is ramp + small noise
    k = (torch.randn(n, nkv, d, generator=g) * 0.05)
    k[:, :, 0] = (ramp / (1.0 / math.sqrt(d))).unsqueeze(1)
    k = k.to(torch.bfloat16)
    ks[0] = k
    for i in range(-(-n // P)):
        m = min(P, n - i * P)
        pages[table[0, i], 0, :, :m] = k[i * P:i * P + m].transpose(0, 1)
    rows = [(0, p) for p in range(n)]
    q = torch.randn(n, nh, d, generator=g) * 0.05
    q[:, :, 0] = 1.0
    q = q.to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    ctx = _Ctx(torch.arange(n, dtype=torch.int32, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV), table.to(DEV), [],
               list(range(n)))
    out = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(q.view(n, nh * d).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, scale, 0.0, window)
    ops.raise_on_device_error()
    pick = sorted(set(range(0, n, 11)) | set(range(n - 70, n)) | set(range(0, 70)))
    ref = torch.stack([_attn_ref(q[i], ks[0], vs[0], i, nh, nkv, scale, 0.0, window) for i in pick])
    got = out.view(n, nh, d)[pick]
    assert not torch.isnan(got.float()).any()
    assert rel_err(got, ref) < 1e-2


def test_prompt_attention_planner_cuts_only_what_repays(ops):
    """The planner's choice of runs per tile: whole prompts stay whole (a second wave of blocks, or partial rows and their
    merge, cost more than a short loop saves), a short portion at a long context is cut so that its blocks fill the GPU."""
    import ctypes
    lib = ops.library()

    def plan(n_tiles, nh, max_keys):
        run_tiles = ctypes.c_int(-1)
        return lib.kf_attention_prefill_tc_plan(n_tiles, nh, max_keys, ctypes.byref(run_tiles)), run_tiles.value

    assert plan(16, 8, 2048) == (1, 0)          # 128 blocks: one wave
    assert plan(4, 8, 512) == (1, 0)            # 32 blocks of at most 8 key tiles: nothing to gain
    assert plan(8, 8, 1024) == (1, 0)
    parts, run_tiles = plan(4, 8, 8192)         # 512 rows at context 8192: 128 key tiles per block
    assert parts == 4 and run_tiles == 0
    assert plan(1, 8, 32768)[0] == 8            # one tile at a very long context: the most runs there are
    assert plan(1, 8, 100) == (1, 0)


@pytest.mark.parametrize("nh,nkv,d,window", [(8, 4, 256, None), (4, 1, 128, 300), (6, 2, 64, None)])
@pytest.mark.parametrize("lens", [[700], [2048], [130, 513, 64]])
def test_prompt_attention_with_keys_cut_into_runs(ops, nh, nkv, d, window, lens):
    """Few blocks of prompt rows (a short portion at a long context, or one long prompt whose last tiles have most of
    the keys) cut every tile's keys into runs with a block each, merged by a second kernel: the same result as one block
    per tile, and as float64."""
    P = 64
    pages, table, ks, vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, lens, seed=31)
    # the last 200 rows of every request (a portion late in its prompt), all rows of short ones
    rows = [(r, p) for r, n in enumerate(lens) for p in range(max(0, n - 200), n)]
    g = torch.Generator().manual_seed(32)
    q = torch.randn(len(rows), nh, d, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
               torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV), [], list(range(len(rows))))
    outs = []
    for split in (True, False):
        ops.prefill_plan_override = (3, 0) if split else (1, 0)     # three runs per tile, whatever the planner would choose
        try:
            out = torch.full((len(rows), nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
            before = ops.launch_count()
            ops.paged_attention(q.view(len(rows), nh * d).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, scale, 50.0, window)
            outs.append((out, ops.launch_count() - before))
        finally:
            ops.prefill_plan_override = None
    ops.raise_on_device_error()
    assert outs[0][1] == 2 and outs[1][1] == 1, "cut into runs: the attention kernel and the merge"
    ref = torch.stack([_attn_ref(q[i], ks[r], vs[r], p, nh, nkv, scale, 50.0, window) for i, (r, p) in enumerate(rows)])
    assert rel_err(outs[0][0].view(len(rows), nh, d), ref) < 1e-2
    assert rel_err(outs[1][0].view(len(rows), nh, d), ref) < 1e-2
    assert rel_err(outs[0][0], outs[1][0]) < 6e-3


@pytest.mark.parametrize("nh,nkv,d,window,lens", [(8, 4, 256, None, [2048]), (16, 4, 64, None, [1500]),
                                                  (8, 2, 128, 1500, [2048]), (8, 4, 256, None, [1100, 300])])
def test_prompt_attention_with_only_the_long_tiles_cut(ops, nh, nkv, d, window, lens):
    """A launch may cut only its long tiles (here: those with more than half of the longest tile's keys, into two runs
    that a second kernel merges) while the others stay whole and write their rows themselves.  Rows of both kinds of
    tile against float64 and against the launch that cuts nothing."""
    P = 64
    pages, table, ks, vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, lens, seed=35)
    rows = [(r, p) for r, n in enumerate(lens) for p in range(n)]
    g = torch.Generator().manual_seed(36)
    q = torch.randn(len(rows), nh, d, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
               torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV), [], list(range(len(rows))))
    outs = []
    key_tiles = (min(max(lens), window + 128 if window else max(lens)) + 63) // 64
    for split in (True, False):
        ops.prefill_plan_override = (2 if split else 1, (key_tiles + 1) // 2 if split else 0)
        try:
            out = torch.full((len(rows), nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
            before = ops.launch_count()
            ops.paged_attention(q.view(len(rows), nh * d).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, scale, 50.0, window)
            outs.append((out, ops.launch_count() - before))
        finally:
            ops.prefill_plan_override = None
    ops.raise_on_device_error()
    assert outs[0][1] == 2 and outs[1][1] == 1, "long tiles cut into runs: the attention kernel and the merge"
    assert not torch.isnan(outs[0][0].float()).any()
    step = 7                                                        # every 7th row and the last rows of every request
    pick = sorted(set(range(0, len(rows), step)) | {i for i, (r, p) in enumerate(rows) if p >= lens[r] - 3})
    ref = torch.stack([_attn_ref(q[i], ks[r], vs[r], p, nh, nkv, scale, 50.0, window) for i, (r, p) in ((i, rows[i]) for i in pick)])
    assert rel_err(outs[0][0].view(len(rows), nh, d)[pick], ref) < 1e-2
    assert rel_err(outs[1][0].view(len(rows), nh, d)[pick], ref) < 1e-2
    assert rel_err(outs[0][0], outs[1][0]) < 6e-3


def _plant(pages, table, req, j, kvh, P, key=None, value=None):
    """Overwrite key and/or value j of a request in its pages (host tensors)."""
    pg = int(table[req, j // P])
    if key is not None:
        pages[pg, 0, kvh, j % P] = key.to(pages.dtype)
    if value is not None:
        pages[pg, 1, kvh, j % P] = value.to(pages.dtype)


@pytest.mark.parametrize("path", ["decode_mma", "decode_simt", "prompt_rows", "generic_f32"])
@pytest.mark.parametrize("nh,nkv,d", [(8, 4, 256), (4, 1, 128), (6, 2, 64)])
def test_attention_finds_a_planted_key(ops, path, nh, nkv, d):
    """Random keys hide a key that is wrongly skipped among thousands (its weight is 1/n).  Here one key is made to match
    the query of head 0, so that it takes almost all the weight: the output must be that key's value when the key is
    visible (the first key of a request, a page's last and first slot, the oldest key inside the window, the row's own
    key) and must not be when it is just outside the window."""
    P, n = 64, 3000
    window = 1000
    dtype = torch.float32 if path == "generic_f32" else torch.bfloat16
    pos = n - 1
    scale = 1.0 / math.sqrt(d)
    cases = [(None, 0), (None, 63), (None, 64), (None, 1471), (None, pos), (window, pos - window + 1), (window, pos - window),
             (window, pos - 1), (window, 0)]
    for win, j in cases:
        pages, table, ks, vs = _paged_setup(dtype, nh, nkv, d, P, [n, 10], seed=40 + j % 7, scramble=True)
        g = torch.Generator().manual_seed(41)
        rows = [(0, pos)] if path != "prompt_rows" else [(0, p) for p in range(pos - 69, pos + 1)]
        q = torch.randn(len(rows), nh, d, generator=g)
        qv = q[-1, 0]                                           # head 0 of the last row looks for key j
        key = qv * (30.0 / (scale * float(qv @ qv)))            # score 30 before the cap, against scores of about +-1
        marker_value = torch.full((d,), 5.0)
        marker_value[::2] = -3.0
        _plant(pages, table, 0, j, 0, P, key=key, value=marker_value)
        ctx_rows = list(range(len(rows)))
        dec, pre = (ctx_rows, []) if path.startswith("decode") else ([], ctx_rows)
        if path == "generic_f32":
            dec, pre = None, None
        ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
                   torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV), dec, pre)
        out = torch.full((len(rows), nh * d), float("nan"), dtype=dtype, device=DEV)
        ops.decode_on_tensor_cores = path != "decode_simt"
        try:
            ops.paged_attention(q.view(len(rows), nh * d).to(dtype).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d,
                                scale, 50.0, win)
        finally:
            ops.decode_on_tensor_cores = True
        got = out.view(len(rows), nh, d)[-1, 0].float().cpu()
        visible = j <= pos and (win is None or pos - j < win)
        dist = float((got - marker_value).norm() / marker_value.norm())
        if visible:
            assert dist < 2e-2, (path, win, j, dist)
        else:
            assert dist > 0.5, (path, win, j, dist)


@pytest.mark.parametrize("nh,nkv,d,P,window,rot", [(8, 4, 256, 64, 1000, 256), (4, 2, 16, 4, 8, 16), (6, 2, 32, 16, None, 16),
                                                   (16, 2, 128, 64, 4096, 128), (5, 5, 64, 32, None, 0), (8, 1, 128, 16, 33, 64)])
@pytest.mark.parametrize("writes", [True, False])
def test_decode_attention_with_rotation_and_append_inside(ops, nh, nkv, d, P, window, rot, writes):
    """A decode step's attention as one launch (the kernel rotates q and k, appends k and v, attends) against the two
    launches it replaces: same bits out and in the pages.  Lengths put the new key at a page's first slot, its last, in
    the middle, and alone in a request."""
    lens = [1, P + 1, 2 * P, 3000, 700, 65]
    pages, table, ks, vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, lens, seed=21)
    T = len(lens)
    g = torch.Generator().manual_seed(22)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g).to(DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    if rot:
        inv = (10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(DEV)
        cos = torch.empty(T, rot // 2, device=DEV)
        sin = torch.empty(T, rot // 2, device=DEV)
        ops.rope_table(pos, inv, cos, sin)
    else:
        cos = sin = None
    ctx = _Ctx(pos, torch.arange(T, dtype=torch.int32, device=DEV), table.to(DEV), list(range(T)), [])
    ctx.n_rows = T
    scale, cap = 1.0 / math.sqrt(d), 50.0
    # the two launches
    pages_a = pages.to(DEV).clone()
    view_a = _View(pages_a, P, writes)
    q = torch.empty(T, nh * d, dtype=torch.bfloat16, device=DEV)
    ops.rope_kv_append(qkv, cos, sin, rot, nh, nkv, d, ctx, view_a, q)
    out_a = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(q, out_a, ctx, view_a, nh, nkv, d, scale, cap, window)
    # the one launch
    pages_b = pages.to(DEV).clone()
    view_b = _View(pages_b, P, writes)
    assert ops.decode_attention_takes_qkv(ctx, view_b, nh, nkv, d)
    out_b = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.rope_append_attend(qkv, cos, sin, rot, out_b, ctx, view_b, nh, nkv, d, scale, cap, window)
    assert bool(torch.isfinite(out_b.float()).all())
    assert torch.equal(pages_a, pages_b)
    assert torch.equal(pages_b, pages.to(DEV)) != writes or T == 0      # the append happened exactly when asked for
    assert torch.equal(out_a, out_b)


@pytest.mark.parametrize("nh,nkv,d,P,window,cap", [(4, 2, 16, 4, 8, 50.0), (6, 2, 32, 16, None, 20.0), (8, 4, 256, 64, 100, 50.0),
                                                   (5, 5, 64, 32, None, 30.0), (16, 2, 128, 64, 70, 50.0), (8, 1, 128, 16, None, 0.0),
                                                   (2, 1, 256, 8, None, 0.0), (4, 2, 64, 64, 100, 30.0), (3, 1, 128, 128, None, 0.0),
                                                   (8, 4, 256, 64, None, 50.0), (8, 8, 128, 64, 200, 20.0)])
def test_prefill_attention(ops, nh, nkv, d, P, window, cap):
    """The tensor-core prompt kernel: a whole prompt from position 0 (several tiles, the last one ragged), a portion
    that continues a long request, a two-row portion, beside single rows that the decode kernel takes."""
    lens = [150, 700, 65, 9, 300]
    pages, table, ks, vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, lens, seed=13)
    rows = ([(0, p) for p in range(150)] + [(1, p) for p in range(570, 700)] + [(2, 64)] + [(3, p) for p in range(7, 9)]
            + [(4, 299)])
    pre = list(range(0, 280)) + [281, 282]
    dec = [280, 283]
    g = torch.Generator().manual_seed(14)
    q = torch.randn(len(rows), nh, d, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
               torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV), dec, pre)
    assert ctx.n_tiles == 3 + 3 + 1
    out = torch.full((len(rows), nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(q.view(len(rows), nh * d).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, scale, cap, window)
    ref = torch.stack([_attn_ref(q[i], ks[r], vs[r], p, nh, nkv, scale, cap, window) for i, (r, p) in enumerate(rows)])
    got = out.view(len(rows), nh, d)
    ops.raise_on_device_error()
    assert bool(torch.isfinite(got.float()).all())
    assert rel_err(got, ref) < 1.5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key(ops, dtype):
    """One key among hundreds carries the answer: its score is made to stand out, on a page of its own."""
    nh, nkv, d, P = 4, 2, 32, 16
    n = 600
    for far in (0, 15, 16, 333, 599 - 1):
        pages, table, ks, vs = _paged_setup(dtype, nh, nkv, d, P, [n], seed=7)
        q = torch.zeros(1, nh, d)
        q[0, :, 3] = 40.0
        k = ks[0].float() * 0.01
        k[far, :, 3] = 10.0
        v = vs[0].float()
        for i in range(-(-n // P)):
            pg = int(table[0, i])
            m = min(P, n - i * P)
            pages[pg, 0, :, :m] = k[i * P:i * P + m].transpose(0, 1).to(dtype)
        ctx = _Ctx(torch.tensor([n - 1], dtype=torch.int32, device=DEV), torch.tensor([0], dtype=torch.int32, device=DEV), table.to(DEV),
                   dec_rows=[0], pre_rows=[])
        out = torch.empty(1, nh * d, dtype=dtype, device=DEV)
        ops.paged_attention(q.view(1, nh * d).to(dtype).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, 1.0, 0.0, None)
        want = torch.stack([v[far, h // 2] for h in range(nh)]).to(dtype).float()
        assert float((out.float().cpu().view(nh, d) - want).abs().max()) < 2e-2, far


def test_window_edge(ops):
    """The key exactly `window` behind must not be seen, the one at window - 1 must."""
    nh, nkv, d, P, W = 2, 1, 16, 4, 8
    n = 30
    pages, table, ks, vs = _paged_setup(torch.float32, nh, nkv, d, P, [n], seed=8)
    pos = n - 1
    for back, seen in ((W - 1, True), (W, False)):
        k = ks[0].clone() * 0.0
        k[pos - back, :, 0] = 30.0
        for i in range(-(-n // P)):
            pg = int(table[0, i])
            m = min(P, n - i * P)
            pages[pg, 0, :, :m] = k[i * P:i * P + m].transpose(0, 1)
        q = torch.zeros(1, nh * d)
        q[0, 0] = 30.0
        q[0, d] = 30.0
        ctx = _Ctx(torch.tensor([pos], dtype=torch.int32, device=DEV), torch.tensor([0], dtype=torch.int32, device=DEV), table.to(DEV))
        out = torch.empty(1, nh * d, device=DEV)
        ops.paged_attention(q.to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, 1.0, 0.0, W)
        target = vs[0][pos - back, 0]
        close = float((out.cpu()[0, :d] - target).abs().max()) < 1e-3
        assert close == seen


@pytest.mark.parametrize("qd,kvd", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("nh,nkv,d,rot,P", [(4, 2, 16, 16, 4), (9, 3, 48, 32, 8), (8, 4, 256, 256, 64), (3, 1, 80, 0, 16)])
def test_rope_kv_append(ops, qd, kvd, nh, nkv, d, rot, P):
    g = torch.Generator().manual_seed(9)
    lens = [20, 7]
    starts = [13, 0]                   # request 0 continues at position 13, request 1 starts
    T = sum(lens)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g)
    positions = torch.tensor([starts[0] + i for i in range(lens[0])] + [starts[1] + i for i in range(lens[1])], dtype=torch.int32)
    row_req = torch.tensor([0] * lens[0] + [1] * lens[1], dtype=torch.int32)
    n_pages = 16
    table = torch.full((2, 12), -1, dtype=torch.int32)
    table[0, :9] = torch.tensor([5, 2, 9, 0, 11, 3, 14, 7, 1])
    table[1, :2] = torch.tensor([4, 8])
    pages = torch.full((n_pages, 2, nkv, P, d), 7.0, dtype=kvd)
    half = rot // 2
    inv = (10000.0 ** (-2.0 * torch.arange(max(half, 1), dtype=torch.float64) / max(rot, 2))).float()
    ang = positions.float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)
    ctx = _Ctx(positions.to(DEV), row_req.to(DEV), table.to(DEV))
    q_out = torch.empty(T, nh * d, dtype=qd, device=DEV)
    view = _View(pages.to(DEV), P)
    ops.rope_kv_append(qkv.to(DEV), cos.to(DEV) if rot else None, sin.to(DEV) if rot else None, rot, nh, nkv, d, ctx, view, q_out)

    def rope(x):                       # x [T, heads, d] double
        x = x.clone()
        if rot:
            a, b = x[..., :half].clone(), x[..., half:rot].clone()
            c, s = cos.double()[:, None, :], sin.double()[:, None, :]
            x[..., :half] = a * c - b * s
            x[..., half:rot] = a * s + b * c
        return x
    q_ref = rope(qkv[:, :nh * d].double().view(T, nh, d))
    k_ref = rope(qkv[:, nh * d:(nh + nkv) * d].double().view(T, nkv, d))
    v_ref = qkv[:, (nh + nkv) * d:].double().view(T, nkv, d)
    tol = 1e-6 if qd == torch.float32 else 5e-3
    assert rel_err(q_out.view(T, nh, d), q_ref) < tol
    got = view.pages.cpu()
    touched = torch.zeros(n_pages, P, dtype=torch.bool)
    for t in range(T):
        r, pos = int(row_req[t]), int(positions[t])
        pg = int(table[r, pos // P])
        touched[pg, pos % P] = True
        assert rel_err(got[pg, 0, :, pos % P], k_ref[t]) < tol
        assert rel_err(got[pg, 1, :, pos % P], v_ref[t]) < tol
    untouched = got.float()[:, :, :, :, :][~touched[:, None, None, :].expand(n_pages, 2, nkv, P)]
    assert bool((untouched == 7.0).all()), "a slot outside the step's positions was written"


@pytest.mark.parametrize("nh,nkv,d,K,lens,writes", [(8, 4, 256, 2304, [700, 330], True), (3, 1, 256, 264, [1500, 1480, 20], True),
                                                    (2, 2, 256, 512, [3100], False), (16, 8, 256, 520, [300, 257], True),
                                                    (16, 8, 256, 328, [1300, 1000], True), (32, 16, 128, 520, [600], True),
                                                    (5, 1, 128, 264, [2000, 1000], True)])
def test_qkv_product_that_rotates_and_files_its_result(ops, nh, nkv, d, K, lens, writes):
    """The q,k,v product of a long prompt with head size 256 or 128 writes rotated q rows and the pages itself.  Against float64
    from the same bfloat16 operands, and against the two-kernel path (32-bit rows, then rotation and append) to within one
    bfloat16 rounding; requests at different positions on scattered pages, padding rows, an odd number of heads (the last CTA
    pair has one head), a K that is no multiple of 64, a cache that is not written; tiles of 128 tokens (the first three
    cases: few tiles) and of 256 (the next two; the second with more tiles than CTA pairs); head size 128 puts two heads
    into a CTA (the last two cases; seven heads leave the last CTA one)."""
    P = 64
    g = torch.Generator().manual_seed(nh * 100 + K)
    starts = [37, 0, 130][:len(lens)]
    T_real = sum(lens)
    T = T_real + 9                                                   # nine padding rows at the end
    N = (nh + 2 * nkv) * d
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * (2.0 / K ** 0.5)).to(torch.bfloat16)
    positions = torch.tensor([s0 + i for s0, n in zip(starts, lens) for i in range(n)] + [0] * 9, dtype=torch.int32)
    row_req = torch.tensor([r for r, n in enumerate(lens) for _ in range(n)] + [-1] * 9, dtype=torch.int32)
    need = [-(-(s0 + n) // P) for s0, n in zip(starts, lens)]
    n_pages = sum(need) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lens), max(need) + 1), -1, dtype=torch.int32)
    for r, n in enumerate(need):
        table[r, :n] = torch.tensor([perm.pop() for _ in range(n)])
    inv = (10000.0 ** (-2.0 * torch.arange(d // 2, dtype=torch.float64) / d)).float()
    ang = positions.float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).to(DEV), torch.sin(ang).to(DEV)
    ctx = _Ctx(positions.to(DEV), row_req.to(DEV), table.to(DEV))
    xd, wd = x.to(DEV), w.to(DEV)

    def run(fused):
        pages = torch.full((n_pages, 2, nkv, P, d), 7.0, dtype=torch.bfloat16, device=DEV)
        view = _View(pages, P, writes)
        q = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        if fused:
            assert ops.linear_rope_kv_append(xd, wd, cos, sin, d, nh, nkv, d, ctx, view, q), "the fused product declined"
        else:
            qkv = torch.empty(T, N, device=DEV)
            ops.linear(xd, wd, qkv)
            ops.rope_kv_append(qkv, cos, sin, d, nh, nkv, d, ctx, view, q)
        ops.raise_on_device_error()
        return q.float().cpu(), pages.float().cpu()

    q_f, pages_f = run(True)
    q_u, pages_u = run(False)
    qkv = x.double() @ w.double().T
    c, s_ = cos.double().cpu()[:, None, :], sin.double().cpu()[:, None, :]

    def rope(h):
        a, b = h[..., :d // 2], h[..., d // 2:]
        return torch.cat([a * c - b * s_, a * s_ + b * c], dim=-1)
    q_ref = rope(qkv[:, :nh * d].view(T, nh, d))
    q_ref[T_real:] = 0                                               # rows of no request give zero q
    k_ref = rope(qkv[:, nh * d:(nh + nkv) * d].view(T, nkv, d))
    v_ref = qkv[:, (nh + nkv) * d:].view(T, nkv, d)
    scale = float(qkv.abs().max())
    assert float((q_f.view(T, nh, d) - q_ref).abs().max()) < 6e-3 * scale
    assert float((q_f - q_u).abs().max()) <= 2 ** -7 * scale, "more than a bfloat16 rounding from the two-kernel path"
    assert float((pages_f - pages_u).abs().max()) <= 2 ** -7 * scale
    touched = torch.zeros(n_pages, P, dtype=torch.bool)
    if writes:
        for t in range(T_real):
            r, pos = int(row_req[t]), int(positions[t])
            pg = int(table[r, pos // P])
            touched[pg, pos % P] = True
            assert float((pages_f[pg, 0, :, pos % P] - k_ref[t]).abs().max()) < 6e-3 * scale
            assert float((pages_f[pg, 1, :, pos % P] - v_ref[t]).abs().max()) < 6e-3 * scale
    untouched = pages_f[~touched[:, None, None, :].expand(n_pages, 2, nkv, P)]
    assert bool((untouched == 7.0).all()), "a slot outside the step's positions was written"


@pytest.mark.parametrize("V", [512, 1000, 256000])
def test_argmax_and_topk(ops, V):
    g = torch.Generator().manual_seed(10)
    logits = torch.randn(5, V, generator=g)
    logits[1, 7] = logits[1, V - 3] = 99.0          # equal maxima: the first wins
    logits[2] = torch.round(logits[2] * 2) / 2       # many ties
    dev = logits.to(DEV)
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(dev, out)
    assert out.tolist() == torch.argmax(logits, -1).tolist() and out[1].item() == 7
    for k in (1, 40, 64):
        ids = torch.empty(5, k, dtype=torch.int32, device=DEV)
        vals = torch.empty(5, k, device=DEV)
        lse = torch.empty(5, device=DEV)
        ops.topk_lse(dev, k, ids, vals, lse)
        order = torch.argsort(-logits.double(), dim=-1, stable=True)[:, :k]
        assert ids.cpu().tolist() == order.tolist()
        assert torch.equal(vals.cpu(), torch.gather(logits, 1, order))
        assert float((lse.cpu().double() - torch.logsumexp(logits.double(), -1)).abs().max()) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_random_weights_are_the_same_bits_on_host_and_device(ops, dtype):
    """The counter-based generator of random-weights mode: the kernel and its numpy restatement give equal tensors."""
    from kungfu_b200.weights.store import TensorSpec, random_tensor, random_tensor_device
    for spec in (TensorSpec("model.layers.0.mlp.up_proj.weight", (333, 517), 0.02), TensorSpec("n", (2304,), 0.1, "norm"),
                 TensorSpec("big", (1 << 21,), 1.7)):
        host = random_tensor(spec, 11, dtype)
        dev = random_tensor_device(spec, 11, dtype, torch.device(DEV))
        assert dev.dtype == dtype and torch.equal(dev.cpu(), host), spec.name
    table = TensorSpec("ids", (1000,), 1.0, "table")
    assert torch.equal(random_tensor_device(table, 5, torch.int32, torch.device(DEV)).cpu(), random_tensor(table, 5))


@pytest.mark.parametrize("ratio", [0.5, 1.0, 3.0])
@pytest.mark.parametrize("path,nh,nkv,d,P,cap", [("prefill tcgen05", 8, 4, 256, 64, 50.0), ("prefill tcgen05", 6, 2, 128, 64, 20.0),
                                                 ("prefill tcgen05 cut", 4, 2, 64, 64, 30.0), ("prefill mma.sync", 6, 2, 32, 16, 20.0),
                                                 ("decode mma", 8, 4, 256, 64, 50.0), ("decode mma", 32, 16, 128, 64, 20.0),
                                                 ("decode simt", 8, 4, 256, 64, 50.0), ("generic", 9, 3, 48, 8, 30.0)])
def test_softcap_where_it_bends(ops, path, nh, nkv, d, P, cap, ratio):
    """Every bfloat16 attention kernel with queries scaled so that the largest scores before the cap reach `ratio` caps:
    half a cap (the polynomial branch of the tcgen05 kernel), one cap, and three caps (its exponential branch, and
    saturation), against float64, with a scale that is not 1/sqrt(head size) (Gemma 2 27B: 1/sqrt(144) with heads of
    128).  The same reference without the cap, or with 1/sqrt(head size), is far outside the tolerance, so a kernel
    that dropped or misplaced the cap or derived the scale from the head size would fail here."""
    lens = [300, 90, 1] if path.startswith("prefill") or path == "generic" else [300, 2100, 65, 1]
    pages, table, ks, vs = _paged_setup(torch.bfloat16, nh, nkv, d, P, lens, seed=61)
    if path.startswith("prefill") or path == "generic":
        rows = [(r, p) for r, n in enumerate(lens[:2]) for p in range(n)]
        dec, pre = [], list(range(len(rows)))
    else:
        rows = [(r, n - 1) for r, n in enumerate(lens)]
        dec, pre = list(range(len(rows))), []
    g = torch.Generator().manual_seed(62)
    scale = 0.6 / math.sqrt(d)
    # scale * q.k has spread 0.6 for unit-variance q and k: three spreads reach ratio * cap
    q = (torch.randn(len(rows), nh, d, generator=g) * (ratio * cap / 1.8)).to(torch.bfloat16)
    ctx = _Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
               torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV), dec, pre)
    out = torch.full((len(rows), nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    was = (ops.prefill_on_tcgen05, ops.decode_on_tensor_cores, ops.use_fast_attention, ops.prefill_plan_override)
    ops.prefill_on_tcgen05 = path.startswith("prefill tcgen05")
    ops.decode_on_tensor_cores = path == "decode mma"
    ops.use_fast_attention = path != "generic"
    ops.prefill_plan_override = (2, 0) if path == "prefill tcgen05 cut" else None
    try:
        ops.paged_attention(q.view(len(rows), nh * d).to(DEV), out, ctx, _View(pages.to(DEV), P), nh, nkv, d, scale, cap, None)
    finally:
        ops.prefill_on_tcgen05, ops.decode_on_tensor_cores, ops.use_fast_attention, ops.prefill_plan_override = was
    ops.raise_on_device_error()
    pick = list(range(0, len(rows), 5)) + [len(rows) - 1]
    ref = torch.stack([_attn_ref(q[i], ks[rows[i][0]], vs[rows[i][0]], rows[i][1], nh, nkv, scale, cap, None) for i in pick])
    nocap = torch.stack([_attn_ref(q[i], ks[rows[i][0]], vs[rows[i][0]], rows[i][1], nh, nkv, scale, 0.0, None) for i in pick])
    by_d = torch.stack([_attn_ref(q[i], ks[rows[i][0]], vs[rows[i][0]], rows[i][1], nh, nkv, 1.0 / math.sqrt(d), cap, None) for i in pick])
    got = out.view(len(rows), nh, d)[pick]
    assert bool(torch.isfinite(got.float()).all())
    assert rel_err(got, ref) < 1e-2
    if ratio >= 1.0:
        assert rel_err(nocap, ref) > 0.1, "the case must be one in which the cap matters"
        assert rel_err(by_d, ref) > 0.1, "and one in which the scale matters"


def test_rope_table_far_positions(ops):
    """cos and sin of position x frequency at positions where the 32-bit product alone is off by 1e-4 rad and more:
    the table keeps the product's rounding error and stays within 1e-6 of float64."""
    d, base = 256, 10000.0
    i = torch.arange(d // 2, dtype=torch.float64)
    inv = (base ** (-2.0 * i / d)).to(torch.float32)
    pos = torch.tensor([0, 1, 777, 4095, 4199, 8191, 131071], dtype=torch.int32)
    cos = torch.empty(len(pos), d // 2, device=DEV)
    sin = torch.empty(len(pos), d // 2, device=DEV)
    ops.rope_table(pos.to(DEV), inv.to(DEV), cos, sin)
    ang = pos.double()[:, None] * inv.double()[None, :]
    assert float((cos.cpu().double() - torch.cos(ang)).abs().max()) < 1e-6
    assert float((sin.cpu().double() - torch.sin(ang)).abs().max()) < 1e-6
    one_product = (pos.float()[:, None] * inv[None, :]).double()           # what a single 32-bit product would give
    assert float((torch.cos(one_product) - torch.cos(ang)).abs().max()) > 1e-4


def _device_sample(ops, logits, rules, seeds, recents, whole):
    """Rows of `logits` through ops.sample, row i under rules[i]; returns ids, states after, candidates."""
    import numpy as np
    from kungfu_b200.sampling import Sampling, pack_state
    n = logits.shape[0]
    st = np.stack([pack_state(Sampling(**rules[i]), seeds[i], recents[i]) for i in range(n)])
    states = torch.from_numpy(st).to(DEV)
    out = torch.full((n,), -7, dtype=torch.int32, device=DEV)
    # a permutation between rows and state slots, as a step has it
    slot_of = torch.arange(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, states, out, logit_rows=torch.arange(n, dtype=torch.int32, device=DEV), row_req=slot_of, req_slot=slot_of,
               whole_ranking=whole)
    return out.cpu().tolist(), states.cpu().numpy()


@pytest.mark.parametrize("V", [300, 5000, 70001])
def test_device_sampler_equals_the_plain_sampler(ops, V):
    """400 fuzzed rows per vocabulary size: every combination of temperature, top-k (within and beyond the 64
    candidates, and none), top-p, min-p and repeat penalty, logits with many equal values, tokens repeated in the window.
    The token, the generator state after the draw and the recorded token equal the plain sampler's
    (the reference checks its two samplers against each other the same way, crates/kf-engine/src/sampler.rs:229-321).
    Where the drawn number lies within 1e-5 of the kept mass from the edge of a token's share, the neighbouring token
    is accepted too: the device's exponential and numpy's may differ in the last bit."""
    import numpy as np
    import plain_sampler
    from kungfu_b200.sampling import RING, generator_state
    g = np.random.default_rng(V)
    rows_per_round, rounds = 8, 50
    exact = close = 0
    for rnd in range(rounds):
        l = (g.normal(size=(rows_per_round, V)) * g.choice([1.0, 3.0, 8.0])).astype(np.float32)
        if rnd % 3 == 0:
            l = np.round(l * 2) / 2                          # many equal values: the lower id ranks first
        if rnd % 7 == 0:
            l = np.clip(l, -2.0, 2.0)                       # hundreds of tokens share the maximum
        rules, seeds, recents = [], [], []
        for i in range(rows_per_round):
            rules.append(dict(temperature=float(g.choice([0.0, 0.7, 1.3])), top_k=int(g.choice([0, 1, 40, 64, 100, V])),
                              top_p=float(g.choice([1.0, 0.9, 0.5])), min_p=float(g.choice([0.0, 0.1])),
                              repeat_penalty=float(g.choice([1.0, 1.3, 0.8])), repeat_window=int(g.choice([0, 5, 64, 256]))))
            seeds.append(int(g.integers(0, 2 ** 62)))
            n_recent = int(g.choice([0, 3, 70, 300]))
            top = np.argsort(-l[i])[:5]
            recents.append([int(t) for t in g.choice(np.concatenate([top, g.integers(0, V, size=20)]), size=n_recent)])
        whole = any(r["temperature"] > 0 and (r["top_k"] == 0 or r["top_k"] > 64) for r in rules)
        got, states = _device_sample(ops, torch.from_numpy(l).to(DEV), rules, seeds, recents, whole)
        for i in range(rows_per_round):
            rng = plain_sampler.Rng(seeds[i])
            want, margin = plain_sampler.sample(l[i], recent=recents[i], rng=rng, **rules[i])
            assert generator_state(states[i]) == rng.state, (rnd, i, rules[i])
            assert states[i][8] == len(recents[i]) + 1 and states[i][16 + len(recents[i]) % RING] == got[i]
            if got[i] == want:
                exact += 1
                continue
            assert margin is not None and margin < 1e-5, (rnd, i, rules[i], got[i], want, margin)
            close += 1
    ops.raise_on_device_error()
    assert exact + close == rows_per_round * rounds and close <= 2, (exact, close)


def test_device_sampler_skips_padding_rows_and_follows_the_maps(ops):
    """Rows reach their request's state through logit_rows -> row_req -> req_slot; a row of request -1 (padding of a
    replayed graph) is skipped and touches no state."""
    import numpy as np
    import plain_sampler
    from kungfu_b200.sampling import Sampling, pack_state
    g = np.random.default_rng(1)
    V = 1000
    l = torch.from_numpy(g.normal(size=(3, V)).astype(np.float32) * 4).to(DEV)
    st = np.stack([pack_state(Sampling(temperature=1.0, top_k=40, top_p=1.0), 100 + s) for s in range(5)])
    states = torch.from_numpy(st).to(DEV)
    out = torch.full((3,), -7, dtype=torch.int32, device=DEV)
    logit_rows = torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV)          # rows of the step whose logits these are
    row_req = torch.tensor([1, 9, -1, 9, 0], dtype=torch.int32, device=DEV)      # request of each row of the step
    req_slot = torch.tensor([3, 2], dtype=torch.int32, device=DEV)               # state slot of each request
    ops.sample(l, states, out, logit_rows=logit_rows, row_req=row_req, req_slot=req_slot)
    after = states.cpu().numpy()
    want0, _ = plain_sampler.sample(l[0].cpu().numpy(), temperature=1.0, top_k=40, rng=plain_sampler.Rng(103))
    want1, _ = plain_sampler.sample(l[1].cpu().numpy(), temperature=1.0, top_k=40, rng=plain_sampler.Rng(102))
    assert out.cpu().tolist() == [want0, want1, 0]
    assert after[3][8] == 1 and after[2][8] == 1 and (after[[0, 1, 4]] == st[[0, 1, 4]]).all()


@pytest.mark.parametrize("T,N,K", [(8, 2304, 2304), (300, 4096, 2304), (16, 256, 2048)])
def test_a_wait_that_runs_out_leaves_a_status_and_a_usable_device(ops, T, N, K):
    """Every wait of the tensor-core kernels on a barrier is bounded.  Here one runs out: a test hook makes the
    weight-streaming product's producer leave out its loads from the second stage on and shortens the limit to 2 ms, so
    the thread that issues the MMAs waits for operands that never arrive.  The kernel must come back by itself (error
    word set, nothing trapped, tensor memory freed, every cluster barrier met), and the same product must be right
    again once the hook is off."""
    import ctypes
    import time
    lib = ops.library()
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    out = torch.zeros(T, N, device=DEV)
    ops.linear(x, w, out)                                    # builds tensor maps and the scratch before the hook is on
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    assert lib.kf_test_gemm_give_up(ctypes.c_ulonglong(2_000_000), 1) == 0
    try:
        t0 = time.perf_counter()
        ops.linear(x, w, out)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        code = ops.device_error()
    finally:
        assert lib.kf_test_gemm_give_up(ctypes.c_ulonglong(0), -1) == 0
    assert code in (1, 2, 3), code                           # operands never arrived / stage never freed / accumulator
    assert waited < 2.0
    with pytest.raises(ops.KernelError, match="gave up waiting"):
        ops.raise_on_device_error()
    ops.clear_device_error()
    again = torch.full((T, N), float("nan"), device=DEV)
    ops.linear(x, w, again)
    torch.cuda.synchronize()
    assert ops.device_error() == 0
    assert rel_err(again, x.double() @ w.double().T) < 2e-6 * math.sqrt(K) + 1e-6


def test_nvtx_ranges_can_be_switched_on(ops):
    x = torch.randn(4, 64, device=DEV)
    w = torch.zeros(64, device=DEV)
    out = torch.empty(4, 64, device=DEV)
    ops.nvtx_ranges = True
    try:
        ops.rmsnorm(x, w, 1e-6, True, out)
        with ops.nvtx_range("a part"):
            ops.rmsnorm(x, w, 1e-6, True, out)
    finally:
        ops.nvtx_ranges = False
    assert rel_err(out, x.double() * torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + 1e-6)) < 1e-5
