"""A slow CPU stand-in for `kungfu_b200.ops`, for tests on machines without a GPU.

It lets the engine's host logic (metadata, block tables, page reuse, scheduling) be checked against
the plain implementation without any kernel.  It is test equipment: the package has no CPU path and
never imports this file.  Each function mirrors the contract of the kernel of the same name.
"""
from __future__ import annotations

import math

import torch


def _act(name, x):
    if name == "gelu_tanh":
        return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    if name == "gelu_erf":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    return x * torch.sigmoid(x)


class CpuOps:
    def check_attention_sizes(self, nh, nkv, d):
        assert nh % nkv == 0 and d % 2 == 0

    def embed(self, tokens, table, scale, out):
        out.copy_(table.float()[tokens.long()] * torch.tensor(scale, dtype=torch.float32))

    def rmsnorm(self, x, weight, eps, plus_one, out, rows=None):
        xs = x if rows is None else x[rows.long()]
        inv = torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + eps)
        g = weight.float() + (1.0 if plus_one else 0.0)
        out.copy_((xs * inv * g).to(out.dtype))

    def add_rmsnorm(self, branch, weight, eps, plus_one, residual, *, next_weight=None, next_eps=0.0,
                    next_plus_one=False, next_out=None):
        inv = torch.rsqrt(branch.pow(2).mean(-1, keepdim=True) + eps)
        residual.add_(branch * inv * (weight.float() + (1.0 if plus_one else 0.0)))
        if next_out is not None:
            self.rmsnorm(residual, next_weight, next_eps, next_plus_one, next_out)

    def add(self, a, x):
        x.add_(a)

    def linear(self, x, weight, out, softcap=0.0):
        y = x.float() @ weight.float().T
        if softcap > 0:
            y = softcap * torch.tanh(y / softcap)
        out.copy_(y.to(out.dtype))

    def linear_gated(self, x, w_gate_up, out, activation, ctx):
        I = out.shape[1]
        gu = x.float() @ w_gate_up.float().T
        out.copy_((_act(activation, gu[:, :I]) * gu[:, I:]).to(out.dtype))

    def rope_table(self, positions, inv_freq, cos, sin):
        ang = positions.float()[:, None] * inv_freq[None, :]
        cos.copy_(torch.cos(ang))
        sin.copy_(torch.sin(ang))

    def linear_rope_kv_append(self, x, wqkv, cos, sin, rot, nh, nkv, d, ctx, cache, q_out):
        return False                                   # no fused product here: the caller runs linear and rope_kv_append

    def rope_kv_append(self, qkv, cos, sin, rot, nh, nkv, d, ctx, cache, q_out):
        T = qkv.shape[0]
        q = qkv[:, :nh * d].view(T, nh, d).clone()
        k = qkv[:, nh * d:(nh + nkv) * d].view(T, nkv, d).clone()
        v = qkv[:, (nh + nkv) * d:].view(T, nkv, d)
        if rot:
            half = rot // 2
            c, s = cos[:, None, :], sin[:, None, :]
            for x in (q, k):
                a, b = x[..., :half].clone(), x[..., half:rot].clone()
                x[..., :half] = a * c - b * s
                x[..., half:rot] = a * s + b * c
        q_out.copy_(q.reshape(T, nh * d).to(q_out.dtype))
        if not cache.writes:
            return
        table = ctx.block_tables[cache.group]
        P = cache.page_size
        for t in range(T):
            r = int(ctx.row_req[t])
            if r < 0:
                continue
            pos = int(ctx.positions[t])
            page = int(table[r, pos // P])
            assert page >= 0
            cache.pages[page, 0, :, pos % P, :] = k[t].to(cache.pages.dtype)
            cache.pages[page, 1, :, pos % P, :] = v[t].to(cache.pages.dtype)

    def paged_attention(self, q, out, ctx, cache, nh, nkv, d, scale, softcap, window):
        T = q.shape[0]
        table = ctx.block_tables[cache.group]
        P = cache.page_size
        group = nh // nkv
        for t in range(T):
            r = int(ctx.row_req[t])
            if r < 0:
                out[t] = 0
                continue
            pos = int(ctx.positions[t])
            lo = max(0, pos - window + 1) if window else 0
            js = list(range(lo, pos + 1))
            pages = [int(table[r, j // P]) for j in js]
            assert all(p >= 0 for p in pages), f"row {t} reads a page that was given back"
            slots = [j % P for j in js]
            K = cache.pages[pages, 0, :, slots, :].float()        # [n, nkv, d]
            V = cache.pages[pages, 1, :, slots, :].float()
            qt = q[t].float().view(nh, d)
            for h in range(nh):
                s = (K[:, h // group] @ qt[h]) * scale
                if softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                p = torch.softmax(s, dim=0)
                out[t, h * d:(h + 1) * d] = (p @ V[:, h // group]).to(out.dtype)

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))

    def sample(self, logits, states, out_ids, *, logit_rows=None, row_req=None, req_slot=None, whole_ranking=False,
               cand_ids=None, cand_vals=None, cand_lse=None):
        """The device sampler's stand-in: the plain sampler of tests/plain_sampler.py on each row, reading and updating
        the per-request state words as the kernels do."""
        import numpy as np
        import plain_sampler
        from kungfu_b200.sampling import RING, generator_state
        st_all = states.numpy()
        for i in range(logits.shape[0]):
            lr = i if logit_rows is None else int(logit_rows[i])
            rq = 0 if row_req is None else int(row_req[lr])
            if rq < 0:
                out_ids[i] = 0
                continue
            st = st_all[rq if req_slot is None else int(req_slot[rq])]
            f = st[2:6].view(np.float32)
            count = int(st[8])
            recent = [int(st[16 + j % RING]) for j in range(max(0, count - RING), count)]
            rng = plain_sampler.Rng(1)
            rng.state = generator_state(st)
            tok, _ = plain_sampler.sample(logits[i].float().numpy(), temperature=float(f[0]), top_k=int(st[6]), top_p=float(f[1]),
                                          min_p=float(f[2]), repeat_penalty=float(f[3]), repeat_window=int(st[7]),
                                          recent=recent, rng=rng)
            st[0:2] = np.array([rng.state & 0xFFFFFFFF, rng.state >> 32], dtype=np.uint32).view(np.int32)
            st[16 + count % RING] = tok
            st[8] = count + 1
            out_ids[i] = tok

    def topk_lse(self, logits, k, out_ids, out_vals, out_lse):
        V = logits.shape[1]
        # falling value, lower id first among equals
        order = torch.argsort(-logits.double() * 1.0, dim=-1, stable=True)[:, :k]
        out_ids.copy_(order.to(torch.int32))
        out_vals.copy_(torch.gather(logits, 1, order))
        out_lse.copy_(torch.logsumexp(logits.double(), dim=-1).float())
