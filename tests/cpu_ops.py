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

    # ---- short convolution, q|k|v preparation, state-space scan (restatements of what the kernels of the same names do) ----------------
    @staticmethod
    def _conv_inputs(proj, col0, in_bias, C, taps, state, ctx, req):
        """[taps - 1 + n, C]: the state of request `req` followed by its biased inputs of this step."""
        r0, n, slot = int(ctx.req_row_start[req]), int(ctx.req_n_rows[req]), int(ctx.req_state_slot[req])
        u = proj[r0:r0 + n, col0:col0 + C].float()
        if in_bias is not None:
            u = u + in_bias.float()[None, :]
        old = state[slot, :taps - 1].float() if (state is not None and taps > 1) else torch.zeros(0, C)
        return torch.cat([old, u], 0), r0, n, slot

    def short_conv(self, proj, col0, in_bias, weight, out_bias, act, state, out, ctx, commit_inline=False):
        C, taps = weight.shape
        for req in range(ctx.n_reqs):
            if int(ctx.req_n_rows[req]) <= 0:
                continue
            u, r0, n, _ = self._conv_inputs(proj, col0, in_bias, C, taps, state, ctx, req)
            y = torch.zeros(n, C)
            for j in range(taps):
                y += u[j:j + n] * weight[:, j].float()[None, :]
            if out_bias is not None:
                y = y + out_bias.float()[None, :]
            if act == "silu":
                y = y * torch.sigmoid(y)
            out[r0:r0 + n] = y
        return False                                   # the state is never moved on here: the caller runs the commit

    def short_conv_commit(self, proj, col0, in_bias, n_channels, taps, state, ctx, w_dtype=None):
        if taps <= 1:
            return
        for req in range(ctx.n_reqs):
            if int(ctx.req_n_rows[req]) <= 0:
                continue
            u, _, _, slot = self._conv_inputs(proj, col0, in_bias, n_channels, taps, state, ctx, req)
            state[slot, :taps - 1] = u[-(taps - 1):]

    def qkv_prepare(self, proj, col0, in_bias, conv_w, conv_state, q_norm, k_norm, eps, cos, sin, rot, interleaved,
                    nh, nkv, dk, dv, ctx, cache, q_out, commit_inline=False):
        T = q_out.shape[0]
        D = cache.pages.shape[-1]
        C = (nh + nkv) * dk + nkv * dv
        x = torch.zeros(T, C)
        if conv_w is not None:
            self.short_conv(proj, col0, in_bias, conv_w, None, None, conv_state, x, ctx)
        else:
            x = proj[:, col0:col0 + C].float() + (in_bias.float()[None, :] if in_bias is not None else 0.0)
        q = x[:, :nh * dk].reshape(T, nh, dk).clone()
        k = x[:, nh * dk:(nh + nkv) * dk].reshape(T, nkv, dk).clone()
        v = x[:, (nh + nkv) * dk:].reshape(T, nkv, dv)
        for y, w in ((q, q_norm), (k, k_norm)):
            if w is not None:
                y.copy_(y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * w.float())
        if rot:
            c, s_ = cos[:, None, :], sin[:, None, :]
            for y in (q, k):
                if interleaved:
                    a, b = y[..., 0:rot:2].clone(), y[..., 1:rot:2].clone()
                    y[..., 0:rot:2] = a * c - b * s_
                    y[..., 1:rot:2] = b * c + a * s_
                else:
                    a, b = y[..., :rot // 2].clone(), y[..., rot // 2:rot].clone()
                    y[..., :rot // 2] = a * c - b * s_
                    y[..., rot // 2:rot] = a * s_ + b * c
        qp = torch.zeros(T, nh, D)
        qp[..., :dk] = q
        valid = (ctx.row_req[:T] >= 0)
        qp[~valid] = 0
        q_out.copy_(qp.reshape(T, nh * D).to(q_out.dtype))
        if not cache.writes:
            return False
        table = ctx.block_tables[cache.group]
        P = cache.page_size
        for t in range(T):
            r = int(ctx.row_req[t])
            if r < 0:
                continue
            pos = int(ctx.positions[t])
            page = int(table[r, pos // P])
            assert page >= 0
            cache.pages[page, :, :, pos % P, :] = 0
            cache.pages[page, 0, :, pos % P, :dk] = k[t].to(cache.pages.dtype)
            cache.pages[page, 1, :, pos % P, :dv] = v[t].to(cache.pages.dtype)
        return False

    def head_gate(self, o, proj, gate_col0, nh, dv, D, out, ctx):
        T = out.shape[0]
        y = o.float().view(T, nh, D)[..., :dv]
        if proj is not None:
            y = y * torch.sigmoid(proj[:, gate_col0:gate_col0 + nh].float())[..., None]
        y = y * (ctx.row_req[:T] >= 0).float()[:, None, None]
        out.copy_(y.reshape(T, nh * dv).to(out.dtype))

    def ssm_scan(self, xbc, proj, dt_col0, dt_bias, a_log, d_skip, state, y, heads, groups, P, N, ctx, writes=True):
        inner = heads * P
        A = -torch.exp(a_log.float())
        for req in range(ctx.n_reqs):
            n = int(ctx.req_n_rows[req])
            if n <= 0:
                continue
            r0, slot = int(ctx.req_row_start[req]), int(ctx.req_state_slot[req])
            S = state[slot].clone()                                   # [heads, P, N]
            for i in range(n):
                row = xbc[r0 + i]
                dt = torch.nn.functional.softplus(proj[r0 + i, dt_col0:dt_col0 + heads].float() + dt_bias.float(), threshold=20.0)
                for h in range(heads):
                    g = h // (heads // groups)
                    x = row[h * P:(h + 1) * P]
                    B = row[inner + g * N:inner + (g + 1) * N]
                    C = row[inner + groups * N + g * N:inner + groups * N + (g + 1) * N]
                    S[h] = torch.exp(A[h] * dt[h]) * S[h] + dt[h] * torch.outer(x, B)
                    y[r0 + i, h * P:(h + 1) * P] = S[h] @ C + d_skip[h].float() * x
            if writes:
                state[slot] = S

    def gated_group_norm(self, y, proj, z_col0, weight, eps, parts, out, ctx):
        T, inner = out.shape
        z = proj[:, z_col0:z_col0 + inner].float()
        v = (y * (z * torch.sigmoid(z))).view(T, parts, inner // parts)
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        v = v.reshape(T, inner) * weight.float()[None, :]
        v = torch.where((ctx.row_req[:T] >= 0)[:, None], v, torch.zeros_like(v))
        out.copy_(v.to(out.dtype))

    def add2_rmsnorm(self, a, b, x, *, next_weight=None, next_eps=0.0, next_plus_one=False, next_out=None):
        x.add_(a if b is None else a + b)
        if next_out is not None:
            self.rmsnorm(x, next_weight, next_eps, next_plus_one, next_out)

    def activation(self, x, out, act):
        out.copy_(_act(act, x.float()).to(out.dtype))

    def linear_act(self, x, w_up, out, activation, ctx):
        out.copy_(_act(activation, x.float() @ w_up.float().T).to(out.dtype))

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
