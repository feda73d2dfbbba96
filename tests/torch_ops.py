"""Plain PyTorch statements of what each CUDA kernel of the engine computes, with the kernels'
own signatures. Used by the tests only: as the reference each kernel is compared with, and to run
the engine's host-side logic (cache, batching, scheduler) on a machine without a GPU.
Math is done in float64 and rounded once to the output's dtype.
"""
from __future__ import annotations


import torch

from nanoinfer_b200.parts.base import as_tensor


class TorchOps:
    name = "torch-reference"

    def embed(self, ids, table, out32, scale=1.0):
        out32.copy_((table[ids.long()].double() * scale).to(torch.float32))

    def rmsnorm(self, x32, gain32, eps, out, rows=None):
        x = x32.double() if rows is None else x32[rows.long()].double()
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gain32.double()
        out.copy_(y.to(out.dtype))

    def linear(self, a, w, bias32, out, mode):
        a = as_tensor(a)
        y = a.double() @ w.double().t()
        if bias32 is not None:
            y = y + bias32.double()
        if mode == "add":
            out.copy_((out.double() + y).to(out.dtype))
        elif mode in ("store", "f32"):
            out.copy_(y.to(out.dtype))
        else:
            raise ValueError(mode)

    def linear_swiglu(self, a, w_gate_up, out):
        a = as_tensor(a)
        inter = w_gate_up.shape[0] // 2
        g = a.double() @ w_gate_up[:inter].double().t()
        u = a.double() @ w_gate_up[inter:].double().t()
        out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))

    def qkv_project(self, a, w_qkv, bias32, qkv, heads, kv_heads, head_dim, positions, req_index, rotary,
                    block_table, page_size, k_pages, v_pages, writes):
        self.linear(a, w_qkv, bias32, qkv, "store")
        self.rope_store(qkv, heads, kv_heads, head_dim, positions, req_index, rotary, block_table, page_size,
                        k_pages, v_pages, writes)

    def rope_store(self, qkv, heads, kv_heads, head_dim, positions, req_index, rotary, block_table,
                   page_size, k_pages, v_pages, writes):
        m = qkv.shape[0]
        x = qkv.double().view(m, heads + 2 * kv_heads, head_dim)
        if rotary is not None:
            cos, sin, dim = rotary
            half = dim // 2
            c = cos[positions.long()].double()[:, None, :]
            s = sin[positions.long()].double()[:, None, :]
            qk = x[:, :heads + kv_heads, :]
            x1, x2 = qk[..., :half].clone(), qk[..., half:dim].clone()
            qk[..., :half] = x1 * c - x2 * s
            qk[..., half:dim] = x2 * c + x1 * s
        qkv.copy_(x.view(m, -1).to(qkv.dtype))
        if not writes:
            return
        pos = positions.long()
        page = block_table[req_index.long(), pos // page_size].long()
        assert (page >= 0).all(), "write to a position without a page"
        off = pos % page_size
        k = qkv.view(m, heads + 2 * kv_heads, head_dim)[:, heads:heads + kv_heads]
        v = qkv.view(m, heads + 2 * kv_heads, head_dim)[:, heads + kv_heads:]
        k_pages[page, :, off, :] = k
        v_pages[page, :, off, :] = v

    def attention(self, qkv, out, heads, kv_heads, head_dim, scale, window, ctx, block_table,
                  page_size, k_pages, v_pages, own_kv=False):
        m = qkv.shape[0]
        q = qkv.view(m, heads + 2 * kv_heads, head_dim)[:, :heads].double()
        n_rep = heads // kv_heads
        res = torch.zeros(m, heads, head_dim, dtype=torch.float64, device=qkv.device)
        positions = ctx.positions.tolist()
        req_index = ctx.req_index.tolist()
        for t in range(m):
            p, r = positions[t], req_index[t]
            lo = max(0, p - window + 1) if window else 0
            idx = torch.arange(lo, p + 1, device=qkv.device)
            pages = block_table[r, idx // page_size].long()
            assert (pages >= 0).all(), "read of a position without a page"
            k = k_pages[pages, :, idx % page_size, :].double()   # [n, kv_heads, d]
            v = v_pages[pages, :, idx % page_size, :].double()
            for h in range(heads):
                s = (k[:, h // n_rep, :] @ q[t, h]) * scale
                e = torch.exp(s - s.max())
                res[t, h] = (e / e.sum()) @ v[:, h // n_rep, :]
        out.copy_(res.view(m, -1).to(out.dtype))

    # ---- row-wise and element-wise kernels of pointwise.cu ------------------------------------------
    def rmsnorm_pair(self, x32, gain_a32, gain_b32, eps, out_a, out_b):
        self.rmsnorm(x32, gain_a32, eps, out_a)
        self.rmsnorm(x32, gain_b32, eps, out_b)

    def poly_norm(self, z32, coef32, eps, out):
        z = z32.double()
        n = lambda y: y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps)
        c = coef32.double()
        out.copy_((c[0] * n(z) + c[1] * n(z ** 2) + c[2] * n(z ** 3) + c[3]).to(out.dtype))

    def depth_mix(self, hist32, x32, coef32, n):
        hist32[n - 1].copy_(x32)
        acc = torch.zeros_like(x32, dtype=torch.float64)
        for j in range(n):
            acc += coef32[j].double() * hist32[j].double()
        x32.copy_(acc.to(torch.float32))

    def depth_mix_norm_pair(self, hist32, x32, coef32, n, gain_a32, gain_b32, eps, out_a, out_b):
        self.depth_mix(hist32, x32, coef32, n)
        self.rmsnorm_pair(x32, gain_a32, gain_b32, eps, out_a, out_b)

    def unary(self, in32, out, kind):
        x = in32.double()
        out.copy_({"tanh": torch.tanh, "copy": lambda v: v, "sigmoid": torch.sigmoid}[kind](x).to(out.dtype))

    def head_norm_gate(self, o32, gate32, gain32, eps, heads, d, out):
        m = o32.shape[0]
        o = o32.double().view(m, heads, d)
        o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_((o.reshape(m, heads * d) * gain32.double() * torch.sigmoid(gate32.double())).to(out.dtype))

    def block_diag_linear(self, a_blocks, w_blocks, bias32, out32, a32=None):
        y = torch.einsum("bmk,bnk->bmn", a_blocks.double(), w_blocks.double())
        if bias32 is not None:
            y = y + bias32.double()[:, None, :]
        out32.copy_(y.to(torch.float32))

    # ---- attention with options (attention_flex.cu) --------------------------------------------------
    def attention_prepare(self, qkv32, q_out, heads, kv_heads, dim, vdim, q_gain32, k_gain32, eps, freq32, rot_dims, ctx,
                          block_table, page_size, k_pages, v_pages, writes, layout="half", unit_norm_after=False,
                          values_are_keys=False, norm_whole=False, v_first32=None, vmix32=None):
        m = qkv32.shape[0]
        nq, nk = heads * dim, kv_heads * dim
        q = qkv32[:, :nq].double().reshape(m, heads, dim)
        k = qkv32[:, nq:nq + nk].double().reshape(m, kv_heads, dim)
        v = k.clone() if values_are_keys else qkv32[:, nq + nk:].double().reshape(m, kv_heads, vdim)
        if v_first32 is not None:
            lam = vmix32.double().reshape(())
            v = (1.0 - lam) * v + lam * v_first32.double().reshape(m, kv_heads, vdim)
        if q_gain32 is not None and norm_whole:
            qf, kf = q.reshape(m, nq), k.reshape(m, nk)
            q = (qf / torch.sqrt(qf.pow(2).mean(-1, keepdim=True) + eps) * q_gain32.double()).reshape(m, heads, dim)
            k = (kf / torch.sqrt(kf.pow(2).mean(-1, keepdim=True) + eps) * k_gain32.double()).reshape(m, kv_heads, dim)
        elif q_gain32 is not None:
            q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_gain32.double()
            k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_gain32.double()
        if rot_dims:
            half = rot_dims // 2
            ang = ctx.positions.double()[:, None] * freq32.double()[None, :]
            c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]

            first = slice(0, half) if layout == "half" else slice(0, rot_dims, 2)
            second = slice(half, rot_dims) if layout == "half" else slice(1, rot_dims, 2)

            def turn(x):
                a, b = x[..., first].clone(), x[..., second].clone()
                x = x.clone()
                x[..., first] = a * c - b * s
                x[..., second] = b * c + a * s
                return x
            q, k = turn(q), turn(k)
        if unit_norm_after:
            q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps)
            k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps)
        q_out.copy_(q.reshape(m, nq).to(q_out.dtype))
        if not writes:
            return
        pos = ctx.positions.long()
        page = block_table[ctx.req_index.long(), pos // page_size].long()
        ok = page >= 0      # padding rows of a replayed step hold no pages
        k_pages[page[ok], :, (pos % page_size)[ok], :] = k[ok].to(k_pages.dtype)
        v_pages[page[ok], :, (pos % page_size)[ok], :] = v[ok].to(v_pages.dtype)

    def attention_flex(self, q, out, heads, kv_heads, dim, vdim, scale, softcap, slopes32, window, chunk, out_scale, ctx,
                       block_table, page_size, k_pages, v_pages, sinks32=None):
        m = q.shape[0]
        qh = q.double().view(m, heads, dim)
        rep = heads // kv_heads
        res = torch.zeros(m, heads, vdim, dtype=torch.float64, device=q.device)
        for t in range(m):
            pos, r = int(ctx.positions[t]), int(ctx.req_index[t])
            lo = max(0, pos - window + 1) if window else 0
            if chunk:
                lo = max(lo, (pos // chunk) * chunk)
            js = torch.arange(lo, pos + 1)
            pages = block_table[r, js // page_size].long()
            if (pages < 0).any():
                continue        # a padding row
            k = k_pages[pages, :, js % page_size, :].double()       # [keys, kv_heads, dim]
            v = v_pages[pages, :, js % page_size, :].double()
            for h in range(heads):
                s = (k[:, h // rep] @ qh[t, h]) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                if slopes32 is not None:
                    s = s - slopes32[h].double() * (pos - js).double()
                if sinks32 is not None:     # one more term of the denominator, with no value
                    w = torch.softmax(torch.cat([s, sinks32[h].double().reshape(1)]), 0)[:-1]
                else:
                    w = torch.softmax(s, 0)
                res[t, h] = w @ v[:, h // rep]
        out.copy_((res.view(m, heads * vdim) * out_scale).to(out.dtype))

    # ---- gate, norm in groups, skip (pointwise.cu) ---------------------------------------------------
    def gated_norm(self, o32, out, groups=0, eps=0.0, gain32=None, gate32=None, gate_kind="none", gate_first=False,
                   skip32=None, skip_coef32=None, out_scale=1.0):
        m, n = o32.shape
        y = o32.double()
        if skip32 is not None:
            y = y + skip32.double() * skip_coef32.double().repeat_interleave(n // skip_coef32.numel())
        act = {"sigmoid": torch.sigmoid, "silu": lambda z: z * torch.sigmoid(z)}.get(gate_kind)
        if act is not None and gate_first:
            y = y * act(gate32.double())
        if groups:
            y = y.view(m, groups, n // groups)
            y = (y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps)).reshape(m, n)
        if gain32 is not None:
            y = y * gain32.double().repeat(n // gain32.numel())
        if act is not None and not gate_first:
            y = y * act(gate32.double())
        out.copy_((y * out_scale).to(out.dtype))

    # ---- matrix states that decay (linear_state.cu) --------------------------------------------------
    def conv_tokens(self, x32, w32, bias32, act, state, state_off, ctx, out32, taps):
        start = 0
        width = x32.shape[1]
        for q_len, slot in zip(ctx.host.q_lens, ctx.host.slots):
            if taps > 1:
                hist = state[slot, state_off:state_off + (taps - 1) * width].double().view(taps - 1, width)
            else:
                hist = torch.zeros(0, width, dtype=torch.float64)
            padded = torch.cat([hist, x32[start:start + q_len].double()], 0)
            u = torch.zeros(q_len, width, dtype=torch.float64)
            for j in range(taps):
                u += padded[j:j + q_len] * w32[:, j].double()
            if bias32 is not None:
                u = u + bias32.double()
            if act == "silu":
                u = u * torch.sigmoid(u)
            out32[start:start + q_len] = u.to(torch.float32)
            start += q_len

    def conv_tail(self, x32, state, state_off, ctx, taps):
        start = 0
        width = x32.shape[1]
        for q_len, slot in zip(ctx.host.q_lens, ctx.host.slots):
            hist = state[slot, state_off:state_off + (taps - 1) * width].view(taps - 1, width)
            padded = torch.cat([hist.clone(), x32[start:start + q_len]], 0)
            hist.copy_(padded[-(taps - 1):])
            start += q_len

    def conv_step(self, x32, w32, bias32, act, state, state_off, ctx, out32, taps):
        self.conv_tokens(x32, w32, bias32, act, state, state_off, ctx, out32, taps)
        if taps > 1:
            self.conv_tail(x32, state, state_off, ctx, taps)

    def token_shift(self, h, mu32, state, state_off, ctx, mixes):
        start = 0
        width = h.shape[1]
        for q_len, slot in zip(ctx.host.q_lens, ctx.host.slots):
            cur = h[start:start + q_len].double()
            prev = torch.cat([state[slot, state_off:state_off + width].double()[None, :], cur[:-1]], 0)
            for s in range(mu32.shape[0]):
                mixes[s, start:start + q_len] = (cur + (prev - cur) * mu32[s].double()).to(mixes.dtype)
            state[slot, state_off:state_off + width] = cur[-1].to(torch.float32)
            start += q_len

    def decay_map(self, z32, out32, kind, param):
        z = z32.double()
        if kind == "sigmoid_root":
            out32.copy_(torch.exp(torch.nn.functional.logsigmoid(z) / param).to(torch.float32))
        elif kind == "exp_neg_exp":
            out32.copy_(torch.exp(-torch.exp(z)).to(torch.float32))
        else:
            raise ValueError(kind)

    def step_sizes(self, dt_raw32, dt_bias32, a_log32, dt_out, decay_out):
        dt = torch.nn.functional.softplus(dt_raw32.double() + dt_bias32.double(), threshold=1e9)
        dt_out.copy_(dt.to(torch.float32))
        decay_out.copy_(torch.exp(-torch.exp(a_log32.double()) * dt_out.double()).to(torch.float32))

    def linear_state_scan(self, q32, k32, v32, w32, state, state_off, ctx, o32, heads, kq_heads, dk, dv, q_scale=1.0,
                          bonus32=None, v_scale32=None, seg_len=None):
        start = 0
        rep = heads // kq_heads
        per_channel = w32.shape[1] == heads * dk
        for q_len, slot in zip(ctx.host.q_lens, ctx.host.slots):
            flat = state[slot, state_off:state_off + heads * dv * dk]
            s = flat.double().view(heads, dv, dk).transpose(1, 2).clone()      # [head, key channel, value channel]
            for t in range(start, start + q_len):
                q = (q32[t].double() * q_scale).view(kq_heads, dk).repeat_interleave(rep, 0)
                k = k32[t].double().view(kq_heads, dk).repeat_interleave(rep, 0)
                v = v32[t].double().view(heads, dv)
                if v_scale32 is not None:
                    v = v * v_scale32[t].double()[:, None]
                w = w32[t].double().view(heads, dk) if per_channel else w32[t].double()[:, None].expand(heads, dk)
                kv = k[:, :, None] * v[:, None, :]
                if bonus32 is not None:
                    o = torch.einsum("hkv,hk->hv", s + bonus32.double()[:, :, None] * kv, q)
                    s = w[:, :, None] * s + kv
                else:
                    s = w[:, :, None] * s + kv
                    o = torch.einsum("hkv,hk->hv", s, q)
                o32[t] = o.reshape(-1).to(torch.float32)
            flat.copy_(s.transpose(1, 2).reshape(-1).to(torch.float32))
            start += q_len

    # ---- recurrent mixers of recurrent.cu -----------------------------------------------------------
    def delta_rule_scan(self, r32, k32, v32, a_logit32, w_logit32, state, ctx, o32, heads, d):
        import math
        start = 0
        for q_len, slot in zip(ctx.host.q_lens, ctx.host.slots):
            S = state[slot].double().transpose(1, 2).clone()            # kept as [head, value, key]; here [head, key, value]
            for t in range(start, start + q_len):
                r, k, v = (x[t].double().view(heads, d) for x in (r32, k32, v32))
                a = torch.sigmoid(a_logit32[t].double()).view(heads, d)
                w = torch.exp(-math.exp(-0.5) * torch.sigmoid(w_logit32[t].double())).view(heads, d)
                u = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
                proj = torch.einsum("hk,hkv->hv", u, S)
                S = w[:, :, None] * S - (a * u)[:, :, None] * proj[:, None, :] + k[:, :, None] * v[:, None, :]
                o32[t] = torch.einsum("hkv,hk->hv", S, r).reshape(-1).to(torch.float32)
            state[slot] = S.transpose(1, 2).to(torch.float32)
            start += q_len

    def causal_conv(self, x32, w32, bias32, state, hist_row0, ctx, u32, u_blocks, taps, blocks):
        start = 0
        m, width = x32.shape
        for q_len, slot in zip(ctx.host.q_lens, ctx.host.slots):
            hist = state[slot, hist_row0:hist_row0 + taps - 1].double()
            padded = torch.cat([hist, x32[start:start + q_len].double()], 0)
            u = bias32.double().expand(q_len, width).clone()
            for j in range(taps):
                u += padded[j:j + q_len] * w32[:, j].double()
            u32[start:start + q_len] = u.to(torch.float32)
            start += q_len
        bw = width // blocks
        u_blocks.copy_(u32.view(m, blocks, bw).transpose(0, 1).to(u_blocks.dtype))

    def rglru_scan(self, u32, gates32, y_logit32, x32, softplus_lam32, state, ctx, out, taps, blocks):
        import math
        m, width = u32.shape
        bw = width // blocks
        g = gates32.double().transpose(0, 1)                                # [m, blocks, 2 bw]
        rg = torch.sigmoid(g[..., :bw]).reshape(m, width)
        ig = torch.sigmoid(g[..., bw:]).reshape(m, width)
        log_a = -8.0 * rg * softplus_lam32.double()
        a = torch.exp(log_a)
        mult = torch.sqrt(-torch.expm1(2.0 * log_a))
        z = y_logit32.double()
        y = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
        start = 0
        for q_len, slot in zip(ctx.host.q_lens, ctx.host.slots):
            S = state[slot, 0].double()
            for t in range(start, start + q_len):
                S = a[t] * S + mult[t] * ig[t] * u32[t].double()
                out[t] = (S * y[t]).to(out.dtype)
            state[slot, 0] = S.to(torch.float32)
            if taps > 1:
                joined = torch.cat([state[slot, 1:taps], x32[start:start + q_len]], 0)
                state[slot, 1:taps] = joined[-(taps - 1):].clone()
            start += q_len

    # ---- attention through a latent (latent_attention.cu) ---------------------------------------------
    @staticmethod
    def _turn(x, positions, freq32, mag, layout="interleaved"):
        """Pairs of the last axis (2i, 2i + 1, or with the layout "half" i, i + n/2) turned by position * freq (angles in
        32-bit, as the kernels form them)."""
        ang = (positions.to(torch.float32)[:, None] * freq32[None, :]).double()
        c, s = ang.cos() * mag, ang.sin() * mag
        while c.dim() < x.dim():
            c, s = c.unsqueeze(1), s.unsqueeze(1)
        n = x.shape[-1]
        first = slice(0, n, 2) if layout == "interleaved" else slice(0, n // 2)
        second = slice(1, n, 2) if layout == "interleaved" else slice(n // 2, n)
        out = torch.empty_like(x)
        out[..., first] = x[..., first] * c - x[..., second] * s
        out[..., second] = x[..., second] * c + x[..., first] * s
        return out

    def latent_store(self, z32, gain32, eps, freq32, mag, ctx, block_table, page_size, pages, rank, rot, layout="interleaved"):
        z = z32.double()
        c = z[:, :rank] / torch.sqrt(z[:, :rank].pow(2).mean(-1, keepdim=True) + eps) * gain32.double()
        kr = self._turn(z[:, rank:], ctx.positions, freq32, mag, layout)
        pos = ctx.positions.long()
        page = block_table[ctx.req_index.long(), pos // page_size].long()
        ok = page >= 0
        pages[page[ok], 0, (pos % page_size)[ok], :] = torch.cat([c, kr], -1)[ok].to(pages.dtype)

    def latent_query_layout(self, dtype, rank, rot):
        return rank + rot, torch.float32

    def latent_query(self, q32, w_uk, freq32, mag, positions, qa32, heads, dn, rank, rot, layout="interleaved"):
        m = q32.shape[0]
        q = q32.double().view(m, heads, dn + rot)
        lat = torch.einsum("thd,hdc->thc", q[..., :dn], w_uk.double().view(heads, dn, rank))
        qa32.copy_(torch.cat([lat, self._turn(q[..., dn:], positions, freq32, mag, layout)], -1).reshape(m, -1).to(torch.float32))

    def latent_attention(self, qa32, lat32, ctx, block_table, page_size, pages, heads, rank, rot, scale, window, sink32=None):
        m = qa32.shape[0]
        q = qa32.double().view(m, heads, rank + rot)
        positions, req_index = ctx.positions.tolist(), ctx.req_index.tolist()
        for t in range(m):
            p, r = positions[t], req_index[t]
            lo = max(0, p - window + 1) if window else 0
            idx = torch.arange(lo, p + 1)
            pg = block_table[r, idx // page_size].long()
            if (pg < 0).any():
                assert (pg < 0).all() and p == 0, "read of a position without a page"     # a padding row sees nothing
                lat32[t] = 0
                continue
            rows = pages[pg, 0, idx % page_size, :].double()             # [n, rank + rot]
            s = torch.einsum("hc,nc->hn", q[t], rows) * scale
            if sink32 is not None:      # one more column in the softmax, with nothing behind it
                s = torch.cat([s, sink32.double()[:, None]], -1)
            w = torch.softmax(s, dim=-1)[:, :rows.shape[0]]
            lat32[t] = (w @ rows[:, :rank]).reshape(-1).to(torch.float32)

    def latent_value(self, lat32, w_uv, out, heads, dv, rank, gate32=None):
        m = lat32.shape[0]
        v = torch.einsum("thc,hjc->thj", lat32.double().view(m, heads, rank), w_uv.double().view(heads, dv, rank)).reshape(m, heads * dv)
        if gate32 is not None:
            v = v * torch.sigmoid(gate32.double())
        out.copy_(v.to(out.dtype))

    # ---- the norm on a branch's output, and routed experts (pointwise.cu, moe.cu) -----------------------------
    def rmsnorm_add(self, y32, gain32, eps, mult, x32, h_out=None, clear=False, next_gain32=None, next_eps=0.0):
        y = y32.double()
        x = x32.double() + mult * y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps) * gain32.double()
        x32.copy_(x.to(torch.float32))
        if h_out is not None and next_gain32 is not None:
            xn = x32.double()
            h_out.copy_((xn / torch.sqrt(xn.pow(2).mean(-1, keepdim=True) + next_eps) * next_gain32.double()).to(h_out.dtype))
        elif h_out is not None:
            h_out.copy_(x32.to(h_out.dtype))
        if clear:
            y32.zero_()

    def moe_route(self, z32, top, sel_e, sel_w, score="sigmoid", renormalize=False, correction32=None, always=0):
        if always:      # the pieces of a shared expert: experts 0..always-1 for every token, weighted by the gate behind the router's logits
            wide = torch.as_strided(z32, (z32.shape[0], z32.shape[1] + 1), z32.stride())
            gate = torch.sigmoid(wide[:, -1:].double()).to(torch.float32)
            e, w = torch.empty_like(sel_e[:, :top]), torch.empty_like(sel_w[:, :top])
            self.moe_route(z32, top, e, w, score, renormalize, correction32)
            sel_e.copy_(torch.cat([e + always, torch.arange(always, dtype=torch.int32).expand(z32.shape[0], always)], dim=1))
            sel_w.copy_(torch.cat([w, gate.expand(z32.shape[0], always)], dim=1))
            return
        z = z32.double()
        if score == "sigmoid" and not renormalize and correction32 is None:
            order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
            sel_e.copy_(order.to(torch.int32))
            sel_w.copy_(torch.sigmoid(torch.gather(z, 1, order)).to(torch.float32))
            return
        sc = torch.softmax(z, -1) if score == "softmax" else torch.sigmoid(z)
        choice = sc if correction32 is None else sc + correction32.double()
        order = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
        w = torch.gather(sc, 1, order)
        if renormalize:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        sel_e.copy_(order.to(torch.int32))
        sel_w.copy_(w.to(torch.float32))

    def moe_experts(self, h, sel_e, sel_w, w_gate_up, w_down, out32, plan=None, gated=True, weight_on="input", outputs=None):
        ff = w_down.shape[2]
        acc = out32.double()
        for t in range(h.shape[0]):
            for c in range(sel_e.shape[1]):
                e, w = int(sel_e[t, c]), sel_w[t, c].double()
                if e >= w_down.shape[0]:
                    continue        # a router output that is no expert
                w_in, w_res = (w, 1.0) if weight_on == "input" else (1.0, w)
                if gated:
                    g = (w_gate_up[e, :ff].double() @ h[t].double()) * w_in
                    u = (w_gate_up[e, ff:].double() @ h[t].double()) * w_in
                    act = (g / (1.0 + torch.exp(-g)) * u).to(h.dtype).double()
                else:
                    act = (torch.relu((w_gate_up[e].double() @ h[t].double()) * w_in) ** 2).to(h.dtype).double()
                acc[t] += w_res * (w_down[e].double() @ act)
        out32.copy_(acc.to(torch.float32))

    def moe_identity(self, h, out32, sel_e, sel_w, n_real):
        w = (sel_w.double() * (sel_e >= n_real)).sum(-1, keepdim=True)
        out32.copy_((out32.double() + w * h.double()).to(torch.float32))

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(out.dtype))

    def repetition_penalty(self, logits, seen, seen_start, penalty, pending=None):
        starts = seen_start.tolist()
        for r in range(logits.shape[0]):
            p = float(penalty[r])
            if p == 1.0:
                continue
            ids = seen[starts[r]:starts[r + 1]].long()
            if pending is not None and int(pending[r]) not in ids.tolist():
                ids = torch.cat([ids, pending[r:r + 1].long()])
            s = logits[r, ids]
            logits[r, ids] = torch.where(s > 0, s / p, s * p)

    def sample(self, logits, temperature, top_k, top_p, uniform, out):
        """Inverse CDF in vocabulary order over the distribution of tests/plain_qwen2.py."""
        import numpy as np
        from plain_qwen2 import sampling_distribution
        for r in range(logits.shape[0]):
            probs = sampling_distribution(logits[r].double().cpu().numpy(), [], float(temperature[r]),
                                          int(top_k[r]), float(top_p[r]), 1.0)
            cdf = np.cumsum(probs)
            i = int(np.searchsorted(cdf, float(uniform[r]) * cdf[-1], side="right"))
            kept = np.nonzero(probs > 0)[0]
            i = min(i, int(kept[-1]))
            while probs[i] == 0:
                i += 1
            out[r] = i
