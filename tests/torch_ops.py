"""The kernels' interface restated in plain torch, for tests only.

Each method has the signature and meaning of the same method of the product's
CUDA bindings (``kernel_rush_kawk_b200/csrc/bindings.py``) and serves two ends:
the reference that each kernel is compared with on the GPU, and a stand-in
backend with which the engine's step, cache and generation logic can be run on
the CPU (the product itself has no CPU path and never imports this file).

Rounding follows the formulas of willzeng274/kernel-rush-kawk that
``tests/plain_qwen3.py`` cites: a value is rounded to the compute dtype wherever
the reference's BF16 path rounds; reductions are float32.
"""

from __future__ import annotations

import math

import torch

PAGE = 64


def _mix32(x: torch.Tensor) -> torch.Tensor:
    m = 0xFFFFFFFF
    x = x & m
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    x = x ^ (x >> 16)
    return x


class TorchOps:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype

    def rt(self, t: torch.Tensor) -> torch.Tensor:
        """Round to the compute dtype, keep float32 for the next wide operation."""
        return t.to(self.dtype).float()

    # -- helpers -----------------------------------------------------------
    def empty_like(self, x):
        return torch.empty_like(x)

    def _resolve(self, x):
        return x.tensor() if hasattr(x, "tensor") and not isinstance(x, torch.Tensor) else x

    # -- elementwise and norms -----------------------------------------------
    def embed(self, table, tokens, n_rows):
        return table[tokens.long()].to(self.dtype)

    def rmsnorm(self, x, gain, eps):
        xf = x.float()
        n = self.rt(xf * torch.rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps))
        return (n * gain.float()).to(self.dtype)

    def add_rmsnorm(self, x, branch, gain, eps, x_new):
        s = (x.float() + branch.float()).to(self.dtype)
        x_new.copy_(s)
        return self.rmsnorm(s, gain, eps)

    def gather_rows(self, x, idx):
        return x[idx.long()]

    # -- matrix products -------------------------------------------------------
    def linear(self, x, w, out_float32=False):
        x = self._resolve(x)
        y = x.float() @ w.float().t()
        return y if out_float32 else y.to(self.dtype)

    def gate_up_swiglu(self, h, w_gate_up, intermediate):
        gu = self.linear(h, w_gate_up).float()
        g, u = gu[:, :intermediate], gu[:, intermediate:]
        return (self.rt(g / (1.0 + torch.exp(-g))) * u).to(self.dtype)

    # -- attention ----------------------------------------------------------
    def qk_norm_rope_write(self, qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache):
        D = head_dim
        half = cos.shape[1] if cos is not None else D // 2  # the rotated width is twice the tables' columns
        rows = qkv.shape[0]
        pos = batch.row_pos.long()
        view = qkv.view(rows, heads + 2 * kv_in_row, D)

        def norm_rope(x, gain):
            x = x.float()
            if gain is not None:
                r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
                x = self.rt(gain.float() * self.rt(x * r))
            if cos is not None:
                c, s = cos[pos].float()[:, None, :], sin[pos].float()[:, None, :]
                x1, x2, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
                x = torch.cat([self.rt(self.rt(x1 * c) + self.rt(-x2 * s)),
                               self.rt(self.rt(x2 * c) + self.rt(x1 * s)), rest], dim=-1)
            return x.to(self.dtype)

        view[:, :heads] = norm_rope(view[:, :heads], q_gain)
        if kv_in_row:
            k = norm_rope(view[:, heads:heads + kv_in_row], k_gain)
            v = view[:, heads + kv_in_row:]
            slot = batch.seq_slot.long()[batch.row_seq.long()]
            page = cache.table.long()[slot, (pos // PAGE) % cache.width]
            off = pos % PAGE
            cache.k[page, :, off] = k
            cache.v[page, :, off] = v

    def rope_attention(self, qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache, scale,
                       window):
        self.qk_norm_rope_write(qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache)
        return self.attention(qkv, heads, kv_in_row, head_dim, batch, cache, scale, window)

    def attention(self, qkv, heads, kv_in_row, head_dim, batch, cache, scale, window):
        D = head_dim
        rows = qkv.shape[0]
        G = heads // cache.kv_heads
        q = qkv.view(rows, heads + 2 * kv_in_row, D)[:, :heads].float()
        out = torch.empty((rows, heads, D), dtype=torch.float32, device=qkv.device)
        table = cache.table.long()
        row0 = 0
        for slot, start, n in zip(batch.slots, batch.starts, batch.q_lens):
            total = start + n
            lo = 0 if window is None else max(0, start - window + 1)
            positions = torch.arange(lo, total, device=qkv.device)
            pages = table[slot, (positions // PAGE) % cache.width]
            k = cache.k[pages, :, positions % PAGE].float()  # [keys, kv_heads, D]
            v = cache.v[pages, :, positions % PAGE].float()
            qpos = torch.arange(start, total, device=qkv.device)
            visible = positions[None, :] <= qpos[:, None]
            if window is not None:
                visible &= positions[None, :] > qpos[:, None] - window
            for h in range(heads):
                s = (q[row0:row0 + n, h] @ k[:, h // G].t()) * scale
                s = s.masked_fill(~visible, float("-inf"))
                m = s.max(dim=-1, keepdim=True).values
                p = torch.exp(s - m)
                l = p.sum(dim=-1, keepdim=True)
                out[row0:row0 + n, h] = (self.rt(p) @ v[:, h // G]) / l
            row0 += n
        return out.to(self.dtype).view(rows, heads * D)

    # -- token selection ------------------------------------------------------
    def select_tokens(self, logits, temperature, seed, requests, step):
        logits = logits.float()
        if temperature == 0.0:
            return logits.argmax(dim=-1).to(torch.int32)
        n, vocab = logits.shape
        t = lambda v: torch.tensor(v & 0xFFFFFFFF, dtype=torch.int64)
        i = torch.arange(vocab, dtype=torch.int64)
        out = torch.empty(n, dtype=torch.int32)
        for r in range(n):
            key = _mix32(_mix32(_mix32(t(seed)) ^ t(int(requests[r]))) ^ t(step))
            h = _mix32(key ^ ((i * 0x9E3779B9) & 0xFFFFFFFF))
            u = ((h >> 9).float() + 0.5) / 8388608.0
            g = -torch.log(-torch.log(u))
            out[r] = int(torch.argmax(logits[r].cpu() / temperature + g))
        return out.to(logits.device)


# ----------------------------------------------------------------------------
# the kernels of models with a 32-bit residual stream, windowed attention with a sink,
# and recurrent state (kernel_rush_kawk_b200/csrc/wide_rows.cu, sink_attention.cu, recurrent.cu)
# ----------------------------------------------------------------------------

def _entry(cache, pos):
    """The page-table entry of a position: the first ``keep_pages`` entries hold their positions for good."""
    b = pos // PAGE
    keep = getattr(cache, "keep_pages", 0)
    if not keep:
        return b % cache.width
    return torch.where(b < keep, b, keep + (b - keep) % max(cache.width - keep, 1))


def _act(z, name):
    if name == "silu":
        return z * torch.sigmoid(z)
    if name == "sigmoid":
        return torch.sigmoid(z)
    if name == "gelu_tanh":
        return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
    raise ValueError(name)


class _WideOps:
    def embed_scaled(self, table, tokens, n_rows, scale, copies=1):
        return (table[tokens.long()].float() * scale).repeat(1, copies)

    def rmsnorm_wide(self, x, branch, gain, offset, eps, x_new, out_dtype, branch2=None, scale=1.0, gain2=None):
        s = x
        if branch is not None:
            b = branch.float() if branch2 is None else branch.float() + branch2.float()
            s = x + (b if scale == 1.0 else b * scale)
            x_new.copy_(s)
        n = s * torch.rsqrt((s * s).mean(dim=-1, keepdim=True) + eps)
        first = (n * (offset + gain.float())).to(out_dtype)
        return first if gain2 is None else (first, (n * (offset + gain2.float())).to(out_dtype))

    def gate_up_act(self, h, w_gate_up, intermediate, activation, act_params=None):
        return self.gated_act(self.linear(h, w_gate_up), intermediate, activation, act_params=act_params)

    def gated_act(self, gu, intermediate, activation, row_gate_col=None, act_params=None):
        g = gu.float()
        if activation == "swish_clamped":
            limit, slope = act_params
            a = torch.clamp(g[:, :intermediate], max=limit)
            b = torch.clamp(g[:, intermediate:2 * intermediate], min=-limit, max=limit)
            out = a * torch.sigmoid(slope * a) * (b + 1.0)
        else:
            out = _act(g[:, :intermediate], activation) * g[:, intermediate:2 * intermediate]
        if row_gate_col is not None:
            out = out * torch.sigmoid(g[:, row_gate_col:row_gate_col + 1])
        return out.to(gu.dtype)

    def latent_norm_write(self, proj, c_col, rank, gain, eps, batch, cache, keep_rows=False):
        c = proj[:, c_col:c_col + rank].float()
        c = c * torch.rsqrt((c * c).mean(dim=-1, keepdim=True) + eps) * gain.float()
        pos = batch.row_pos.long()
        slot = batch.seq_slot.long()[batch.row_seq.long()]
        page = cache.table.long()[slot, _entry(cache, pos)]
        cache.k[page, 0, pos % PAGE] = c.to(proj.dtype)
        return c.to(proj.dtype) if keep_rows else None

    def head_linear(self, x, w, out=None, out_col=0, out_scale=1.0):
        heads, n, k = w.shape
        rows = x.shape[0]
        y = torch.einsum("rhk,hnk->rhn", x.float().reshape(rows, heads, k), w.float()).reshape(rows, heads * n) * out_scale
        if out is None:
            return y.to(x.dtype)
        out[:, out_col:out_col + heads * n] = y.to(out.dtype)
        return out

    def moe_route(self, x, w, b, top, gate_row=False, over_all=False, sigmoid_groups=None):
        z = x.float() @ w.float().t()
        row_gate = torch.sigmoid(z[:, -1]) if gate_row else None
        z = z[:, :-1] if gate_row else z
        if sigmoid_groups is not None:
            return (*self._route_sigmoid_groups(z, top, *sigmoid_groups), row_gate)
        if b is not None:
            z = z + b.float()
        best = torch.topk(z, top, dim=-1)  # ties are not exercised: equal logits do not occur with random weights
        if over_all:
            return best.indices.to(torch.int32), torch.softmax(z, dim=-1).gather(1, best.indices), row_gate
        return best.indices.to(torch.int32), torch.softmax(best.values, dim=-1), row_gate

    # -- pair-hash embedding, per-head norms with pair rotation, attention with mixed head scores over blocks
    # of keys, norms of several outputs summed, plain activations, sigmoid routing within groups --------------
    def embed_bigram(self, table, pairs, state, buckets, mul_prev, mul_cur, batch):
        tok = batch.tokens.long()
        prev = torch.empty_like(tok)
        prev[1:] = tok[:-1]
        first = torch.zeros(tok.shape[0], dtype=torch.bool)
        row0 = 0
        for slot, start, n in zip(batch.slots, batch.starts, batch.q_lens):
            prev[row0] = state[slot, 0]
            first[row0] = start == 0
            state[slot, 0] = tok[row0 + n - 1]
            row0 += n
        row = (prev * mul_prev + tok * mul_cur) % buckets
        row = torch.where(first, torch.full_like(row, buckets), row)
        return table[tok].float() + pairs[row].float()

    def bias_norm_rotate_write(self, proj, q_col, k_col, v_col, heads, kv_heads, dim, vdim, bias, qk_gain, eps, inv_freq,
                               rot_dims, pairs, batch, cache):
        rows = proj.shape[0]
        pos = batch.row_pos.long()
        half = rot_dims // 2
        end = v_col + kv_heads * vdim
        x = proj[:, q_col:end].float()
        if bias is not None:
            x = x + bias
        q = x[:, :k_col - q_col].reshape(rows, heads, dim)
        k = x[:, k_col - q_col:v_col - q_col].reshape(rows, kv_heads, dim)
        v = x[:, v_col - q_col:].reshape(rows, kv_heads, vdim)
        if qk_gain is not None:
            q = q * torch.rsqrt((q * q).mean(dim=-1, keepdim=True) + eps) * qk_gain[:dim]
            k = k * torch.rsqrt((k * k).mean(dim=-1, keepdim=True) + eps) * qk_gain[dim:]

        def rotate(t):
            if not half:
                return t
            f = inv_freq[:half].double() + inv_freq[half:].double()
            a = pos.double()[:, None] * f[None, :]
            c, sn = torch.cos(a).float()[:, None, :], torch.sin(a).float()[:, None, :]
            if pairs:
                u, w = t[..., 0:rot_dims:2], t[..., 1:rot_dims:2]
                turned = torch.stack([u * c - w * sn, w * c + u * sn], dim=-1).reshape(t.shape[0], t.shape[1], rot_dims)
            else:
                u, w = t[..., :half], t[..., half:rot_dims]
                turned = torch.cat([u * c - w * sn, w * c + u * sn], dim=-1)
            return torch.cat([turned, t[..., rot_dims:]], dim=-1)

        proj[:, q_col:q_col + heads * dim] = rotate(q).reshape(rows, heads * dim).to(proj.dtype)
        slot = batch.seq_slot.long()[batch.row_seq.long()]
        page = cache.table.long()[slot, _entry(cache, pos)]
        cache.k[page, :, pos % PAGE] = rotate(k).to(proj.dtype)
        cache.v[page, :, pos % PAGE] = v.to(proj.dtype)

    def mixed_attention(self, proj, q_col, heads, dim, vdim, sink, talk, scale, chunk, batch, cache, out, out_col, out_scale,
                        gate=None):
        rows = proj.shape[0]
        G = heads // cache.kv_heads
        q = proj[:, q_col:q_col + heads * dim].reshape(rows, heads, dim).float()
        res = torch.empty((rows, heads, vdim), dtype=torch.float32, device=proj.device)
        table = cache.table.long()
        row0 = 0
        for slot, start, n in zip(batch.slots, batch.starts, batch.q_lens):
            total = start + n
            lo = (start // chunk) * chunk if chunk else 0
            positions = torch.arange(lo, total, device=proj.device)
            pages = table[slot, _entry(cache, positions)]
            k = cache.k[pages, :, positions % PAGE].float()  # [keys, kv heads, dim]
            v = cache.v[pages, :, positions % PAGE].float()
            qpos = torch.arange(start, total, device=proj.device)
            visible = positions[None, :] <= qpos[:, None]
            if chunk:
                visible &= (positions[None, :] // chunk) == (qpos[:, None] // chunk)
            kh = torch.arange(heads) // G
            s = torch.einsum("qhd,khd->hqk", q[row0:row0 + n], k[:, kh]) * scale
            if talk is not None:
                s = torch.einsum("hg,gqk->hqk", talk.float(), s)
            s = s.masked_fill(~visible[None], float("-inf"))
            m = s.max(dim=-1, keepdim=True).values
            extra = 0.0
            if sink is not None:
                m = torch.maximum(m, sink.float()[:, None, None])
                extra = torch.exp(sink.float()[:, None, None] - m)
            p = torch.exp(s - m)
            o = torch.einsum("hqk,khd->hqd", p, v[:, kh]) / (p.sum(dim=-1, keepdim=True) + extra)
            res[row0:row0 + n] = o.transpose(0, 1)
            row0 += n
        if gate is not None:
            col, mode = gate
            width = heads * (vdim if mode == "element" else 1)
            res = res * torch.sigmoid(proj[:, col:col + width].float()).reshape(rows, heads, -1)
        out[:, out_col:out_col + heads * vdim] = (res * out_scale).to(out.dtype).view(rows, heads * vdim)

    def norm_sum(self, outs, gains, eps, scale):
        total = 0.0
        for y, g in zip(outs, gains):
            yf = y.float()
            total = total + yf * torch.rsqrt((yf * yf).mean(dim=-1, keepdim=True) + eps) * g.float()
        return (total * scale).to(outs[0].dtype)

    def act_rows(self, z, activation, params=(0.0, 0.0)):
        zf = z.float()
        if activation == "xielu":
            a, b = params
            out = torch.where(zf > 0, a * zf * zf + 0.5 * zf, b * (torch.expm1(zf) - zf) + 0.5 * zf)
        else:
            out = _act(zf, activation)
        return out.to(z.dtype)

    def _route_sigmoid_groups(self, z, top, correction, groups, keep, scale):
        rows, E = z.shape
        s = torch.sigmoid(z)
        c = s + correction.float()
        size = E // groups
        score = c.view(rows, groups, size).topk(min(2, size), dim=-1).values.sum(dim=-1)
        best = score.topk(keep, dim=-1).indices
        allowed = torch.zeros((rows, groups), dtype=torch.bool).scatter_(1, best, True)
        c = c.masked_fill(~allowed.repeat_interleave(size, dim=1), float("-inf"))
        idx = c.topk(top, dim=-1).indices
        w = s.gather(1, idx)
        return idx.to(torch.int32), w / (w.sum(dim=-1, keepdim=True) + 1e-20) * scale

    # -- hyper-connections, the state-space mixer, biases and row norms of attention --------------------
    def hyper_rmsnorm(self, x, branch, fold, read, gain, offset, eps, x_new, out_dtype):
        S = read.shape[0]
        rows, C = x.shape[0], x.shape[1] // S
        X = x.view(rows, S, C)
        if branch is not None:
            M, b = fold[:S * S].view(S, S), fold[S * S:]
            X = torch.einsum("st,rsc->rtc", M, X) + b[None, :, None] * branch.float()[:, None, :]
            x_new.copy_(X.reshape(rows, S * C))
        u = torch.einsum("s,rsc->rc", read, X)
        n = u * torch.rsqrt((u * u).mean(dim=-1, keepdim=True) + eps)
        return (n * (offset + gain.float())).to(out_dtype)

    def bias_row_norm(self, proj, cols, bias, gain, eps):
        q0, k0, v0, end = cols
        x = proj[:, q0:end].float()
        if bias is not None:
            x = x + bias
        if gain is not None:
            for a, b in ((q0, k0), (k0, v0)):
                seg = x[:, a - q0:b - q0]
                x[:, a - q0:b - q0] = seg * torch.rsqrt((seg * seg).mean(dim=-1, keepdim=True) + eps) * gain[a - q0:b - q0]
        proj[:, q0:end] = x.to(proj.dtype)

    def causal_conv_silu(self, x, w, b, tail, batch):
        rows, ch = x.shape
        taps = w.shape[0]  # tap-major weights [taps, channels]
        out = torch.empty((rows, ch), dtype=torch.float32)
        row0 = 0
        for slot, n in zip(batch.slots, batch.q_lens):
            seq = torch.cat([tail[slot][-(taps - 1):].float(), x[row0:row0 + n].float()]) if taps > 1 else x[row0:row0 + n].float()
            acc = b.float()[None, :].repeat(n, 1)
            for j in range(taps):
                acc += seq[j:j + n] * w[j].float()
            out[row0:row0 + n] = acc
            if taps > 1:
                tail[slot][-(taps - 1):] = seq[n:].to(tail.dtype)
            row0 += n
        return (out * torch.sigmoid(out)).to(x.dtype)

    def ssd_scan(self, x, B, C, dt, dt_bias, a_log, skip, heads, P, N, groups, state, batch):
        rows = x.shape[0]
        xf, Bf, Cf = x.float().reshape(rows, heads, P), B.float().reshape(rows, groups, N), C.float().reshape(rows, groups, N)
        step = torch.nn.functional.softplus(dt.float() + dt_bias, threshold=30.0)
        decay = torch.exp(-torch.exp(a_log) * step)
        g_of = torch.arange(heads) // (heads // groups)
        y = torch.empty((rows, heads, P), dtype=torch.float32)
        row0 = 0
        for slot, n in zip(batch.slots, batch.q_lens):
            S = state[slot].clone()  # [heads, N, P]
            for t in range(row0, row0 + n):
                S = decay[t][:, None, None] * S + step[t][:, None, None] * Bf[t][g_of][:, :, None] * xf[t][:, None, :]
                y[t] = torch.einsum("hn,hnp->hp", Cf[t][g_of], S) + skip[:, None] * xf[t]
            state[slot] = S
            row0 += n
        return y.reshape(rows, heads * P)

    def gated_group_norm(self, y, gate_rows, weight, parts, eps, out, out_col, out_scale):
        rows, inner = y.shape
        z = gate_rows.float()
        v = (y * (z * torch.sigmoid(z))).view(rows, parts, inner // parts)
        v = v * torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps)
        out[:, out_col:out_col + inner] = (v.reshape(rows, inner) * weight * out_scale).to(out.dtype)

    def moe_experts(self, x, w_gate_up, w_down, experts, weights, intermediate, activation, add=None, add_gate=None,
                    batch=None):
        rows, top = experts.shape
        out = torch.zeros((rows, w_down.shape[1]), dtype=torch.float32) if add is None else add.float().clone()
        if add is not None and add_gate is not None:
            out = out * add_gate[:, None]
        xf = x.float()
        for r in range(rows):
            for j in range(top):
                e = int(experts[r, j])
                gu = xf[r] @ w_gate_up[e].float().t()
                a = (_act(gu[:intermediate], activation) * gu[intermediate:]).to(self.dtype).float()
                out[r] += weights[r, j] * (a @ w_down[e].float().t())
        return out.to(self.dtype)

    def rotate_norm_write(self, proj, q_col, k_col, v_col, heads, kv_heads, dim, vdim, inv_freq, rot_dims, value_eps,
                          batch, cache, value_mix=None):
        rows = proj.shape[0]
        pos = batch.row_pos.long()
        half = rot_dims // 2

        def rotate(x):
            x = x.float()
            if not half:
                return x
            f = inv_freq[:half].double() + inv_freq[half:].double()  # the frequencies come as two floats each
            a = pos.double()[:, None] * f[None, :]
            c, s = torch.cos(a).float()[:, None, :], torch.sin(a).float()[:, None, :]
            u, v, rest = x[..., :half], x[..., half:rot_dims], x[..., rot_dims:]
            return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)

        q = proj[:, q_col:q_col + heads * dim].view(rows, heads, dim)
        q.copy_(rotate(q).to(proj.dtype))
        k = rotate(proj[:, k_col:k_col + kv_heads * dim].reshape(rows, kv_heads, dim)).to(proj.dtype)
        v = proj[:, v_col:v_col + kv_heads * vdim].reshape(rows, kv_heads, vdim).float()
        if value_mix is not None:
            first, lam = value_mix
            v = (1.0 - lam) * v + lam * first.float().reshape(rows, kv_heads, vdim)
        if value_eps is not None:
            v = v * torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + value_eps)
        slot = batch.seq_slot.long()[batch.row_seq.long()]
        page = cache.table.long()[slot, _entry(cache, pos)]
        cache.k[page, :, pos % PAGE] = k
        cache.v[page, :, pos % PAGE] = v.to(proj.dtype)

    def sink_attention(self, proj, q_col, heads, dim, vdim, sink, scale, window, batch, cache, out, out_col, out_scale,
                       keep_first=0, gate=None, gate_rows=None):
        rows = proj.shape[0]
        G = heads // cache.kv_heads
        q = proj[:, q_col:q_col + heads * dim].reshape(rows, heads, dim).float()
        res = torch.empty((rows, heads, vdim), dtype=torch.float32, device=proj.device)
        table = cache.table.long()
        row0 = 0
        for slot, start, n in zip(batch.slots, batch.starts, batch.q_lens):
            total = start + n
            lo = 0 if window is None else max(0, start - window + 1)
            positions = torch.arange(lo, total, device=proj.device)
            if window is not None and keep_first:
                positions = torch.cat([torch.arange(0, min(keep_first, lo), device=proj.device), positions])
            pages = table[slot, _entry(cache, positions)]
            k = cache.k[pages, :, positions % PAGE].float()
            v = cache.v[pages, :, positions % PAGE].float()
            qpos = torch.arange(start, total, device=proj.device)
            visible = positions[None, :] <= qpos[:, None]
            if window is not None:
                visible &= (positions[None, :] > qpos[:, None] - window) | (positions[None, :] < keep_first)
            for h in range(heads):
                s = (q[row0:row0 + n, h] @ k[:, h // G].t()) * scale
                s = s.masked_fill(~visible, float("-inf"))
                m = s.max(dim=-1, keepdim=True).values
                extra = 0.0
                if sink is not None:
                    m = torch.maximum(m, sink[h].float())
                    extra = torch.exp(sink[h].float() - m)
                p = torch.exp(s - m)
                res[row0:row0 + n, h] = (p @ v[:, h // G]) / (p.sum(dim=-1, keepdim=True) + extra)
            row0 += n
        if gate is not None:
            col, mode = gate
            src = proj if gate_rows is None else gate_rows
            width = heads * (vdim if mode == "element" else 1)
            res = res * torch.sigmoid(src[:, col:col + width].float()).reshape(rows, heads, -1)
        out[:, out_col:out_col + heads * vdim] = (res * out_scale).to(out.dtype).view(rows, heads * vdim)

    def sink_attention_step(self, proj, q_col, k_col, v_col, heads, kv_heads, dim, vdim, inv_freq, rot_dims, value_eps, sink,
                            scale, window, batch, cache, out, out_col, out_scale):
        self.rotate_norm_write(proj, q_col, k_col, v_col, heads, kv_heads, dim, vdim, inv_freq, rot_dims, value_eps, batch,
                               cache)
        self.sink_attention(proj, q_col, heads, dim, vdim, sink, scale, window, batch, cache, out, out_col, out_scale)
        return True

    def token_shift(self, h, last_state, mu, batch, store=False):
        hf = h.float()
        prev = torch.empty_like(hf)
        prev[1:] = hf[:-1]
        row0 = 0
        for slot, n in zip(batch.slots, batch.q_lens):
            prev[row0] = last_state[slot]
            if store:
                last_state[slot] = hf[row0 + n - 1]
            row0 += n
        return (hf[None] + (prev - hf)[None] * mu.float()[:, None, :]).to(h.dtype)

    def linear_recurrence(self, kind, r, k, v, gate, lora, w2, w0, heads, dim, norm_w, eps, state, batch, out, out_col,
                          out_scale, rate=None, rate_bias=None, decay_scale=1.0, bonus=None, last_rows=None):
        rows, H, N = r.shape[0], heads, dim
        f = lambda t: t.float().reshape(rows, H, N)
        z = torch.tanh(lora.float()).to(self.dtype).float() @ w2.float().t() + w0.float()
        if kind == "delta":
            decay = torch.exp(-decay_scale * torch.sigmoid(z)).view(rows, H, N)
            a = torch.sigmoid(rate.float() + rate_bias.float()).view(rows, H, N)
            g = torch.sigmoid(gate.float())
        else:
            decay = torch.exp(-torch.exp(z)).view(rows, H, N)
            g = gate.float() * torch.sigmoid(gate.float())
            bon = bonus.float().view(H, N)
        rr, kk, vv = f(r), f(k), f(v)
        o = torch.empty((rows, H, N), dtype=torch.float32, device=r.device)
        row0 = 0
        for slot, n in zip(batch.slots, batch.q_lens):
            S = state[slot].clone()
            for t in range(row0, row0 + n):
                kv = kk[t][:, :, None] * vv[t][:, None, :]
                if kind == "delta":
                    u = kk[t] / torch.sqrt((kk[t] * kk[t]).sum(dim=-1, keepdim=True) + 1e-6)
                    uS = torch.einsum("hi,hij->hj", u, S)
                    S = decay[t][:, :, None] * S - (a[t] * u)[:, :, None] * uS[:, None, :] + kv
                    o[t] = torch.einsum("hi,hij->hj", rr[t], S)
                else:
                    o[t] = torch.einsum("hi,hij->hj", rr[t], S + bon[:, :, None] * kv)
                    S = decay[t][:, :, None] * S + kv
            state[slot] = S
            if last_rows is not None:
                last_rows[1][slot] = last_rows[0][row0 + n - 1].float()
            row0 += n
        o = o * torch.rsqrt((o * o).mean(dim=-1, keepdim=True) + eps)
        res = o.reshape(rows, H * N) * norm_w.float() * g * out_scale
        out[:, out_col:out_col + H * N] = res.to(out.dtype)


for _name, _fn in vars(_WideOps).items():
    if not _name.startswith("__"):
        setattr(TorchOps, _name, _fn)
