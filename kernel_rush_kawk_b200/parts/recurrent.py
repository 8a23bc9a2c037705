"""Mixers with a matrix-valued recurrent state per head.

Each head keeps S [N, N] (key channel x value channel) in 32-bit, zero at the
start of a sequence and carried from token to token. With r, k, v [N] of a
token, a decay w and (for the delta rule) a removal rate a per key channel:

* ``DeltaRule`` (generalized delta rule): u = k / sqrt(sum k^2 + 1e-6);
  S <- diag(w) S - (a * u)(u^T S) + k v^T, both first terms read the old S;
  o = S^T r. w = exp(-decay_scale * sigmoid(W2 tanh(W1 h) + w0)),
  a = sigmoid(Wa h + b), output gate sigmoid(Wg h).
* ``TimeMixWKV`` (RWKV-style time mixing): every projection reads its own blend
  h + (h_prev - h) * mu of the token and the one before it (zeros before the
  first; the last token's h is part of the state); o = (S + diag(bonus) k v^T)^T r
  with the old S, then S <- diag(w) S + k v^T; w = exp(-exp(W2 tanh(W1 h_w) + w0)),
  output gate silu(Wg h_g).

Either way each head's o is divided by its root mean square, multiplied by a plain
weight over all heads' channels and by the gate, and projected by Wo. Decays,
rates, unit keys, the state and o are 32-bit on every path; the projections and
their activations run in the path's dtype.
"""

from __future__ import annotations

import math

import torch

from .base import StateNeed, TensorSpec, register_mixer
from .branches import Branch, pad_rows


class DeltaRule(Branch):
    """params: hidden, heads, dim, rank, eps, decay_scale (default exp(-1/2))."""

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.rank = int(p["rank"])
        self.eps = float(p["eps"])
        self.decay_scale = float(p.get("decay_scale", math.exp(-0.5)))
        self.channels = self.heads * self.dim

    def tensor_specs(self):
        C, HN, R = self.hidden, self.channels, self.rank
        specs = {k: TensorSpec((HN, C)) for k in ("r", "k", "v", "g", "a")}
        specs.update({"a.b": TensorSpec((HN,), "vector"), "w1": TensorSpec((R, C)), "w2": TensorSpec((HN, R)),
                      "w0": TensorSpec((HN,), "vector"), "norm": TensorSpec((HN,), "gain"), "o": TensorSpec((C, HN))})
        return specs

    def cache_need(self):
        return StateNeed((self.heads, self.dim, self.dim), "float32")

    def bind(self, tensors, runtime):
        self.w = dict(tensors)
        f = lambda key: tensors[key].float().contiguous()
        self.rate_bias, self.w0, self.norm_w = f("a.b"), f("w0"), f("norm")
        self.w2 = tensors["w2"].contiguous()
        self.bind_standalone()

    def in_weight(self):
        return torch.cat([self.w[k] for k in ("r", "k", "v", "g", "a", "w1")], dim=0)

    def out_weight(self):
        return self.w["o"]

    def middle(self, ctx, proj, cache, out, col0, scale):
        HN = self.channels
        cut = lambda i, n=HN: proj[:, i * HN:i * HN + n]
        ctx.ops.linear_recurrence("delta", cut(0), cut(1), cut(2), cut(3), cut(5, self.rank), self.w2, self.w0,
                                  self.heads, self.dim, self.norm_w, self.eps, cache.state, ctx.batch, out, col0, scale,
                                  rate=cut(4), rate_bias=self.rate_bias, decay_scale=self.decay_scale)


class TimeMixWKV(Branch):
    """params: hidden, heads, dim, rank, eps. Its projections do not read one shared input, so it
    stands alone (``in_weight`` is not offered)."""

    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.rank = int(p["rank"])
        self.eps = float(p["eps"])
        self.channels = self.heads * self.dim

    def tensor_specs(self):
        C, HN, R = self.hidden, self.channels, self.rank
        specs = {"mu." + s: TensorSpec((C,), "vector") for s in self.MIXES}
        specs.update({k: TensorSpec((HN, C)) for k in ("r", "k", "v", "g")})
        specs.update({"w1": TensorSpec((R, C)), "w2": TensorSpec((HN, R)), "w0": TensorSpec((HN,), "vector"),
                      "u": TensorSpec((self.heads, self.dim), "vector"), "norm": TensorSpec((HN,), "gain"),
                      "o": TensorSpec((C, HN))})
        return specs

    def cache_need(self):
        return (StateNeed((self.heads, self.dim, self.dim), "float32"), StateNeed((self.hidden,), "float32"))

    def bind(self, tensors, runtime):
        f = lambda key: tensors[key].float().contiguous()
        self.mu = torch.stack([f("mu." + s) for s in self.MIXES]).contiguous()
        self.w_proj = [pad_rows(tensors[k]) for k in ("r", "k", "v", "g", "w1")]
        self.w2 = tensors["w2"].contiguous()
        self.w0, self.bonus, self.norm_w = f("w0"), f("u").reshape(-1).contiguous(), f("norm")
        self._w_out = tensors["o"].contiguous()

    def forward(self, ctx, h, cache):
        ops = ctx.ops
        state, last = cache
        rows = h.tensor() if not isinstance(h, torch.Tensor) else h
        mixes = ops.token_shift(rows, last.state, self.mu, ctx.batch)  # [5, rows, hidden]
        HN = self.channels
        r, k, v, g, lora = (ops.linear(mixes[i], w) for i, w in enumerate(self.w_proj))
        out = torch.empty((rows.shape[0], HN), dtype=r.dtype, device=r.device)
        ops.linear_recurrence("wkv", r[:, :HN], k[:, :HN], v[:, :HN], g[:, :HN], lora[:, :self.rank], self.w2, self.w0,
                              self.heads, self.dim, self.norm_w, self.eps, state.state, ctx.batch, out, 0, 1.0,
                              bonus=self.bonus, last_rows=(rows, last.state))
        return ops.linear(out, self._w_out)


register_mixer("delta_rule", DeltaRule)
register_mixer("wkv_time_mix", TimeMixWKV)
