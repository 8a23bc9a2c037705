"""Parts for models whose residual stream is kept in 32-bit on every path.

* ``ScaledEmbedding``: x = table[token] * scale, written as float32 rows.
* ``WideRMSNorm``: y = x / sqrt(mean(x^2) + eps) * (offset + w) with x, the sum
  x + branch and all arithmetic in float32; only y is rounded to the path's
  dtype. ``offset`` 1 serves weights that are stored around zero, 0 the usual
  gain. The stream it leaves behind (``x_new``) is float32. A stream with two
  pending outputs and a multiplier is folded as x + scale * (branch + branch2);
  ``forward_pair`` gives two norms of the same x (two gains, one pass over x) for
  a layer whose mixer and feed-forward both read it.
* ``GatedMLP``: down(act(gate h) * (up h)) with the activation as a parameter
  (``gelu_tanh``: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), or ``silu``);
  the activation and the product are computed in float32 and rounded once.
  ``swish_clamped`` (parameters ``limit`` L and ``slope`` a) clamps both inputs first,
  g' = min(g, L), u' = clamp(u, -L, L), and gives g' sigmoid(a g') (u' + 1).
* ``DenseMLP``: down(act(up h)) without a gate. ``xielu`` has two learned numbers (p, q) in a tensor of its own:
  z > 0: softplus(p) z^2 + z/2; z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2. ``gelu_tanh`` and ``silu``
  have none.
"""

from __future__ import annotations

import torch

from .base import Embedding, FeedForward, Norm, Stream, TensorSpec, register_embedding, register_feed_forward, register_norm
from .norm import Normed

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "sigmoid": 2}


class ScaledEmbedding(Embedding):
    """params: vocab, hidden, scale, copies (default 1: the row is written that many times side by side, the
    equal streams that hyper-connections start from)."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.scale = float(params.get("scale", 1.0))
        self.copies = int(params.get("copies", 1))
        self.table = None

    def tensor_specs(self):
        return {"table": TensorSpec((self.vocab, self.hidden), "table")}

    def bind(self, tensors, runtime):
        self.table = tensors["table"]

    def forward(self, ctx):
        if self.copies == 1:
            return ctx.ops.embed_scaled(self.table, ctx.batch.tokens, ctx.batch.n_rows, self.scale)
        return ctx.ops.embed_scaled(self.table, ctx.batch.tokens, ctx.batch.n_rows, self.scale, copies=self.copies)


class WideRMSNorm(Norm):
    """params: size, eps, gain_offset (default 0)."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.offset = float(params.get("gain_offset", 0.0))
        self.gain = None
        self.dtype = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), "vector" if self.offset else "gain")}

    def bind(self, tensors, runtime):
        self.gain = tensors["weight"].float().contiguous()
        self.dtype = runtime.dtype

    def forward(self, ctx, stream: Stream) -> Normed:
        return self._run(ctx, stream, None)[0]

    def forward_pair(self, ctx, stream: Stream, other: "WideRMSNorm"):
        """This norm and ``other`` of the same x (the pending outputs folded in once): two Normed."""
        if other.eps != self.eps or other.offset != self.offset or other.size != self.size:
            raise ValueError("two norms of one x share their size, eps and gain offset")
        return self._run(ctx, stream, other.gain)

    def _run(self, ctx, stream: Stream, gain2):
        x = stream.x
        if x.dtype != torch.float32:
            raise TypeError("a wide norm follows a float32 residual stream (an embedding or norm of the same family)")
        branch, branch2 = stream.branch, stream.branch2
        if branch is None and branch2 is not None:
            branch, branch2 = branch2, None
        x_new = ctx.ops.empty_like(x) if branch is not None else x
        if branch2 is None and gain2 is None and stream.scale == 1.0:
            rows = ctx.ops.rmsnorm_wide(x, branch, self.gain, self.offset, self.eps, x_new, self.dtype)
        else:
            rows = ctx.ops.rmsnorm_wide(x, branch, self.gain, self.offset, self.eps, x_new, self.dtype, branch2=branch2,
                                        scale=stream.scale, gain2=gain2)
        out = []
        for r, g in zip(rows if gain2 is not None else (rows,), (self.gain, gain2)):
            normed = Normed(ctx.ops, x, branch, g, self.eps, x_new)
            normed.mark_fused(r)  # computed here and now: a product never folds this norm into its prologue
            out.append(normed)
        stream.x = x_new
        stream.branch = stream.branch2 = None
        stream.scale = 1.0
        return out


class GatedMLP(FeedForward):
    """params: hidden, intermediate, activation; for "swish_clamped" also limit and slope."""

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.activation = str(params.get("activation", "silu"))
        if self.activation not in ("silu", "gelu_tanh", "swish_clamped"):
            raise ValueError(f"unknown activation '{self.activation}' for a gated feed-forward")
        self.act_params = None
        if self.activation == "swish_clamped":
            self.act_params = (float(params["limit"]), float(params.get("slope", 1.702)))
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        return {"gate": TensorSpec((self.intermediate, self.hidden)),
                "up": TensorSpec((self.intermediate, self.hidden)),
                "down": TensorSpec((self.hidden, self.intermediate))}

    def bind(self, tensors, runtime):
        self.w_gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.w_down = tensors["down"].contiguous()

    def forward(self, ctx, h):
        if self.act_params is None:
            act = ctx.ops.gate_up_act(h, self.w_gate_up, self.intermediate, self.activation)
        else:
            act = ctx.ops.gate_up_act(h, self.w_gate_up, self.intermediate, self.activation, act_params=self.act_params)
        return ctx.ops.linear(act, self.w_down)


class DenseMLP(FeedForward):
    """params: hidden, intermediate, activation ("xielu", "gelu_tanh" or "silu"). Tensors: up, down and, for
    xielu, act [2]."""

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.activation = str(params.get("activation", "xielu"))
        if self.activation not in ("xielu", "gelu_tanh", "silu"):
            raise ValueError(f"unknown activation '{self.activation}' for a dense feed-forward")
        self.w_up = self.w_down = None
        self.act_params = (0.0, 0.0)

    def tensor_specs(self):
        specs = {"up": TensorSpec((self.intermediate, self.hidden)), "down": TensorSpec((self.hidden, self.intermediate))}
        if self.activation == "xielu":
            specs["act"] = TensorSpec((2,), "vector")
        return specs

    def bind(self, tensors, runtime):
        self.w_up, self.w_down = tensors["up"].contiguous(), tensors["down"].contiguous()
        if self.activation == "xielu":  # the two slopes, once, in 64-bit: softplus(p) and 1/2 + softplus(q)
            p, q = torch.nn.functional.softplus(tensors["act"].double().cpu()).tolist()
            self.act_params = (p, 0.5 + q)

    def forward(self, ctx, h):
        return ctx.ops.linear(ctx.ops.act_rows(ctx.ops.linear(h, self.w_up), self.activation, self.act_params), self.w_down)


register_embedding("scaled_embedding", ScaledEmbedding)
register_feed_forward("dense_mlp", DenseMLP)
register_norm("rmsnorm_wide", WideRMSNorm)
register_feed_forward("gated_mlp", GatedMLP)
