"""Hyper-connections: several residual streams, read and written through small learned weights.

Instead of one x a model keeps S streams x_1 .. x_S (all equal to the embedding at the start), stored
side by side as one float32 row [S * size] per token. A sublayer with weights a [S], b [S] and M [S, S]
(indexed [from, to]) reads u = sum_s a_s x_s through an RMS norm, and when its output y comes back every
stream is rewritten at once from the old ones: x_t <- sum_s M[s, t] x_s + b_t y. With S = 1, a = b = M = 1
this is the plain residual sum.

``HyperRMSNorm`` is the norm in front of such a sublayer. Like the other norms it folds what is pending on
the stream first: the previous sublayer's output and that sublayer's (M, b), which the previous norm left
on the stream when it ran (``Stream.fold``). So a layer's arrangement stays the pre-norm one, and one
kernel does the write-back of one sublayer, the weighted read of the next and its norm, all in 32-bit.
``read`` "sum" makes a norm that reads the plain sum of the streams and owns no hyper-connection (a
model's last norm).
"""

from __future__ import annotations

import torch

from .base import Norm, Stream, TensorSpec, register_norm
from .norm import Normed


class HyperRMSNorm(Norm):
    """params: size, eps, streams, read ("weights", the default, or "sum"), gain_offset (default 0)."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.streams = int(params["streams"])
        self.read = str(params.get("read", "weights"))
        self.offset = float(params.get("gain_offset", 0.0))
        if self.read not in ("weights", "sum"):
            raise ValueError(f"read must be 'weights' or 'sum', got {self.read!r}")
        if not 1 <= self.streams <= 8:
            raise ValueError(f"between 1 and 8 streams, got {self.streams}")
        self.gain = self.read_w = self.fold = None
        self.dtype = None

    def tensor_specs(self):
        specs = {"weight": TensorSpec((self.size,), "vector" if self.offset else "gain")}
        if self.read == "weights":
            S = self.streams
            specs.update({"in": TensorSpec((S,), "vector"), "out": TensorSpec((S,), "vector"),
                          "mix": TensorSpec((S, S), "vector")})
        return specs

    def bind(self, tensors, runtime):
        self.gain = tensors["weight"].float().contiguous()
        self.dtype = runtime.dtype
        S = self.streams
        if self.read == "weights":
            self.read_w = tensors["in"].float().contiguous()
            # what this sublayer's output is folded in with, when it comes back: M [from, to] then b
            self.fold = torch.cat([tensors["mix"].float().reshape(S * S), tensors["out"].float().reshape(S)]).contiguous()
        else:
            self.read_w = torch.ones(S, dtype=torch.float32, device=runtime.device)
            self.fold = None

    def forward(self, ctx, stream: Stream) -> Normed:
        x = stream.x
        S, C = self.streams, self.size
        if x.dtype != torch.float32 or x.shape[1] != S * C:
            raise TypeError(f"a hyper-connection norm follows {S} float32 streams of {C} side by side")
        branch = stream.branch
        if stream.branch2 is not None or stream.scale != 1.0:
            raise TypeError("hyper-connections fold one pending output at a time")
        if branch is not None and stream.fold is None:
            raise TypeError("an output is pending but no hyper-connection to fold it with")
        x_new = ctx.ops.empty_like(x) if branch is not None else x
        rows = ctx.ops.hyper_rmsnorm(x, branch, stream.fold if branch is not None else None, self.read_w, self.gain,
                                     self.offset, self.eps, x_new, self.dtype)
        normed = Normed(ctx.ops, x, branch, self.gain, self.eps, x_new)
        normed.mark_fused(rows)
        stream.x = x_new
        stream.branch = None
        stream.fold = self.fold  # the sublayer behind this norm comes back through these
        return normed


register_norm("hyper_rmsnorm", HyperRMSNorm)
