"""A state-space mixer with a matrix state per head and a scalar decay (Mamba-2).

One input product gives, side by side, z [inner], x [inner], B [groups * N], C [groups * N] and dt [heads],
with inner = heads * head_dim. x, B and C together pass a short causal convolution per channel (``taps``
taps, the last one on the current token, zeros before the start of a sequence, a bias) and silu. Then per
head h, which reads the B and C of group h // (heads / groups):

    dt = softplus(dt + dt_bias_h)                     (no clamp)
    S <- exp(-exp(A_log_h) dt) S + dt B x^T           (S is N x head_dim, zero at the start of a sequence)
    y = S^T C + D_h x

The heads' y side by side are multiplied by silu(z), divided by their root mean square in ``norm_groups``
equal parts, multiplied by a weight, and projected. dt, the decay, the state and y are 32-bit on every path;
the projections and the convolution with its silu run in the path's dtype. What a sequence carries from
token to token is S and the convolution's last ``taps - 1`` inputs.
"""

from __future__ import annotations

import torch

from .base import StateNeed, TensorSpec, register_mixer
from .branches import Branch


class Mamba2(Branch):
    """params: hidden, heads, head_dim, state, groups, taps, norm_groups, eps."""

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.head_dim = int(p["head_dim"])
        self.state = int(p["state"])
        self.groups = int(p.get("groups", 1))
        self.taps = int(p["taps"])
        self.norm_groups = int(p.get("norm_groups", 1))
        self.eps = float(p["eps"])
        self.inner = self.heads * self.head_dim
        self.conv_channels = self.inner + 2 * self.groups * self.state
        if self.heads % self.groups:
            raise ValueError(f"heads ({self.heads}) must be a multiple of groups ({self.groups})")
        if self.inner % self.norm_groups:
            raise ValueError(f"norm_groups ({self.norm_groups}) must divide heads * head_dim ({self.inner})")
        if self.taps < 1:
            raise ValueError("the convolution has at least one tap")

    def tensor_specs(self):
        H, ch = self.heads, self.conv_channels
        return {"in": TensorSpec((2 * self.inner + 2 * self.groups * self.state + H, self.hidden)),
                "conv": TensorSpec((ch, self.taps), "vector"), "conv.b": TensorSpec((ch,), "vector"),
                "dt_bias": TensorSpec((H,), "vector"), "A_log": TensorSpec((H,), "vector"), "D": TensorSpec((H,), "gain"),
                "norm": TensorSpec((self.inner,), "gain"), "o": TensorSpec((self.hidden, self.inner))}

    def cache_need(self):
        # the convolution's inputs are rows of the input product: the path's dtype holds them exactly
        return (StateNeed((self.heads, self.state, self.head_dim), "float32"),
                StateNeed((max(self.taps - 1, 1), self.conv_channels), "compute"))

    def bind(self, tensors, runtime):
        self.w = {"in": tensors["in"], "o": tensors["o"]}
        f = lambda key: tensors[key].float().contiguous()
        self.conv_w, self.conv_b = f("conv").t().contiguous(), f("conv.b")  # tap-major [taps, channels] for the kernel
        self.dt_bias, self.a_log, self.skip, self.norm_w = f("dt_bias"), f("A_log"), f("D"), f("norm")
        self.bind_standalone()

    def in_weight(self):
        return self.w["in"]

    def out_weight(self):
        return self.w["o"]

    def middle(self, ctx, proj, cache, out, col0, scale):
        ops = ctx.ops
        state, tail = cache
        inner, GN = self.inner, self.groups * self.state
        xbc = ops.causal_conv_silu(proj[:, inner:inner + self.conv_channels], self.conv_w, self.conv_b, tail.state, ctx.batch)
        y = ops.ssd_scan(xbc[:, :inner], xbc[:, inner:inner + GN], xbc[:, inner + GN:inner + 2 * GN],
                         proj[:, inner + self.conv_channels:inner + self.conv_channels + self.heads], self.dt_bias,
                         self.a_log, self.skip, self.heads, self.head_dim, self.state, self.groups, state.state, ctx.batch)
        ops.gated_group_norm(y, proj[:, :inner], self.norm_w, self.norm_groups, self.eps, out, col0, scale)


register_mixer("mamba2", Mamba2)
