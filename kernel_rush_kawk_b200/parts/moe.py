"""A feed-forward of routed experts, with an optional shared expert.

Router: z = Wr h + b in 32-bit (h as the path holds it); a token takes the ``top``
experts with the largest z (ties: the lower index), weighted by the softmax over
the chosen logits only. Expert e: Wdown_e (act(Wgate_e h) * (Wup_e h)). The result
is the weighted sum of the chosen experts' outputs. The shared expert has the same
form with its own size, runs for every token, and is multiplied by sigmoid(Wsg h),
one number per token, before it is added.

The routing never leaves the device: a routing kernel writes each row's experts and
weights; few rows (single-token steps) read each chosen expert's weights once per
(row, expert) pair; many rows are counted, ordered by expert and multiplied by all
experts in one batched product. The shared expert is a gated feed-forward of its own
(stacked [gate; up] product with the activation, a down product); its gate's weights
ride in the router's product as one more row, the routing kernel writes the token's
sigmoid beside the routing, and the kernel that adds the experts' weighted results
onto the shared expert's output multiplies that output by it.
"""

from __future__ import annotations

import torch

from .base import FeedForward, TensorSpec, register_feed_forward


class RoutedExperts(FeedForward):
    """params: hidden, experts, top, intermediate, activation ("silu"), shared_intermediate (None or int),
    shared_gate (bool: the shared expert sits behind sigmoid(Wsg h)), router_bias (default True: the router
    has a bias "router.b"), weights ("chosen", the default: softmax over the chosen logits; "all": each chosen
    expert's share of the softmax over all experts, not renormalised)."""

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden"])
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.intermediate = int(p["intermediate"])
        self.activation = str(p.get("activation", "silu"))
        self.shared = None if p.get("shared_intermediate") is None else int(p["shared_intermediate"])
        self.shared_gate = bool(p.get("shared_gate", False)) and self.shared is not None
        self.router_bias = bool(p.get("router_bias", True))
        self.weights = str(p.get("weights", "chosen"))
        if self.weights not in ("chosen", "all"):
            raise ValueError(f"weights must be 'chosen' or 'all', got {self.weights!r}")
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"a token takes between 1 and {self.experts} experts, got top = {self.top}")
        if self.top > 32:
            raise ValueError("at most 32 experts per token")

    def tensor_specs(self):
        H, F = self.hidden, self.intermediate
        specs = {"router": TensorSpec((self.experts, H))}
        if self.router_bias:
            specs["router.b"] = TensorSpec((self.experts,), "vector")
        for e in range(self.experts):
            specs[f"e{e}.gate"] = TensorSpec((F, H))
            specs[f"e{e}.up"] = TensorSpec((F, H))
            specs[f"e{e}.down"] = TensorSpec((H, F))
        if self.shared is not None:
            specs["shared.gate"] = TensorSpec((self.shared, H))
            specs["shared.up"] = TensorSpec((self.shared, H))
            specs["shared.down"] = TensorSpec((H, self.shared))
            if self.shared_gate:
                specs["shared.sg"] = TensorSpec((1, H))
        return specs

    def bind(self, tensors, runtime):
        E = self.experts
        # in the path's dtype: the logits' product accumulates in 32-bit; the shared expert's gate is its last row
        self.router_w = torch.cat([tensors["router"]] + ([tensors["shared.sg"]] if self.shared_gate else []), dim=0).contiguous()
        self.router_b = tensors["router.b"].float().contiguous() if self.router_bias else None
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0) for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()
        self.w_shared_in = self.w_shared_down = None
        if self.shared is not None:
            self.w_shared_in = torch.cat([tensors["shared.gate"], tensors["shared.up"]], dim=0).contiguous()
            self.w_shared_down = tensors["shared.down"].contiguous()

    def forward(self, ctx, h):
        ops = ctx.ops
        x = h.tensor() if hasattr(h, "tensor") and not isinstance(h, torch.Tensor) else h
        base = None
        if self.shared is not None:
            base = ops.linear(ops.gate_up_act(x, self.w_shared_in, self.shared, self.activation), self.w_shared_down)
        if self.weights == "all":
            experts, weights, row_gate = ops.moe_route(x, self.router_w, self.router_b, self.top, gate_row=self.shared_gate,
                                                       over_all=True)
        else:
            experts, weights, row_gate = ops.moe_route(x, self.router_w, self.router_b, self.top, gate_row=self.shared_gate)
        return ops.moe_experts(x, self.w_gate_up, self.w_down, experts, weights, self.intermediate, self.activation,
                               add=base, add_gate=row_gate, batch=ctx.batch)


register_feed_forward("routed_experts", RoutedExperts)
