"""A feed-forward of routed experts, with an optional shared expert.

Router: z = Wr h + b in 32-bit (h as the path holds it); a token takes the ``top``
experts with the largest z (ties: the lower index), weighted by the softmax over
the chosen logits only. Expert e: Wdown_e (act(Wgate_e h) * (Wup_e h)). The result
is the weighted sum of the chosen experts' outputs. The shared expert has the same
form with its own size, runs for every token, and is multiplied by sigmoid(Wsg h),
one number per token, before it is added.

``scoring`` "sigmoid_groups" is another way to choose and weigh: s = sigmoid(z); the choice is made by
s + c with a stored correction c per expert ("correction"), the weights by s alone. The experts form ``groups``
equal groups of neighbours; a group's score is the sum of its two largest choice scores (its one score where a group
has one expert), only the ``keep_groups`` best groups' experts can be chosen, and the weights are the chosen
experts' s divided by their sum (+ 1e-20) and multiplied by ``route_scale``.

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
    expert's share of the softmax over all experts, not renormalised), scoring (None or "sigmoid_groups", with
    groups, keep_groups and route_scale; it has the tensor "correction" and no router bias)."""

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
        self.scoring = p.get("scoring")
        if self.scoring not in (None, "sigmoid_groups"):
            raise ValueError(f"scoring must be None or 'sigmoid_groups', got {self.scoring!r}")
        self.groups = int(p.get("groups", 1))
        self.keep_groups = int(p.get("keep_groups", self.groups))
        self.route_scale = float(p.get("route_scale", 1.0))
        if self.scoring:
            self.router_bias = False
            if self.experts % self.groups or not 1 <= self.keep_groups <= self.groups:
                raise ValueError(f"{self.experts} experts do not form {self.groups} equal groups of which {self.keep_groups} are kept")
            if self.top > self.keep_groups * (self.experts // self.groups):
                raise ValueError("a token cannot take more experts than the kept groups hold")
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
        if self.scoring:
            specs["correction"] = TensorSpec((self.experts,), "vector")
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
        self.correction = tensors["correction"].float().contiguous() if self.scoring else None
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
        if self.scoring:
            experts, weights, row_gate = ops.moe_route(x, self.router_w, None, self.top, gate_row=self.shared_gate,
                                                       sigmoid_groups=(self.correction, self.groups, self.keep_groups,
                                                                       self.route_scale))
        elif self.weights == "all":
            experts, weights, row_gate = ops.moe_route(x, self.router_w, self.router_b, self.top, gate_row=self.shared_gate,
                                                       over_all=True)
        else:
            experts, weights, row_gate = ops.moe_route(x, self.router_w, self.router_b, self.top, gate_row=self.shared_gate)
        return ops.moe_experts(x, self.w_gate_up, self.w_down, experts, weights, self.intermediate, self.activation,
                               add=base, add_gate=row_gate, batch=ctx.batch)


register_feed_forward("routed_experts", RoutedExperts)
