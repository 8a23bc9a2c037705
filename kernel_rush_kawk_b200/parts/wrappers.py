"""Mixers that are built around other mixers.

* ``TokenShifted`` (kind "token_shifted"): the inner mixer does not read the layer's normalised rows n but
  s_t = n_t + (n_(t-1) - n_t) * shift, element by element, with a learned vector ``shift`` and n_(t-1) the row of
  the token before (zeros before a sequence's first token). The last n of every sequence is kept as fixed-size
  state (32-bit), so that a step may start anywhere in a sequence. Whatever else reads the layer's norm (a
  feed-forward beside the mixer) still reads n.
* ``NormedSum`` (kind "normed_sum"): several mixers read the same input; the result is
  scale * sum_b rmsnorm(mixer_b(h)) * gain_b, each output normalised over the model width (eps under the root,
  plain gains) in 32-bit before the sum. Any registered mixer may stand inside either of them; their storage needs
  are passed through, in order.
"""

from __future__ import annotations

import torch

from .base import Mixer, StateNeed, TensorSpec, mixer_class, register_mixer


def _needs_of(mixer) -> tuple[list, bool]:
    need = mixer.cache_need()
    many = isinstance(need, (tuple, list))
    return (list(need) if many else ([] if need is None else [need])), many


def _views_for(views: tuple, first: int, count: int, many: bool):
    return tuple(views[first:first + count]) if many else (views[first] if count else None)


class TokenShifted(Mixer):
    """params: hidden, inner: {"kind", "params"}. Tensor keys: "shift" and "inner.<the inner mixer's key>"."""

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden"])
        self.inner = mixer_class(params["inner"]["kind"])(params["inner"]["params"])
        self.graph_safe = self.inner.graph_safe
        self.shift = None

    def tensor_specs(self):
        specs = {"shift": TensorSpec((self.hidden,), "vector")}
        specs.update({"inner." + key: spec for key, spec in self.inner.tensor_specs().items()})
        return specs

    def cache_need(self):
        inner, self._inner_many = _needs_of(self.inner)
        self._inner_count = len(inner)
        return (StateNeed((self.hidden,), "float32"), *inner)

    def attention_head_dims(self):
        return tuple(getattr(self.inner, "attention_head_dims", lambda: ())())

    def bind(self, tensors, runtime):
        self.shift = tensors["shift"].float().reshape(1, self.hidden).contiguous()
        self.inner.bind({key[6:]: t for key, t in tensors.items() if key.startswith("inner.")}, runtime)
        self.cache_need()

    def forward(self, ctx, h, cache):
        rows = h.tensor() if not isinstance(h, torch.Tensor) else h
        shifted = ctx.ops.token_shift(rows, cache[0].state, self.shift, ctx.batch, store=True)[0]
        return self.inner.forward(ctx, shifted, _views_for(cache, 1, self._inner_count, self._inner_many))


class NormedSum(Mixer):
    """params: hidden, eps, scale (default 1), branches: a list of {"name", "kind", "params"}. Tensor keys:
    "<name>.<the branch's key>" and, for the gain of a branch's norm, "out.<name>"."""

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden"])
        self.eps = float(params["eps"])
        self.scale = float(params.get("scale", 1.0))
        self.names = [str(b["name"]) for b in params["branches"]]
        self.branches = [mixer_class(b["kind"])(b["params"]) for b in params["branches"]]
        if not 1 <= len(self.branches) <= 4:
            raise ValueError("between one and four mixers stand side by side")
        self.graph_safe = all(b.graph_safe for b in self.branches)
        self.gains = None

    def tensor_specs(self):
        specs = {f"{name}.{key}": spec for name, b in zip(self.names, self.branches) for key, spec in b.tensor_specs().items()}
        specs.update({f"out.{name}": TensorSpec((self.hidden,), "gain") for name in self.names})
        return specs

    def cache_need(self):
        needs, self._slices = [], []
        for b in self.branches:
            group, many = _needs_of(b)
            self._slices.append((len(needs), len(group), many))
            needs.extend(group)
        return tuple(needs) if needs else None

    def attention_head_dims(self):
        return tuple(d for b in self.branches for d in getattr(b, "attention_head_dims", lambda: ())())

    def bind(self, tensors, runtime):
        for name, b in zip(self.names, self.branches):
            b.bind({key[len(name) + 1:]: t for key, t in tensors.items() if key.startswith(name + ".")}, runtime)
        self.gains = torch.stack([tensors[f"out.{name}"].float() for name in self.names]).contiguous()
        self.cache_need()

    def forward(self, ctx, h, cache):
        rows = h.tensor() if not isinstance(h, torch.Tensor) else h
        views = cache if isinstance(cache, tuple) else (() if cache is None else (cache,))
        outs = [b.forward(ctx, rows, _views_for(views, *s)) for b, s in zip(self.branches, self._slices)]
        return ctx.ops.norm_sum(outs, self.gains, self.eps, self.scale)


register_mixer("token_shifted", TokenShifted)
register_mixer("normed_sum", NormedSum)
