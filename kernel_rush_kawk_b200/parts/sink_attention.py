"""Grouped-query attention over a sliding window with a softmax sink.

q = Wq h, k = Wk h, v = Wv h (no biases); the first ``rot_dims`` elements of every
q and k head are rotated by the position (element i with element i + rot_dims/2,
angle p * rot_base^(-2i/rot_dims), positions and angles in 32-bit or better); with
``value_norm`` every value head is divided by its root mean square before it is
cached; a query at position p sees keys p - window + 1 .. p (``window`` None: all
of 0..p); score = (q . k) * scale with ``scale`` a parameter; with ``sink`` each
head's softmax has one more term in its denominator, exp(sink_h), which carries
no value. Key and value heads may differ in size (``dim``, ``vdim``). Scores and
weights are 32-bit; the weights multiply the values unrounded.

Three more options, each off by default. ``keep_first``: a windowed query also sees
the sequence's first ``keep_first`` keys, at their true positions (the cache keeps
their pages out of the window's ring). ``gate``: the heads' outputs are multiplied
by sigmoid(Wg h) before the output projection, one number per head ("head") or per
element ("element"); Wg h rides in the stacked input product. ``value_mix``: values
are blended across layers of one step: the layer marked "first" leaves its values of
the step's tokens under ``value_mix_key``, a layer marked "blend" caches
(1 - lambda) v + lambda v_first with its own scalar lambda (tensor "vmix").

Three options of the projections and the sink. ``bias``: q, k and v have biases (tensors "q.b", "k.b", "v.b").
``qk_norm`` "row": the whole q row (all heads together) is divided by its root mean square and multiplied
by a weight of the row's size ("q.norm"), and the k row likewise ("k.norm"), after the biases and before the
rotation, in 32-bit. ``sink`` "zero": the extra term of the softmax's denominator is exp(0) for every head,
p_j = exp(s_j) / (1 + sum exp(s_j)), and no tensor is read for it.

Options of a second kind of this attention, which come with kernels of their own (a fused bias + norm + rotation +
cache write, and an attention kernel whose block holds all heads of a row). ``qk_norm`` "head": every q head and
every k head is divided by its own root mean square and multiplied by a weight of the head's size, shared by the
heads ("q.norm", "k.norm" of ``dim`` elements), after the biases and before the rotation. ``rot_pairs``: the rotation
pairs element 2i with element 2i + 1 instead of i with i + rot_dims/2. ``rot_factor``: every rotation frequency is
divided by it. ``chunk``: a query at position p sees the keys of its own block of ``chunk`` positions only,
(p // chunk) * chunk .. p, blocks counted from the sequence's first position. ``talk``: the heads' scaled scores of
a (query, key) pair are mixed before the softmax, s'_h = sum_g T[h, g] s_g with a learned T ("talk", [heads, heads]).
"""

from __future__ import annotations

import torch

from .base import KVNeed, TensorSpec, register_mixer
from .branches import Branch


class SinkWindowAttention(Branch):
    """params: hidden, heads, kv_heads, dim, vdim, scale, window (None or int), rot_dims, rot_base,
    value_norm (bool), sink (bool), eps, keep_first (int), gate (None, "head" or "element"),
    value_mix (None, "first" or "blend"), value_mix_key, bias (bool), qk_norm (None, "row" or "head"); sink may
    be "zero"; rot_pairs (bool), rot_factor, chunk (None or int), talk (bool)."""

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p.get("vdim") or self.dim)
        self.scale = float(p["scale"])
        self.window = None if p.get("window") is None else int(p["window"])
        self.rot_dims = int(p.get("rot_dims", 0))
        self.rot_base = float(p.get("rot_base", 10000.0))
        self.value_norm = bool(p.get("value_norm", False))
        self.zero_sink = p.get("sink") == "zero"
        self.has_sink = bool(p.get("sink", False)) and not self.zero_sink
        self.bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        if self.qk_norm not in (None, "row", "head"):
            raise ValueError(f"qk_norm must be None, 'row' or 'head', got {self.qk_norm!r}")
        self.rot_pairs = bool(p.get("rot_pairs", False))
        self.rot_factor = float(p.get("rot_factor", 1.0))
        self.chunk = None if p.get("chunk") is None else int(p["chunk"])
        self.talk = bool(p.get("talk", False))
        #: the second kind of this attention (see the module text)
        self._mixed = self.qk_norm == "head" or self.rot_pairs or self.chunk is not None or self.talk
        self.eps = float(p.get("eps", 0.0))
        self.keep_first = int(p.get("keep_first") or 0) if self.window is not None else 0
        self.gate = p.get("gate")
        self.value_mix = p.get("value_mix")
        self.value_mix_key = str(p.get("value_mix_key", "value_mix"))
        if self.gate not in (None, "head", "element"):
            raise ValueError(f"gate must be None, 'head' or 'element', got {self.gate!r}")
        if self.value_mix not in (None, "first", "blend"):
            raise ValueError(f"value_mix must be None, 'first' or 'blend', got {self.value_mix!r}")
        if self.heads % self.kv_heads:
            raise ValueError(f"heads ({self.heads}) must be a multiple of kv_heads ({self.kv_heads})")
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ValueError(f"rot_dims ({self.rot_dims}) must be even and at most dim ({self.dim})")
        if self._mixed and (self.window is not None or self.value_norm or self.value_mix or self.qk_norm == "row"
                            or self.gate == "element" or (self.chunk is not None and self.chunk < 1)):
            raise ValueError("per-head norms, pair rotation, blocks of keys and mixed scores come without a window, value "
                             "norm, value blend, row norm or per-element gate")

    def tensor_specs(self):
        specs = {"q": TensorSpec((self.heads * self.dim, self.hidden)),
                 "k": TensorSpec((self.kv_heads * self.dim, self.hidden)),
                 "v": TensorSpec((self.kv_heads * self.vdim, self.hidden)),
                 "o": TensorSpec((self.hidden, self.heads * self.vdim))}
        if self.has_sink:
            specs["sink"] = TensorSpec((self.heads,), "vector")
        if self.gate:
            specs["g"] = TensorSpec((self.heads * (self.vdim if self.gate == "element" else 1), self.hidden))
        if self.bias:
            specs.update({"q.b": TensorSpec((self.heads * self.dim,), "vector"),
                          "k.b": TensorSpec((self.kv_heads * self.dim,), "vector"),
                          "v.b": TensorSpec((self.kv_heads * self.vdim,), "vector")})
        if self.qk_norm == "row":
            specs.update({"q.norm": TensorSpec((self.heads * self.dim,), "gain"),
                          "k.norm": TensorSpec((self.kv_heads * self.dim,), "gain")})
        if self.qk_norm == "head":
            specs.update({"q.norm": TensorSpec((self.dim,), "gain"), "k.norm": TensorSpec((self.dim,), "gain")})
        if self.talk:
            specs["talk"] = TensorSpec((self.heads, self.heads), "mixing")
        if self.value_mix:
            specs["vmix"] = TensorSpec((), "vector")  # the first layer of a blend stores one too and never reads it
        return specs

    def cache_need(self):
        return KVNeed(self.kv_heads, self.dim, self.window, None if self.vdim == self.dim else self.vdim,
                      keep_first=self.keep_first)

    @property
    def _plain(self) -> bool:
        return not (self.keep_first or self.gate or self.value_mix)

    def attention_head_dims(self):
        if self._mixed:
            return (self.dim,) if self.dim == self.vdim and self.dim % 16 == 0 and self.dim <= 256 else ()
        """Steps of many tokens in bfloat16 run on the tensor cores where key and value heads have one size that
        is a multiple of 16: that kernel is compiled per head size."""
        return (self.dim,) if self.dim == self.vdim and self.dim % 16 == 0 and self.dim <= 256 else ()

    def bind(self, tensors, runtime):
        self.w = {k: tensors[k] for k in ("q", "k", "v", "o") + (("g",) if self.gate else ())}
        self.lam = float(tensors["vmix"].float().item()) if self.value_mix == "blend" else None
        self.sink = tensors["sink"].float().contiguous() if self.has_sink else None
        if self.zero_sink:
            self.sink = torch.zeros(self.heads, dtype=torch.float32, device=runtime.device)
        f = lambda *keys: torch.cat([tensors[k].float().reshape(-1) for k in keys]).contiguous()
        self.qkv_bias = f("q.b", "k.b", "v.b") if self.bias else None
        self.qk_gain = f("q.norm", "k.norm") if self.qk_norm else None
        # the few rotation frequencies come from the host in 64-bit, so that they depend on no device's pow()
        # and as two floats each (the float32 value, then what float32 leaves of the float64 value)
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        f = self.rot_base ** (-2.0 * i / max(self.rot_dims, 1)) / self.rot_factor
        self.talk_w = tensors["talk"].float().contiguous() if self.talk else None
        hi = f.to(torch.float32)
        self.inv_freq = torch.cat([hi, (f - hi.double()).to(torch.float32)]).contiguous().to(runtime.device)
        self.bind_standalone()

    def in_weight(self):
        return torch.cat([self.w["q"], self.w["k"], self.w["v"]] + ([self.w["g"]] if self.gate else []), dim=0)

    def out_weight(self):
        return self.w["o"]

    def middle(self, ctx, proj, cache, out, col0, scale):
        ops = ctx.ops
        k_col = self.heads * self.dim
        v_col = k_col + self.kv_heads * self.dim
        value_eps = self.eps if self.value_norm else None
        if self._mixed:
            ops.bias_norm_rotate_write(proj, 0, k_col, v_col, self.heads, self.kv_heads, self.dim, self.vdim, self.qkv_bias,
                                       self.qk_gain, self.eps, self.inv_freq, self.rot_dims, self.rot_pairs, ctx.batch, cache)
            gate = (v_col + self.kv_heads * self.vdim, self.gate) if self.gate else None
            ops.mixed_attention(proj, 0, self.heads, self.dim, self.vdim, self.sink, self.talk_w, self.scale, self.chunk,
                                ctx.batch, cache, out, col0, scale, gate=gate)
            return
        if self.bias or self.qk_norm:  # biases onto q, k, v; q and k rows divided by their root mean square
            ops.bias_row_norm(proj, (0, k_col, v_col, v_col + self.kv_heads * self.vdim), self.qkv_bias, self.qk_gain,
                              self.eps)
        if not self._plain:
            blend = None
            if self.value_mix == "first":
                ctx.shared[self.value_mix_key] = proj[:, v_col:v_col + self.kv_heads * self.vdim]
            elif self.value_mix == "blend":
                first = ctx.shared.get(self.value_mix_key)
                if first is None or first.shape[1] != self.kv_heads * self.vdim:
                    raise RuntimeError("a layer that blends values runs after the layer that leaves them, with value "
                                       "heads of the same number and size")
                blend = (first, self.lam)
            ops.rotate_norm_write(proj, 0, k_col, v_col, self.heads, self.kv_heads, self.dim, self.vdim, self.inv_freq,
                                  self.rot_dims, value_eps, ctx.batch, cache, value_mix=blend)
            gate = (v_col + self.kv_heads * self.vdim, self.gate) if self.gate else None
            ops.sink_attention(proj, 0, self.heads, self.dim, self.vdim, self.sink, self.scale, self.window, ctx.batch,
                               cache, out, col0, scale, keep_first=self.keep_first, gate=gate)
            return
        if ctx.batch.is_decode and ops.sink_attention_step(proj, 0, k_col, v_col, self.heads, self.kv_heads, self.dim,
                                                           self.vdim, self.inv_freq, self.rot_dims, value_eps, self.sink,
                                                           self.scale, self.window, ctx.batch, cache, out, col0, scale):
            return  # a single-token step: one kernel rotates, writes the cache and attends
        ops.rotate_norm_write(proj, 0, k_col, v_col, self.heads, self.kv_heads, self.dim, self.vdim, self.inv_freq,
                              self.rot_dims, self.eps if self.value_norm else None, ctx.batch, cache)
        ops.sink_attention(proj, 0, self.heads, self.dim, self.vdim, self.sink, self.scale, self.window, ctx.batch, cache,
                           out, col0, scale)


register_mixer("sink_window_attention", SinkWindowAttention)
