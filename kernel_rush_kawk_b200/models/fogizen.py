"""The Fogizen decoder as a plan.

The embedding of a token is the sum of its own row and a row of a second table chosen by a hash of the
token and the one before it; the residual stream is 32-bit. Every layer has one RMS norm, whose output n feeds a
mixer and a feed-forward side by side: x <- x + mixer(shift(n)) + ff(n). The mixer reads n blended with the row
of the token before (a learned vector of blend weights), and is itself two mixers side by side on that input, each
followed by an RMS norm over the model width, averaged:

* left: grouped-query attention with biases, an RMS norm per q and k head (one weight of the head's size),
  rotation of neighbouring pairs with scaled-down frequencies, keys of the query's own block of positions only,
  the heads' scores mixed by a learned matrix before the softmax, one more learned term per head in the softmax's
  denominator, and a sigmoid gate per head;
* right: RWKV-style time mixing with a matrix state per head and decays computed from the input.

The feed-forward is dense (one up and one down product around the xIELU activation) or a set of routed SwiGLU
experts chosen by sigmoid scores with a correction and a limit on the groups of experts, or absent.

Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head`` and, for layer i, ``l<i>.norm1``, ``l<i>.shift``,
``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mix.left.out``, ``l<i>.mix.right.out`` and ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.fogizen import FogizenConfig, decay_rank
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

#: the design gives no longest sequence; tables and caches are sized by what the caller asks for
MAX_POSITIONS = 1 << 20

LEFT_KEYS = ("q", "k", "v", "o", "q.b", "k.b", "v.b", "q.norm", "k.norm", "talk", "sink", "g")
RIGHT_KEYS = ("mu.r", "mu.k", "mu.v", "mu.g", "mu.w", "r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")


def fogizen_plan(cfg: FogizenConfig) -> ModelPlan:
    C = cfg.width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        left, right = layer["mixer"]["left"], layer["mixer"]["right"]
        rot = left["rot"] or {"dims": 0, "base": 10000.0, "scaling": {"factor": 1.0}}
        branches = [
            {"name": "left", "kind": "sink_window_attention",
             "params": {"hidden": C, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"],
                        "vdim": left["vdim"], "scale": left["scale"], "window": None, "rot_dims": rot["dims"],
                        "rot_base": rot["base"], "rot_factor": rot["scaling"]["factor"], "rot_pairs": True,
                        "chunk": left["mask"]["size"] if left["mask"] else None, "talk": True, "sink": True,
                        "gate": "head", "bias": True, "qk_norm": "head", "eps": cfg.eps}},
            {"name": "right", "kind": "wkv_time_mix",
             "params": {"hidden": C, "heads": right["heads"], "dim": right["dim"], "rank": decay_rank(right), "eps": cfg.eps}},
        ]
        names = {"shift": p + "shift", "inner.out.left": p + "mix.left.out", "inner.out.right": p + "mix.right.out"}
        names.update({f"inner.left.{k}": f"{p}mix.left.{k}" for k in LEFT_KEYS})
        names.update({f"inner.right.{k}": f"{p}mix.right.{k}" for k in RIGHT_KEYS})
        mixer = PartSpec("token_shifted",
                         {"hidden": C, "inner": {"kind": "normed_sum",
                                                 "params": {"hidden": C, "eps": cfg.eps, "scale": 0.5, "branches": branches}}},
                         names)
        mlp, ffn = layer["mlp"], None
        if mlp is not None and mlp["kind"] == "dense":
            ffn = PartSpec("dense_mlp", {"hidden": C, "intermediate": mlp["ff"], "activation": "xielu"},
                           {k: f"{p}mlp.{k}" for k in ("up", "down", "act")})
        elif mlp is not None:
            r = mlp["router"]
            keys = ["router", "correction"] + [f"e{e}.{k}" for e in range(r["experts"]) for k in ("gate", "up", "down")]
            ffn = PartSpec("routed_experts",
                           {"hidden": C, "experts": r["experts"], "top": r["top"], "intermediate": mlp["expert"]["ff"],
                            "activation": "silu", "scoring": "sigmoid_groups", "groups": r["groups"]["count"],
                            "keep_groups": r["groups"]["keep"], "route_scale": r["scale"]},
                           {k: f"{p}mlp.{k}" for k in keys})
        norm = PartSpec("rmsnorm_wide", {"size": C, "eps": cfg.eps}, {"weight": p + "norm1"})
        layers.append(LayerSpec("parallel_residual", norm, mixer, None, ffn))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=C,
        vocab_size=cfg.vocab,
        embedding=PartSpec("bigram_embedding", {"vocab": cfg.vocab, "hidden": C, "buckets": cfg.buckets,
                                                "mul_prev": cfg.mul_prev, "mul_cur": cfg.mul_cur},
                           {"table": "embed", "pairs": "bigram"}),
        position=None,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm_wide", {"size": C, "eps": cfg.eps}, {"weight": "final.norm"}),
        head=PartSpec("output_head", {"vocab": cfg.vocab, "hidden": C}, {"weight": "head"}),
        max_positions=MAX_POSITIONS,
    )


register_architecture(FogizenConfig.architecture, FogizenConfig, fogizen_plan)
