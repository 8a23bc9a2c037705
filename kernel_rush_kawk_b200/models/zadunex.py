"""The Zadunex decoder as a plan.

A token embedding starts ``streams`` equal copies of a 32-bit residual stream. Every sublayer (a layer's
mixer, then its feed-forward if it has one) reads a weighted sum of the streams through an RMS norm and
writes back through a hyper-connection: every stream becomes a mix of the old streams plus the sublayer's
output times a weight of its own. A layer's mixer is a state-space layer (Mamba-2: a short causal
convolution, a matrix state per head with a scalar decay, a gated grouped norm) or grouped-query attention
with biases, an RMS norm over the whole query and key rows, a rotation of part of each head and one more
term, exp(0), in the softmax's denominator. The feed-forward is dense with clamped inputs or a set of
routed SwiGLU experts weighted by the softmax over all experts. A span of layers may run several times in a
row with the same weights, each run with storage of its own. The sum of the streams goes through a final
norm and a head of its own, and the logits are multiplied by a constant.

Tensor names: ``embed``, ``final.norm``, ``head`` and, for layer i, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.hc<q>.{in,out,mix}`` (q = 1: mixer, 2: feed-forward), ``l<i>.mix.*`` and ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zadunex import ZadunexConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

#: the design gives no longest sequence; tables and caches are sized by what the caller asks for
MAX_POSITIONS = 1 << 20


def _names(prefix: str, keys) -> dict:
    return {k: prefix + k for k in keys}


def zadunex_plan(cfg: ZadunexConfig) -> ModelPlan:
    C, S = cfg.width, cfg.streams

    def norm(weight: str, hc: str | None):
        if not cfg.hyper:
            return PartSpec("rmsnorm_wide", {"size": C, "eps": cfg.eps}, {"weight": weight})
        if hc is None:  # the model's last norm reads the plain sum of the streams and writes nothing back
            return PartSpec("hyper_rmsnorm", {"size": C, "eps": cfg.eps, "streams": S, "read": "sum"}, {"weight": weight})
        return PartSpec("hyper_rmsnorm", {"size": C, "eps": cfg.eps, "streams": S},
                        {"weight": weight, "in": hc + ".in", "out": hc + ".out", "mix": hc + ".mix"})

    layers, ignored = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "mamba2":
            mixer = PartSpec("mamba2", {"hidden": C, "heads": m["heads"], "head_dim": m["vdim"], "state": m["state"],
                                        "groups": m["groups"], "taps": m["conv"], "norm_groups": m["norm_groups"],
                                        "eps": cfg.eps},
                             _names(p + "mix.", ["in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o"]))
        else:
            mixer = PartSpec("sink_window_attention",
                             {"hidden": C, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                              "scale": m["scale"], "window": None, "rot_dims": m["rot"]["dims"], "rot_base": m["rot"]["base"],
                              "sink": "zero", "bias": True, "qk_norm": "row", "eps": cfg.eps},
                             _names(p + "mix.", ["q", "k", "v", "o", "q.b", "k.b", "v.b", "q.norm", "k.norm"]))
        ffn_norm = ffn = None
        mlp = layer["mlp"]
        if mlp is None:  # should a checkpoint still carry the absent sublayer's norm and hyper-connection
            ignored += [p + "norm2", p + "hc2.in", p + "hc2.out", p + "hc2.mix"]
        if mlp is not None:
            ffn_norm = norm(p + "norm2", p + "hc2")
            if mlp["kind"] == "dense":
                ffn = PartSpec("gated_mlp", {"hidden": C, "intermediate": mlp["ff"], "activation": "swish_clamped",
                                             "limit": mlp["limit"], "slope": 1.702},
                               _names(p + "mlp.", ["gate", "up", "down"]))
            else:
                E = mlp["router"]["experts"]
                keys = ["router"] + [f"e{e}.{k}" for e in range(E) for k in ("gate", "up", "down")]
                ffn = PartSpec("routed_experts",
                               {"hidden": C, "experts": E, "top": mlp["router"]["top"], "intermediate": mlp["expert"]["ff"],
                                "activation": "silu", "router_bias": False, "weights": "all"}, _names(p + "mlp.", keys))
        layers.append(LayerSpec("prenorm", norm(p + "norm1", p + "hc1"), mixer, ffn_norm, ffn))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=C,
        vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_embedding", {"vocab": cfg.vocab, "hidden": C, "scale": 1.0,
                                                "copies": S if cfg.hyper else 1}, {"table": "embed"}),
        position=None,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in cfg.layer_runs()),
        final_norm=norm("final.norm", None),
        head=PartSpec("output_head", {"vocab": cfg.vocab, "hidden": C, "scale": cfg.logit_scale}, {"weight": "head"}),
        max_positions=MAX_POSITIONS,
        ignored=tuple(ignored),
    )


register_architecture(ZadunexConfig.architecture, ZadunexConfig, zadunex_plan)
