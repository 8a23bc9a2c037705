"""Configuration of the Fogizen decoder, read from its own config.json keys.

    {"architecture": "Fogizen", "vocab": V, "width": C, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": m, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "parallel", "mixer": {"left": {...}, "right": {...}}, "mlp": {...} | null}, ...]}

``left`` (attention): ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (keys are seen
within the query's own block of that many positions; absent: every earlier key), ``rot`` (``dims``, ``base``,
``scaling.factor``; absent: no rotation). ``right`` (time mixing): ``heads``, ``dim``; the rank of the decay's two
small matrices is read off the checkpoint (``with_tensor_shapes``), or defaults for random weights.
``mlp``: ``kind`` "dense" with ``ff``, or ``kind`` "moe" with ``expert.ff`` and ``router`` (``experts``, ``top``,
``scale``, ``groups.count``, ``groups.keep``; without ``groups`` all experts form one group); or null.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field, replace
from pathlib import Path

from .base import ConfigError, ModelConfig, positive, require
from .taredra import DEFAULT_DECAY_RANK, _int, _number, _section

PRESET_DIR = Path(__file__).parent / "presets" / "fogizen"

LAYER_TYPES = ("parallel",)


def _read_left(raw: dict, where: str) -> dict:
    out = {"heads": _int(raw, "heads", where), "kv_heads": _int(raw, "kv_heads", where), "dim": _int(raw, "dim", where),
           "vdim": _int(raw, "vdim", where), "scale": _number(raw, "scale", where), "mask": None, "rot": None}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of kv_heads ({out['kv_heads']})")
    if raw.get("mask") is not None:
        out["mask"] = {"size": _int(_section(raw, "mask", where), "size", where + "mask.")}
    if raw.get("rot") is not None:
        rot = _section(raw, "rot", where)
        dims = rot.get("dims")
        if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > out["dim"]:
            raise ConfigError(f"config.json: {where}rot.dims ({dims!r}) must be even and at most dim ({out['dim']})")
        base = _number(rot, "base", where + "rot.")
        factor = 1.0
        if rot.get("scaling") is not None:
            factor = _number(_section(rot, "scaling", where + "rot."), "factor", where + "rot.scaling.")
        if not base > 0 or not factor > 0:
            raise ConfigError(f"config.json: {where}rot.base and rot.scaling.factor must be positive")
        out["rot"] = {"dims": dims, "base": base, "scaling": {"factor": factor}}
    return out


def _read_mlp(raw, where: str):
    if raw is None:
        return None
    kind = raw.get("kind") if isinstance(raw, dict) else None
    if kind == "dense":
        return {"kind": "dense", "ff": _int(raw, "ff", where + "mlp.")}
    if kind == "moe":
        router = _section(raw, "router", where + "mlp.")
        r = {"experts": _int(router, "experts", where + "mlp.router."), "top": _int(router, "top", where + "mlp.router."),
             "scale": _number(router, "scale", where + "mlp.router.") if "scale" in router else 1.0,
             "groups": {"count": 1, "keep": 1}}
        if router.get("groups") is not None:
            g = _section(router, "groups", where + "mlp.router.")
            r["groups"] = {"count": _int(g, "count", where + "mlp.router.groups."),
                           "keep": _int(g, "keep", where + "mlp.router.groups.")}
        count, keep = r["groups"]["count"], r["groups"]["keep"]
        if r["experts"] % count or keep > count:
            raise ConfigError(f"config.json: {where}mlp.router: {r['experts']} experts do not form {count} equal groups "
                              f"of which {keep} are kept")
        if r["top"] > keep * (r["experts"] // count):
            raise ConfigError(f"config.json: {where}mlp.router.top ({r['top']}) exceeds the experts of the kept groups")
        return {"kind": "moe", "expert": {"ff": _int(_section(raw, "expert", where + "mlp."), "ff", where + "mlp.expert.")},
                "router": r}
    raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense' or 'moe', got {raw!r}")


def _read_layer(raw: dict, i: int) -> dict:
    where = f"layers[{i}]."
    kind = raw.get("type") if isinstance(raw, dict) else None
    if kind not in LAYER_TYPES:
        raise ConfigError(f"config.json: {where}type '{kind}' is not a layer of this design {LAYER_TYPES}")
    mixer = _section(raw, "mixer", where)
    right = _section(mixer, "right", where + "mixer.")
    r = {"heads": _int(right, "heads", where + "mixer.right."), "dim": _int(right, "dim", where + "mixer.right.")}
    if right.get("rank") is not None:
        r["rank"] = _int(right, "rank", where + "mixer.right.")
    return {"type": kind, "mixer": {"left": _read_left(_section(mixer, "left", where + "mixer."), where + "mixer.left."),
                                    "right": r}, "mlp": _read_mlp(raw.get("mlp"), where)}


@dataclass(frozen=True)
class FogizenConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    #: one normalised dict per layer (type, mixer, mlp); treated as read-only
    layers: tuple = field(default_factory=tuple)

    architecture = "Fogizen"

    @classmethod
    def from_dict(cls, raw: dict) -> "FogizenConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        bigram = _section(_section(raw, "embedding", ""), "bigram", "embedding.")
        for key in ("mul_prev", "mul_cur"):
            v = bigram.get(key)
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                raise ConfigError(f"config.json: embedding.bigram.{key} must be a non-negative integer, got {v!r}")
        cfg = cls(vocab=require(raw, "vocab", int), width=require(raw, "width", int),
                  eps=_number(_section(raw, "norm", ""), "eps", "norm."),
                  buckets=_int(bigram, "buckets", "embedding.bigram."), mul_prev=bigram["mul_prev"],
                  mul_cur=bigram["mul_cur"], layers=tuple(_read_layer(layer, i) for i, layer in enumerate(layers)))
        positive("vocab", cfg.vocab)
        positive("width", cfg.width)
        if not cfg.eps >= 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {cfg.eps!r}")
        return cfg

    def with_tensor_shapes(self, shapes: dict) -> "FogizenConfig":
        """The decays' rank is the first size of each layer's ``mix.right.w1``."""
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            shape = shapes.get(f"l{i}.mix.right.w1")
            if shape is not None:
                layer["mixer"]["right"]["rank"] = int(shape[0])
        return replace(self, layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
                "layers": copy.deepcopy(list(self.layers))}

    @classmethod
    def preset_names(cls) -> list[str]:
        return sorted(p.stem for p in PRESET_DIR.glob("*.json"))

    @classmethod
    def preset(cls, name: str) -> "FogizenConfig":
        path = PRESET_DIR / f"{name}.json"
        if not path.is_file():
            raise ConfigError(f"unknown preset '{name}'; known presets: {cls.preset_names()}")
        return cls.from_dict(json.loads(path.read_text()))


def decay_rank(right: dict) -> int:
    return int(right.get("rank", DEFAULT_DECAY_RANK))
