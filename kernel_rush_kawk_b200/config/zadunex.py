"""Configuration of the Zadunex decoder, read from its own config.json keys.

    {"architecture": "Zadunex", "vocab": V, "width": C, "norm": {"eps": e}, "streams": S, "logit_scale": a,
     "loop": {"start": i, "stop": j, "times": n},
     "layers": [{"type": T, "mixer": {...}, "mlp": {...} | null}, ...]}

Mixer types and their keys:

* ``mamba2``: ``heads``, ``vdim`` (channels per head), ``state``, ``groups`` (heads share B and C within a
  group), ``conv`` (taps of the short convolution), ``norm_groups`` (parts of the gated norm).
* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` (``dims``, ``base``).

Feed-forward (``mlp``): ``kind`` "dense" with ``ff`` and ``limit``, or ``kind`` "moe" with ``expert.ff``,
``router.experts`` and ``router.top``; or null. ``loop`` (optional) repeats the layers start .. stop-1
``times`` times in a row; ``streams`` (default 1) is the number of residual streams that the layers'
hyper-connections read and write. Whether the layers carry hyper-connection weights is read off the
checkpoint where ``streams`` is 1 (``with_tensor_shapes``); with more streams they always do.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field, replace
from pathlib import Path

from .base import ConfigError, ModelConfig, positive, require
from .taredra import _int, _number, _section

PRESET_DIR = Path(__file__).parent / "presets" / "zadunex"

MIXER_TYPES = ("mamba2", "attention")


def _read_mixer(kind: str, raw: dict, where: str) -> dict:
    if kind == "mamba2":
        out = {k: _int(raw, k, where) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")}
        if out["heads"] % out["groups"]:
            raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of groups ({out['groups']})")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"config.json: {where}norm_groups ({out['norm_groups']}) must divide heads * vdim "
                              f"({out['heads'] * out['vdim']})")
        return out
    out = {"heads": _int(raw, "heads", where), "kv_heads": _int(raw, "kv_heads", where), "dim": _int(raw, "dim", where),
           "vdim": _int(raw, "vdim", where), "scale": _number(raw, "scale", where)}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of kv_heads ({out['kv_heads']})")
    rot = raw.get("rot")
    if rot is None:
        out["rot"] = {"dims": 0, "base": 10000.0}
    else:
        rot = _section(raw, "rot", where)
        dims = rot.get("dims")
        if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > out["dim"]:
            raise ConfigError(f"config.json: {where}rot.dims ({dims!r}) must be even and at most dim ({out['dim']})")
        out["rot"] = {"dims": dims, "base": _number(rot, "base", where + "rot.")}
        if not out["rot"]["base"] > 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
    return out


def _read_mlp(raw, where: str):
    if raw is None:
        return None
    kind = raw.get("kind") if isinstance(raw, dict) else None
    if kind == "dense":
        limit = _number(raw, "limit", where + "mlp.")
        if not limit > 0:
            raise ConfigError(f"config.json: {where}mlp.limit must be positive, got {limit!r}")
        return {"kind": "dense", "ff": _int(raw, "ff", where + "mlp."), "limit": limit}
    if kind == "moe":
        router = _section(raw, "router", where + "mlp.")
        out = {"kind": "moe", "expert": {"ff": _int(_section(raw, "expert", where + "mlp."), "ff", where + "mlp.expert.")},
               "router": {"experts": _int(router, "experts", where + "mlp.router."),
                          "top": _int(router, "top", where + "mlp.router.")}}
        if out["router"]["top"] > out["router"]["experts"]:
            raise ConfigError(f"config.json: {where}mlp.router.top exceeds the number of experts")
        return out
    raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense' or 'moe', got {raw!r}")


def _read_layer(raw: dict, i: int) -> dict:
    where = f"layers[{i}]."
    kind = raw.get("type") if isinstance(raw, dict) else None
    if kind not in MIXER_TYPES:
        raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design {MIXER_TYPES}")
    return {"type": kind, "mixer": _read_mixer(kind, _section(raw, "mixer", where), where + "mixer."),
            "mlp": _read_mlp(raw.get("mlp"), where)}


@dataclass(frozen=True)
class ZadunexConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    streams: int = 1
    logit_scale: float = 1.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    #: whether the layers carry hyper-connection weights (always with several streams)
    hyper: bool = True
    #: one normalised dict per layer (type, mixer, mlp); treated as read-only
    layers: tuple = field(default_factory=tuple)

    architecture = "Zadunex"

    @classmethod
    def from_dict(cls, raw: dict) -> "ZadunexConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        loop = raw.get("loop")
        start, stop, times = 0, 0, 1
        if loop is not None:
            loop = _section(raw, "loop", "")
            for key in ("start", "stop"):
                v = loop.get(key)
                if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                    raise ConfigError(f"config.json: loop.{key} must be a non-negative integer, got {v!r}")
            start, stop, times = loop["start"], loop["stop"], _int(loop, "times", "loop.")
            if not start <= stop <= len(layers):
                raise ConfigError(f"config.json: loop.start <= loop.stop <= {len(layers)} layers must hold, got {start}, {stop}")
        streams = raw.get("streams", 1)
        if isinstance(streams, bool) or not isinstance(streams, int) or streams < 1:
            raise ConfigError(f"config.json: 'streams' must be a positive integer, got {streams!r}")
        cfg = cls(vocab=require(raw, "vocab", int), width=require(raw, "width", int),
                  eps=_number(_section(raw, "norm", ""), "eps", "norm."), streams=streams,
                  logit_scale=_number(raw, "logit_scale", "") if "logit_scale" in raw else 1.0,
                  loop_start=start, loop_stop=stop, loop_times=times, hyper=bool(raw.get("hyper", True)),
                  layers=tuple(_read_layer(layer, i) for i, layer in enumerate(layers)))
        positive("vocab", cfg.vocab)
        positive("width", cfg.width)
        if not cfg.eps >= 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {cfg.eps!r}")
        if cfg.streams > 1 and not cfg.hyper:
            raise ConfigError("config.json: several streams need the layers' hyper-connection weights")
        return cfg

    def with_tensor_shapes(self, shapes: dict) -> "ZadunexConfig":
        """One stream may come with or without hyper-connection weights: the checkpoint tells."""
        if self.streams == 1:
            return replace(self, hyper="l0.hc1.in" in shapes)
        return self

    def layer_runs(self) -> list[int]:
        """The order in which the layers run, the looped span repeated."""
        a, b = self.loop_start, self.loop_stop
        return list(range(a)) + list(range(a, b)) * self.loop_times + list(range(b, len(self.layers)))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "streams": self.streams, "logit_scale": self.logit_scale,
               "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
               "layers": copy.deepcopy(list(self.layers))}
        if not self.hyper:
            out["hyper"] = False
        return out

    @classmethod
    def preset_names(cls) -> list[str]:
        return sorted(p.stem for p in PRESET_DIR.glob("*.json"))

    @classmethod
    def preset(cls, name: str) -> "ZadunexConfig":
        path = PRESET_DIR / f"{name}.json"
        if not path.is_file():
            raise ConfigError(f"unknown preset '{name}'; known presets: {cls.preset_names()}")
        return cls.from_dict(json.loads(path.read_text()))
