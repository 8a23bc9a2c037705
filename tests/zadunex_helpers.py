"""Shared by the Zadunex tests: small configurations, model folders, comparisons.

The configurations differ from one another in every size and constant, and sizes that a model could make
equal by accident are unequal: heads, groups and norm parts of the state-space layers (one group, as many as
heads, in between), state and head sizes, two to five taps, key and value heads of different sizes, one kv
head and as many as query heads, rotation of a part of a head, all of it and of two elements, one to four
streams, a looped span at the start, in the middle and none, a logit scale of 1 and others, dense and routed
feed-forwards and none, a token taking one, some or all experts, and one model with nothing a multiple of 4.

  za  width 64, vocab 211, 2 streams, layers 1..2 three times, logits x 0.5:
      mamba2 4 heads x 16, state 24, 2 groups, 4 taps, 2 norm parts + dense ff 40 limit 1.5
      | attention 4/2 heads dim 16 vdim 24 rot 8 + 5 experts top 2 ff 24
      | mamba2 2 heads x 32, state 16, 1 group, 3 taps, 1 norm part + 4 experts top 1 ff 32
      | attention 6/1 heads dim 32 vdim 32 rot 32, no feed-forward
  zb  width 96, vocab 301, 3 streams, no loop, logits x 1.7:
      attention 3/3 heads dim 8 vdim 40 rot 2 + dense ff 56 limit 0.8
      | mamba2 6 heads x 8, state 40, 6 groups, 2 taps, 3 norm parts + 4 experts top 4 ff 16
      | mamba2 1 head x 64, state 8, 1 group, 5 taps, 4 norm parts, no feed-forward
  zc  width 50, vocab 97, 1 stream (with hyper-connection weights), layers 0..1 twice, logits x 1:
      mamba2 3 heads x 10, state 7, 3 groups, 4 taps, 2 norm parts + 3 experts top 2 ff 11
      | attention 3/1 heads dim 6 vdim 5 rot 4 + dense ff 9 limit 0.7
  zd  width 32, vocab 64, 1 stream without hyper-connection weights, 4 streams' worth of nothing:
      mamba2 2 heads x 12, state 5, 2 groups, 1 tap, 1 norm part + dense ff 24 limit 2.0
      | attention 2/2 heads dim 16 vdim 16 rot 0 + 2 experts top 1 ff 8
  ze  width 48, vocab 80, 4 streams, the only layer twice:
      mamba2 4 heads x 12, state 12, 2 groups, 4 taps, 4 norm parts + 6 experts top 3 ff 20
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_zadunex as plain


def _ssm(heads, vdim, state, groups, conv, parts):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": parts}


def _attn(heads, kv, dim, vdim, rot, base, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot, "base": base}}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


CONFIGS = {
    "za": {"architecture": "Zadunex", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "streams": 2, "logit_scale": 0.5,
           "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
        {"type": "mamba2", "mixer": _ssm(4, 16, 24, 2, 4, 2), "mlp": _dense(40, 1.5)},
        {"type": "attention", "mixer": _attn(4, 2, 16, 24, 8, 100.0, 0.3), "mlp": _moe(5, 2, 24)},
        {"type": "mamba2", "mixer": _ssm(2, 32, 16, 1, 3, 1), "mlp": _moe(4, 1, 32)},
        {"type": "attention", "mixer": _attn(6, 1, 32, 32, 32, 5000.0, 0.2), "mlp": None},
    ]},
    "zb": {"architecture": "Zadunex", "vocab": 301, "width": 96, "norm": {"eps": 1e-6}, "streams": 3, "logit_scale": 1.7,
           "layers": [
        {"type": "attention", "mixer": _attn(3, 3, 8, 40, 2, 10.0, 0.5), "mlp": _dense(56, 0.8)},
        {"type": "mamba2", "mixer": _ssm(6, 8, 40, 6, 2, 3), "mlp": _moe(4, 4, 16)},
        {"type": "mamba2", "mixer": _ssm(1, 64, 8, 1, 5, 4), "mlp": None},
    ]},
    "zc": {"architecture": "Zadunex", "vocab": 97, "width": 50, "norm": {"eps": 1e-5}, "streams": 1, "logit_scale": 1.0,
           "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
        {"type": "mamba2", "mixer": _ssm(3, 10, 7, 3, 4, 2), "mlp": _moe(3, 2, 11)},
        {"type": "attention", "mixer": _attn(3, 1, 6, 5, 4, 7.0, 0.4), "mlp": _dense(9, 0.7)},
    ]},
    "zd": {"architecture": "Zadunex", "vocab": 64, "width": 32, "norm": {"eps": 1e-5}, "streams": 1, "hyper": False,
           "layers": [
        {"type": "mamba2", "mixer": _ssm(2, 12, 5, 2, 1, 1), "mlp": _dense(24, 2.0)},
        {"type": "attention", "mixer": _attn(2, 2, 16, 16, 0, 10000.0, 0.25), "mlp": _moe(2, 1, 8)},
    ]},
    "ze": {"architecture": "Zadunex", "vocab": 80, "width": 48, "norm": {"eps": 1e-6}, "streams": 4, "logit_scale": 2.0,
           "loop": {"start": 0, "stop": 1, "times": 2}, "layers": [
        {"type": "mamba2", "mixer": _ssm(4, 12, 12, 2, 4, 4), "mlp": _moe(6, 3, 20)},
    ]},
}
SEEDS = {"za": 21, "zb": 22, "zc": 23, "zd": 24, "ze": 25}


def config(name: str):
    from kernel_rush_kawk_b200 import ZadunexConfig

    return ZadunexConfig.from_dict(CONFIGS[name])


def shaped_tensors(cfg, seed: int) -> dict:
    """Random weights, shaped so that every mechanism carries weight in the logits: projections of std 0.08,
    biases and routers of order one, decays slow enough that a state remembers hundreds of tokens in some heads
    and a few in others, step sizes on both sides of softplus's knee, hyper-connections that are neither the
    identity nor small."""
    from kernel_rush_kawk_b200.config.registry import get_architecture
    from kernel_rush_kawk_b200.engine.model import expected_tensors
    from kernel_rush_kawk_b200.weights.random_init import random_tensors

    names = expected_tensors(get_architecture(cfg.architecture).plan(cfg))
    t = random_tensors(names, seed, 0.08, "cpu", 0.1)
    S = cfg.streams
    for n in names:
        f = t[n].float()
        if n.endswith((".q.b", ".k.b", ".v.b")):
            f = f * 6.0
        elif n.endswith(".router"):
            f = f * 5.0
        elif n.endswith(".A_log"):
            f = f * 12.0 - 2.5      # rates exp(A_log) from 0.03 to 0.3
        elif n.endswith(".dt_bias"):
            f = f * 10.0 - 0.5
        elif n.endswith(".mix.in"):
            f = f * 2.0             # step sizes and gates of order one
        elif n.endswith(".conv"):
            f = f * 4.0
        elif n.endswith(".conv.b"):
            f = f * 3.0
        elif n.endswith((".hc1.in", ".hc2.in")):
            f = f * 3.0 + 1.0 / S
        elif n.endswith((".hc1.out", ".hc2.out")):
            f = f * 3.0 + 1.0
        elif n.endswith((".hc1.mix", ".hc2.mix")):
            f = f * 2.0 + torch.eye(S)
        t[n] = f.to(torch.bfloat16)
    return t


def write_folder(folder, name: str):
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config(name)
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=2) + "\n")
    save_file({k: v.contiguous() for k, v in shaped_tensors(cfg, SEEDS[name]).items()}, str(folder / "model.safetensors"))
    return folder


def prompts(name: str, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist() for n in lengths]


_cache: dict = {}


def plain_logits(folder, ids) -> torch.Tensor:
    """float64 logits [T, vocab] of the plain implementation (cached per folder and sequence)."""
    key = (str(folder), tuple(ids))
    if key not in _cache:
        cfg, w = plain.read_folder(folder, torch.float64)
        _cache[key] = plain.forward(cfg, w, ids)
    return _cache[key]


def spread(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference with its mean taken off, over the reference's own spread.
    A wrong key, a lost state or a wrong expert moves this by tenths to ones; rounding by 1e-6 in 32-bit."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    r = ref - ref.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / r.pow(2).mean().sqrt()


TOL = {"float32": 5e-5, "bfloat16": 1e-1}


def assert_logits(got, ref, dtype: str, what: str) -> None:
    """32-bit: every row within the tolerance. bfloat16: a token whose two best router scores lie closer than
    the rounding of its input may take another expert than the 64-bit implementation does, and the rows after
    it feel that; so nineteen rows in twenty are held to the tolerance and the rest to five times it."""
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    s = spread(got, ref)
    worst = int(s.argmax())
    if dtype == "float32":
        assert s.max().item() <= TOL[dtype], f"{what}: row {worst} differs by {s.max().item():.3e} of the logits' spread (allowed {TOL[dtype]:.0e})"
        return
    over = int((s > TOL[dtype]).sum())
    assert over <= max(1, s.numel() // 20), f"{what}: {over} of {s.numel()} rows differ by more than {TOL[dtype]:.0e}; worst row {worst}: {s.max().item():.3e}"
    assert s.max().item() <= 5 * TOL[dtype], f"{what}: row {worst} differs by {s.max().item():.3e} of the logits' spread"
