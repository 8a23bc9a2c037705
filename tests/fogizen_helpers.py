"""Shared by the Fogizen tests: small configurations, model folders, comparisons.

The configurations differ from one another in every size and constant, and none of a model's sizes coincide by
accident (key and value heads of different sizes, a rotation of part of a head or of none, head counts that do not
divide the width, ranks other than the default, sizes that are no multiple of 4 or 8, layers with a dense
feed-forward, with routed experts and with none in different orders, groups of one expert, every group kept, blocks
of keys shorter than a page, longer than a page and absent).

  name  width vocab  layers (left heads/kv dim vdim block rot | right heads x dim, rank | feed-forward)
  fa     64   211    4/2 16 32 10 rot 8 | 3 x 16 r8 | moe 6 experts top 2, 3 groups keep 2, ff 24
                     2/2 24  8 37 rot 24 | 1 x 48 r12 | dense 72
                     4/1  8 16 70 rot 0 | 2 x 8 r4 | none
  fb     96   301    6/1 32 32 100 rot 16 | 2 x 32 r16 | dense 136
                     3/3  8 40  5 rot 2 | 5 x 8 r6 | moe 4 experts top 4, 4 groups keep 4 (groups of one, all kept), ff 16
                     2/1 16 24 none rot 16 | 3 x 16 r5 | moe 8 experts top 3, 2 groups keep 1, ff 40
  fc     50    97    3/3  6  5  3 rot 4 | 1 x 7 r3 | moe 9 experts top 2, 3 groups keep 2, ff 11
                     5/1 10  6 64 rot 10 | 3 x 9 r5 | dense 33
                     (nothing a multiple of 4 or 8: every kernel's plain path, the products' fallbacks)
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_fogizen as plain


def _left(heads, kv, dim, vdim, block, rot, base, factor, scale):
    out = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if block is not None:
        out["mask"] = {"size": block}
    if rot:
        out["rot"] = {"dims": rot, "base": base, "scaling": {"factor": factor}}
    return out


def _moe(experts, top, count, keep, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}


def _layer(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


CONFIGS = {
    "fa": {"architecture": "Fogizen", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
           "embedding": {"bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 3}},
           "layers": [
               _layer(_left(4, 2, 16, 32, 10, 8, 100.0, 2.0, 0.31), {"heads": 3, "dim": 16, "rank": 8}, _moe(6, 2, 3, 2, 24, 1.5)),
               _layer(_left(2, 2, 24, 8, 37, 24, 5000.0, 1.0, 0.2), {"heads": 1, "dim": 48, "rank": 12}, {"kind": "dense", "ff": 72}),
               _layer(_left(4, 1, 8, 16, 70, 0, 1.0, 1.0, 0.4), {"heads": 2, "dim": 8, "rank": 4}, None),
           ]},
    "fb": {"architecture": "Fogizen", "vocab": 301, "width": 96, "norm": {"eps": 1e-6},
           "embedding": {"bigram": {"buckets": 1009, "mul_prev": 100003, "mul_cur": 65537}},
           "layers": [
               _layer(_left(6, 1, 32, 32, 100, 16, 15000.0, 4.0, 0.18), {"heads": 2, "dim": 32}, {"kind": "dense", "ff": 136}),
               _layer(_left(3, 3, 8, 40, 5, 2, 10.0, 1.5, 0.5), {"heads": 5, "dim": 8, "rank": 6}, _moe(4, 4, 4, 4, 16, 0.7)),
               _layer(_left(2, 1, 16, 24, None, 16, 300.0, 3.0, 0.25), {"heads": 3, "dim": 16, "rank": 5}, _moe(8, 3, 2, 1, 40, 2.5)),
           ]},
    "fc": {"architecture": "Fogizen", "vocab": 97, "width": 50, "norm": {"eps": 1e-5},
           "embedding": {"bigram": {"buckets": 11, "mul_prev": 1, "mul_cur": 5}},
           "layers": [
               _layer(_left(3, 3, 6, 5, 3, 4, 7.0, 1.25, 0.4), {"heads": 1, "dim": 7, "rank": 3}, _moe(9, 2, 3, 2, 11, 1.0)),
               _layer(_left(5, 1, 10, 6, 64, 10, 50.0, 2.0, 0.3), {"heads": 3, "dim": 9, "rank": 5}, {"kind": "dense", "ff": 33}),
           ]},
}
SEEDS = {"fa": 31, "fb": 32, "fc": 33}


def config(name: str):
    from kernel_rush_kawk_b200 import FogizenConfig

    return FogizenConfig.from_dict(CONFIGS[name])


def shaped_tensors(cfg, seed: int) -> dict:
    """Random weights, shaped so that every mechanism carries weight in the logits: projections of std 0.08, the
    attention's queries and keys scaled up (sharp softmax: a wrong key shows), a mixing matrix that is far from the
    identity, sinks near the scores' size, biases, blends and corrections of order one, decays spread over (0, 1)."""
    from kernel_rush_kawk_b200.config.registry import get_architecture
    from kernel_rush_kawk_b200.engine.model import expected_tensors
    from kernel_rush_kawk_b200.weights.random_init import random_tensors

    names = expected_tensors(get_architecture(cfg.architecture).plan(cfg))
    t = random_tensors(names, seed, 0.08, "cpu", 0.1)
    for n in names:
        f = t[n].float()
        if n.endswith((".left.q", ".left.k")):
            f = f * 3.0
        elif n.endswith((".q.b", ".k.b", ".v.b")):
            f = f * 6.0
        elif n.endswith((".q.norm", ".k.norm")):
            f = f * 1.5
        elif n.endswith(".talk"):
            f = (f - torch.eye(f.shape[0])) * 5.0 + 0.7 * torch.eye(f.shape[0])
        elif n.endswith(".sink"):
            f = f * 20.0
        elif n.endswith(".left.g"):
            f = f * 4.0
        elif n.endswith(".shift") or ".mu." in n:
            f = f * 4.0 + 0.4
        elif n.endswith(".w0"):
            f = f * 20.0 - 1.0
        elif n.endswith((".w1", ".w2")):
            f = f * 3.0
        elif n.endswith(".u"):
            f = f * 8.0
        elif n.endswith(".router"):
            f = f * 5.0
        elif n.endswith(".correction"):
            f = f * 4.0
        elif n.endswith(".act"):
            f = f * 10.0
        elif n == "bigram":
            f = f * 3.0
        t[n] = f.to(torch.bfloat16)
    return t


def write_folder(folder, name: str, change=None):
    """``change(tensors)`` may edit the tensors before they are written (a test that plants a key)."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config(name)
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=2) + "\n")
    tensors = shaped_tensors(cfg, SEEDS[name])
    if change is not None:
        change(tensors)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
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
    """32-bit: every row within the tolerance. bfloat16: a token whose router scores lie closer than the rounding
    of its input may take another expert than the 64-bit implementation does, and the rows after it feel that; so
    nineteen rows in twenty are held to the tolerance and the rest to five times it."""
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
