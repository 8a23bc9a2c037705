"""A plain, slow restatement of the Zadunex decoder, one function per mechanism.

Written from the design's equations for the tests only; it shares no code with
the package. Everything runs in the dtype of the tensors it is given (float64 in
the tests). Notation: X is the set of residual streams [S, T, C]; h a sublayer's
normalised input [T, C]; positions count from 0.

  norm         y = x / sqrt(mean(x^2) + eps) * g
  embedding    every stream starts as E[token]
  sublayer q   u = sum_s a_s X_s;  y = f(norm(u));  X'_t = sum_s M[s, t] X_s + b_t y   (a, M, b per sublayer)
  layer        sublayer 1 is the mixer, sublayer 2 the feed-forward (if the layer has one)
  loop         layers start .. stop-1 run ``times`` times in a row with the same weights; every run keeps
               a cache or state of its own
  output       logits = scale * W_head . norm_final(sum_s X_s)

Mixers:
  mamba2     state-space layer: one input product, a short causal convolution with silu over (x, B, C),
             per head S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, gate silu(z), grouped RMS norm
  attention  grouped-query heads, biases, RMS norm over the whole q (and k) row, rotation of part of each
             head, causal, one more term exp(0) in the softmax's denominator
Feed-forward: dense with clamps, g' = min(g, L), u' = clamp(u, -L, L), g' sigmoid(1.702 g') (u' + 1); or
routed SwiGLU experts weighted by the softmax over all experts' logits, the largest ``top`` taken as they are.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def read_folder(folder, dtype=torch.float64):
    from safetensors import safe_open

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {}
    for shard in sorted(folder.glob("*.safetensors")):
        with safe_open(str(shard), framework="pt", device="cpu") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                w[name] = t.to(dtype) if t.dtype.is_floating_point else t
    return cfg, w


# ---------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------

def rms_norm(x, g, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * g


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_part(x, positions, dims, base):
    """x [T, heads, D]: element i < dims/2 of a head is paired with element i + dims/2 and the pair is
    turned by the angle position * base^(-2i/dims); elements from ``dims`` on pass."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]  # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------
# mixers. Each takes h [T, C] of ONE sequence from position 0 and returns [T, C].
# ---------------------------------------------------------------------------

def causal_conv(x, kernel, bias):
    """x [T, channels]; kernel [channels, taps], its last column multiplies the current token, the one
    before it the previous token, and so on; zeros before the start."""
    T, _ = x.shape
    taps = kernel.shape[1]
    out = torch.zeros_like(x) + bias
    for j in range(taps):
        back = taps - 1 - j  # how many tokens back column j looks
        if back < T:
            out[back:] += x[:T - back] * kernel[:, j]
    return out


def mamba2(h, w, p, m, eps):
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * P
    T = h.shape[0]
    proj = h @ w[p + "in"].T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt = proj[:, 2 * inner + 2 * G * N:]
    assert dt.shape[1] == heads
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)  # [T, heads]
    per = heads // G
    y = torch.zeros(T, heads, P, dtype=h.dtype)
    for hd in range(heads):
        g = hd // per
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ Cm[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = y.reshape(T, parts, inner // parts)
    y = y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)
    y = y.reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def attention(h, w, p, m, eps):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, D)
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(T, G, D)
    v = v.reshape(T, G, V)
    q = rotate_part(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_part(k, pos, m["rot"]["dims"], m["rot"]["base"])
    out = torch.zeros(T, H, V, dtype=h.dtype)
    per = H // G
    for hd in range(H):
        g = hd // per
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, hd]) * m["scale"]
            big = torch.clamp(s.max(), min=0.0)  # the extra term's score is 0
            e = torch.exp(s - big)
            out[t, hd] = (e / (torch.exp(-big) + e.sum())) @ v[:t + 1, g]
    return out.reshape(T, H * V) @ w[p + "o"].T


# ---------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------

def dense_ff(h, w, p, mlp):
    L = mlp["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=L)
    u = torch.clamp(h @ w[p + "up"].T, min=-L, max=L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def routed_ff(h, w, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)  # over all experts
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        chosen = torch.topk(scores[t], top).indices
        for e in chosen.tolist():
            q = f"{p}e{e}."
            y = (silu(h[t] @ w[q + "gate"].T) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T
            out[t] += scores[t, e] * y
    return out


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------

def layer_runs(cfg):
    """The order in which layers run, the looped span repeated."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sublayer(X, w, p, q, f, gain, eps):
    """X [S, T, C] -> the new streams after sublayer q ("hc1" or "hc2") whose function is f."""
    if p + q + ".in" not in w:  # one stream without hyper-connection weights: the plain residual sum
        return X + f(rms_norm(X[0], gain, eps))[None]
    a, b, M = w[p + q + ".in"], w[p + q + ".out"], w[p + q + ".mix"]
    u = torch.einsum("s,stc->tc", a, X)
    y = f(rms_norm(u, gain, eps))
    return torch.einsum("sr,stc->rtc", M, X) + b[:, None, None] * y[None]


def forward(cfg, w, tokens, per_layer=None):
    """tokens: list of ids of one sequence -> logits [T, vocab]. ``per_layer``: a list that receives the
    sum of the streams after every run of a layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    S = int(cfg.get("streams", 1))
    X = x[None].repeat(S, 1, 1)
    for i in layer_runs(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        m = layer["mixer"]
        mix = {"mamba2": mamba2, "attention": attention}[layer["type"]]
        X = sublayer(X, w, p, "hc1", lambda h: mix(h, w, p + "mix.", m, eps), w[p + "norm1"], eps)
        mlp = layer["mlp"]
        if mlp is not None:
            ff = dense_ff if mlp["kind"] == "dense" else routed_ff
            X = sublayer(X, w, p, "hc2", lambda h: ff(h, w, p + "mlp.", mlp), w[p + "norm2"], eps)
        if per_layer is not None:
            per_layer.append(X.sum(dim=0))
    x = X.sum(dim=0)
    return (rms_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg.get("logit_scale", 1.0)
