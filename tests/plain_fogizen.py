"""A plain, slow restatement of the Fogizen decoder, one function per mechanism.

Written from the design's equations for the tests only; it shares no code with
the package. Everything runs in the dtype of the tensors it is given (float64
in the tests), one token, one head or one key after the other where that is the
clearest way to write it. Notation: x is the residual stream [T, C]; n = norm1(x);
a mixer returns [T, C]; tokens of one sequence only, positions 0 .. T-1.

  embedding  x_t = E[id_t] + B[(id_(t-1) a + id_t b) mod m]   (B[m] for t = 0)
  layer      n = norm1(x); s_t = n_t + (n_(t-1) - n_t) * shift; x += mixer(s) + ff(n)
  mixer      (norm_L(attention(s)) + norm_R(time_mix(s))) / 2
  output     logits = H . norm_final(x)
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ---------------------------------------------------------------------------
# reading a model folder (the file format read directly: a length, a JSON table, the data)
# ---------------------------------------------------------------------------

def read_folder(folder, dtype=torch.float64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    blob = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    table = json.loads(blob[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16, "F64": torch.float64}
    w = {}
    for name, info in table.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(blob[8 + n + a:8 + n + b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        w[name] = t.to(dtype) if t.dtype.is_floating_point else t
    return cfg, w


# ---------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------

def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, g, eps):
    return unit_rms(x, eps) * g


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def silu(z):
    return z * torch.sigmoid(z)


def previous_rows(h):
    """Row t holds row t - 1 of h; row 0 is zero."""
    return torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)


def bigram_rows(ids, buckets, mul_prev, mul_cur):
    rows = [buckets]
    for t in range(1, len(ids)):
        rows.append((int(ids[t - 1]) * mul_prev + int(ids[t]) * mul_cur) % buckets)
    return torch.tensor(rows, dtype=torch.long)


def embed(ids, table, bigram, e):
    ids = torch.as_tensor(ids, dtype=torch.long)
    return table[ids] + bigram[bigram_rows(ids, e["buckets"], e["mul_prev"], e["mul_cur"])]


# ---------------------------------------------------------------------------
# left mixer: chunked attention with mixed head scores, a sink and a gate per head
# ---------------------------------------------------------------------------

def rotate_pairs(x, positions, dims, base, factor):
    """x [T, heads, D]; elements (2i, 2i + 1), i < dims / 2, turned by position * base^(-2i / dims) / factor."""
    out = x.clone()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims) / factor
        ang = positions.to(x.dtype) * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def mixed_chunk_attention(q, k, v, scale, talk, sink, chunk):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]. Query t sees keys j <= t of its own chunk
    (t // chunk == j // chunk; chunk None: all j <= t). The H raw scores of a (query, key) pair are mixed
    by ``talk`` [H, H] before the softmax, whose denominator has one more term exp(sink_h)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        first = 0 if chunk is None else (t // chunk) * chunk
        keys = range(first, t + 1)
        raw = torch.stack([torch.stack([(q[t, h] * k[j, h // (H // G)]).sum() * scale for j in keys]) for h in range(H)])
        mixed = talk @ raw  # [H, keys]
        for h in range(H):
            top = torch.maximum(mixed[h].max(), sink[h])
            e = torch.exp(mixed[h] - top)
            p = e / (e.sum() + torch.exp(sink[h] - top))
            for n, j in enumerate(keys):
                out[t, h] += p[n] * v[j, h // (H // G)]
    return out


def left_branch(s, w, p, m, eps, positions):
    T = s.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (s @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    k = (s @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
    v = (s @ w[p + "v"].T + w[p + "v.b"]).view(T, G, Dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot is not None and rot["dims"]:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_pairs(q, positions, rot["dims"], rot["base"], factor)
        k = rotate_pairs(k, positions, rot["dims"], rot["base"], factor)
    chunk = (m.get("mask") or {}).get("size")
    o = mixed_chunk_attention(q, k, v, m["scale"], w[p + "talk"], w[p + "sink"], chunk)
    o = o * torch.sigmoid(s @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * Dv) @ w[p + "o"].T


# ---------------------------------------------------------------------------
# right mixer: time mixing with a matrix state per head
# ---------------------------------------------------------------------------

def state_scan(r, k, v, decay, bonus):
    """r, k, v, decay [T, H, N]; bonus [H, N]. o_t = (S + diag(bonus) k_t v_t^T)^T r_t with the state before
    token t; then S <- diag(decay_t) S + k_t v_t^T. S starts at zero."""
    T, H, N = r.shape
    out = torch.zeros_like(v)
    for h in range(H):
        S = torch.zeros(N, N, dtype=r.dtype)
        for t in range(T):
            kv = torch.outer(k[t, h], v[t, h])
            out[t, h] = (S + bonus[h][:, None] * kv).T @ r[t, h]
            S = decay[t, h][:, None] * S + kv
    return out


def right_branch(s, w, p, m, eps):
    T = s.shape[0]
    H, N = m["heads"], m["dim"]
    d = previous_rows(s) - s
    mix = {c: s + d * w[p + "mu." + c] for c in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).view(T, H, N)
    k = (mix["k"] @ w[p + "k"].T).view(T, H, N)
    v = (mix["v"] @ w[p + "v"].T).view(T, H, N)
    gate = silu(mix["g"] @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, N)
    o = unit_rms(state_scan(r, k, v, decay, w[p + "u"]), eps).reshape(T, H * N)
    return (o * w[p + "norm"] * gate) @ w[p + "o"].T


def mixer(s, w, p, m, eps, positions):
    a = rms_norm(left_branch(s, w, p + "left.", m["left"], eps, positions), w[p + "left.out"], eps)
    b = rms_norm(right_branch(s, w, p + "right.", m["right"], eps), w[p + "right.out"], eps)
    return 0.5 * (a + b)


# ---------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------

def xielu(z, p, q):
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (torch.expm1(z) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(n, w, p):
    a = w[p + "act"]
    return xielu(n @ w[p + "up"].T, a[0], a[1]) @ w[p + "down"].T


def route(n, w, p, router):
    """Per row: the chosen experts and their weights. Choice by sigmoid + correction inside the best groups
    (a group's score: the sum of its two largest choice scores); weights from the sigmoids alone."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(n @ w[p + "router"].T)
    c = s + w[p + "correction"]
    chosen, weights = [], []
    size = E // groups["count"]
    for t in range(n.shape[0]):
        per_group = c[t].view(groups["count"], size)
        score = per_group.topk(min(2, size), dim=1).values.sum(dim=1)
        best = score.topk(groups["keep"]).indices.tolist()
        allowed = torch.full((E,), -math.inf, dtype=n.dtype)
        for g in best:
            allowed[g * size:(g + 1) * size] = c[t, g * size:(g + 1) * size]
        idx = allowed.topk(top).indices
        wt = s[t, idx]
        chosen.append(idx)
        weights.append(wt / (wt.sum() + 1e-20) * router["scale"])
    return torch.stack(chosen), torch.stack(weights)


def routed_ff(n, w, p, mlp):
    idx, wt = route(n, w, p, mlp["router"])
    out = torch.zeros_like(n)
    for t in range(n.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            q = f"{p}e{e}."
            out[t] += a * ((silu(n[t] @ w[q + "gate"].T) * (n[t] @ w[q + "up"].T)) @ w[q + "down"].T)
    return out


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------

def forward(cfg, w, ids, per_layer=None):
    """Logits [T, vocab] of one sequence; ``per_layer`` (a list) receives x after every layer."""
    eps = cfg["norm"]["eps"]
    x = embed(ids, w["embed"], w["bigram"], cfg["embedding"]["bigram"])
    positions = torch.arange(len(ids))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = rms_norm(x, w[p + "norm1"], eps)
        s = n + (previous_rows(n) - n) * w[p + "shift"]
        y = mixer(s, w, p + "mix.", layer["mixer"], eps, positions)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ff(n, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(n, w, p + "mlp.", mlp))
        x = x + y
        if per_layer is not None:
            per_layer.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
