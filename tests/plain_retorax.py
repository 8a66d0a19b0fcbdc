"""A plain, slow Retorax: every mechanism of the design as one small function over whole
sequences, in float64 (or float32) torch on the CPU.  It shares no code with the package:
it reads a configuration dictionary and a dictionary of tensors by their names in the
file, and knows nothing of pages, slots, steps or batches.

Notation.  x: [T, W] rows of one sequence, positions 0..T-1.  A matrix named `m` is applied
as rows @ m.T.
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def xielu(z, p, q):
    """Above zero a parabola through the origin with slope 1/2 there; below zero a curve
    that leaves the origin with the same slope and bends by an exponential."""
    sp = lambda a: torch.log1p(torch.exp(a))
    pos = sp(p) * z * z + 0.5 * z
    neg = (0.5 + sp(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h, up, down, act):
    return xielu(h @ up.T, act[0], act[1]) @ down.T


def mingru_candidate(u):
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru(h, t, state=None):
    """t: the mixer's tensors by short name (z, z.b, x, x.b, g, o).  Returns (rows, last state)."""
    z = torch.sigmoid(h @ t["z"].T + t["z.b"])
    c = mingru_candidate(h @ t["x"].T + t["x.b"])
    gate = h @ t["g"].T
    gate = gate * torch.sigmoid(gate)
    s = torch.zeros(z.shape[1], dtype=h.dtype) if state is None else state
    rows = []
    for i in range(h.shape[0]):
        s = (1 - z[i]) * s + z[i] * c[i]
        rows.append(s * gate[i])
    return torch.stack(rows) @ t["o"].T, s


def rotate(x, positions, dims, base):
    """x: [T, heads, d]; the first `dims` dimensions of every head turn, i with i + dims/2.
    The design forms positions and angles in float32: the angle is the float32 product of the
    position and the float32 frequency (its sine and cosine are then taken in x's type)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = (base ** (-2.0 * i / dims)).to(torch.float32)
    a = (positions.to(torch.float32)[:, None] * f[None, :]).to(x.dtype)
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def attention_keys_values(h, t, m):
    """Rotated keys [T, G, d] and values [T, G, dv] of a layer that has projections."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    k = rotate((h @ t["k"].T).view(T, G, d), pos, m["rot"]["dims"], m["rot"]["base"])
    v = (h @ t["v"].T).view(T, G, dv)
    return k, v


def attention_core(q, k, v, scale, talk=None, sink=None, chunk=None, window=None, first=0):
    """q: [T, H, d] rotated queries at positions first..first+T-1; k: [S, G, d], v: [S, G, dv]
    for positions 0..S-1 (S >= first + T).  Returns [T, H, dv]."""
    T, H = q.shape[0], q.shape[1]
    S, G = k.shape[0], k.shape[1]
    kv_of = torch.arange(H) // (H // G)
    raw = torch.einsum("ihd,jhd->hij", q, k[:, kv_of, :]) * scale
    mixed = raw if talk is None else torch.einsum("hg,gij->hij", talk, raw)
    i, j = (first + torch.arange(T))[:, None], torch.arange(S)[None, :]
    see = j <= i
    if chunk:
        see = see & (i // chunk == j // chunk)
    if window:
        see = see & (j > i - window)
    mixed = mixed.masked_fill(~see[None], -math.inf)
    top = mixed.max(-1).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None])
    e = torch.exp(mixed - top[..., None])
    denom = e.sum(-1)
    if sink is not None:
        denom = denom + torch.exp(sink[:, None] - top)
    return torch.einsum("hij,jhd->ihd", e / denom[..., None], v[:, kv_of, :])


def attention(h, t, m, k, v):
    """t: the mixer's tensors (q, talk, sink, g, o); k, v: keys and values of all positions,
    this layer's own or another layer's."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = rotate((h @ t["q"].T).view(T, H, d), torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    heads = attention_core(q, k, v, m["scale"], t["talk"], t["sink"],
                           (m.get("mask") or {}).get("size")).reshape(T, H * dv)
    heads = heads * torch.sigmoid(h @ t["g"].T)
    return heads @ t["o"].T


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, dtype=torch.float64, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after each layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kv = {}
    after = []
    for li, layer in enumerate(config["layers"]):
        p = f"l{li}."
        norm = lambda name, rows: layer_norm(rows, w[p + name], w[p + name + ".b"], eps)
        h = norm("norm1", x)
        mix = sub(w, p + "mix.")
        if layer["type"] == "mingru":
            y, _ = mingru(h, mix)
        elif layer["type"] == "attention":
            m = layer["mixer"]
            if m.get("kv_from") is None:
                kv[li] = attention_keys_values(h, mix, m)
            k, v = kv[li if m.get("kv_from") is None else m["kv_from"]]
            y = attention(h, mix, m, k, v)
        else:
            raise ValueError(layer["type"])
        x = x + norm("norm1b", y)
        if layer.get("mlp") is not None:
            ff = sub(w, p + "mlp.")
            x = x + norm("norm2b", dense_ff(norm("norm2", x), ff["up"], ff["down"], ff["act"]))
        after.append(x)
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T
    return (logits, torch.stack(after)) if keep_layers else logits
