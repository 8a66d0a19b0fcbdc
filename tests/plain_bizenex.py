"""Bizenex in float64 NumPy, one function per mechanism, token by token where that is the
plainest form.  It shares no code with the package: the tests compare the engine with it.

A model is a dict `cfg` (the nested config.json of the design) and a dict of float64 arrays
by tensor name.  `forward(cfg, w, tokens)` gives the logits of every position of one
sequence; `forward(..., layers_out=[])` also collects the residual stream after every layer.

    layer:   x <- x + mixer(LN1(x));  x <- x + moe(LN2(x))
    output:  cap * tanh(head . LN(x) / cap)
"""
from __future__ import annotations

import math

import numpy as np


def layer_norm(x, w, b, eps):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    return x / np.sqrt((x ** 2).mean(axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.clip(z, -700.0, 700.0)))


def softmax_with_sink(scores, sink):
    """Weights of the keys when the denominator holds one more term exp(sink) that has no key."""
    m = max(scores.max(), sink)
    e = np.exp(scores - m)
    return e / (e.sum() + math.exp(sink - m))


def query_temperature(p, coef, every):
    return 1.0 + coef * math.log((p + 1) // every + 1)


def latent_attention(h, m, t, eps, latents=None):
    """h [T, W] -> [T, W].  `latents` given: another layer's latent rows are read instead of
    projecting this layer's own.  Returns (output, latent rows used)."""
    H, d, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    q = (h @ t["q"].T).reshape(T, H, d)
    if latents is None:
        latents = rms_unit(h @ t["dkv"].T, eps) * t["dkv.norm"]
    k = (latents @ t["uk"].T).reshape(T, H, d)
    v = (latents @ t["uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for i in range(T):
        for hh in range(H):
            s = k[:i + 1, hh] @ q[i, hh] * m["scale"]
            out[i, hh] = softmax_with_sink(s, float(t["sink"][hh])) @ v[:i + 1, hh]
    gated = out.reshape(T, H * dv) * sigmoid(h @ t["g"].T)
    return gated @ t["o"].T, latents


def grouped_attention(h, m, t, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_unit((h @ t["q"].T).reshape(T, H, d), eps)
    k = rms_unit((h @ t["k"].T).reshape(T, G, d), eps)
    v = (h @ t["v"].T).reshape(T, G, dv)
    out = np.zeros((T, H, dv))
    for i in range(T):
        temp = query_temperature(i, m["q_temp"]["coef"], m["q_temp"]["every"]) \
            if m.get("q_temp") else 1.0
        for hh in range(H):
            g = hh // (H // G)
            s = k[:i + 1, g] @ (q[i, hh] * temp) * m["scale"]
            out[i, hh] = softmax_with_sink(s, 0.0) @ v[:i + 1, g]
    return out.reshape(T, H * dv) @ t["o"].T


def route(scores, top, n_groups, keep):
    """Chosen experts and their weights for one token's scores [E]."""
    E = scores.shape[0]
    size = E // n_groups
    group_score = []
    for g in range(n_groups):
        best = np.sort(scores[g * size:(g + 1) * size])[::-1][:2]
        group_score.append(best.sum())
    kept = np.argsort(-np.asarray(group_score), kind="stable")[:keep]
    allowed = np.full(E, -np.inf)
    for g in kept:
        allowed[g * size:(g + 1) * size] = scores[g * size:(g + 1) * size]
    chosen = np.argsort(-allowed, kind="stable")[:top]
    weights = scores[chosen] / (scores[chosen].sum() + 1e-20)
    return chosen, weights


def expert(x, gate, up, down):
    z = gate @ x
    return down @ (z * sigmoid(z) * (up @ x))


def moe(h, mlp, t):
    r = mlp["router"]
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        s = sigmoid(t["router"] @ h[i])
        groups = r.get("groups") or {"count": 1, "keep": 1}      # no groups: one group of all
        chosen, weights = route(s, r["top"], groups["count"], groups["keep"])
        for e, wgt in zip(chosen, weights):
            out[i] += wgt * expert(h[i], t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"])
    return out


def _sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(cfg, w, tokens, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        m, t = layer["mixer"], _sub(w, p + "mix.")
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            y, latents[i] = latent_attention(h, m, t, eps, None if src is None else latents[src])
        elif layer["type"] == "attention":
            y = grouped_attention(h, m, t, eps)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            x = x + moe(h, layer["mlp"], _sub(w, p + "mlp."))
        if layers_out is not None:
            layers_out.append(x.copy())
    h = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = h @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(logits / cap) if cap else logits
