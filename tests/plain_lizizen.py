"""Plain, slow float64 implementation of the Lizizen design: one function per mechanism, written
from the equations, with loops over heads and no cache.  Tokens of one sequence at a time.

A layer:   x <- x + mixer(shift(norm1(x))) + ff(norm2(x)),  norms of the same x with factor (1 + w);
``shift`` replaces row t by ``h_t + (h_(t-1) - h_t) * s`` (zeros before row 0).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_around_zero(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def token_shift(h, s):
    """Row t becomes h_t + (h_(t-1) - h_t) * s; the row before the first is zero."""
    before = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (before - h) * s


def query_temperature(positions, coef, every):
    return 1.0 + coef * np.log(np.floor((positions + 1.0) / every) + 1.0)


def distance_bias(r1, r2, n):
    """[n, n]: r1 ln(1 + r2 (i - j)) for j <= i (0 above the diagonal, which is masked anyway)."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    return r1 * np.log1p(r2 * np.maximum(i - j, 0))


def softmax_with_zero_sink(scores, visible):
    """Rows of exp(s_j) / (1 + sum_j exp(s_j)) over the visible keys."""
    e = np.where(visible, np.exp(np.where(visible, scores, 0.0)), 0.0)
    return e / (1.0 + e.sum(-1, keepdims=True))


def softmax(scores, visible):
    s = np.where(visible, scores, -np.inf)
    s = s - s.max(-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(-1, keepdims=True)


def causal(n):
    return np.arange(n)[None, :] <= np.arange(n)[:, None]


def same_chunk(n, size):
    i = np.arange(n)
    return (i[:, None] // size) == (i[None, :] // size)


def rotate_half(x, positions, base, dims):
    """x [n, ..., d]: dims i and i + dims/2 (i < dims/2) turn by positions * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    a = positions[:, None] * f[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return np.concatenate([u * c - v * s, v * c + u * s, rest], axis=-1)


def softcap(s, cap):
    return cap * np.tanh(s / cap)


def scored_attention(h, W, p, m):
    """The mixer 'attention'."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(n, H, d)
    k = (h @ W[p + "k"].T).reshape(n, G, d)
    v = (h @ W[p + "v"].T).reshape(n, G, dv)
    positions = np.arange(n, dtype=np.float64)
    if m.get("q_temp") is not None:
        q = q * query_temperature(positions, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    out = np.zeros((n, H, dv))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"] - distance_bias(W[p + "r1"][head], W[p + "r2"][head], n)
        out[:, head] = softmax_with_zero_sink(s, causal(n)) @ v[:, g]
    return out.reshape(n, H * dv) @ W[p + "o"].T


def differential_lambda(W, p, diff):
    return (math.exp(float(np.sum(W[p + "lq1"] * W[p + "lk1"]))) - math.exp(float(np.sum(W[p + "lq2"] * W[p + "lk2"])))
            + diff)


def differential_attention(h, W, p, m, eps):
    """The mixer 'attention_2'."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(n, H, 2, d)
    k = (h @ W[p + "k"].T).reshape(n, G, 2, d)
    v = (h @ W[p + "v"].T).reshape(n, G, dv)
    q = rms_unit(q, eps) * W[p + "q.norm"]
    k = rms_unit(k, eps) * W[p + "k.norm"]
    positions = np.arange(n, dtype=np.float64)
    if m.get("rot") is not None:
        q = rotate_half(q, positions, m["rot"]["base"], m["rot"]["dims"])
        k = rotate_half(k, positions, m["rot"]["base"], m["rot"]["dims"])
    visible = causal(n)
    if m.get("mask") is not None:
        visible = visible & same_chunk(n, m["mask"]["size"])
    lam = differential_lambda(W, p, m["diff"])
    out = np.zeros((n, H, dv))
    for head in range(H):
        g = head // (H // G)
        maps = []
        for which in range(2):
            s = (q[:, head, which] @ k[:, g, which].T) * m["scale"]
            if m.get("softcap") is not None:
                s = softcap(s, m["softcap"])
            maps.append(softmax(s, visible) @ v[:, g])
        out[:, head] = rms_unit(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    gate = sigmoid(h @ W[p + "g"].T)
    return (out.reshape(n, H * dv) * gate) @ W[p + "o"].T


def feed_forward(h, W, p, f):
    g = h @ W[p + "gate"].T + W[p + "gate.b"]
    u = h @ W[p + "up"].T + W[p + "up.b"]
    if f.get("limit") is not None:
        g = np.minimum(g, f["limit"])
        u = np.clip(u, -f["limit"], f["limit"])
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T + W[p + "down.b"]


def run_order(cfg) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    return (list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"]
            + list(range(loop["stop"], n)))


def forward(cfg: Dict[str, Any], W: Dict[str, np.ndarray], tokens, collect: Optional[list] = None) -> np.ndarray:
    """Logits [tokens, vocab]; ``collect`` receives the stream after every layer run."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    for index in run_order(cfg):
        layer = cfg["layers"][index]
        p = f"l{index}."
        h = token_shift(norm_around_zero(x, W[p + "norm1"], eps), W[p + "shift"])
        if layer["type"] == "attention":
            y = scored_attention(h, W, p + "mix.", layer["mixer"])
        else:
            y = differential_attention(h, W, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + feed_forward(norm_around_zero(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
        x = x + y
        if collect is not None:
            collect.append(x.copy())
    return norm_around_zero(x, W["final.norm"], eps) @ W["head"].T
