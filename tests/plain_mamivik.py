"""A plain, slow Mamivik in float64 numpy: one function per mechanism, dense masks, an explicit
loop over tokens for the recurrence, keys and values expanded per head, no cache.  It shares no
code with the engine; the tests hold the engine against it.

``tensors`` maps checkpoint names to float arrays, ``cfg`` is the dict of a config.json.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def causal_conv(h, w):
    """h [T, E], w [E, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    T, E = h.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, E)), h])
    out = np.zeros_like(h)
    for j in range(taps):
        out += padded[j : j + T] * w[:, j]
    return out


def frequencies(rot):
    """Angle per position of every pair, and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    magnitude = 1.0
    s = rot.get("scaling")
    if s:
        def turn(t):
            return dims * math.log(s["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turn(s["fast"])), 0)
        hi = min(math.ceil(turn(s["slow"])), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / s["factor"] * ramp + f * (1.0 - ramp)
        magnitude = 0.1 * math.log(s["factor"]) + 1.0
    return f, magnitude


def rotate_halves(x, rot, positions):
    """x [T, heads, D]: dim i of the first rot.dims turns with dim i + dims / 2."""
    dims = int(rot["dims"])
    half = dims // 2
    f, magnitude = frequencies(rot)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return np.concatenate([u * c - v * s, v * c + u * s, x[..., dims:]], axis=-1)


def window_mask(T, size):
    d = np.arange(T)[:, None] - np.arange(T)[None, :]
    return (d >= 0) & (d < size)


def attend(scores, mask, values, sink=None):
    """scores [H, T, T], values [H, T, dv]; with a sink exp(sink_h) joins every denominator."""
    scores = np.where(mask[None], scores, -np.inf)
    top = scores.max(-1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink[:, None, None])
    e = np.exp(scores - top)
    den = e.sum(-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink[:, None, None] - top)
    return (e / den) @ values


def latent_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    cq = rms_unit(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(T, H, D + R)
    down = h @ W[p + "dkv"].T
    c = rms_unit(down[:, :rank], eps) * W[p + "dkv.norm"]
    k_rot = rotate_halves(down[:, rank:].reshape(T, 1, R), m["rot"], pos)[:, 0]
    q_rot = rotate_halves(q[..., D:], m["rot"], pos)
    k = (c @ W[p + "uk"].T).reshape(T, H, D)
    v = (c @ W[p + "uv"].T).reshape(T, H, Dv)
    scores = (np.einsum("thd,shd->hts", q[..., :D], k) + np.einsum("thd,sd->hts", q_rot, k_rot)) * m["scale"]
    o = attend(scores, window_mask(T, m["mask"]["size"]), v.transpose(1, 0, 2), W[p + "sink"])
    o = o.transpose(1, 0, 2).reshape(T, H * Dv) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def key_value_attention(h, W, p, m):
    """Grouped heads over a window; the values are the keys before the rotation."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = np.arange(T)
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, D)
    v = k
    q, k = rotate_halves(q, m["rot"], pos), rotate_halves(k, m["rot"], pos)
    k = np.repeat(k, H // G, axis=1)
    v = np.repeat(v, H // G, axis=1)
    scores = np.einsum("thd,shd->hts", q, k) * m["scale"]
    o = attend(scores, window_mask(T, m["mask"]["size"]), v.transpose(1, 0, 2))
    return o.transpose(1, 0, 2).reshape(T, H * D) @ W[p + "o"].T


def delta_rule_states(r, k, v, w, a, S=None):
    """One head: r, k, w, a [T, Dk], v [T, Dv].  Returns (outputs [T, Dv], last state [Dk, Dv])."""
    T, Dk = k.shape
    S = np.zeros((Dk, v.shape[1])) if S is None else S.copy()
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        u = k[t] / math.sqrt(float(np.sum(k[t] * k[t])) + 1e-6)
        S = w[t][:, None] * S - np.outer(a[t] * u, u @ S) + np.outer(k[t], v[t])
        out[t] = S.T @ r[t]
    return out, S


def delta_rule(h, W, p, m, eps):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ W[p + "r"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, D)
    w = np.exp(-math.exp(-0.5) * sigmoid(np.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, H, D)
    a = sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).reshape(T, H, D)
    o = np.stack([delta_rule_states(r[:, i], k[:, i], v[:, i], w[:, i], a[:, i])[0] for i in range(H)], axis=1)
    o = rms_unit(o, eps).reshape(T, H * D) * W[p + "norm"] * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def feed_forward(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def mixer_input(x, W, layer, eps):
    h = rms_unit(x, eps) * W[layer + "norm1"]
    return h + causal_conv(h, W[layer + "canon1"])


def forward(cfg, W, tokens, collect=None):
    """Logits [T, vocab] of one sequence; ``collect`` (a list) gets the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    for index, layer in enumerate(cfg["layers"]):
        L = f"l{index}."
        h = mixer_input(x, W, L, eps)
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            x = x + latent_attention(h, W, L + "mix.", m, eps)
        elif layer["type"] == "parallel":
            x = x + (m["left_scale"] * key_value_attention(h, W, L + "mix.left.", m["left"])
                     + m["right_scale"] * delta_rule(h, W, L + "mix.right.", m["right"], eps))
        else:
            raise ValueError(layer["type"])
        if layer["mlp"] is not None:
            x = x + feed_forward(rms_unit(x, eps) * W[L + "norm2"], W, L + "mlp.")
        if collect is not None:
            collect.append(x.copy())
    return (rms_unit(x, eps) * W["final.norm"]) @ W["head"].T
