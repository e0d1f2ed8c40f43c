"""Position encodings applied to q and k inside an attention mixer.

``rotary_half`` is the reference's RoPE: float32 tables ``angle[p, i] = (p / factor) *
theta^(-2i/R)`` (src/rope.py:45-56) and the rotate-half form ``lo' = lo*cos - hi*sin``,
``hi' = lo*sin + hi*cos`` on the two halves of the first R dims of every head
(src/rope_inplace.py:25-47).  ``none`` rotates nothing.  Both write k and v into the paged
cache in the same kernel that rotates.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .base import PositionEncoding
from .registry import register_part


def stretch_slow_pairs(inv_freq: torch.Tensor, rotary_dim: int, base: float, scaling) -> tuple:
    """YaRN: ``scaling`` = {factor, original, fast, slow}.  With ``turn(t) = rotary_dim *
    ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(turn(fast)), 0)``, ``hi =
    min(ceil(turn(slow)), rotary_dim - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001),
    0, 1)``, pair i turns by ``f_i / factor * ramp_i + f_i * (1 - ramp_i)`` per position, and cos and
    sin are multiplied by ``0.1 ln(factor) + 1``.  Returns (frequencies, that magnitude)."""
    import math

    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), rotary_dim - 1)
    index = torch.arange(inv_freq.numel(), dtype=torch.float64)
    ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    inv_freq = inv_freq.to(torch.float64)
    return inv_freq / factor * ramp + inv_freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


@register_part("position", "rotary_half")
class RotaryHalf(PositionEncoding):
    """``scaling`` = {factor, original, fast, slow} stretches the slow pairs (``stretch_slow_pairs``;
    the angles are then formed in float64).  ``layout`` tells a mixer that rotates with its own
    kernel which dims are a pair: dim i with dim i + rotary_dim / 2."""

    layout = "half"

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.scaling_factor = float(params.get("scaling_factor", 1.0))
        self.max_position = int(params["max_position"])
        if self.rotary_dim % 2 != 0 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(
                f"rotary_dim={self.rotary_dim} must be even and within head_dim={self.head_dim}"
            )
        # ``angles``: "float32" forms position * frequency in float32 (the reference's tables);
        # "float64" forms it in float64 and rounds the cosine and sine once.
        scaling = params.get("scaling")
        precise = params.get("angles", "float32") == "float64" or bool(scaling)
        work = torch.float64 if precise else torch.float32
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=work) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponent)
        magnitude = 1.0
        if scaling:
            inv_freq, magnitude = stretch_slow_pairs(inv_freq, self.rotary_dim, self.theta, scaling)
        positions = torch.arange(self.max_position, dtype=work)
        if self.scaling_factor != 1.0:
            positions = positions / self.scaling_factor
        angles = torch.outer(positions, inv_freq)
        cos, sin = angles.cos(), angles.sin()
        if magnitude != 1.0:
            cos, sin = cos * magnitude, sin * magnitude
        self.pairs = self.rotary_dim // 2
        self.cos = cos.to(torch.float32).to(device).contiguous()
        self.sin = sin.to(torch.float32).to(device).contiguous()

    def rotate_and_store(self, qkv, ctx, slots, k_cache, v_cache, num_heads, num_kv_heads, values_from_keys=False):
        """``values_from_keys``: the rows hold q | k; the values written to the cache are the keys
        before the rotation."""
        kernels.rope_cache_write(
            qkv, ctx.positions, self.cos, self.sin, slots, k_cache, v_cache, ctx.num_tokens,
            num_heads, num_kv_heads, self.head_dim, self.rotary_dim, ctx.status, values_from_keys=values_from_keys,
        )

    def full_rotation_tables(self):
        """(cos, sin) [max_position, head_dim / 2] when every dim of a head rotates, which is
        what a projection that rotates in its epilogue needs; else None."""
        return (self.cos, self.sin) if self.rotary_dim == self.head_dim else None


@register_part("position", "none")
class NoPosition(PositionEncoding):
    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.head_dim = int(params["head_dim"])

    def rotate_and_store(self, qkv, ctx, slots, k_cache, v_cache, num_heads, num_kv_heads):
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * self.head_dim:
            # The projection's rows hold more than q | k | v: the kernel that takes a row pitch.
            kernels.pair_rope_cache_write(qkv, ctx.positions, None, None, slots, k_cache, v_cache, ctx.num_tokens,
                                          num_heads, num_kv_heads, self.head_dim, 0, ctx.status)
            return
        kernels.rope_cache_write(
            qkv, ctx.positions, None, None, slots, k_cache, v_cache, ctx.num_tokens,
            num_heads, num_kv_heads, self.head_dim, 0, ctx.status,
        )


@register_part("position", "log_temperature")
class LogTemperature(NoPosition):
    """No rotation; instead the scores of the query at position p are multiplied by
    ``1 + coef * ln(floor((p + 1) / every) + 1)``.  The part owns the float32 table ``row_scale``
    [max_position] (formed in float64, rounded once), which the attention kernels apply to a
    row's scores; q itself is left as the projection made it."""

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.coef = float(params["coef"])
        self.every = int(params["every"])
        self.max_position = int(params["max_position"])
        if self.every < 1:
            raise ValueError(f"log_temperature: every={self.every} must be at least 1")
        p = torch.arange(self.max_position, dtype=torch.float64)
        table = 1.0 + self.coef * torch.log(torch.floor((p + 1.0) / self.every) + 1.0)
        self.row_scale = table.to(torch.float32).to(device).contiguous()


@register_part("position", "rotary_interleaved")
class RotaryInterleaved(PositionEncoding):
    """Rotation of neighbouring pairs: dims ``2i`` and ``2i + 1`` of the first ``rotary_dim`` dims
    of a vector are a pair ``(u, v) -> (u cos a - v sin a, v cos a + u sin a)`` with ``a =
    position * base^(-2i / rotary_dim)``; the other dims pass.  The part owns the float32 tables
    ``cos``/``sin`` [max_position, rotary_dim / 2] (angles formed in float64, rounded once); the
    mixer that applies it passes them to its kernel, or calls ``rotate_and_store`` (``head_dim``
    given), which rotates q in place and k on its way into the paged cache.

    ``scaling`` = {factor, original, fast, slow} stretches the slow pairs (YaRN): with
    ``turn(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(turn(fast)),
    0)``, ``hi = min(ceil(turn(slow)), rotary_dim - 1)`` and ``ramp_i = clamp((i - lo) / max(hi -
    lo, 0.001), 0, 1)``, pair i turns by ``f_i / factor * ramp_i + f_i * (1 - ramp_i)`` per
    position, and cos and sin are multiplied by ``0.1 ln(factor) + 1``."""

    layout = "pairs"

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.rotary_dim = int(params["rotary_dim"])
        self.base = float(params["base"])
        self.max_position = int(params["max_position"])
        if self.rotary_dim % 2 != 0 or self.rotary_dim < 0:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even")
        pairs = self.rotary_dim // 2
        exponent = torch.arange(pairs, dtype=torch.float64) * (2.0 / max(self.rotary_dim, 1))
        inv_freq = torch.pow(torch.tensor(self.base, dtype=torch.float64), -exponent)
        self.head_dim = int(params["head_dim"]) if params.get("head_dim") else None
        magnitude = 1.0
        scaling = params.get("scaling")
        if scaling:
            inv_freq, magnitude = stretch_slow_pairs(inv_freq, self.rotary_dim, self.base, scaling)
        angles = torch.outer(torch.arange(self.max_position, dtype=torch.float64), inv_freq)
        width = max(pairs, 1)
        cos = torch.ones((self.max_position, width), dtype=torch.float32)
        sin = torch.zeros((self.max_position, width), dtype=torch.float32)
        cos[:, :pairs] = (angles.cos() * magnitude).to(torch.float32)
        sin[:, :pairs] = (angles.sin() * magnitude).to(torch.float32)
        self.pairs = pairs
        self.cos = cos.to(device).contiguous()
        self.sin = sin.to(device).contiguous()

    def rotate_and_store(self, qkv, ctx, slots, k_cache, v_cache, num_heads, num_kv_heads):
        if self.head_dim is None:
            raise ValueError("rotary_interleaved needs head_dim to rotate heads of a q | k | v projection")
        kernels.pair_rope_cache_write(qkv, ctx.positions, self.cos, self.sin, slots, k_cache, v_cache,
                                      ctx.num_tokens, num_heads, num_kv_heads, self.head_dim,
                                      self.rotary_dim if self.pairs else 0, ctx.status)
