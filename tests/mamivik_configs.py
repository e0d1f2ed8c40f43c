"""Small Mamivik configurations and weights for the tests.

The configurations differ in every size and make sizes differ that a model may happen to make
equal or 1: heads and KV heads of the left mixer (1, 2, 3, 4 heads per KV head), head sizes that
are no multiples of 16, rotation of some or all dims of a head, with and without stretched slow
pairs, windows of one key, of a few, of more than a page, longer than any prompt, latents and
ranks that are no multiples of eight, one head, a convolution of 1, 2, 3, 4 and 5 taps, layers
without feed-forward, widths that are no multiples of eight, every order of the two kinds of
layer, scales of the two sides that differ from 1 and from each other.  ``make_weights`` draws
weights at a scale at which every mechanism does something: a unit-variance stream, taps that
reorder what a token reads, sinks that take a good share of the weight, decays and removal rates
away from their ends.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch


def rot(base, dims, scaling=None) -> Dict[str, Any]:
    out: Dict[str, Any] = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, window, base, scaling=None, dims=None) -> Dict[str, Any]:
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "scale": scale, "mask": {"size": window}, "rot": rot(base, rot_dim if dims is None else dims, scaling)}


def left(heads, kv_heads, dim, scale, window, base, dims, scaling=None) -> Dict[str, Any]:
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": window},
            "rot": rot(base, dims, scaling)}


def parallel(left_mixer, heads, dim, left_scale, right_scale) -> Dict[str, Any]:
    return {"left": left_mixer, "right": {"heads": heads, "dim": dim}, "left_scale": left_scale,
            "right_scale": right_scale}


def dense(ff) -> Dict[str, Any]:
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp) -> Dict[str, Any]:
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, taps, layers, eps=1e-5) -> Dict[str, Any]:
    return {"architecture": "Mamivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "layers": layers}


# Both kinds of layer; a window shorter than a page of 16 and no multiple of a page of 4; two heads
# per KV head; a layer without feed-forward; stretched slow pairs in the latent layer.
SMALL = config(64, 120, 3, [
    layer("parallel", parallel(left(4, 2, 16, 0.3, 10, 100.0, 8), 2, 16, 1.3, 0.7), dense(40)),
    layer("latent_attention", latent(3, 16, 8, 24, 32, 24, 0.25, 7, 1000.0, (4.0, 16, 8.0, 1.0)), None),
    layer("parallel", parallel(left(2, 1, 8, 0.35, 33, 50.0, 8), 4, 8, 0.6, 1.1), dense(24)),
], eps=1e-6)

# Sizes of one and widths that are no multiples of eight: one head, no grouping, a window of one
# key, two taps, ranks that need padding, a decay rank that is no multiple of eight, latent layers
# next to each other, a window longer than any prompt.
ODD = config(100, 331, 2, [
    layer("latent_attention", latent(1, 20, 4, 12, 28, 10, 0.3, 1, 50.0), dense(52)),
    layer("latent_attention", latent(5, 12, 12, 20, 20, 36, 0.3, 1000, 10000.0, (8.0, 32, 4.0, 0.5)), dense(17)),
    layer("parallel", parallel(left(3, 3, 12, 0.3, 1, 5000.0, 12), 1, 24, 1.0, 2.0), None),
    layer("parallel", parallel(left(6, 2, 20, 0.25, 5, 20.0, 4, (3.0, 20, 2.0, 0.25)), 3, 12, 0.4, 0.4), dense(36)),
], eps=1e-5)

# Sizes near a real model's: heads of 64 and 128 for the tensor-memory attention kernels, a latent
# row of 160 and one of 256, state heads of 64, windows across pages and key tiles, five taps.
WIDE = config(256, 500, 5, [
    layer("latent_attention", latent(6, 64, 32, 48, 128, 72, 0.1, 150, 10000.0, (4.0, 256, 16.0, 1.0)), dense(384)),
    layer("parallel", parallel(left(6, 3, 64, 0.125, 200, 100000.0, 32), 2, 64, 1.4, 0.8), dense(256)),
    layer("parallel", parallel(left(4, 1, 128, 0.09, 64, 500000.0, 64), 3, 32, 0.8, 1.1), None),
    layer("latent_attention", latent(4, 32, 64, 48, 192, 96, 0.12, 65, 500.0), dense(128)),
], eps=2e-5)

# Head sizes between the common ones, one tap (no convolution state); three heads per KV head; a
# state head of 48; both mixers' windows are equal, so they share a cache group; only 16 of the latent
# layer's 24 rotated dims turn.
MID = config(192, 700, 1, [
    layer("parallel", parallel(left(6, 2, 72, 0.12, 100, 300000.0, 24), 2, 48, 1.5, 0.5), dense(320)),
    layer("latent_attention", latent(6, 40, 24, 56, 88, 64, 0.13, 100, 20000.0, dims=16), dense(200)),
], eps=1e-6)

# Four taps with prompts shorter than the taps; only parallel layers.
TAPS = config(48, 90, 4, [
    layer("parallel", parallel(left(2, 2, 16, 0.3, 12, 100.0, 16), 2, 8, 1.0, 1.0), dense(32)),
    layer("parallel", parallel(left(4, 1, 8, 0.4, 3, 100.0, 2), 1, 16, 1.1, 0.9), None),
], eps=1e-5)

# Latents wider than the attention kernels' widest cached row: these layers run with keys and
# values expanded per head.  One of them stretches its slow pairs, one has a value size above its
# query size.
BROAD = config(72, 150, 3, [
    layer("latent_attention", latent(2, 16, 8, 24, 264, 20, 0.2, 11, 300.0, (2.0, 32, 8.0, 1.0)), dense(48)),
    layer("parallel", parallel(left(2, 1, 16, 0.3, 20, 100.0, 8), 1, 16, 1.0, 1.0), None),
    layer("latent_attention", latent(3, 8, 16, 40, 300, 44, 0.25, 1000, 5000.0), dense(40)),
], eps=1e-5)

# More query heads on one cached row or KV head than an attention tile has rows: a token's heads are
# cut across tiles, in the layer whose rows the sink's merge finishes and in the one beside the
# delta rule.
MANY = config(80, 200, 2, [
    layer("latent_attention", latent(20, 8, 8, 8, 24, 16, 0.3, 30, 100.0), dense(64)),
    layer("parallel", parallel(left(18, 1, 16, 0.25, 25, 1000.0, 8), 2, 8, 1.0, 0.7), None),
    layer("latent_attention", latent(17, 16, 4, 12, 40, 24, 0.25, 1000, 100.0, (2.0, 16, 4.0, 1.0)), dense(40)),
], eps=1e-5)

ALL = {"small": SMALL, "odd": ODD, "wide": WIDE, "mid": MID, "taps": TAPS, "broad": BROAD, "many": MANY}

# The inner size of the decay's two small matrices is a tensor shape, not a configuration key.
DECAY_RANKS = {"small": 8, "odd": 5, "wide": 16, "mid": 24, "taps": 3, "broad": 8, "many": 4}


def build_spec(cfg: Dict[str, Any], decay_rank: Optional[int] = None):
    from velox_b200.config.registry import architecture_of

    arch = architecture_of(cfg)
    typed = arch.parse_config(cfg)
    ranks = None
    if decay_rank is not None:
        ranks = {i: decay_rank for i, l in enumerate(cfg["layers"]) if l["type"] == "parallel"}
    return arch.build_spec(typed, decay_ranks=ranks)


def make_weights(cfg: Dict[str, Any], seed: int, sharp: float = 1.0, decay_rank: Optional[int] = None
                 ) -> Dict[str, torch.Tensor]:
    """Tensors under the checkpoint's names, bfloat16.  ``sharp`` scales the query projections:
    at 3 or more the softmax puts most of its weight on a few keys."""
    spec = build_spec(cfg, decay_rank)
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, source in sorted(spec.checkpoint_tensors().items()):
        shape = tuple(source.shape)
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = torch.randn(shape, generator=gen)
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif name.endswith((".dq.norm", ".dkv.norm", ".right.norm")):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif last == "canon1":
            t = 0.5 * torch.randn(shape, generator=gen)
        elif last == "sink":
            t = 1.5 * torch.randn(shape, generator=gen)
        elif last in ("w0", "b") and ".right." in name:
            t = 1.5 * torch.randn(shape, generator=gen)
        elif last == "w2":
            t = 2.0 * torch.randn(shape, generator=gen) / shape[-1] ** 0.5
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / shape[-1] ** 0.5
            if last in ("q", "uq"):
                t = t * sharp
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(folder: str, cfg: Dict[str, Any], tensors: Dict[str, torch.Tensor]) -> None:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(cfg, handle)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))


def as_numpy(tensors: Dict[str, torch.Tensor]):
    return {k: v.double().numpy() for k, v in tensors.items()}
