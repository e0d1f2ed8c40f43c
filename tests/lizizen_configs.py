"""Small Lizizen configurations and weights for the tests.

The configurations differ in every size and make sizes differ that a model may happen to make
equal or 1: query/key and value sizes of a head, heads per KV head (1, 2, 3, 4), rotation of some
or all dims of a map or none, a chunked mask of one key, of a few, of more than a page, or none,
capped scores or not, a query temperature that changes every position, every few, or none, a
feed-forward with and without clamps or none at all, a looped stretch at the start, in the middle,
run once, or none, widths that are no multiples of eight.  ``make_weights`` draws weights at a
scale at which every mechanism does something: a unit-variance stream, clamps that cut, shifts
between 0 and 0.8, distance slopes that reorder keys, lambdas away from the constant.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch


def scored(heads, kv_heads, dim, vdim, scale, q_temp=None) -> Dict[str, Any]:
    out: Dict[str, Any] = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp is not None:
        out["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return out


def differential(heads, kv_heads, dim, vdim, scale, diff, chunk=None, rot=None, softcap=None) -> Dict[str, Any]:
    out: Dict[str, Any] = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if chunk is not None:
        out["mask"] = {"size": chunk}
    if rot is not None:
        out["rot"] = {"base": rot[0], "dims": rot[1]}
    if softcap is not None:
        out["softcap"] = softcap
    return out


def dense(ff, limit=None) -> Dict[str, Any]:
    out: Dict[str, Any] = {"kind": "dense", "ff": ff}
    if limit is not None:
        out["limit"] = limit
    return out


def layer(kind, mixer, mlp) -> Dict[str, Any]:
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, layers, eps=1e-5, loop=None) -> Dict[str, Any]:
    out = {"architecture": "Lizizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# Both mixers; value size above and below the query/key size; three heads on one KV head; a
# layer without feed-forward; a loop over the first two layers; a chunk shorter than a page of 16
# and no multiple of a page of 4.
SMALL = config(64, 120, [
    layer("attention_2", differential(4, 2, 16, 24, 0.25, 0.3, chunk=10, rot=(100.0, 8), softcap=4.0), dense(40, 1.0)),
    layer("attention", scored(3, 1, 24, 8, 0.2, q_temp=(0.5, 4)), None),
    layer("attention_2", differential(2, 1, 8, 16, 0.35, 0.6), dense(24)),
], eps=1e-6, loop=(0, 2, 2))

# Sizes of one and widths that are no multiples of eight: no grouping of heads, a chunk of one
# key, rotation of all dims of a map, a temperature that changes at every position and a layer
# without one, a looped stretch that runs once, no clamps, one head.
ODD = config(100, 331, [
    layer("attention", scored(5, 5, 12, 20, 0.3), dense(52, 0.7)),
    layer("attention_2", differential(3, 3, 12, 20, 0.3, 0.2, chunk=1, rot=(50.0, 12)), dense(17, 2.0)),
    layer("attention_2", differential(1, 1, 20, 12, 0.2, 0.45, chunk=7, softcap=1.5), None),
    layer("attention", scored(4, 2, 8, 8, 0.4, q_temp=(1.0, 1)), dense(36)),
    layer("attention_2", differential(6, 2, 10, 6, 0.3, 0.8, chunk=33, rot=(10000.0, 4), softcap=30.0), dense(20, 1.2)),
], eps=1e-5, loop=(1, 3, 1))

# Heads of 64 and 128 (two maps of 128 fill the widest cached row), a chunk longer than a page
# and a key tile, a loop over the middle that runs three times.
WIDE = config(256, 500, [
    layer("attention", scored(8, 2, 64, 64, 0.125, q_temp=(0.2, 50)), dense(384, 1.5)),
    layer("attention_2", differential(4, 1, 128, 96, 0.09, 0.45, chunk=150, rot=(500000.0, 64), softcap=20.0),
          dense(256, 1.0)),
    layer("attention_2", differential(8, 4, 32, 64, 0.18, 0.35, chunk=64, rot=(500.0, 32)), None),
    layer("attention", scored(4, 4, 128, 32, 0.09), dense(128, 3.0)),
], eps=2e-5, loop=(1, 3, 3))

# Head sizes between the common ones (cached rows of 80 and 112), rotated dims whose half is no
# multiple of eight, a chunk that is no multiple of a page, three heads per KV head in both mixers,
# a loop over the last two layers.
MID = config(192, 700, [
    layer("attention_2", differential(6, 2, 56, 40, 0.13, 0.4, chunk=100, rot=(300000.0, 24), softcap=40.0), dense(320, 1.2)),
    layer("attention", scored(6, 2, 72, 72, 0.12, q_temp=(0.25, 64)), dense(200, 2.5)),
    layer("attention_2", differential(3, 1, 40, 80, 0.16, 0.6, chunk=90, rot=(20000.0, 20)), dense(144)),
], eps=1e-6, loop=(1, 3, 2))

ALL = {"small": SMALL, "odd": ODD, "wide": WIDE, "mid": MID}


def make_weights(cfg: Dict[str, Any], seed: int, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """Tensors under the checkpoint's names, bfloat16.  ``sharp`` scales the query projections:
    at 3 or more the softmax puts most of its weight on a few keys."""
    from velox_b200.config.registry import architecture_of

    arch = architecture_of(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, source in sorted(spec.checkpoint_tensors().items()):
        shape = tuple(source.shape)
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = torch.randn(shape, generator=gen)
        elif name.endswith(("q.norm", "k.norm")):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = 0.3 * torch.randn(shape, generator=gen)  # stored around zero
        elif last == "shift":
            t = 0.8 * torch.rand(shape, generator=gen)
        elif last == "r1":
            t = 2.0 * torch.rand(shape, generator=gen)
        elif last == "r2":
            t = 0.05 + 0.45 * torch.rand(shape, generator=gen)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.8 * torch.randn(shape, generator=gen) / shape[0] ** 0.25
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / shape[-1] ** 0.5
            if last == "q":
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
    return {k: v.float().numpy() for k, v in tensors.items()}
