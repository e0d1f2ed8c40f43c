"""``Mamivik`` as a model spec.

Pre-norm layers over the float32 stream x, every norm an RMS norm times one number:

    h = norm1(x);   h_t <- h_t + sum_j canon[:, j] * h_(t - taps + 1 + j);   x <- x + mixer(h)
    x <- x + feed_forward(norm2(x))                                   (a layer may have none)

with one of two mixers, listed layer by layer:

* ``latent_attention``: per token the layer caches a normed latent and one rotated key part that
  all heads share; the queries come through a normed latent of their own; the rotated parts turn
  in halves (dim i with dim i + dims / 2) with the slow pairs stretched; a query sees a window of
  keys; a learned number per head joins the softmax denominator; the heads' outputs pass
  ``sigmoid(W_g h)`` element by element.
* ``parallel``: ``left_scale * left + right_scale * right`` of two mixers on the same h.  Left:
  grouped heads over a window, biases on q and k, the first dims of every head rotated in halves,
  and no value projection: a token's values are its keys before the rotation.  Right: the
  generalized delta rule (``parts.recurrent.DeltaRule``).

The feed-forward is ``W_down (gelu_tanh(W_gate h) * (W_up h))``.  After the last layer: the same
kind of norm and the head.

This module only maps configuration keys to part parameters and checkpoint names to part
weights.  It has no forward pass.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

from ..config.model_config import (DeltaRuleConfig, GatedFeedForwardConfig, MamivikConfig, ModelConfig,
                                   WindowAttentionConfig, WindowedLatentConfig)
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSource, WeightSpec

ARCHITECTURE = "Mamivik"

# Constants of the design.  The decay of the delta rule is exp(-exp(-1/2) * sigmoid(.)); its unit
# key has 1e-6 under the root.  The gate's activation is the tanh form of GELU, written as
# g * sigmoid(alpha * (g + cubic * g^3)) with alpha = 2 sqrt(2 / pi).
DECAY_SCALE = math.exp(-0.5)
KEY_EPS = 1e-6
GELU_ALPHA = 2.0 * math.sqrt(2.0 / math.pi)
GELU_CUBIC = 0.044715


def _matrix(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="matrix")


def _vector(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="vector")


def _rms(name: str, size: int, eps: float) -> PartSpec:
    """An RMS norm whose weight is one number."""
    return PartSpec(kind="rms", params={"size": size, "eps": eps, "scalar_weight": True},
                    weights={"weight": _vector(TensorSource(name, (), init="one_plus_normal"))})


def _ceil16(n: int) -> int:
    return -(-n // 16) * 16


def _scaling(rot) -> Optional[Dict[str, float]]:
    return None if rot[2] is None else dict(zip(("factor", "original", "fast", "slow"), rot[2]))


def _latent(prefix: str, a: WindowedLatentConfig, width: int, eps: float) -> PartSpec:
    params = {
        "hidden_size": width, "num_heads": a.heads, "dim": a.dim, "rot_dim": a.rot_dim, "value_dim": a.vdim,
        "kv_rank": a.kv_rank, "query_rank": a.q_rank, "softmax_scale": a.scale, "eps": eps, "window": a.window,
        "sink": True, "output_gate": True, "gate": "element",
    }
    q_head = a.dim + a.rot_dim
    weights = {
        "in.weight": _matrix(TensorSource(prefix + "dq", (a.q_rank, width)),
                             TensorSource(prefix + "dkv", (a.kv_rank + a.rot_dim, width)),
                             TensorSource(prefix + "g", (a.heads * a.vdim, width))),
        "query_norm.weight": _vector(TensorSource(prefix + "dq.norm", (a.q_rank,), init="one_plus_normal")),
        "uq.weight": _matrix(TensorSource(prefix + "uq", (a.heads * q_head, a.q_rank))),
        "latent_norm.weight": _vector(TensorSource(prefix + "dkv.norm", (a.kv_rank,), init="one_plus_normal")),
        "uk.weight": _matrix(TensorSource(prefix + "uk", (a.heads * a.dim, a.kv_rank))),
        "uv.weight": _matrix(TensorSource(prefix + "uv", (a.heads * a.vdim, a.kv_rank))),
        "sink": _vector(TensorSource(prefix + "sink", (a.heads,), init="normal_wide")),
        "out.weight": _matrix(TensorSource(prefix + "o", (width, a.heads * a.vdim))),
    }
    return PartSpec(kind="latent_attention", params=params, weights=weights)


def left_head_dim(a: WindowAttentionConfig) -> int:
    """The head size the attention kernels run for the left mixer of a ``parallel`` layer."""
    return _ceil16(max(a.dim, a.vdim))


def _left(a: WindowAttentionConfig, width: int) -> Dict:
    return {"kind": "attention", "params": {
        "hidden_size": width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": left_head_dim(a),
        "key_dim": a.dim, "value_dim": a.vdim, "window": a.window, "softmax_scale": a.scale, "qkv_bias": True,
        "values_from_keys": True,
    }}


def _right(d: DeltaRuleConfig, width: int, eps: float, rank: int) -> Dict:
    return {"kind": "delta_rule", "params": {
        "hidden_size": width, "heads": d.heads, "dim": d.dim, "eps": eps, "decay_scale": DECAY_SCALE,
        "key_eps": KEY_EPS, "decay_rank": rank,
    }}


def _parallel(prefix: str, layer, width: int, eps: float, rank: int) -> PartSpec:
    a, d = layer.left, layer.right
    inner = d.heads * d.dim
    lp, rp = prefix + "left.", prefix + "right."
    weights = {
        "left.q.weight": _matrix(TensorSource(lp + "q", (a.heads * a.dim, width))),
        "left.q.bias": _vector(TensorSource(lp + "q.b", (a.heads * a.dim,))),
        "left.k.weight": _matrix(TensorSource(lp + "k", (a.kv_heads * a.dim, width))),
        "left.k.bias": _vector(TensorSource(lp + "k.b", (a.kv_heads * a.dim,))),
        "left.out.weight": _matrix(TensorSource(lp + "o", (width, a.heads * a.vdim))),
        "right.in.weight": _matrix(*(TensorSource(rp + name, (inner, width)) for name in ("r", "k", "v", "g", "a")),
                                   TensorSource(rp + "w1", (rank, width))),
        "right.decay_up.weight": _matrix(TensorSource(rp + "w2", (inner, rank), init="normal_wide")),
        "right.decay_bias": _vector(TensorSource(rp + "w0", (inner,), init="normal_wide")),
        "right.removal_bias": _vector(TensorSource(rp + "a.b", (inner,), init="normal_wide")),
        "right.norm.weight": _vector(TensorSource(rp + "norm", (inner,), init="one_plus_normal")),
        "right.out.weight": _matrix(TensorSource(rp + "o", (width, inner))),
    }
    params = {"hidden_size": width, "join": "weighted_sum", "left_scale": layer.left_scale,
              "right_scale": layer.right_scale, "left": _left(a, width), "right": _right(d, width, eps, rank)}
    return PartSpec(kind="side_by_side", params=params, weights=weights)


def _feed_forward(prefix: str, f: GatedFeedForwardConfig, width: int) -> PartSpec:
    return PartSpec(
        kind="clamped_glu",
        params={"hidden_size": width, "intermediate_size": f.ff, "limit": 0.0, "alpha": GELU_ALPHA,
                "cubic": GELU_CUBIC, "up_shift": 0.0, "biases": False},
        weights={
            "gate_up.weight": _matrix(TensorSource(prefix + "gate", (f.ff, width)),
                                      TensorSource(prefix + "up", (f.ff, width))),
            "down.weight": _matrix(TensorSource(prefix + "down", (width, f.ff))),
        },
    )


def build_mamivik_spec(config: ModelConfig, decay_ranks: Optional[Dict[int, int]] = None) -> ModelSpec:
    """``decay_ranks``: per ``parallel`` layer, the inner size of the decay's two small matrices.  No
    configuration key names it: a checkpoint's tensor shapes do (``checkpoint_sizes``, which the
    loader of a model folder calls); without a checkpoint it is ``default_decay_rank``."""
    if not isinstance(config, MamivikConfig):
        raise TypeError(f"expected a MamivikConfig, got {type(config).__name__}")
    c = config
    E, V = c.hidden_size, c.vocab_size
    positions: Dict[tuple, PartSpec] = {}

    def position(key: tuple, make) -> PartSpec:
        if key not in positions:
            positions[key] = make()
        return positions[key]

    layers = []
    for index, layer in enumerate(c.layers):
        p = f"l{index}.mix."
        if layer.type == "latent_attention":
            a = layer.latent
            mixer = _latent(p, a, E, c.norm_eps)
            base, dims, _ = a.rot
            pos = position(("latent", a.rot, a.rot_dim), lambda: PartSpec(
                kind="rotary_half",
                params={"head_dim": a.rot_dim, "rotary_dim": dims, "theta": base, "scaling": _scaling(a.rot),
                        "max_position": c.max_position_embeddings, "angles": "float64"}))
        else:
            a = layer.left
            rank = (decay_ranks or {}).get(index, default_decay_rank(layer.right))
            mixer = _parallel(p, layer, E, c.norm_eps, rank)
            base, dims, _ = a.rot
            D = left_head_dim(a)
            pos = position(("left", a.rot, D), lambda: PartSpec(
                kind="rotary_half",
                params={"head_dim": D, "rotary_dim": dims, "theta": base, "scaling": _scaling(a.rot),
                        "max_position": c.max_position_embeddings, "angles": "float64"}))
        feed_forward = None if layer.mlp is None else _feed_forward(f"l{index}.mlp.", layer.mlp, E)
        norms = {"mixer": _rms(f"l{index}.norm1", E, c.norm_eps)}
        if feed_forward is not None:
            norms["feed_forward"] = _rms(f"l{index}.norm2", E, c.norm_eps)
        layers.append(LayerSpec(
            block="pre_norm", mixer=mixer, feed_forward=feed_forward, norms=norms, position=pos,
            block_params={"input_conv": True},
            block_weights={"conv": _vector(TensorSource(f"l{index}.canon1", (E, c.canon_taps), init="normal_wide"))}))
    spec = ModelSpec(
        architecture=c.architecture,
        hidden_size=E,
        vocab_size=V,
        max_position=c.max_position_embeddings,
        embedding=PartSpec(kind="token_embedding", params={"vocab_size": V, "hidden_size": E},
                           weights={"weight": _matrix(TensorSource("embed", (V, E)))}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
        final_norm=_rms("final.norm", E, c.norm_eps),
        lm_head=PartSpec(kind="linear_head", params={"hidden_size": E, "vocab_size": V},
                         weights={"weight": _matrix(TensorSource("head", (V, E)))}),
        eos_token_ids=tuple(c.eos_token_ids),
        # A layer without feed-forward has no use for a second norm; a file may still carry one.
        ignored_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(c.layers) if layer.mlp is None),
    )
    spec.validate()
    return spec


def default_decay_rank(d: DeltaRuleConfig) -> int:
    """The inner size of the decay's small matrices where no checkpoint gives it."""
    return max(8, (d.heads * d.dim) // 8 // 8 * 8)


def checkpoint_sizes(config: ModelConfig, shape_of) -> Dict[str, Dict[int, int]]:
    """Sizes that only the checkpoint gives, as keyword arguments for ``build_mamivik_spec``:
    ``shape_of(name)`` returns a tensor's shape or None."""
    ranks: Dict[int, int] = {}
    for index, layer in enumerate(config.layers):
        if layer.type == "parallel":
            shape = shape_of(f"l{index}.mix.right.w1")
            if shape is not None and len(shape) == 2:
                ranks[index] = int(shape[0])
    return {"decay_ranks": ranks}


register_architecture(ARCHITECTURE, MamivikConfig.from_dict, build_mamivik_spec, checkpoint_sizes)
