"""``Lizizen`` as a model spec.

Every layer reads the float32 stream x through two RMS norms whose weights are stored around
zero (the factor is ``1 + w``):

    h = norm1(x);   h_t <- h_t + (h_(t-1) - h_t) * shift;   x <- x + mixer(h) + feed_forward(norm2(x))

(a layer may have no feed-forward), with one of two mixers, listed layer by layer:

* ``attention``: grouped heads over all keys, no rotation; the scores of the query at position
  p are multiplied by ``1 + coef ln(floor((p + 1) / every) + 1)``, ``r1_h ln(1 + r2_h (i - j))`` is
  taken off the score of query i and key j, and the softmax denominator has one more term of
  score 0 that carries no value.
* ``attention_2``: two maps per head over the same values (q and k hold both maps' rows head by
  head), RMS norm of q and k per head and map, rotation of the first dims of every map,
  ``cap tanh(score / cap)``, a mask of chunks counted from position 0, then
  ``o = a1 - lambda a2`` with ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff``, o scaled to
  unit RMS per head, times ``1 - diff``, times ``sigmoid(W_g h)``.

The feed-forward is ``W_down (g sigmoid(1.702 g) (u + 1))`` with ``g = min(W_gate h + b, limit)``
and ``u = clamp(W_up h + b, -limit, limit)``.  A stretch of layers may run several times in a
row with the same weights (``loop``): every run is a schedule entry with a cache and a shift
state of its own.  After the last layer: the same kind of norm and the head.

This module only maps configuration keys to part parameters and checkpoint names to part
weights.  It has no forward pass.
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config.model_config import (ClampedFeedForwardConfig, DifferentialAttentionConfig, LizizenConfig, ModelConfig,
                                   ScoredAttentionConfig)
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSource, WeightSpec

ARCHITECTURE = "Lizizen"

# Constants of the design: the gate's activation is g * sigmoid(1.702 g), the up branch is u + 1.
GATE_ALPHA = 1.702
UP_SHIFT = 1.0


def _matrix(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="matrix")


def _vector(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="vector")


def _rms(name: str, size: int, eps: float) -> PartSpec:
    """An RMS norm whose stored weight lies around zero."""
    return PartSpec(kind="rms", params={"size": size, "eps": eps, "weight_offset": 1.0},
                    weights={"weight": _vector(TensorSource(name, (size,)))})


def _ceil16(n: int) -> int:
    return -(-n // 16) * 16


def scored_head_dim(a: ScoredAttentionConfig) -> int:
    """The head size the attention kernels run for an ``attention`` layer."""
    return _ceil16(max(a.dim, a.vdim))


def differential_head_dim(a: DifferentialAttentionConfig) -> int:
    """The same for ``attention_2``: a cached key row holds both maps' keys side by side."""
    return _ceil16(max(2 * a.dim, a.vdim))


def _scored(prefix: str, a: ScoredAttentionConfig, width: int) -> PartSpec:
    params = {
        "hidden_size": width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": scored_head_dim(a),
        "key_dim": a.dim, "value_dim": a.vdim, "window": None, "softmax_scale": a.scale, "qkv_bias": False,
        "sink_zero": True, "distance_bias": True,
    }
    weights = {
        "q.weight": _matrix(TensorSource(prefix + "q", (a.heads * a.dim, width))),
        "k.weight": _matrix(TensorSource(prefix + "k", (a.kv_heads * a.dim, width))),
        "v.weight": _matrix(TensorSource(prefix + "v", (a.kv_heads * a.vdim, width))),
        "out.weight": _matrix(TensorSource(prefix + "o", (width, a.heads * a.vdim))),
        "bias_r1": _vector(TensorSource(prefix + "r1", (a.heads,), init="uniform:0:2")),
        "bias_r2": _vector(TensorSource(prefix + "r2", (a.heads,), init="uniform:0.05:0.5")),
    }
    return PartSpec(kind="attention", params=params, weights=weights)


def _differential(prefix: str, a: DifferentialAttentionConfig, width: int, eps: float) -> PartSpec:
    params = {
        "hidden_size": width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "dim": a.dim, "value_dim": a.vdim,
        "head_dim": differential_head_dim(a), "softmax_scale": a.scale, "softcap": a.softcap, "chunk": a.chunk,
        "lambda_init": a.diff, "eps": eps, "qk_norm": True, "output_gate": True,
    }
    dim = a.dim
    weights = {
        "q.weight": _matrix(TensorSource(prefix + "q", (a.heads * 2 * dim, width))),
        "k.weight": _matrix(TensorSource(prefix + "k", (a.kv_heads * 2 * dim, width))),
        "v.weight": _matrix(TensorSource(prefix + "v", (a.kv_heads * a.vdim, width))),
        "gate.weight": _matrix(TensorSource(prefix + "g", (a.heads * a.vdim, width))),
        "out.weight": _matrix(TensorSource(prefix + "o", (width, a.heads * a.vdim))),
        "q_norm": _vector(TensorSource(prefix + "q.norm", (dim,), init="one_plus_normal")),
        "k_norm": _vector(TensorSource(prefix + "k.norm", (dim,), init="one_plus_normal")),
    }
    for name in ("lq1", "lk1", "lq2", "lk2"):
        weights[name] = _vector(TensorSource(prefix + name, (dim,), init="normal_wide"))
    return PartSpec(kind="differential_attention", params=params, weights=weights)


def _feed_forward(prefix: str, f: ClampedFeedForwardConfig, width: int) -> PartSpec:
    return PartSpec(
        kind="clamped_glu",
        params={"hidden_size": width, "intermediate_size": f.ff, "limit": f.limit, "alpha": GATE_ALPHA,
                "up_shift": UP_SHIFT, "biases": True},
        weights={
            "gate_up.weight": _matrix(TensorSource(prefix + "gate", (f.ff, width)),
                                      TensorSource(prefix + "up", (f.ff, width))),
            "gate_up.bias": _vector(TensorSource(prefix + "gate.b", (f.ff,)), TensorSource(prefix + "up.b", (f.ff,))),
            "down.weight": _matrix(TensorSource(prefix + "down", (width, f.ff))),
            "down.bias": _vector(TensorSource(prefix + "down.b", (width,))),
        },
    )


def build_lizizen_spec(config: ModelConfig) -> ModelSpec:
    if not isinstance(config, LizizenConfig):
        raise TypeError(f"expected a LizizenConfig, got {type(config).__name__}")
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
        pos: Optional[PartSpec]
        if layer.type == "attention":
            a = layer.scored
            mixer = _scored(p, a, E)
            D = scored_head_dim(a)
            if a.q_temp is None:
                pos = position(("none", D), lambda: PartSpec(kind="none", params={"head_dim": D}))
            else:
                coef, every = a.q_temp
                pos = position(("temp", coef, every, D), lambda: PartSpec(
                    kind="log_temperature",
                    params={"head_dim": D, "coef": coef, "every": every, "max_position": c.max_position_embeddings}))
        else:
            d = layer.differential
            mixer = _differential(p, d, E, c.norm_eps)
            if d.rot is None:
                pos = position(("none", d.dim), lambda: PartSpec(kind="none", params={"head_dim": d.dim}))
            else:
                base, dims = d.rot
                pos = position(("rot", base, dims, d.dim), lambda: PartSpec(
                    kind="rotary_half",
                    params={"rotary_dim": dims, "theta": base, "max_position": c.max_position_embeddings,
                            "head_dim": d.dim, "angles": "float64"}))
        feed_forward = None if layer.mlp is None else _feed_forward(f"l{index}.mlp.", layer.mlp, E)
        norms = {"input": _rms(f"l{index}.norm1", E, c.norm_eps)}
        if feed_forward is not None:
            norms["feed_forward"] = _rms(f"l{index}.norm2", E, c.norm_eps)
        layers.append(LayerSpec(
            block="parallel", mixer=mixer, feed_forward=feed_forward, norms=norms, position=pos,
            block_params={"token_shift": True},
            block_weights={"shift": _vector(TensorSource(f"l{index}.shift", (E,), init="uniform:0:0.8"))}))
    spec = ModelSpec(
        architecture=c.architecture,
        hidden_size=E,
        vocab_size=V,
        max_position=c.max_position_embeddings,
        embedding=PartSpec(kind="token_embedding", params={"vocab_size": V, "hidden_size": E},
                           weights={"weight": _matrix(TensorSource("embed", (V, E)))}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in c.run_order()),
        final_norm=_rms("final.norm", E, c.norm_eps),
        lm_head=PartSpec(kind="linear_head", params={"hidden_size": E, "vocab_size": V},
                         weights={"weight": _matrix(TensorSource("head", (V, E)))}),
        eos_token_ids=tuple(c.eos_token_ids),
        # A layer without feed-forward has no use for a second norm; a file may still carry one.
        ignored_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(c.layers) if layer.mlp is None),
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, LizizenConfig.from_dict, build_lizizen_spec)
