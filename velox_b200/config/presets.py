"""Named example configurations of the Qwen2.5 dense family, and of the Peratar, Redalix, Lizizen and
Mamivik designs at the same widths, as ``config.json`` dictionaries.

They exist for runs with random weights (``--model-size`` of the benchmark command line): no
checkpoint is needed to time the layer sizes of a published model.  Nothing in the engine
reads them; a model folder's own ``config.json`` is what a model is built from.  The sizes are
those of the published Qwen2.5 checkpoints (0.5B ... 14B) and of two tiny test shapes.
"""
from __future__ import annotations

import copy
from typing import Any, Dict


def _qwen2(layers, hidden, heads, kv_heads, inter, vocab, tied, eps, max_pos=32768, theta=1000000.0,
           head_dim=None) -> Dict[str, Any]:
    cfg = {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers,
        "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
        "intermediate_size": inter, "vocab_size": vocab, "rope_theta": theta, "rms_norm_eps": eps,
        "tie_word_embeddings": tied, "use_sliding_window": False, "max_position_embeddings": max_pos,
        "hidden_act": "silu",
    }
    if head_dim is not None:
        cfg["head_dim"] = head_dim
    return cfg


MODEL_SIZES: Dict[str, Dict[str, Any]] = {
    "tiny-a": _qwen2(2, 64, 4, 2, 128, 256, True, 1e-6, max_pos=128, theta=10000.0, head_dim=16),
    "tiny-b": _qwen2(3, 256, 8, 1, 704, 512, False, 1e-5, max_pos=256, head_dim=32),
    "0.5b": _qwen2(24, 896, 14, 2, 4864, 151936, True, 1e-6),
    "1.5b": _qwen2(28, 1536, 12, 2, 8960, 151936, True, 1e-6),
    "3b": _qwen2(36, 2048, 16, 2, 11008, 151936, True, 1e-6),
    "7b": _qwen2(28, 3584, 28, 4, 18944, 152064, False, 1e-6),
    "14b": _qwen2(48, 5120, 40, 8, 13824, 152064, False, 1e-5),
}


def _peratar(like: str, rot_dim: int = 32, kv_rank: int = 96, share_every: int = 2) -> Dict[str, Any]:
    """A Peratar configuration with the width, head count, layer count and vocabulary of the named
    Qwen2.5 size: query heads as wide as that model's (``rot_dim`` of their dims rotate), values as
    wide as its heads, a latent of ``kv_rank`` values, every ``share_every``-th layer reading the
    cache of the layer before it, and a dense inner width that gives a layer (gates included)
    as many weights in its feed-forward as the gated feed-forward of that size has."""
    base = MODEL_SIZES[like]
    width, heads, layers = base["hidden_size"], base["num_attention_heads"], base["num_hidden_layers"]
    head = base.get("head_dim") or width // heads
    inner = max(64, (3 * base["intermediate_size"] - 2 * width) // 2 // 64 * 64)
    entries = []
    for index in range(layers):
        mixer = {"heads": heads, "dim": head - rot_dim, "rot_dim": rot_dim, "vdim": head, "kv_rank": kv_rank,
                 "scale": (head ** -0.5), "rot": {"base": base["rope_theta"], "dims": rot_dim}}
        if share_every > 1 and index % share_every == share_every - 1:
            mixer["kv_from"] = index - 1
        entries.append({"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": inner}})
    return {"architecture": "Peratar", "vocab": base["vocab_size"], "width": width, "norm": {"eps": 1e-5},
            "logit_softcap": 30.0, "layers": entries, "max_position_embeddings": base["max_position_embeddings"]}


def _peratar_tiny() -> Dict[str, Any]:
    """A tiny Peratar configuration for smoke runs of the command lines: three layers of different
    sizes, the second without feed-forward, the third on the first one's cache."""
    def mixer(heads, dim, rot_dim, vdim, kv_rank, scale, kv_from=None):
        out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
               "rot": {"base": 10000.0, "dims": rot_dim}}
        if kv_from is not None:
            out["kv_from"] = kv_from
        return out

    layers = [
        {"type": "latent_attention", "mixer": mixer(4, 16, 8, 16, 24, 0.2), "mlp": {"kind": "dense", "ff": 160}},
        {"type": "latent_attention", "mixer": mixer(2, 24, 16, 32, 32, 0.15), "mlp": None},
        {"type": "latent_attention", "mixer": mixer(4, 8, 8, 24, 24, 0.25, kv_from=0), "mlp": {"kind": "dense", "ff": 96}},
    ]
    return {"architecture": "Peratar", "vocab": 384, "width": 128, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
            "layers": layers, "max_position_embeddings": 512}


def _redalix(like: str, experts: int = 16, top: int = 2) -> Dict[str, Any]:
    """A Redalix configuration with the width, head counts, layer count and vocabulary of the named
    Qwen2.5 size.  Its layers repeat the pattern parallel, attention, parallel, mamba2; attention
    heads are as wide as that model's; the recurrence is as wide as the model, in eight parts; the
    state-space layer has twice the model's width in heads of 64 values over a state of 128; every
    feed-forward is ``experts`` experts of a quarter of that model's inner width, ``top`` per
    token, beside a shared expert of the whole inner width, so that a token meets as many
    feed-forward weights as in the gated feed-forward of that size."""
    base = MODEL_SIZES[like]
    width, heads, kv_heads = base["hidden_size"], base["num_attention_heads"], base["num_key_value_heads"]
    head = base.get("head_dim") or width // heads
    inner = base["intermediate_size"]
    mlp = {"kind": "moe", "expert": {"ff": max(64, inner // 4 // 64 * 64)}, "router": {"experts": experts, "top": top},
           "shared": {"ff": inner}}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5,
            "mask": {"size": 1024, "keep_first": 64}}
    right = {"width": width, "blocks": 8, "conv": 4}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5,
                 "mask": {"size": 4096},
                 "rot": {"base": base["rope_theta"], "dims": head,
                         "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    mamba = {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 2, "norm_groups": 2, "conv": 4}
    pattern = [
        {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp},
        {"type": "attention", "mixer": attention, "mlp": mlp},
        {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp},
        {"type": "mamba2", "mixer": mamba, "mlp": mlp},
    ]
    entries = [copy.deepcopy(pattern[index % len(pattern)]) for index in range(base["num_hidden_layers"])]
    return {"architecture": "Redalix", "vocab": base["vocab_size"], "width": width, "norm": {"eps": 1e-5},
            "layers": entries, "max_position_embeddings": base["max_position_embeddings"]}


def _redalix_tiny() -> Dict[str, Any]:
    """A tiny Redalix configuration for smoke runs of the command lines: one layer of each kind."""
    left = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.25, "mask": {"size": 24, "keep_first": 4}}
    attention = {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 16, "scale": 0.18, "mask": {"size": 40},
                 "rot": {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}}}
    mlp = {"kind": "moe", "expert": {"ff": 48}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 64}}
    layers = [
        {"type": "parallel", "mixer": {"left": left, "right": {"width": 96, "blocks": 3, "conv": 4}},
         "mlp": {"kind": "dense", "ff": 160}},
        {"type": "attention", "mixer": attention, "mlp": mlp},
        {"type": "mamba2", "mixer": {"heads": 8, "vdim": 16, "state": 24, "groups": 2, "norm_groups": 2, "conv": 3},
         "mlp": mlp},
    ]
    return {"architecture": "Redalix", "vocab": 384, "width": 128, "norm": {"eps": 1e-5}, "layers": layers,
            "max_position_embeddings": 512}


def _lizizen(like: str, chunk: int = 1024) -> Dict[str, Any]:
    """A Lizizen configuration with the width, head counts, layer count, feed-forward width and
    vocabulary of the named Qwen2.5 size.  Its layers alternate ``attention_2`` and ``attention``.
    An ``attention`` head is as wide as that model's; an ``attention_2`` head has two maps of half
    that size and values of the whole size, so both mixers have that model's q, k, v and o
    matrices (``attention_2`` one more of the size of q, for its gate) and cache as many values
    per key."""
    base = MODEL_SIZES[like]
    width, heads, kv_heads = base["hidden_size"], base["num_attention_heads"], base["num_key_value_heads"]
    head = base.get("head_dim") or width // heads
    mlp = {"kind": "dense", "ff": base["intermediate_size"], "limit": 7.0}
    two_maps = {"heads": heads, "kv_heads": kv_heads, "dim": head // 2, "vdim": head, "scale": (head // 2) ** -0.5,
                "diff": 0.5, "mask": {"size": chunk}, "rot": {"base": base["rope_theta"], "dims": head // 4},
                "softcap": 50.0}
    all_keys = {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5,
                "q_temp": {"coef": 0.1, "every": 1024}}
    pattern = [{"type": "attention_2", "mixer": two_maps, "mlp": mlp}, {"type": "attention", "mixer": all_keys, "mlp": mlp}]
    entries = [copy.deepcopy(pattern[index % len(pattern)]) for index in range(base["num_hidden_layers"])]
    return {"architecture": "Lizizen", "vocab": base["vocab_size"], "width": width, "norm": {"eps": 1e-6},
            "layers": entries, "max_position_embeddings": base["max_position_embeddings"]}


def _lizizen_tiny() -> Dict[str, Any]:
    """A tiny Lizizen configuration for smoke runs of the command lines: both mixers, a layer
    without feed-forward, the first two layers run twice."""
    layers = [
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.25, "diff": 0.4,
                                          "mask": {"size": 24}, "rot": {"base": 10000.0, "dims": 8}, "softcap": 10.0},
         "mlp": {"kind": "dense", "ff": 160, "limit": 2.0}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 16, "scale": 0.18,
                                        "q_temp": {"coef": 0.2, "every": 16}}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.25},
         "mlp": {"kind": "dense", "ff": 96, "limit": 1.0}},
    ]
    return {"architecture": "Lizizen", "vocab": 384, "width": 128, "norm": {"eps": 1e-5}, "layers": layers,
            "loop": {"start": 0, "stop": 2, "times": 2}, "max_position_embeddings": 512}


def _mamivik(like: str, rot_dim: int = 32, kv_rank: int = 96, window: int = 1024) -> Dict[str, Any]:
    """A Mamivik configuration with the width, head counts, layer count, feed-forward width and
    vocabulary of the named Qwen2.5 size.  Its layers alternate ``latent_attention`` (query heads as
    wide as that model's, ``rot_dim`` of their dims rotating, values as wide as its heads, a
    latent of ``kv_rank`` values, queries through a latent of a quarter of the width) and
    ``parallel`` (left: that model's heads over a window; right: a delta rule of as many channels
    as the left mixer has key channels, in heads of 64)."""
    base = MODEL_SIZES[like]
    width, heads, kv_heads = base["hidden_size"], base["num_attention_heads"], base["num_key_value_heads"]
    head = base.get("head_dim") or width // heads
    mlp = {"kind": "dense", "ff": base["intermediate_size"]}
    latent = {"heads": heads, "dim": head - rot_dim, "rot_dim": rot_dim, "vdim": head, "kv_rank": kv_rank,
              "q_rank": width // 4 // 8 * 8, "scale": head ** -0.5, "mask": {"size": window},
              "rot": {"base": 10000.0, "dims": rot_dim,
                      "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5,
            "mask": {"size": window}, "rot": {"base": base["rope_theta"], "dims": head // 2}}
    both = {"left": left, "right": {"heads": max(1, kv_heads * head // 64), "dim": 64}, "left_scale": 1.0,
            "right_scale": 1.0}
    pattern = [{"type": "latent_attention", "mixer": latent, "mlp": mlp}, {"type": "parallel", "mixer": both, "mlp": mlp}]
    entries = [copy.deepcopy(pattern[index % len(pattern)]) for index in range(base["num_hidden_layers"])]
    return {"architecture": "Mamivik", "vocab": base["vocab_size"], "width": width, "norm": {"eps": 1e-6},
            "canon": {"taps": 4}, "layers": entries, "max_position_embeddings": base["max_position_embeddings"]}


def _mamivik_tiny() -> Dict[str, Any]:
    """A tiny Mamivik configuration for smoke runs of the command lines: both kinds of layer, a
    layer without feed-forward."""
    layers = [
        {"type": "parallel", "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 24},
                     "rot": {"base": 10000.0, "dims": 8}},
            "right": {"heads": 2, "dim": 16}, "left_scale": 1.1, "right_scale": 0.8},
         "mlp": {"kind": "dense", "ff": 160}},
        {"type": "latent_attention", "mixer": {
            "heads": 4, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "q_rank": 32, "scale": 0.2,
            "mask": {"size": 40}, "rot": {"base": 1000.0, "dims": 8,
                                           "scaling": {"factor": 2.0, "original": 64, "fast": 8.0, "slow": 1.0}}},
         "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.18, "mask": {"size": 100},
                     "rot": {"base": 500.0, "dims": 32}},
            "right": {"heads": 1, "dim": 32}, "left_scale": 0.9, "right_scale": 1.2},
         "mlp": {"kind": "dense", "ff": 96}},
    ]
    return {"architecture": "Mamivik", "vocab": 384, "width": 128, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
            "layers": layers, "max_position_embeddings": 512}


MODEL_SIZES.update({
    "tiny-m": _mamivik_tiny(),
    "mamivik-0.5b": _mamivik("0.5b"),
    "mamivik-1.5b": _mamivik("1.5b"),
    "mamivik-3b": _mamivik("3b"),
    "tiny-r": _redalix_tiny(),
    "redalix-0.5b": _redalix("0.5b"),
    "redalix-1.5b": _redalix("1.5b"),
    "redalix-3b": _redalix("3b"),
    "tiny-p": _peratar_tiny(),
    "peratar-0.5b": _peratar("0.5b"),
    "peratar-1.5b": _peratar("1.5b"),
    "peratar-3b": _peratar("3b"),
    "peratar-7b": _peratar("7b"),
    "tiny-l": _lizizen_tiny(),
    "lizizen-0.5b": _lizizen("0.5b"),
    "lizizen-1.5b": _lizizen("1.5b"),
    "lizizen-3b": _lizizen("3b"),
})


def with_layers(config_json: Dict[str, Any], layers: int) -> Dict[str, Any]:
    """The configuration with another number of layers of the same sizes (a list of layers is cut,
    or repeated from its start with every ``kv_from`` kept at its distance; a ``loop`` over the list
    as it was is dropped)."""
    out = copy.deepcopy(config_json)
    if "layers" not in out:
        out["num_hidden_layers"] = layers
        return out
    given = out["layers"]
    if layers != len(given):
        out.pop("loop", None)  # a looped stretch names layers of the list as it was
    entries = []
    for index in range(layers):
        entry = copy.deepcopy(given[index % len(given)])
        source = entry["mixer"].get("kv_from")
        if source is not None:
            entry["mixer"]["kv_from"] = index - (index % len(given) - source)
        entries.append(entry)
    out["layers"] = entries
    return out


def model_size(name: str) -> Dict[str, Any]:
    """A copy of the named configuration; KeyError lists the names."""
    try:
        return copy.deepcopy(MODEL_SIZES[name])
    except KeyError:
        raise KeyError(f"unknown model size {name!r}; known: {', '.join(sorted(MODEL_SIZES))}") from None
