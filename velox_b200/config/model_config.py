"""Typed model configuration, read from an architecture's own ``config.json`` keys.

Every size and constant of a model comes from here; no kernel, part or engine module carries a
model size of its own.  The field list follows the reference's ``ModelConfig``
(src/config.py:6-42) and adds the keys the reference leaves implicit: ``head_dim`` (the
reference derives it as ``hidden_size // num_attention_heads``, src/transformer.py:19),
``hidden_act`` (fixed to SiLU in src/mlp.py:15) and the sliding-window keys that Qwen2
checkpoints carry and the reference never reads.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the offending key named."""


def _require(cfg: Mapping[str, Any], key: str) -> Any:
    if key not in cfg or cfg[key] is None:
        raise ConfigError(f"config.json is missing required key {key!r}")
    return cfg[key]


def _positive_int(cfg: Mapping[str, Any], key: str, default: Optional[int] = None) -> int:
    value = cfg.get(key)
    if value is None:
        value = default if default is not None else _require(cfg, key)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json key {key!r} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class ModelConfig:
    """Fields shared by every architecture; an architecture subclasses this with its own keys."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_ids: Tuple[int, ...] = ()

    def to_json_dict(self) -> Dict[str, Any]:  # pragma: no cover - overridden
        raise NotImplementedError


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """``Qwen2ForCausalLM``: dense decoder, q/k/v bias, SwiGLU, pre-RMSNorm, rotate-half RoPE.

    Defaults of absent keys follow src/config.py:29-42: ``num_key_value_heads`` falls back to
    ``num_attention_heads``, ``rms_norm_eps`` to ``layer_norm_eps`` then 1e-6,
    ``max_position_embeddings`` to ``seq_length`` then 4096, ``rope_theta`` to 10000 and
    ``tie_word_embeddings`` to False.
    """

    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    # Linear position scaling only (positions are divided by this), as in src/rope.py:11-18.
    rope_scaling_factor: float = 1.0
    hidden_act: str = "silu"
    # Window of keys a query may see (itself included) in the layers that use one; None = all keys.
    sliding_window: Optional[int] = None
    # Layers with index >= max_window_layers use the window when it is enabled.
    max_window_layers: int = 0
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------ derived
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        """Key window of one layer: the first ``max_window_layers`` layers see every key."""
        if self.sliding_window is None or layer < self.max_window_layers:
            return None
        return self.sliding_window

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "Qwen2Config":
        archs = cfg.get("architectures") or ["Qwen2ForCausalLM"]
        hidden = _positive_int(cfg, "hidden_size")
        heads = _positive_int(cfg, "num_attention_heads")
        kv_heads = _positive_int(cfg, "num_key_value_heads", heads)
        if cfg.get("head_dim") is not None:
            head_dim = _positive_int(cfg, "head_dim")
        else:
            if hidden % heads != 0:
                raise ConfigError(
                    f"hidden_size={hidden} is not divisible by num_attention_heads={heads} "
                    "and config.json gives no head_dim"
                )
            head_dim = hidden // heads
        if heads % kv_heads != 0:
            raise ConfigError(
                f"num_attention_heads={heads} must be a multiple of num_key_value_heads={kv_heads}"
            )
        if head_dim % 2 != 0:
            raise ConfigError(f"head_dim={head_dim} must be even for rotate-half RoPE")

        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r} is not supported (Qwen2 uses 'silu')")

        scaling = cfg.get("rope_scaling")
        factor = 1.0
        if scaling:
            kind = scaling.get("type") or scaling.get("rope_type")
            if kind in (None, "default"):
                factor = 1.0
            elif kind == "linear":
                factor = float(scaling.get("factor", 1.0))
                if not factor > 0.0:
                    raise ConfigError(f"rope_scaling.factor must be positive, got {factor}")
            else:
                raise ConfigError(
                    f"rope_scaling type {kind!r} is not supported (only 'linear' is); "
                    "refusing to run with wrong rotation angles"
                )

        window: Optional[int] = None
        layers = _positive_int(cfg, "num_hidden_layers")
        max_window_layers = layers
        if cfg.get("use_sliding_window", False):
            window = _positive_int(cfg, "sliding_window")
            max_window_layers = int(cfg.get("max_window_layers", layers))
            if max_window_layers < 0:
                raise ConfigError("max_window_layers must be non-negative")

        eps = cfg.get("rms_norm_eps", cfg.get("layer_norm_eps", 1e-6))
        max_pos = cfg.get("max_position_embeddings", cfg.get("seq_length", 4096))
        eos = cfg.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(t) for t in eos)

        return Qwen2Config(
            architecture=str(archs[0]),
            vocab_size=_positive_int(cfg, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=layers,
            max_position_embeddings=int(max_pos),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_positive_int(cfg, "intermediate_size"),
            rms_norm_eps=float(eps),
            rope_theta=float(cfg.get("rope_theta", 10000.0)),
            rope_scaling_factor=factor,
            hidden_act=act,
            sliding_window=window,
            max_window_layers=max_window_layers,
            torch_dtype=str(cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))),
        )

    def to_json_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": (
                None
                if self.rope_scaling_factor == 1.0
                else {"type": "linear", "factor": self.rope_scaling_factor}
            ),
            "hidden_act": self.hidden_act,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.sliding_window is not None,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _mapping(cfg: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = cfg.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}: key {key!r} must be an object, got {value!r}")
    return value


def _number(cfg: Mapping[str, Any], key: str, where: str) -> float:
    value = cfg.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{where}: key {key!r} must be a number, got {value!r}")
    return float(value)


def _count(cfg: Mapping[str, Any], key: str, where: str) -> int:
    value = cfg.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"{where}: key {key!r} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class LatentMixerConfig:
    """One layer's latent attention: ``heads`` heads of ``dim`` unrotated and ``rot_dim`` rotated
    query/key dims and ``vdim`` value dims over a cached latent of ``kv_rank`` values; pairs of
    the first ``rot_dims`` rotated dims turn with ``rot_base``; ``kv_from`` names the layer whose
    cached latent this layer reads instead of making its own."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: Optional[int] = None

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
            "kv_rank": self.kv_rank, "scale": self.scale,
            "rot": {"base": self.rot_base, "dims": self.rot_dims},
        }
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class PeratarLayerConfig:
    mixer: LatentMixerConfig
    # Inner width of the dense feed-forward; None: the layer has none.
    ff: Optional[int]


@dataclass(frozen=True)
class PeratarConfig(ModelConfig):
    """``Peratar``: every layer is latent attention and, optionally, a dense xIELU feed-forward,
    each followed by a gate, a weight-only layer norm and the residual add; a layer's input is
    a learned weighted sum of the results of all layers before it.  config.json keys: ``vocab``,
    ``width``, ``norm.eps``, ``logit_softcap`` and ``layers`` (a list of ``{type, mixer, mlp}``).
    ``max_position_embeddings`` is optional (the design has no limit of its own)."""

    layers: Tuple[PeratarLayerConfig, ...] = ()
    norm_eps: float = 1e-5
    logit_softcap: Optional[float] = None
    torch_dtype: str = "bfloat16"

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "PeratarConfig":
        name = cfg.get("architecture") or (cfg.get("architectures") or ["Peratar"])[0]
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"config.json layers[{index}]"
            if not isinstance(raw, Mapping):
                raise ConfigError(f"{where} must be an object")
            kind = raw.get("type")
            if kind != "latent_attention":
                raise ConfigError(f"{where}: mixer type {kind!r} is not supported (only 'latent_attention' is)")
            m = _mapping(raw, "mixer", where)
            rot = _mapping(m, "rot", where + ".mixer")
            kv_from = m.get("kv_from")
            if kv_from is not None:
                if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < index:
                    raise ConfigError(f"{where}: kv_from={kv_from!r} must name an earlier layer")
            mixer = LatentMixerConfig(
                heads=_count(m, "heads", where), dim=_count(m, "dim", where), rot_dim=_count(m, "rot_dim", where),
                vdim=_count(m, "vdim", where), kv_rank=_count(m, "kv_rank", where),
                scale=_number(m, "scale", where), rot_base=_number(rot, "base", where + ".mixer.rot"),
                rot_dims=_count(rot, "dims", where + ".mixer.rot"), kv_from=kv_from,
            )
            if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                raise ConfigError(f"{where}: rot.dims={mixer.rot_dims} must be even and at most rot_dim={mixer.rot_dim}")
            if kv_from is not None:
                source = layers[kv_from].mixer
                if source.kv_from is not None:
                    raise ConfigError(f"{where}: layer {kv_from} has no cached latent of its own to read")
                if (source.kv_rank, source.rot_dim, source.rot_base, source.rot_dims) != (
                        mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims):
                    raise ConfigError(f"{where}: kv_rank, rot_dim and rotation must equal those of layer {kv_from}")
            mlp = raw.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{where}: key 'mlp' must be an object or null")
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}: mlp kind {mlp.get('kind')!r} is not supported (only 'dense' is)")
                ff = _count(mlp, "ff", where + ".mlp")
            layers.append(PeratarLayerConfig(mixer=mixer, ff=ff))
        cap = cfg.get("logit_softcap")
        if cap is not None and not float(cap) > 0.0:
            raise ConfigError(f"logit_softcap must be positive, got {cap!r}")
        eos = cfg.get("eos_token_id")
        eos_ids: Tuple[int, ...] = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(t) for t in eos))
        return PeratarConfig(
            architecture=str(name),
            vocab_size=_count(cfg, "vocab", "config.json"),
            hidden_size=_count(cfg, "width", "config.json"),
            num_hidden_layers=len(layers),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 1 << 20)),
            tie_word_embeddings=False,
            eos_token_ids=eos_ids,
            layers=tuple(layers),
            norm_eps=_number(_mapping(cfg, "norm", "config.json"), "eps", "config.json norm"),
            logit_softcap=None if cap is None else float(cap),
            torch_dtype=str(cfg.get("torch_dtype", "bfloat16")),
        )

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": self.architecture,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [
                {"type": "latent_attention", "mixer": layer.mixer.to_json_dict(),
                 "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}}
                for layer in self.layers
            ],
            "torch_dtype": self.torch_dtype,
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.max_position_embeddings != 1 << 20:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _window(cfg: Mapping[str, Any], where: str, keep_allowed: bool) -> Tuple[int, int]:
    mask = _mapping(cfg, "mask", where)
    size = _count(mask, "size", where + ".mask")
    keep = mask.get("keep_first", 0)
    if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
        raise ConfigError(f"{where}.mask: keep_first={keep!r} must be a non-negative integer")
    if keep and not keep_allowed:
        raise ConfigError(f"{where}.mask: keep_first is not a key of this mixer")
    return size, keep


@dataclass(frozen=True)
class WindowAttentionConfig:
    """Softmax attention with grouped heads over a sliding window.  ``keep_first`` keys stay
    visible behind the window; ``rot`` (or None) = (base, dims, scaling or None) with scaling =
    (factor, original, fast, slow); ``biases``, ``sink`` and ``head_gate`` say which further
    tensors the mixer has."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int = 0
    rot: Optional[Tuple[float, int, Optional[Tuple[float, float, float, float]]]] = None
    biases: bool = False
    sink: bool = False
    head_gate: bool = False

    @staticmethod
    def parse(m: Mapping[str, Any], where: str, *, rotated: bool, biases: bool, sink: bool, head_gate: bool,
              keep_allowed: bool) -> "WindowAttentionConfig":
        heads, kv_heads = _count(m, "heads", where), _count(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"{where}: heads={heads} must be a multiple of kv_heads={kv_heads}")
        window, keep = _window(m, where, keep_allowed)
        rot = None
        if rotated:
            r = _mapping(m, "rot", where)
            dims = _count(r, "dims", where + ".rot")
            dim = _count(m, "dim", where)
            if dims % 2 or dims > dim:
                raise ConfigError(f"{where}.rot: dims={dims} must be even and at most dim={dim}")
            scaling = None
            if r.get("scaling") is not None:
                sc = _mapping(r, "scaling", where + ".rot")
                scaling = tuple(_number(sc, key, where + ".rot.scaling") for key in ("factor", "original", "fast", "slow"))
                if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
                    raise ConfigError(f"{where}.rot.scaling: factor, original, fast and slow must be positive")
            rot = (_number(r, "base", where + ".rot"), dims, scaling)
        elif m.get("rot") is not None:
            raise ConfigError(f"{where}: this mixer has no rotation, but 'rot' is given")
        return WindowAttentionConfig(
            heads=heads, kv_heads=kv_heads, dim=_count(m, "dim", where), vdim=_count(m, "vdim", where),
            scale=_number(m, "scale", where), window=window, keep_first=keep, rot=rot, biases=biases, sink=sink,
            head_gate=head_gate)

    def to_json_dict(self) -> Dict[str, Any]:
        mask: Dict[str, Any] = {"size": self.window}
        if self.keep_first or self.sink:
            # the mixer beside a recurrence always names its kept keys, even none
            mask["keep_first"] = self.keep_first
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "mask": mask}
        if self.rot is not None:
            base, dims, scaling = self.rot
            out["rot"] = {"base": base, "dims": dims}
            if scaling is not None:
                out["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
        return out


@dataclass(frozen=True)
class RecurrenceConfig:
    """The gated linear recurrence: ``width`` channels in ``blocks`` parts, a convolution of
    ``conv`` taps."""

    width: int
    blocks: int
    conv: int

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "RecurrenceConfig":
        out = RecurrenceConfig(width=_count(m, "width", where), blocks=_count(m, "blocks", where),
                               conv=_count(m, "conv", where))
        if out.width % out.blocks:
            raise ConfigError(f"{where}: width={out.width} must be a multiple of blocks={out.blocks}")
        return out

    def to_json_dict(self) -> Dict[str, Any]:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "StateSpaceConfig":
        out = StateSpaceConfig(heads=_count(m, "heads", where), vdim=_count(m, "vdim", where),
                               state=_count(m, "state", where), groups=_count(m, "groups", where),
                               norm_groups=_count(m, "norm_groups", where), conv=_count(m, "conv", where))
        if out.heads % out.groups:
            raise ConfigError(f"{where}: heads={out.heads} must be a multiple of groups={out.groups}")
        if (out.heads * out.vdim) % out.norm_groups:
            raise ConfigError(f"{where}: heads * vdim must be a multiple of norm_groups={out.norm_groups}")
        return out

    def to_json_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "norm_groups": self.norm_groups, "conv": self.conv}


@dataclass(frozen=True)
class RedalixFeedForwardConfig:
    """``kind`` dense: ``ff``.  ``kind`` moe: ``experts`` of inner width ``expert_ff``, ``top`` per
    token, and ``shared_ff`` (None: no shared expert)."""

    kind: str
    ff: int = 0
    experts: int = 0
    top: int = 0
    expert_ff: int = 0
    shared_ff: Optional[int] = None

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "RedalixFeedForwardConfig":
        kind = m.get("kind")
        if kind == "dense":
            return RedalixFeedForwardConfig(kind="dense", ff=_count(m, "ff", where))
        if kind == "moe":
            router = _mapping(m, "router", where)
            experts, top = _count(router, "experts", where + ".router"), _count(router, "top", where + ".router")
            if top > experts:
                raise ConfigError(f"{where}.router: top={top} is more than experts={experts}")
            shared = m.get("shared")
            return RedalixFeedForwardConfig(
                kind="moe", experts=experts, top=top,
                expert_ff=_count(_mapping(m, "expert", where), "ff", where + ".expert"),
                shared_ff=None if shared is None else _count(_mapping(m, "shared", where), "ff", where + ".shared"))
        raise ConfigError(f"{where}: mlp kind {kind!r} is not supported ('dense' and 'moe' are)")

    def to_json_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.expert_ff},
                               "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class RedalixLayerConfig:
    """``type`` parallel: ``left`` (attention) and ``right`` (recurrence); attention: ``left``;
    mamba2: ``state_space``."""

    type: str
    left: Optional[WindowAttentionConfig] = None
    right: Optional[RecurrenceConfig] = None
    state_space: Optional[StateSpaceConfig] = None
    mlp: Optional[RedalixFeedForwardConfig] = None


@dataclass(frozen=True)
class RedalixConfig(ModelConfig):
    """``Redalix``: every layer is ``x <- x + mixer(h) + ff(h)`` with ``h = rms_norm(x)``; the
    mixer is windowed attention with rotation, biases and a gate per head (``attention``), a
    state-space layer (``mamba2``), or windowed attention with a sink and kept first keys beside
    a gated linear recurrence (``parallel``); the feed-forward is dense or a set of experts
    chosen by a table over token ids, with a gated shared expert.  config.json keys: ``vocab``,
    ``width``, ``norm.eps`` and ``layers`` (a list of ``{type, mixer, mlp}``)."""

    layers: Tuple[RedalixLayerConfig, ...] = ()
    norm_eps: float = 1e-5
    torch_dtype: str = "bfloat16"

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "RedalixConfig":
        name = cfg.get("architecture") or (cfg.get("architectures") or ["Redalix"])[0]
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"config.json layers[{index}]"
            if not isinstance(raw, Mapping):
                raise ConfigError(f"{where} must be an object")
            kind = raw.get("type")
            m = _mapping(raw, "mixer", where)
            mlp = None
            if raw.get("mlp") is not None:
                mlp = RedalixFeedForwardConfig.parse(_mapping(raw, "mlp", where), where + ".mlp")
            if kind == "parallel":
                layer = RedalixLayerConfig(
                    type=kind,
                    left=WindowAttentionConfig.parse(_mapping(m, "left", where + ".mixer"), where + ".mixer.left",
                                                     rotated=False, biases=False, sink=True, head_gate=False,
                                                     keep_allowed=True),
                    right=RecurrenceConfig.parse(_mapping(m, "right", where + ".mixer"), where + ".mixer.right"),
                    mlp=mlp)
            elif kind == "attention":
                layer = RedalixLayerConfig(
                    type=kind,
                    left=WindowAttentionConfig.parse(m, where + ".mixer", rotated=True, biases=True, sink=False,
                                                     head_gate=True, keep_allowed=False),
                    mlp=mlp)
            elif kind == "mamba2":
                layer = RedalixLayerConfig(type=kind, state_space=StateSpaceConfig.parse(m, where + ".mixer"), mlp=mlp)
            else:
                raise ConfigError(f"{where}: layer type {kind!r} is not supported "
                                  "('parallel', 'attention' and 'mamba2' are)")
            layers.append(layer)
        eos = cfg.get("eos_token_id")
        eos_ids: Tuple[int, ...] = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(t) for t in eos))
        return RedalixConfig(
            architecture=str(name),
            vocab_size=_count(cfg, "vocab", "config.json"),
            hidden_size=_count(cfg, "width", "config.json"),
            num_hidden_layers=len(layers),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 1 << 20)),
            tie_word_embeddings=False,
            eos_token_ids=eos_ids,
            layers=tuple(layers),
            norm_eps=_number(_mapping(cfg, "norm", "config.json"), "eps", "config.json norm"),
            torch_dtype=str(cfg.get("torch_dtype", "bfloat16")),
        )

    def to_json_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            if layer.type == "parallel":
                mixer: Dict[str, Any] = {"left": layer.left.to_json_dict(), "right": layer.right.to_json_dict()}
            elif layer.type == "attention":
                mixer = layer.left.to_json_dict()
            else:
                mixer = layer.state_space.to_json_dict()
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.mlp is None else layer.mlp.to_json_dict()})
        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps}, "layers": layers, "torch_dtype": self.torch_dtype,
        }
        if self.max_position_embeddings != 1 << 20:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


@dataclass(frozen=True)
class ScoredAttentionConfig:
    """Causal softmax attention over all keys with grouped heads, no rotation, a term of score 0
    in every denominator and a distance bias per head; ``q_temp`` (or None) = (coef, every): the
    query at position p is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[Tuple[float, int]] = None

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "ScoredAttentionConfig":
        heads, kv_heads = _count(m, "heads", where), _count(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"{where}: heads={heads} must be a multiple of kv_heads={kv_heads}")
        for key in ("rot", "mask", "softcap", "diff"):
            if m.get(key) is not None:
                raise ConfigError(f"{where}: {key!r} is not a key of this mixer")
        q_temp = None
        if m.get("q_temp") is not None:
            t = _mapping(m, "q_temp", where)
            q_temp = (_number(t, "coef", where + ".q_temp"), _count(t, "every", where + ".q_temp"))
        return ScoredAttentionConfig(heads=heads, kv_heads=kv_heads, dim=_count(m, "dim", where),
                                     vdim=_count(m, "vdim", where), scale=_number(m, "scale", where), q_temp=q_temp)

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.q_temp is not None:
            out["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        return out


@dataclass(frozen=True)
class DifferentialAttentionConfig:
    """Two softmax maps per head over the same values, combined as ``a1 - lambda a2``.  ``rot``
    (or None) = (base, dims); ``chunk`` (or None): the size of the chunks a query stays inside;
    ``softcap`` (or None); ``diff``: the constant in lambda and in the output's factor."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    rot: Optional[Tuple[float, int]] = None
    chunk: Optional[int] = None
    softcap: Optional[float] = None

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "DifferentialAttentionConfig":
        heads, kv_heads = _count(m, "heads", where), _count(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"{where}: heads={heads} must be a multiple of kv_heads={kv_heads}")
        dim = _count(m, "dim", where)
        if m.get("q_temp") is not None:
            raise ConfigError(f"{where}: 'q_temp' is not a key of this mixer")
        rot = None
        if m.get("rot") is not None:
            r = _mapping(m, "rot", where)
            dims = _count(r, "dims", where + ".rot")
            if dims % 2 or dims > dim:
                raise ConfigError(f"{where}.rot: dims={dims} must be even and at most dim={dim}")
            base = _number(r, "base", where + ".rot")
            if base <= 0:
                raise ConfigError(f"{where}.rot: base={base} must be positive")
            rot = (base, dims)
        chunk = None
        if m.get("mask") is not None:
            mask = _mapping(m, "mask", where)
            if mask.get("keep_first"):
                raise ConfigError(f"{where}.mask: keep_first is not a key of this mixer")
            chunk = _count(mask, "size", where + ".mask")
        softcap = None
        if m.get("softcap") is not None:
            softcap = _number(m, "softcap", where)
            if softcap <= 0:
                raise ConfigError(f"{where}: softcap={softcap} must be positive")
        return DifferentialAttentionConfig(
            heads=heads, kv_heads=kv_heads, dim=dim, vdim=_count(m, "vdim", where), scale=_number(m, "scale", where),
            diff=_number(m, "diff", where), rot=rot, chunk=chunk, softcap=softcap)

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "diff": self.diff}
        if self.rot is not None:
            out["rot"] = {"base": self.rot[0], "dims": self.rot[1]}
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class ClampedFeedForwardConfig:
    """A gated feed-forward of inner width ``ff`` whose gate and up values are clamped at
    ``limit`` (None: no clamps)."""

    ff: int
    limit: Optional[float] = None

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "ClampedFeedForwardConfig":
        kind = m.get("kind")
        if kind != "dense":
            raise ConfigError(f"{where}: mlp kind {kind!r} is not supported ('dense' is)")
        limit = None
        if m.get("limit") is not None:
            limit = _number(m, "limit", where)
            if limit <= 0:
                raise ConfigError(f"{where}: limit={limit} must be positive")
        return ClampedFeedForwardConfig(ff=_count(m, "ff", where), limit=limit)

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"kind": "dense", "ff": self.ff}
        if self.limit is not None:
            out["limit"] = self.limit
        return out


@dataclass(frozen=True)
class LizizenLayerConfig:
    """``type`` attention: ``scored``; attention_2: ``differential``."""

    type: str
    scored: Optional[ScoredAttentionConfig] = None
    differential: Optional[DifferentialAttentionConfig] = None
    mlp: Optional[ClampedFeedForwardConfig] = None


@dataclass(frozen=True)
class LizizenConfig(ModelConfig):
    """``Lizizen``: every layer is ``x <- x + mixer(shift(norm1(x))) + ff(norm2(x))`` with two RMS
    norms of the same x whose weights are stored around zero, and a token shift in front of the
    mixer; the mixer is ``attention`` (all keys, no rotation, query temperature, distance bias,
    a term of score 0 in the denominator) or ``attention_2`` (two maps per head, query/key norm,
    partial rotation, capped scores, chunked mask, an output gate); the feed-forward is gated
    with clamps and biases.  ``loop`` = (start, stop, times): layers start .. stop - 1 run
    ``times`` times in a row.  config.json keys: ``vocab``, ``width``, ``norm.eps``, ``layers``
    (a list of ``{type, mixer, mlp}``) and ``loop``."""

    layers: Tuple[LizizenLayerConfig, ...] = ()
    loop: Optional[Tuple[int, int, int]] = None
    norm_eps: float = 1e-6
    torch_dtype: str = "bfloat16"

    def run_order(self) -> Tuple[int, ...]:
        """Layer indices in the order they run, a looped stretch repeated."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        start, stop, times = self.loop
        return tuple(range(start)) + tuple(range(start, stop)) * times + tuple(range(stop, n))

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "LizizenConfig":
        name = cfg.get("architecture") or (cfg.get("architectures") or ["Lizizen"])[0]
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"config.json layers[{index}]"
            if not isinstance(raw, Mapping):
                raise ConfigError(f"{where} must be an object")
            kind = raw.get("type")
            m = _mapping(raw, "mixer", where)
            mlp = None
            if raw.get("mlp") is not None:
                mlp = ClampedFeedForwardConfig.parse(_mapping(raw, "mlp", where), where + ".mlp")
            if kind == "attention":
                layers.append(LizizenLayerConfig(type=kind, scored=ScoredAttentionConfig.parse(m, where + ".mixer"),
                                                 mlp=mlp))
            elif kind == "attention_2":
                layers.append(LizizenLayerConfig(
                    type=kind, differential=DifferentialAttentionConfig.parse(m, where + ".mixer"), mlp=mlp))
            else:
                raise ConfigError(f"{where}: layer type {kind!r} is not supported "
                                  "('attention' and 'attention_2' are)")
        loop = None
        if cfg.get("loop") is not None:
            lp = _mapping(cfg, "loop", "config.json")
            start, stop = lp.get("start"), lp.get("stop")
            for key, value in (("start", start), ("stop", stop)):
                if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                    raise ConfigError(f"config.json loop: {key}={value!r} must be a non-negative integer")
            times = _count(lp, "times", "config.json loop")
            if not start <= stop <= len(layers):
                raise ConfigError(f"config.json loop: start={start}, stop={stop} do not fit {len(layers)} layers")
            loop = (start, stop, times)
        eos = cfg.get("eos_token_id")
        eos_ids: Tuple[int, ...] = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(t) for t in eos))
        return LizizenConfig(
            architecture=str(name),
            vocab_size=_count(cfg, "vocab", "config.json"),
            hidden_size=_count(cfg, "width", "config.json"),
            num_hidden_layers=len(layers),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 1 << 20)),
            tie_word_embeddings=False,
            eos_token_ids=eos_ids,
            layers=tuple(layers),
            loop=loop,
            norm_eps=_number(_mapping(cfg, "norm", "config.json"), "eps", "config.json norm"),
            torch_dtype=str(cfg.get("torch_dtype", "bfloat16")),
        )

    def to_json_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            mixer = (layer.scored if layer.type == "attention" else layer.differential).to_json_dict()
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.mlp is None else layer.mlp.to_json_dict()})
        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps}, "layers": layers, "torch_dtype": self.torch_dtype,
        }
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_position_embeddings != 1 << 20:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _rotation(m: Mapping[str, Any], where: str, limit: int, what: str):
    """``rot`` = {base, dims[, scaling: {factor, original, fast, slow}]} -> (base, dims, scaling or None)."""
    r = _mapping(m, "rot", where)
    dims = _count(r, "dims", where + ".rot")
    if dims % 2 or dims > limit:
        raise ConfigError(f"{where}.rot: dims={dims} must be even and at most {what}={limit}")
    scaling = None
    if r.get("scaling") is not None:
        sc = _mapping(r, "scaling", where + ".rot")
        scaling = tuple(_number(sc, key, where + ".rot.scaling") for key in ("factor", "original", "fast", "slow"))
        if min(scaling) <= 0:
            raise ConfigError(f"{where}.rot.scaling: factor, original, fast and slow must be positive")
    base = _number(r, "base", where + ".rot")
    if base <= 1.0:
        raise ConfigError(f"{where}.rot: base={base} must be above 1")
    return base, dims, scaling


def _rotation_json(rot) -> Dict[str, Any]:
    base, dims, scaling = rot
    out: Dict[str, Any] = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


@dataclass(frozen=True)
class WindowedLatentConfig:
    """Latent attention over a sliding window: ``heads`` heads of ``dim`` unrotated and ``rot_dim``
    rotated query/key dims and ``vdim`` value dims over a cached latent of ``kv_rank`` values; the
    queries come through a normed latent of ``q_rank`` values; ``rot`` = (base, dims, scaling or
    None) turns the first ``dims`` of the rotated part in halves; a learned sink per head joins the softmax denominator
    and the heads' outputs pass an element-wise gate."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: int
    rot: Tuple[float, int, Optional[Tuple[float, float, float, float]]]

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "WindowedLatentConfig":
        rot_dim = _count(m, "rot_dim", where)
        rot = _rotation(m, where, rot_dim, "rot_dim")
        window, _ = _window(m, where, keep_allowed=False)
        return WindowedLatentConfig(
            heads=_count(m, "heads", where), dim=_count(m, "dim", where), rot_dim=rot_dim, vdim=_count(m, "vdim", where),
            kv_rank=_count(m, "kv_rank", where), q_rank=_count(m, "q_rank", where), scale=_number(m, "scale", where),
            window=window, rot=rot)

    def to_json_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale, "mask": {"size": self.window},
                "rot": _rotation_json(self.rot)}


@dataclass(frozen=True)
class DeltaRuleConfig:
    """The generalized delta rule: ``heads`` heads whose state is ``dim`` x ``dim``."""

    heads: int
    dim: int

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "DeltaRuleConfig":
        return DeltaRuleConfig(heads=_count(m, "heads", where), dim=_count(m, "dim", where))

    def to_json_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim}


@dataclass(frozen=True)
class GatedFeedForwardConfig:
    """A gated feed-forward of inner width ``ff``."""

    ff: int

    @staticmethod
    def parse(m: Mapping[str, Any], where: str) -> "GatedFeedForwardConfig":
        kind = m.get("kind")
        if kind != "dense":
            raise ConfigError(f"{where}: mlp kind {kind!r} is not supported ('dense' is)")
        return GatedFeedForwardConfig(ff=_count(m, "ff", where))

    def to_json_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class MamivikLayerConfig:
    """``type`` latent_attention: ``latent``; parallel: ``left`` (attention whose values are its
    keys) and ``right`` (delta rule), summed with ``left_scale`` and ``right_scale``."""

    type: str
    latent: Optional[WindowedLatentConfig] = None
    left: Optional[WindowAttentionConfig] = None
    right: Optional[DeltaRuleConfig] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: Optional[GatedFeedForwardConfig] = None


@dataclass(frozen=True)
class MamivikConfig(ModelConfig):
    """``Mamivik``: pre-norm layers ``x <- x + mixer(h + conv(h))`` with ``h = norm1(x)`` and a
    causal convolution of ``canon_taps`` taps per channel, then ``x <- x + ff(norm2(x))``; every
    norm is an RMS norm times one number.  The mixer is latent attention over a window with a
    sink and an output gate (``latent_attention``), or windowed attention whose values are its
    unrotated keys beside a generalized delta rule (``parallel``); the feed-forward is gated with
    the tanh form of GELU.  config.json keys: ``vocab``, ``width``, ``norm.eps``, ``canon.taps``
    and ``layers`` (a list of ``{type, mixer, mlp}``)."""

    layers: Tuple[MamivikLayerConfig, ...] = ()
    norm_eps: float = 1e-5
    canon_taps: int = 1
    torch_dtype: str = "bfloat16"

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "MamivikConfig":
        name = cfg.get("architecture") or (cfg.get("architectures") or ["Mamivik"])[0]
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"config.json layers[{index}]"
            if not isinstance(raw, Mapping):
                raise ConfigError(f"{where} must be an object")
            kind = raw.get("type")
            m = _mapping(raw, "mixer", where)
            mlp = None
            if raw.get("mlp") is not None:
                mlp = GatedFeedForwardConfig.parse(_mapping(raw, "mlp", where), where + ".mlp")
            if kind == "latent_attention":
                layer = MamivikLayerConfig(type=kind, latent=WindowedLatentConfig.parse(m, where + ".mixer"), mlp=mlp)
            elif kind == "parallel":
                left = WindowAttentionConfig.parse(_mapping(m, "left", where + ".mixer"), where + ".mixer.left",
                                                   rotated=True, biases=True, sink=False, head_gate=False,
                                                   keep_allowed=False)
                if left.vdim != left.dim:
                    raise ConfigError(f"{where}.mixer.left: the values are the keys, so vdim={left.vdim} must equal "
                                      f"dim={left.dim}")
                layer = MamivikLayerConfig(
                    type=kind, left=left,
                    right=DeltaRuleConfig.parse(_mapping(m, "right", where + ".mixer"), where + ".mixer.right"),
                    left_scale=_number(m, "left_scale", where + ".mixer"),
                    right_scale=_number(m, "right_scale", where + ".mixer"), mlp=mlp)
            else:
                raise ConfigError(f"{where}: layer type {kind!r} is not supported "
                                  "('latent_attention' and 'parallel' are)")
            layers.append(layer)
        eos = cfg.get("eos_token_id")
        eos_ids: Tuple[int, ...] = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(t) for t in eos))
        return MamivikConfig(
            architecture=str(name),
            vocab_size=_count(cfg, "vocab", "config.json"),
            hidden_size=_count(cfg, "width", "config.json"),
            num_hidden_layers=len(layers),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 1 << 20)),
            tie_word_embeddings=False,
            eos_token_ids=eos_ids,
            layers=tuple(layers),
            norm_eps=_number(_mapping(cfg, "norm", "config.json"), "eps", "config.json norm"),
            canon_taps=_count(_mapping(cfg, "canon", "config.json"), "taps", "config.json canon"),
            torch_dtype=str(cfg.get("torch_dtype", "bfloat16")),
        )

    def to_json_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            if layer.type == "parallel":
                mixer: Dict[str, Any] = {"left": layer.left.to_json_dict(), "right": layer.right.to_json_dict(),
                                         "left_scale": layer.left_scale, "right_scale": layer.right_scale}
            else:
                mixer = layer.latent.to_json_dict()
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.mlp is None else layer.mlp.to_json_dict()})
        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps}, "layers": layers,
            "torch_dtype": self.torch_dtype,
        }
        if self.max_position_embeddings != 1 << 20:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path, "r", encoding="utf-8") as handle:
        cfg = json.load(handle)
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return cfg
