"""Typed configuration of the Fovudra decoder, read from ``config.json`` keys.

``config.json`` gives ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list in which every entry
names its ``type`` (``"attention"``, ``"mlstm"`` or ``"lightning"``), the sizes and constants of its
``mixer`` and its feed-forward ``mlp`` (``{"kind": "moe", "router": {"experts", "top"}, "expert":
{"ff"}, "shared": {"ff"} or null}``, or null for a layer without one).  Nothing has a default: a key
that is missing is an error that names it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .qwen2_config import ConfigError
from .zelasun_config import _count, _divides, _get, _number


@dataclass(frozen=True)
class RotaryScaling:
    """Frequencies rescaled by wavelength: long waves divided by ``factor``, short ones kept, a blend between."""

    factor: float
    low: float
    high: float
    original: float

    @classmethod
    def read(cls, raw, where: str) -> "RotaryScaling":
        out = cls(_number(raw, "factor", where), _number(raw, "low", where), _number(raw, "high", where),
                  _number(raw, "original", where))
        if out.high == out.low:
            raise ConfigError(f"{where}high and {where}low must differ")
        return out


@dataclass(frozen=True)
class WindowedAttentionSizes:
    """Grouped-query softmax attention whose values are its keys, with a window that keeps the first tokens."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int
    rot_dims: int
    rot_base: float
    rot_scaling: RotaryScaling | None

    @classmethod
    def read(cls, raw, where: str) -> "WindowedAttentionSizes":
        mask = _get(raw, "mask", where)
        rot = _get(raw, "rot", where)
        keep = _get(mask, "keep_first", where + "mask.")
        if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
            raise ConfigError(f"{where}mask.keep_first must be a non-negative integer, got {keep!r}")
        scaling = rot.get("scaling") if isinstance(rot, Mapping) else None
        out = cls(_count(raw, "heads", where), _count(raw, "kv_heads", where), _count(raw, "dim", where),
                  _count(raw, "vdim", where), _number(raw, "scale", where), _count(mask, "size", where + "mask."),
                  keep, _count(rot, "dims", where + "rot."), _number(rot, "base", where + "rot."),
                  RotaryScaling.read(scaling, where + "rot.scaling.") if scaling is not None else None)
        _divides(out.kv_heads, out.heads, where + "heads / kv_heads")
        if out.vdim != out.dim:
            raise ConfigError(f"{where}vdim ({out.vdim}) must equal {where}dim ({out.dim}): the values are the keys")
        if out.rot_dims % 2 or out.rot_dims > out.dim:
            raise ConfigError(f"{where}rot.dims ({out.rot_dims}) must be even and at most dim ({out.dim})")
        return out


@dataclass(frozen=True)
class MlstmSizes:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def read(cls, raw, where: str) -> "MlstmSizes":
        return cls(_count(raw, "heads", where), _count(raw, "dim", where), _count(raw, "vdim", where),
                   _number(raw, "gate_cap", where))


@dataclass(frozen=True)
class LightningSizes:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @classmethod
    def read(cls, raw, where: str) -> "LightningSizes":
        decay = _get(raw, "decay", where)
        heads = _count(raw, "heads", where)
        if not isinstance(decay, (list, tuple)) or len(decay) != heads or any(
                isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"{where}decay must list one number per head ({heads})")
        return cls(heads, _count(raw, "dim", where), _count(raw, "vdim", where), tuple(float(d) for d in decay))


@dataclass(frozen=True)
class RoutedFeedForwardSizes:
    experts: int
    top: int
    ff: int
    shared_ff: int | None  # None: no shared expert

    @classmethod
    def read(cls, raw, where: str) -> "RoutedFeedForwardSizes":
        kind = _get(raw, "kind", where)
        if kind != "moe":
            raise ConfigError(f"{where}kind {kind!r}: this design has routed ('moe') feed-forwards only")
        router = _get(raw, "router", where)
        shared = raw.get("shared")
        out = cls(_count(router, "experts", where + "router."), _count(router, "top", where + "router."),
                  _count(_get(raw, "expert", where), "ff", where + "expert."),
                  _count(shared, "ff", where + "shared.") if shared is not None else None)
        if out.top > out.experts:
            raise ConfigError(f"{where}router.top ({out.top}) exceeds {where}router.experts ({out.experts})")
        return out


_MIXERS = {"attention": WindowedAttentionSizes, "mlstm": MlstmSizes, "lightning": LightningSizes}


@dataclass(frozen=True)
class FovudraLayer:
    type: str                                  # "attention" | "mlstm" | "lightning"
    mixer: Any
    mlp: RoutedFeedForwardSizes | None         # None: the layer has no feed-forward


@dataclass(frozen=True)
class FovudraConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[FovudraLayer, ...]
    eos_token_id: int | None = None
    architecture: str = "Fovudra"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FovudraConfig":
        listed = _get(raw, "layers", "")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for index, entry in enumerate(listed):
            where = f"layers[{index}]."
            kind = _get(entry, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}type {kind!r}: this design has {', '.join(repr(k) for k in _MIXERS)} layers")
            mixer = _MIXERS[kind].read(_get(entry, "mixer", where), where + "mixer.")
            mlp = entry.get("mlp")
            layers.append(FovudraLayer(kind, mixer, RoutedFeedForwardSizes.read(mlp, where + "mlp.") if mlp is not None else None))
        eos = raw.get("eos_token_id")
        known = {"architecture", "architectures", "layers", "norm", "vocab", "width", "eos_token_id"}
        return cls(
            vocab=_count(raw, "vocab", ""),
            width=_count(raw, "width", ""),
            eps=_number(_get(raw, "norm", ""), "eps", "norm."),
            layers=tuple(layers),
            eos_token_id=int(eos) if eos is not None else None,
            extra={k: v for k, v in raw.items() if k not in known},
        )
