"""Typed configuration of the Zelasun decoder, read from ``config.json`` keys.

``config.json`` gives ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list in which every
entry names its ``type`` (``"parallel"`` or ``"mamba2"``), the sizes of its ``mixer`` and its
feed-forward ``mlp`` (``{"kind": "dense", "ff": n}`` or null for none).  Nothing has a default:
a key that is missing is an error that names it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .qwen2_config import ConfigError


def _get(raw: Mapping[str, Any], key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw:
        raise ConfigError(f"config.json lacks {where}{key}")
    return raw[key]


def _count(raw, key: str, where: str) -> int:
    value = _get(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or value < 1:
        raise ConfigError(f"{where}{key} must be a positive integer, got {value!r}")
    return value


def _number(raw, key: str, where: str) -> float:
    value = _get(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{where}{key} must be a number, got {value!r}")
    return float(value)


def _divides(small: int, large: int, what: str) -> None:
    if large % small:
        raise ConfigError(f"{what}: {large} is no multiple of {small}")


@dataclass(frozen=True)
class ChunkedAttentionSizes:
    """The softmax half of a ``parallel`` mixer: grouped queries, no rotation, keys of the token's own chunk."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int

    @classmethod
    def read(cls, raw, where: str) -> "ChunkedAttentionSizes":
        out = cls(_count(raw, "heads", where), _count(raw, "kv_heads", where), _count(raw, "dim", where),
                  _count(raw, "vdim", where), _number(raw, "scale", where),
                  _count(_get(raw, "mask", where), "size", where + "mask."))
        _divides(out.kv_heads, out.heads, where + "heads / kv_heads")
        return out


@dataclass(frozen=True)
class DeltaRuleSizes:
    """The recurrent half of a ``parallel`` mixer: the gated delta rule."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def read(cls, raw, where: str) -> "DeltaRuleSizes":
        out = cls(_count(raw, "heads", where), _count(raw, "kv_heads", where), _count(raw, "dim", where),
                  _count(raw, "vdim", where), _count(raw, "conv", where))
        _divides(out.kv_heads, out.heads, where + "heads / kv_heads")
        return out


@dataclass(frozen=True)
class ParallelMixerSizes:
    left: ChunkedAttentionSizes
    right: DeltaRuleSizes
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class Mamba2Sizes:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @classmethod
    def read(cls, raw, where: str) -> "Mamba2Sizes":
        out = cls(_count(raw, "heads", where), _count(raw, "vdim", where), _count(raw, "state", where),
                  _count(raw, "groups", where), _count(raw, "norm_groups", where), _count(raw, "conv", where))
        _divides(out.groups, out.heads, where + "heads / groups")
        _divides(out.norm_groups, out.inner, where + "heads * vdim / norm_groups")
        return out


@dataclass(frozen=True)
class ZelasunLayer:
    type: str                      # "parallel" | "mamba2"
    mixer: Any                     # ParallelMixerSizes | Mamba2Sizes
    ff: int | None                 # width of the dense feed-forward, None: the layer has none


@dataclass(frozen=True)
class ZelasunConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[ZelasunLayer, ...]
    eos_token_id: int | None = None
    architecture: str = "Zelasun"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZelasunConfig":
        layers = []
        listed = _get(raw, "layers", "")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("layers must be a non-empty list")
        for index, entry in enumerate(listed):
            where = f"layers[{index}]."
            kind = _get(entry, "type", where)
            sizes = _get(entry, "mixer", where)
            if kind == "parallel":
                mixer = ParallelMixerSizes(
                    ChunkedAttentionSizes.read(_get(sizes, "left", where + "mixer."), where + "mixer.left."),
                    DeltaRuleSizes.read(_get(sizes, "right", where + "mixer."), where + "mixer.right."),
                    _number(sizes, "left_scale", where + "mixer."), _number(sizes, "right_scale", where + "mixer."),
                )
            elif kind == "mamba2":
                mixer = Mamba2Sizes.read(sizes, where + "mixer.")
            else:
                raise ConfigError(f"{where}type {kind!r}: this design has 'parallel' and 'mamba2' layers")
            mlp = entry.get("mlp")  # null, or absent: the layer has no feed-forward
            ff = None
            if mlp is not None:
                if _get(mlp, "kind", where + "mlp.") != "dense":
                    raise ConfigError(f"{where}mlp.kind {mlp['kind']!r}: this design has dense feed-forwards only")
                ff = _count(mlp, "ff", where + "mlp.")
            layers.append(ZelasunLayer(kind, mixer, ff))
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
