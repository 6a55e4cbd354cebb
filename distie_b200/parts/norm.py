"""Norms: float32 statistics; each part also does the residual sum that precedes it, in the same kernel.

``rmsnorm``: formula of the reference (worker/src/inference/qwen2/model.py:85-90), the weight
applied after the cast back.
``layernorm``: ``(x - mean) / sqrt(variance + eps) * weight + bias`` with the variance the mean of the
squared deviations, all in float32 up to the store.
"""

from __future__ import annotations

from ..config.model_spec import PartSpec
from ..kernels.interface import Terms
from .base import NORMS, BuildContext, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm:
    """params: ``eps``.  tensors: ``<prefix>weight [hidden]``."""

    def __init__(self, weight, eps: float, kernels) -> None:
        self.weight = weight
        self.eps = float(eps)
        self.kernels = kernels

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        return [TensorSpec(spec.prefix + "weight", (hidden_size,), "norm")]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "RMSNorm":
        return cls(ctx.weights.vector(spec.prefix + "weight"), spec.params["eps"], ctx.kernels)

    def apply(self, delta, residual, out, rows=None) -> None:
        """``residual += delta`` (if any), ``out = norm(residual)``; with ``rows`` only those rows, residual kept."""
        if isinstance(delta, Terms):
            delta = delta.total()
        self.kernels.add_rmsnorm(delta, residual, self.weight, self.eps, out, rows)


@NORMS.register("layernorm")
class LayerNorm:
    """params: ``eps``; ``weight`` and ``bias``: what the tensors' names add to the prefix (defaults
    ``"weight"`` and ``"bias"``)."""

    def __init__(self, weight, bias, eps: float, kernels) -> None:
        self.weight = weight
        self.bias = bias
        self.eps = float(eps)
        self.kernels = kernels

    @staticmethod
    def _names(spec: PartSpec) -> tuple[str, str]:
        return spec.prefix + spec.params.get("weight", "weight"), spec.prefix + spec.params.get("bias", "bias")

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        weight, bias = cls._names(spec)
        return [TensorSpec(weight, (hidden_size,), "norm"), TensorSpec(bias, (hidden_size,), "bias")]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "LayerNorm":
        weight, bias = cls._names(spec)
        return cls(ctx.weights.vector(weight), ctx.weights.vector(bias), spec.params["eps"], ctx.kernels)

    def apply(self, delta, residual, out, rows=None) -> None:
        """``residual += delta`` (if any; a :class:`Terms` is summed in the kernel), ``out = norm(residual)``."""
        self.kernels.add_layernorm(delta, residual, self.weight, self.bias, self.eps, out, rows)
