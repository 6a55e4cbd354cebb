"""SwiGLU feed-forward, dense: ``down(silu(gate(x)) * up(x))``, no biases.

Formula of the reference (worker/src/inference/qwen2/model.py:228-236).  Gate and
up are one product against the row-stacked weight ``[2 * inter, hidden]``.
``none`` is the feed-forward of a layer that has none: it declares nothing and adds nothing.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import FEED_FORWARDS, BuildContext, LayerRun, TensorSpec
from .linear import Linear, fuse_rows


@FEED_FORWARDS.register("swiglu")
class SwiGluFeedForward:
    """params: ``intermediate_size``; optional ``names``: what the names of the gate, up and down matrices add to
    the prefix (default ``gate_proj.weight``, ``up_proj.weight``, ``down_proj.weight``)."""

    _NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")

    def __init__(self, gate_up: Linear, down: Linear, inter: int, kernels) -> None:
        self.gate_up = gate_up
        self.down = down
        self.inter = inter
        self.kernels = kernels

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        p, inter = spec.prefix, int(spec.params["intermediate_size"])
        gate, up, down = spec.params.get("names", cls._NAMES)
        return [
            TensorSpec(p + gate, (inter, hidden_size)),
            TensorSpec(p + up, (inter, hidden_size)),
            TensorSpec(p + down, (hidden_size, inter)),
        ]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "SwiGluFeedForward":
        p, w = spec.prefix, ctx.weights
        gate, up, down = spec.params.get("names", cls._NAMES)
        gate_up = fuse_rows([w.matrix(p + gate), w.matrix(p + up)])
        return cls(
            Linear(gate_up, None, ctx.kernels),
            Linear(w.matrix(p + down), None, ctx.kernels),
            int(spec.params["intermediate_size"]),
            ctx.kernels,
        )

    def forward(self, x: torch.Tensor, run: LayerRun) -> torch.Tensor:
        # The down product's float32 slices are summed by the norm that follows (or by the stream).
        return self.kernels.linear_split(self.kernels.linear_swiglu(x, self.gate_up.weight), self.down.weight)


@FEED_FORWARDS.register("none")
class NoFeedForward:
    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        return []

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "NoFeedForward":
        return cls()

    def forward(self, x: torch.Tensor, run: LayerRun):
        return None
