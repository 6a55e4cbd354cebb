"""Two mixers side by side: both read the same input and their outputs are added with fixed weights.

``side_by_side``: ``left_scale * left(h) + right_scale * right(h)``.  The sum is not done here: the
mixer returns the two outputs as a weighted sum still to be done, and the next norm kernel adds it to
the float32 residual.  The pair owns one cache slot; at most one of the two may keep keys in pages, and
their per-request state tensors are told apart by the prefixes ``left.`` and ``right.``.
"""

from __future__ import annotations

from dataclasses import replace

import torch

from ..config.model_spec import PartSpec
from ..kernels.interface import Terms
from .base import MIXERS, BuildContext, LayerRun, StateNeed, TensorSpec, build_part


def _sides(spec: PartSpec):
    return (("left", spec.params["left"]), ("right", spec.params["right"]))


def _named(need, side: str) -> dict:
    if need is None:
        return {}
    if isinstance(need, StateNeed):
        return {side: need}
    return {f"{side}.{name}": item for name, item in need.items()}


@MIXERS.register("side_by_side")
class SideBySide:
    """params: ``left``, ``right`` (PartSpecs of mixers, prefixes included), ``left_scale``, ``right_scale``."""

    def __init__(self, left, right, left_scale: float, right_scale: float) -> None:
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", True) for part in (self.left, self.right))

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        return [t for _, part in _sides(spec) for t in MIXERS.get(part.kind).tensor_specs(part, hidden_size)]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        needs = [need for _, part in _sides(spec) if (need := MIXERS.get(part.kind).cache_need(part)) is not None]
        if len(needs) > 1:
            raise ValueError("only one of two mixers side by side may keep keys and values in pages")
        return needs[0] if needs else None

    @classmethod
    def state_need(cls, spec: PartSpec):
        merged = {}
        for side, part in _sides(spec):
            merged.update(_named(MIXERS.get(part.kind).state_need(part), side))
        return merged or None

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "SideBySide":
        left, right = (build_part(MIXERS, part, ctx) for _, part in _sides(spec))
        return cls(left, right, spec.params["left_scale"], spec.params["right_scale"])

    @staticmethod
    def _state_of(state, side: str):
        if not isinstance(state, dict):
            return None
        if side in state:
            return state[side]
        own = {name[len(side) + 1 :]: t for name, t in state.items() if name.startswith(side + ".")}
        return own or None

    def branches(self, x: torch.Tensor, run: LayerRun):
        """The two mixers as jobs that a block may run side by side; each returns its weighted output."""
        left_run = replace(run, state=self._state_of(run.state, "left"))
        right_run = replace(run, state=self._state_of(run.state, "right"))
        return (lambda: Terms.of(self.left.forward(x, left_run), self.left_scale),
                lambda: Terms.of(self.right.forward(x, right_run), self.right_scale))

    def forward(self, x: torch.Tensor, run: LayerRun):
        left, right = (job() for job in self.branches(x, run))
        return left + right
