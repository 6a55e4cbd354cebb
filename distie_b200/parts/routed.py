"""Routed feed-forward: every token goes through a few of many small SwiGLU experts, and through a shared one.

``routed_swiglu``: router scores ``s = sigmoid(W_router h)`` from float32 logits; the ``top`` experts with the
largest scores are chosen (ties to the lower index) and weighted by their scores as they are; with
``weight_on="input"`` the weight multiplies what the expert reads, ``sum_e expert_e(s_e h)``, with ``"output"``
what it returns.  A shared expert of the same form runs for every token and is added.  The output stays a sum
still to be done (the routed slices and the shared expert's), which the norm kernel that follows adds up.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..kernels.interface import Terms
from .base import FEED_FORWARDS, Branches, BuildContext, LayerRun, TensorSpec
from .linear import fuse_rows


@FEED_FORWARDS.register("routed_swiglu")
class RoutedSwiGlu:
    """params: ``experts``, ``top``, ``intermediate_size``, ``shared_size`` (None: no shared expert), optional
    ``weight_on`` (``"input"``, default, or ``"output"``).
    tensors (prefix +): ``router [experts, hidden]``; ``e<j>.gate, e<j>.up [ff, hidden]``, ``e<j>.down [hidden, ff]``;
    ``shared.gate, shared.up, shared.down``."""

    graph_safe = True

    def __init__(self, router, gate_up, down, shared_gate_up, shared_down, prm: dict, kernels) -> None:
        self.router, self.gate_up, self.down = router, gate_up, down
        self.shared_gate_up, self.shared_down = shared_gate_up, shared_down
        self.experts, self.top = int(prm["experts"]), int(prm["top"])
        self.scale_input = prm.get("weight_on", "input") == "input"
        self.kernels = kernels

    @staticmethod
    def _check(prm) -> None:
        experts, top = int(prm["experts"]), int(prm["top"])
        if experts < 1 or top < 1 or top > experts or top > 32:
            raise ValueError(f"experts {experts}, top {top}: 1 <= top <= min(experts, 32)")
        if prm.get("weight_on", "input") not in ("input", "output"):
            raise ValueError(f"weight_on {prm['weight_on']!r}: 'input' or 'output'")

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        cls._check(spec.params)
        p, prm = spec.prefix, spec.params
        ff = int(prm["intermediate_size"])
        specs = []
        for e in range(int(prm["experts"])):
            specs += [TensorSpec(f"{p}e{e}.gate", (ff, hidden_size)), TensorSpec(f"{p}e{e}.up", (ff, hidden_size)),
                      TensorSpec(f"{p}e{e}.down", (hidden_size, ff))]
        specs.append(TensorSpec(p + "router", (int(prm["experts"]), hidden_size)))
        if prm.get("shared_size") is not None:
            shared = int(prm["shared_size"])
            specs += [TensorSpec(p + "shared.gate", (shared, hidden_size)), TensorSpec(p + "shared.up", (shared, hidden_size)),
                      TensorSpec(p + "shared.down", (hidden_size, shared))]
        return specs

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "RoutedSwiGlu":
        cls._check(spec.params)
        p, prm, w = spec.prefix, spec.params, ctx.weights
        experts = range(int(prm["experts"]))
        gate_up = torch.stack([fuse_rows([w.matrix(f"{p}e{e}.gate"), w.matrix(f"{p}e{e}.up")]) for e in experts]).contiguous()
        down = torch.stack([w.matrix(f"{p}e{e}.down") for e in experts]).contiguous()
        shared_gate_up = shared_down = None
        if prm.get("shared_size") is not None:
            shared_gate_up = fuse_rows([w.matrix(p + "shared.gate"), w.matrix(p + "shared.up")])
            shared_down = w.matrix(p + "shared.down")
        return cls(w.matrix(p + "router"), gate_up, down, shared_gate_up, shared_down, dict(prm), ctx.kernels)

    def forward(self, x: torch.Tensor, run: LayerRun):
        k = self.kernels

        def routed():
            ids, weights = k.route_top(x, self.router, self.top, "sigmoid")
            return k.routed_swiglu(x, ids, weights, self.gate_up, self.down, self.scale_input)

        if self.shared_gate_up is None:
            return Terms.of(routed())
        # The routed experts and the shared one read the same input and nothing of one another: in a step of few
        # tokens, where each is a chain of short kernels, they run side by side.
        both = Branches.run([routed, lambda: k.linear_split(k.linear_swiglu(x, self.shared_gate_up), self.shared_down)],
                            x.shape[0], x.device)
        return Terms.of(both[0]) + Terms.of(both[1])
