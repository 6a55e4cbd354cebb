"""Mixers with a matrix state per head and request instead of a cache of keys: linear recurrences.

Both kinds here keep, per request, a float32 state ``S [key size, value size]`` per head and the last
``taps - 1`` inputs of a short causal convolution, in the cache manager's state slots; a step moves
them on by the tokens it brings, however a prompt was cut.  Per token and head

    S <- g S;   S <- S + k u^T;   o = S^T q

``gated_delta_rule``: ``u = beta (v - S^T k)`` with the decayed S (the write corrects what the state
already returns for this key); q, k and v each pass a short convolution and SiLU; q and k are unit
vectors per head (q times ``key_dim**-0.5``); ``beta = sigmoid(W_b h)``;
``g = exp(-exp(A_log) softplus(W_a h + dt_bias))``; the read-out is RMS-normed per head, scaled by a
weight shared by the heads and gated by ``silu(W_g h)``.

``mamba2`` (state-space duality): one input projection laid out ``[z | x | B | C | dt]``; x, B and C
pass the convolution (with bias) and SiLU; ``dt = softplus(dt + dt_bias)``; ``g = exp(-exp(A_log) dt)``;
``k = B``, ``u = dt x``, ``q = C``, plus a skip ``D x``; the read-out is gated by ``silu(z)`` first and
then RMS-normed in ``norm_groups`` equal parts.

Everything between the projections and the output projection is float32: the projections leave
float32 (the product's accumulator), the convolution, the activations, decays, step sizes, gates and
the state are float32, and only the normed read-out is cast for the output projection.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, BuildContext, LayerRun, StateNeed, TensorSpec
from .linear import Linear, fuse_rows


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule:
    """params: ``heads`` (value heads), ``groups`` (q/k heads; head h reads group ``h // (heads / groups)``),
    ``key_dim``, ``value_dim``, ``taps``, ``eps`` (of the read-out norm).

    tensors (prefix +): ``q, k, v`` (projections), ``q.conv, k.conv, v.conv [channels, taps]``, ``b`` (beta),
    ``a`` (decay), ``A_log, dt_bias [heads]``, ``g`` (gate), ``norm [value_dim]``, ``o``.
    """

    graph_safe = True

    def __init__(self, proj: Linear, conv, out: Linear, vectors: dict, prm: dict, kernels) -> None:
        self.proj, self.conv, self.out = proj, conv, out
        self.vectors = vectors
        self.heads, self.groups = int(prm["heads"]), int(prm["groups"])
        self.key_dim, self.value_dim, self.taps = int(prm["key_dim"]), int(prm["value_dim"]), int(prm["taps"])
        self.eps = float(prm["eps"])
        self.kernels = kernels

    @staticmethod
    def _sizes(prm) -> tuple[int, int, int]:
        heads, groups = int(prm["heads"]), int(prm["groups"])
        if heads < 1 or groups < 1 or heads % groups:
            raise ValueError(f"heads ({heads}) must be a positive multiple of groups ({groups})")
        if int(prm["taps"]) < 1 or int(prm["taps"]) > 16:
            raise ValueError("the short convolution takes 1 to 16 taps")
        return groups * int(prm["key_dim"]), heads * int(prm["value_dim"]), heads

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        p, prm = spec.prefix, spec.params
        qk, vv, heads = cls._sizes(prm)
        taps = int(prm["taps"])
        return [
            TensorSpec(p + "q", (qk, hidden_size)), TensorSpec(p + "q.conv", (qk, taps), "bias"),
            TensorSpec(p + "k", (qk, hidden_size)), TensorSpec(p + "k.conv", (qk, taps), "bias"),
            TensorSpec(p + "v", (vv, hidden_size)), TensorSpec(p + "v.conv", (vv, taps), "bias"),
            TensorSpec(p + "b", (heads, hidden_size)), TensorSpec(p + "A_log", (heads,), "bias"),
            TensorSpec(p + "norm", (int(prm["value_dim"]),), "norm"), TensorSpec(p + "a", (heads, hidden_size)),
            TensorSpec(p + "dt_bias", (heads,), "bias"), TensorSpec(p + "g", (vv, hidden_size)),
            TensorSpec(p + "o", (hidden_size, vv)),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return None

    @classmethod
    def state_need(cls, spec: PartSpec):
        prm = spec.params
        qk, vv, heads = cls._sizes(prm)
        need = {"matrix": StateNeed((heads, int(prm["value_dim"]), int(prm["key_dim"])), torch.float32)}
        if int(prm["taps"]) > 1:
            need["conv"] = StateNeed((int(prm["taps"]) - 1, 2 * qk + vv), torch.float32)
        return need

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "GatedDeltaRule":
        p, w = spec.prefix, ctx.weights
        cls._sizes(spec.params)
        # One product for everything that reads the mixer's input: [q | k | v | beta | decay | gate].
        proj = fuse_rows([w.matrix(p + n) for n in ("q", "k", "v", "b", "a", "g")])
        conv = torch.cat([w.vector(p + n + ".conv") for n in ("q", "k", "v")], dim=0).contiguous()
        vectors = {n: w.vector(p + n) for n in ("A_log", "dt_bias", "norm")}
        return cls(Linear(proj, None, ctx.kernels), conv, Linear(w.matrix(p + "o"), None, ctx.kernels), vectors,
                   dict(spec.params), ctx.kernels)

    def forward(self, x: torch.Tensor, run: LayerRun):
        k = self.kernels
        qk, vv, heads = self.groups * self.key_dim, self.heads * self.value_dim, self.heads
        # The projection stays float32 slices [S, T, n] (the accumulators of a product whose reduction was split over
        # thread blocks, or one slice): what reads it adds the slices up on the way in.
        y = k.linear_split(x, self.proj.weight)
        state = run.state
        mixed = k.short_conv(y[:, :, : 2 * qk + vv], self.conv, None, state["conv"] if self.taps > 1 else None,
                             run.step, "silu")
        at = 2 * qk + vv
        read = k.linear_recurrence(
            "delta", mixed[:, :qk], mixed[:, qk : 2 * qk], mixed[:, 2 * qk :], y[:, :, at + heads : at + 2 * heads],
            y[:, :, at : at + heads], state["matrix"], run.step, heads, self.groups, self.key_dim, self.value_dim,
            decay_rate=self.vectors["A_log"], decay_bias=self.vectors["dt_bias"],
        )
        normed = torch.empty((x.shape[0], vv), dtype=x.dtype, device=x.device)
        k.gated_rmsnorm(read, y[:, :, at + 2 * heads :], self.vectors["norm"], self.eps, self.value_dim, False, normed)
        return k.linear_split(normed, self.out.weight)


@MIXERS.register("mamba2")
class Mamba2:
    """params: ``heads``, ``value_dim``, ``state`` (N), ``groups`` (of B and C; head h reads group
    ``h // (heads / groups)``), ``norm_groups``, ``taps``, ``eps``.

    tensors (prefix +): ``in [2 inner + 2 groups N + heads, hidden]``, ``conv [inner + 2 groups N, taps]``,
    ``conv.b``, ``dt_bias, A_log, D [heads]``, ``norm [inner]``, ``o [hidden, inner]``.
    """

    graph_safe = True

    def __init__(self, proj: Linear, conv, conv_bias, out: Linear, vectors: dict, prm: dict, kernels) -> None:
        self.proj, self.conv, self.conv_bias, self.out = proj, conv, conv_bias, out
        self.vectors = vectors
        self.heads, self.value_dim, self.n = int(prm["heads"]), int(prm["value_dim"]), int(prm["state"])
        self.groups, self.norm_groups, self.taps = int(prm["groups"]), int(prm["norm_groups"]), int(prm["taps"])
        self.eps = float(prm["eps"])
        self.kernels = kernels

    @staticmethod
    def _sizes(prm) -> tuple[int, int]:
        heads, groups = int(prm["heads"]), int(prm["groups"])
        inner = heads * int(prm["value_dim"])
        if heads < 1 or groups < 1 or heads % groups:
            raise ValueError(f"heads ({heads}) must be a positive multiple of groups ({groups})")
        if int(prm["norm_groups"]) < 1 or inner % int(prm["norm_groups"]):
            raise ValueError(f"heads * value_dim ({inner}) must be a multiple of norm_groups ({prm['norm_groups']})")
        if int(prm["taps"]) < 1 or int(prm["taps"]) > 16:
            raise ValueError("the short convolution takes 1 to 16 taps")
        return inner, groups * int(prm["state"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        p, prm = spec.prefix, spec.params
        inner, gn = cls._sizes(prm)
        heads = int(prm["heads"])
        return [
            TensorSpec(p + "in", (2 * inner + 2 * gn + heads, hidden_size)),
            TensorSpec(p + "conv", (inner + 2 * gn, int(prm["taps"])), "bias"),
            TensorSpec(p + "conv.b", (inner + 2 * gn,), "bias"),
            TensorSpec(p + "dt_bias", (heads,), "bias"), TensorSpec(p + "A_log", (heads,), "bias"),
            TensorSpec(p + "D", (heads,), "bias"), TensorSpec(p + "norm", (inner,), "norm"),
            TensorSpec(p + "o", (hidden_size, inner)),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return None

    @classmethod
    def state_need(cls, spec: PartSpec):
        prm = spec.params
        inner, gn = cls._sizes(prm)
        need = {"matrix": StateNeed((int(prm["heads"]), int(prm["value_dim"]), int(prm["state"])), torch.float32)}
        if int(prm["taps"]) > 1:
            need["conv"] = StateNeed((int(prm["taps"]) - 1, inner + 2 * gn), torch.float32)
        return need

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "Mamba2":
        p, w = spec.prefix, ctx.weights
        cls._sizes(spec.params)
        vectors = {n: w.vector(p + n) for n in ("A_log", "dt_bias", "D", "norm")}
        return cls(Linear(w.matrix(p + "in"), None, ctx.kernels), w.vector(p + "conv"), w.vector(p + "conv.b"),
                   Linear(w.matrix(p + "o"), None, ctx.kernels), vectors, dict(spec.params), ctx.kernels)

    def forward(self, x: torch.Tensor, run: LayerRun):
        k = self.kernels
        inner, gn, heads = self.heads * self.value_dim, self.groups * self.n, self.heads
        y = k.linear_split(x, self.proj.weight)  # float32 slices [S, T, n], added up by what reads them
        state = run.state
        mixed = k.short_conv(y[:, :, inner : 2 * inner + 2 * gn], self.conv, self.conv_bias,
                             state["conv"] if self.taps > 1 else None, run.step, "silu")
        dt = y[:, :, 2 * inner + 2 * gn :]
        read = k.linear_recurrence(
            "ssd", mixed[:, inner + gn :], mixed[:, inner : inner + gn], mixed[:, :inner], dt, dt, state["matrix"],
            run.step, heads, self.groups, self.n, self.value_dim, decay_rate=self.vectors["A_log"],
            decay_bias=self.vectors["dt_bias"], skip=self.vectors["D"],
        )
        normed = torch.empty((x.shape[0], inner), dtype=x.dtype, device=x.device)
        k.gated_rmsnorm(read, y[:, :, :inner], self.vectors["norm"], self.eps, inner // self.norm_groups, True, normed)
        return k.linear_split(normed, self.out.weight)
