"""Mixers with a matrix memory per head and request whose decay and write strength are plain numbers.

Both keep, per request and head, a float32 matrix ``S [key size, value size]`` in the cache manager's state
slots and move it on token by token, however a prompt was cut: ``S <- g S + w k v^T``, ``o = S^T q``.

``decay_attention``: q, k and v pass SiLU; ``g`` is a constant per head (a parameter), ``w = 1``; the heads'
read-outs are RMS-normed together with a weight, multiplied by ``sigmoid(W_g h)`` and projected.

``exp_gate_memory``: q is scaled by ``key_dim**-0.5``; a log input gate ``i = cap tanh((W_i h + b_i) / cap)`` and
a log forget gate ``f = logsigmoid(cap tanh((W_f h + b_f) / cap))`` per head, stabilised by a running maximum
``m_t = max(f + m_(t-1), i)`` that starts at 0: ``g = exp(f + m_(t-1) - m_t)``, ``w = exp(i - m_t)``; a vector
``n <- g n + w k`` rides along as one more column of S; the read-out is ``S^T q / (max(|n . q|, exp(-m_t)) + 1e-6)``,
RMS-normed per head, times a weight over all heads, times ``sigmoid(W_g h)``, then projected.

Everything between the projections and the output projection is float32: the projections leave float32 (the
product's accumulators), activations, gates, the running maximum, the state and the read-out stay float32 and
only the normed read-out is cast for the output projection.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, BuildContext, LayerRun, StateNeed, TensorSpec
from .linear import Linear, fuse_rows


def _sizes(prm) -> tuple[int, int, int]:
    heads, key_dim, value_dim = int(prm["heads"]), int(prm["key_dim"]), int(prm["value_dim"])
    if heads < 1 or key_dim < 1 or key_dim > 256 or value_dim < 1:
        raise ValueError(f"heads {heads}, key_dim {key_dim}, value_dim {value_dim}: at least 1 each, key_dim at most 256")
    return heads, key_dim, value_dim


@MIXERS.register("decay_attention")
class DecayAttention:
    """params: ``heads``, ``key_dim``, ``value_dim``, ``decay`` (one number per head), ``eps`` (of the read-out norm).
    tensors (prefix +): ``q, k [heads * key_dim, hidden]``, ``v, g [heads * value_dim, hidden]``,
    ``norm [heads * value_dim]``, ``o [hidden, heads * value_dim]``."""

    graph_safe = True

    def __init__(self, proj: Linear, out: Linear, norm, decay, prm: dict, kernels) -> None:
        self.proj, self.out, self.norm, self.decay = proj, out, norm, decay
        self.heads, self.key_dim, self.value_dim = _sizes(prm)
        self.eps = float(prm["eps"])
        self.kernels = kernels

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        p = spec.prefix
        heads, key_dim, value_dim = _sizes(spec.params)
        if len(spec.params["decay"]) != heads:
            raise ValueError("decay lists one number per head")
        return [
            TensorSpec(p + "q", (heads * key_dim, hidden_size)), TensorSpec(p + "k", (heads * key_dim, hidden_size)),
            TensorSpec(p + "v", (heads * value_dim, hidden_size)), TensorSpec(p + "g", (heads * value_dim, hidden_size)),
            TensorSpec(p + "o", (hidden_size, heads * value_dim)), TensorSpec(p + "norm", (heads * value_dim,), "norm"),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return None

    @classmethod
    def state_need(cls, spec: PartSpec):
        heads, key_dim, value_dim = _sizes(spec.params)
        return {"matrix": StateNeed((heads, value_dim, key_dim), torch.float32)}

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "DecayAttention":
        p, w = spec.prefix, ctx.weights
        proj = fuse_rows([w.matrix(p + n) for n in ("q", "k", "v", "g")])  # one product for all that reads the input
        decay = torch.tensor([float(d) for d in spec.params["decay"]], dtype=torch.float32, device=ctx.device)
        return cls(Linear(proj, None, ctx.kernels), Linear(w.matrix(p + "o"), None, ctx.kernels), w.vector(p + "norm"),
                   decay, dict(spec.params), ctx.kernels)

    def forward(self, x: torch.Tensor, run: LayerRun):
        k = self.kernels
        qk, vv = self.heads * self.key_dim, self.heads * self.value_dim
        y = k.linear_split(x, self.proj.weight)  # float32 slices [S, T, n], added up by what reads them
        act = k.activation(y[:, :, : 2 * qk + vv], "silu")
        read = k.linear_recurrence("gated", act[:, :qk], act[:, qk : 2 * qk], act[:, 2 * qk :], None, None,
                                   run.state["matrix"], run.step, self.heads, self.heads, self.key_dim, self.value_dim,
                                   decay_rate=self.decay)
        normed = torch.empty((x.shape[0], vv), dtype=x.dtype, device=x.device)
        k.gated_rmsnorm(read, y[:, :, 2 * qk + vv :], self.norm, self.eps, vv, False, normed, activation="sigmoid")
        return k.linear_split(normed, self.out.weight)


@MIXERS.register("exp_gate_memory")
class ExpGateMemory:
    """params: ``heads``, ``key_dim``, ``value_dim``, ``gate_cap``, ``eps`` (of the read-out norm).
    tensors (prefix +): ``q, k [heads * key_dim, hidden]``, ``v, g [heads * value_dim, hidden]``, ``i, f [heads,
    hidden]`` with biases ``i.b, f.b [heads]``, ``norm [heads * value_dim]``, ``o [hidden, heads * value_dim]``."""

    graph_safe = True

    def __init__(self, proj: Linear, out: Linear, vectors: dict, prm: dict, kernels) -> None:
        self.proj, self.out, self.vectors = proj, out, vectors
        self.heads, self.key_dim, self.value_dim = _sizes(prm)
        self.cap, self.eps = float(prm["gate_cap"]), float(prm["eps"])
        self.kernels = kernels

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        p = spec.prefix
        heads, key_dim, value_dim = _sizes(spec.params)
        return [
            TensorSpec(p + "q", (heads * key_dim, hidden_size)), TensorSpec(p + "k", (heads * key_dim, hidden_size)),
            TensorSpec(p + "v", (heads * value_dim, hidden_size)),
            TensorSpec(p + "i", (heads, hidden_size)), TensorSpec(p + "i.b", (heads,), "bias"),
            TensorSpec(p + "f", (heads, hidden_size)), TensorSpec(p + "f.b", (heads,), "bias"),
            TensorSpec(p + "g", (heads * value_dim, hidden_size)), TensorSpec(p + "o", (hidden_size, heads * value_dim)),
            TensorSpec(p + "norm", (heads * value_dim,), "norm"),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return None

    @classmethod
    def state_need(cls, spec: PartSpec):
        heads, key_dim, value_dim = _sizes(spec.params)
        # The matrix has one more column per head than a value has elements: the normaliser n.
        return {"matrix": StateNeed((heads, value_dim + 1, key_dim), torch.float32),
                "max": StateNeed((heads,), torch.float32)}

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "ExpGateMemory":
        p, w = spec.prefix, ctx.weights
        proj = fuse_rows([w.matrix(p + n) for n in ("q", "k", "v", "i", "f", "g")])
        vectors = {n: w.vector(p + n) for n in ("i.b", "f.b", "norm")}
        return cls(Linear(proj, None, ctx.kernels), Linear(w.matrix(p + "o"), None, ctx.kernels), vectors,
                   dict(spec.params), ctx.kernels)

    def forward(self, x: torch.Tensor, run: LayerRun):
        k = self.kernels
        heads, qk, vv = self.heads, self.heads * self.key_dim, self.heads * self.value_dim
        y = k.linear_split(x, self.proj.weight)
        at = 2 * qk + vv
        qkv = k.activation(y[:, :, :at], "none", scale=self.key_dim ** -0.5, scaled_columns=qk)
        keep, take, floor = k.exp_gate_scan(y[:, :, at : at + heads], y[:, :, at + heads : at + 2 * heads],
                                            self.vectors["i.b"], self.vectors["f.b"], self.cap, run.state["max"], run.step)
        read = k.linear_recurrence("gated", qkv[:, :qk], qkv[:, qk : 2 * qk], qkv[:, 2 * qk :], keep, take,
                                   run.state["matrix"], run.step, heads, heads, self.key_dim, self.value_dim + 1,
                                   unit_column=True)
        plain = k.stabilized_readout(read, floor, heads, self.value_dim)
        normed = torch.empty((x.shape[0], vv), dtype=x.dtype, device=x.device)
        k.gated_rmsnorm(plain, y[:, :, at + 2 * heads :], self.vectors["norm"], self.eps, self.value_dim, False, normed,
                        activation="sigmoid")
        return k.linear_split(normed, self.out.weight)
