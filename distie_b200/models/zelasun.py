"""Recipe of the Zelasun decoder: typed configuration -> parts and run order.

The design: a token embedding; layers in the order the configuration lists them, each a
``parallel`` block (one layer norm with weight and bias; mixer and dense SwiGLU feed-forward both
read it, and both are added to the residual); a final layer norm; a head that is the embedding
table.  A layer's mixer is either

* ``parallel``: a chunked, unrotated, grouped-query softmax attention with a sigmoid gate per head
  side by side with a gated delta rule, summed with the configuration's two weights, or
* ``mamba2``: a state-space-duality layer.

Tensor names: ``embed``; ``l<i>.norm1`` / ``l<i>.norm1.b``; ``l<i>.mix.*`` (``left.*`` and ``right.*``
in a parallel mixer); ``l<i>.mlp.gate|up|down``; ``final.norm`` / ``final.norm.b``.  Every layer owns
one cache slot: pages of keys and values for the attention of a parallel mixer, state slots for the
recurrences.
"""

from __future__ import annotations

from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture
from ..config.zelasun_config import ZelasunConfig


def _mixer(layer, prefix: str, eps: float) -> PartSpec:
    m = layer.mixer
    if layer.type == "mamba2":
        return PartSpec("mamba2", {"heads": m.heads, "value_dim": m.vdim, "state": m.state, "groups": m.groups,
                                   "norm_groups": m.norm_groups, "taps": m.conv, "eps": eps}, prefix)
    left = PartSpec(
        "gqa_attention",
        {"num_heads": m.left.heads, "num_kv_heads": m.left.kv_heads, "head_dim": m.left.dim,
         "value_dim": m.left.vdim, "scale": m.left.scale, "chunk": m.left.chunk, "gate": "head_sigmoid",
         "qkv_bias": False, "out_bias": False, "window": None, "position": PartSpec("none"),
         "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"}},
        prefix + "left.",
    )
    right = PartSpec(
        "gated_delta_rule",
        {"heads": m.right.heads, "groups": m.right.kv_heads, "key_dim": m.right.dim, "value_dim": m.right.vdim,
         "taps": m.right.conv, "eps": eps},
        prefix + "right.",
    )
    return PartSpec("side_by_side", {"left": left, "right": right, "left_scale": m.left_scale,
                                     "right_scale": m.right_scale}, prefix)


def zelasun_recipe(cfg: ZelasunConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norm = PartSpec("layernorm", {"eps": cfg.eps, "weight": "", "bias": ".b"}, p + "norm1")
        if layer.ff is None:
            feed_forward = PartSpec("none")
        else:
            feed_forward = PartSpec("swiglu", {"intermediate_size": layer.ff, "names": ("gate", "up", "down")}, p + "mlp.")
        layers.append(LayerSpec("parallel", _mixer(layer, p + "mix.", cfg.eps), feed_forward, {"input": norm}))
    return ModelSpec(
        architecture="Zelasun",
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        layers=tuple(layers),
        order=tuple(LayerCall(i, i, True) for i in range(len(layers))),
        final_norm=PartSpec("layernorm", {"eps": cfg.eps, "weight": "", "bias": ".b"}, "final.norm"),
        embedding_name="embed",
        head_name=None,
        eos_token_id=cfg.eos_token_id,
    )


register_architecture("Zelasun", ZelasunConfig, zelasun_recipe)
