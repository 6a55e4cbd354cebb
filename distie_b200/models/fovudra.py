"""Recipe of the Fovudra decoder: typed configuration -> parts and run order.

The design: a token embedding followed by an RMS norm; layers in the order the configuration lists them, each
a ``sandwich`` block (an RMS norm before and after each sublayer, all with a scale stored around zero:
``x += norm_1b(mixer(norm_1(x)))``, ``x += norm_2b(ff(norm_2(x)))``); a final norm; an untied head.  A layer's
mixer is one of

* ``attention``: grouped-query softmax attention with biases on q and k, no value projection (a token's value is
  its key before rotation and norm), rotary positions on part of each head with the frequencies of long waves
  divided, q and k divided by their root mean square per head after the rotation, a window that also keeps the
  request's first tokens;
* ``mlstm``: a matrix memory with exponential input and forget gates under a running maximum;
* ``lightning``: linear attention with a fixed decay per head;

and its feed-forward routes every token through the top few of many small SwiGLU experts, weighted by sigmoid
scores on the expert's input, beside a shared expert.

Tensor names: ``embed``, ``embed.norm``; ``l<i>.norm1|norm1b|norm2|norm2b``; ``l<i>.mix.*`` (biases add ``.b``);
``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.shared.gate|up|down``; ``final.norm``; ``head``.
Every layer owns one cache slot: pages of keys and values for an attention layer, state slots for the others.
"""

from __future__ import annotations

from ..config.fovudra_config import FovudraConfig
from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture


def _norm(eps: float, prefix: str, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"eps": eps, "name": name, "offset": 1.0}, prefix)


def _mixer(layer, prefix: str, eps: float) -> PartSpec:
    m = layer.mixer
    if layer.type == "lightning":
        return PartSpec("decay_attention", {"heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
                                            "decay": tuple(m.decay), "eps": eps}, prefix)
    if layer.type == "mlstm":
        return PartSpec("exp_gate_memory", {"heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
                                            "gate_cap": m.gate_cap, "eps": eps}, prefix)
    scaling = m.rot_scaling
    position = PartSpec("rotary", {
        "head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
        "scaling": None if scaling is None else {"factor": scaling.factor, "low": scaling.low, "high": scaling.high,
                                                 "original": scaling.original},
    })
    return PartSpec(
        "gqa_attention",
        {"num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale, "window": m.window,
         "keep_first": m.keep_first, "values": "keys", "qk_norm": eps, "qkv_bias": True, "out_bias": False,
         "position": position, "bias_suffix": ".b", "names": {"q": "q", "k": "k", "o": "o"}},
        prefix,
    )


def _feed_forward(mlp, prefix: str) -> PartSpec:
    if mlp is None:
        return PartSpec("none")
    return PartSpec("routed_swiglu", {"experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff,
                                      "shared_size": mlp.shared_ff, "weight_on": "input"}, prefix)


def fovudra_recipe(cfg: FovudraConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norms = {"input": _norm(cfg.eps, p, "norm1"), "mixer_out": _norm(cfg.eps, p, "norm1b"),
                 "post_mixer": _norm(cfg.eps, p, "norm2"), "ff_out": _norm(cfg.eps, p, "norm2b")}
        layers.append(LayerSpec("sandwich", _mixer(layer, p + "mix.", cfg.eps), _feed_forward(layer.mlp, p + "mlp."), norms))
    return ModelSpec(
        architecture="Fovudra",
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        layers=tuple(layers),
        order=tuple(LayerCall(i, i, True) for i in range(len(layers))),
        final_norm=_norm(cfg.eps, "final.", "norm"),
        embedding_name="embed",
        head_name="head",
        eos_token_id=cfg.eos_token_id,
        embedding_norm=_norm(cfg.eps, "embed.", "norm"),
    )


register_architecture("Fovudra", FovudraConfig, fovudra_recipe)
