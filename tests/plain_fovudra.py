"""A plain, slow Fovudra decoder: one function per mechanism, whole sequences, no cache.

Written from the design's equations only; it shares no code with the engine.  A sequence is run
from its first token, token by token where the design has a recurrence, so it is the oracle for
every way of cutting and batching.

Notation: ``h`` is a mixer's input ``[T, width]``; weights are ``[out, in]`` and applied as
``h @ W.T``; ``w`` maps a tensor name to its tensor; ``cfg`` is the dictionary of ``config.json``.
"""

from __future__ import annotations

import math

import torch


STORED = None  # a torch dtype: what an engine of that type hands from one product to the next is rounded to it


def stored(x):
    """``x`` as a 16-bit engine stores it between two products (norm outputs, q, k and v, gated read-outs, what an
    expert reads and what it hands to its down projection); unchanged unless :func:`stored_as` is active."""
    return x if STORED is None else x.to(STORED).to(x.dtype)


class stored_as:
    """``with stored_as(torch.bfloat16): forward(...)``: the plain implementation with the roundings of a 16-bit engine
    (everything else stays in the precision of the call): what such an engine may lose, and nothing more."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global STORED
        self.before, STORED = STORED, self.dtype

    def __exit__(self, *exc):
        global STORED
        STORED = self.before


def silu(z):
    return z * torch.sigmoid(z)


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, weight, eps):
    """RMS norm whose weight is stored around zero."""
    return rms_unit(x, eps) * (1.0 + weight)


def normed_input(x, weight, eps):
    """What a sublayer reads: the norm of the residual, as the engine stores it."""
    return stored(zero_centred_norm(x, weight, eps))


# -- rotary positions with scaled frequencies ------------------------------------------------------
def rotary_frequencies(dims, base, scaling=None, dtype=torch.float64):
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for n in range(dims // 2):
        wavelength = 2.0 * math.pi / float(f[n])
        if wavelength < original / high:
            continue
        if wavelength > original / low:
            out[n] = f[n] / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[n] = (1.0 - s) * f[n] / factor + s * f[n]
    return out


def rotate_half(x, positions, freqs, dims):
    """``x [T, heads, dim]``: dimension i of the first ``dims`` is paired with i + dims/2."""
    angles = positions.to(freqs.dtype)[:, None] * freqs[None, :]
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2 : dims]
    out = x.clone()
    out[..., : dims // 2] = u * cos - v * sin
    out[..., dims // 2 : dims] = v * cos + u * sin
    return out


# -- softmax attention with a window and kept first tokens -------------------------------------------
def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def windowed_softmax(q, k, v, scale, size, keep_first):
    """``q [T, heads, dim]``, ``k, v [T, kv_heads, dim]`` -> ``[T, heads, dim]``."""
    tokens, heads, _ = q.shape
    rep = heads // k.shape[1]
    out = torch.zeros(tokens, heads, v.shape[2], dtype=q.dtype)
    for i in range(tokens):
        seen = [j for j in range(i + 1) if visible(i, j, size, keep_first)]
        for head in range(heads):
            g = head // rep
            scores = (k[seen, g] @ q[i, head]) * scale
            weights = torch.softmax(scores, dim=0)
            out[i, head] = weights @ v[seen, g]
    return out


def attention_mixer(h, w, p, m, eps):
    tokens = h.shape[0]
    heads, kv_heads, dim = m["heads"], m["kv_heads"], m["dim"]
    if m["vdim"] != dim:
        raise ValueError("the values are the keys: vdim equals dim")
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(tokens, heads, dim)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(tokens, kv_heads, dim)
    v = stored(k)
    rot = m["rot"]
    freqs = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
    positions = torch.arange(tokens)
    q = stored(rms_unit(rotate_half(q, positions, freqs, rot["dims"]), eps))
    k = stored(rms_unit(rotate_half(k, positions, freqs, rot["dims"]), eps))
    o = windowed_softmax(q, k, v, m["scale"], m["mask"]["size"], m["mask"]["keep_first"])
    return stored(o.reshape(tokens, heads * dim)) @ w[p + "o"].T


# -- matrix memory with exponential gates --------------------------------------------------------------
def soft_cap(z, cap):
    return cap * torch.tanh(z / cap)


def mlstm_mixer(h, w, p, m, eps):
    tokens = h.shape[0]
    heads, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(tokens, heads, dim) * dim ** -0.5
    k = (h @ w[p + "k"].T).reshape(tokens, heads, dim)
    v = (h @ w[p + "v"].T).reshape(tokens, heads, vdim)
    log_in = soft_cap(h @ w[p + "i"].T + w[p + "i.b"], cap)
    log_forget = torch.nn.functional.logsigmoid(soft_cap(h @ w[p + "f"].T + w[p + "f.b"], cap))
    out = torch.zeros(tokens, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        n = torch.zeros(dim, dtype=h.dtype)
        top = torch.zeros((), dtype=h.dtype)
        for t in range(tokens):
            new_top = torch.maximum(log_forget[t, head] + top, log_in[t, head])
            keep = torch.exp(log_forget[t, head] + top - new_top)
            take = torch.exp(log_in[t, head] - new_top)
            S = keep * S + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            top = new_top
            floor = torch.maximum((n @ q[t, head]).abs(), torch.exp(-top))
            out[t, head] = (S.T @ q[t, head]) / (floor + 1e-6)
    out = rms_unit(out, eps).reshape(tokens, heads * vdim) * w[p + "norm"]
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return stored(out) @ w[p + "o"].T


# -- linear attention with a fixed decay per head -------------------------------------------------------
def lightning_mixer(h, w, p, m, eps):
    tokens = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(tokens, heads, dim)
    k = silu(h @ w[p + "k"].T).reshape(tokens, heads, dim)
    v = silu(h @ w[p + "v"].T).reshape(tokens, heads, vdim)
    out = torch.zeros(tokens, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        decay = float(m["decay"][head])
        for t in range(tokens):
            S = decay * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    out = rms_unit(out.reshape(tokens, heads * vdim), eps) * w[p + "norm"]
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return stored(out) @ w[p + "o"].T


# -- routed feed-forward ---------------------------------------------------------------------------------
def expert(h, w, p):
    h = stored(h)
    return stored(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_feed_forward(h, w, p, mlp, margins=None):
    """``margins`` (a list) receives, per token, the gap between the logits of the last expert chosen and the first
    one left out (infinite when every expert is chosen)."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ w[p + "router"].T
    scores = torch.sigmoid(logits)
    if margins is not None:
        ranked = torch.sort(logits, dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < experts else torch.full_like(ranked[:, 0], float("inf")))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(scores[t], top).indices
        for e in chosen.tolist():
            out[t] += expert(scores[t, e] * h[t : t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + expert(h, w, p + "shared.")
    return out


# -- the model -------------------------------------------------------------------------------------------
MIXERS = {"attention": attention_mixer, "mlstm": mlstm_mixer, "lightning": lightning_mixer}


def forward(cfg, w, tokens, dtype=torch.float64, trace=None, margins=None):
    """Logits ``[T, vocab]`` of one sequence; ``trace`` (a list) receives the residual after every layer, ``margins``
    (a list) every router's margins."""
    w = {name: t.to(dtype) for name, t in w.items() if t.is_floating_point()}
    eps = float(cfg["norm"]["eps"])
    x = zero_centred_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
    for index, layer in enumerate(cfg["layers"]):
        p = f"l{index}."
        mixed = MIXERS[layer["type"]](normed_input(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        x = x + zero_centred_norm(mixed, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            fed = routed_feed_forward(normed_input(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"], margins)
            x = x + zero_centred_norm(fed, w[p + "norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return normed_input(x, w["final.norm"], eps) @ w["head"].T


# -- tensors of a configuration, and random ones ---------------------------------------------------------
def tensor_shapes(cfg):
    width, shapes = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "embed.norm": (cfg["width"],)}
    for index, layer in enumerate(cfg["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (width,)
        q = p + "mix."
        if layer["type"] == "attention":
            shapes.update({q + "q": (m["heads"] * m["dim"], width), q + "q.b": (m["heads"] * m["dim"],),
                           q + "k": (m["kv_heads"] * m["dim"], width), q + "k.b": (m["kv_heads"] * m["dim"],),
                           q + "o": (width, m["heads"] * m["vdim"])})
        else:
            qk, vv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            shapes.update({q + "q": (qk, width), q + "k": (qk, width), q + "v": (vv, width), q + "g": (vv, width),
                           q + "o": (width, vv), q + "norm": (vv,)})
            if layer["type"] == "mlstm":
                shapes.update({q + "i": (m["heads"], width), q + "i.b": (m["heads"],), q + "f": (m["heads"], width),
                               q + "f.b": (m["heads"],)})
        mlp = layer.get("mlp")
        if mlp is not None:
            shapes[p + "norm2"] = shapes[p + "norm2b"] = (width,)
            q = p + "mlp."
            shapes[q + "router"] = (mlp["router"]["experts"], width)
            blocks = [(f"e{e}.", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared") is not None:
                blocks.append(("shared.", mlp["shared"]["ff"]))
            for name, ff in blocks:
                shapes.update({q + name + "gate": (ff, width), q + name + "up": (ff, width), q + name + "down": (width, ff)})
    shapes["final.norm"] = (width,)
    shapes["head"] = (cfg["vocab"], width)
    return shapes


def random_weights(cfg, seed, scale=1.0):
    """Weights rounded to bfloat16 (as checkpoints store them), sized so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = torch.randn(shape, generator=g)
        elif leaf == "router":
            t = torch.randn(shape, generator=g) * 6.0 / math.sqrt(shape[1])  # scores well apart: few close calls
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * scale / math.sqrt(shape[1])
        elif leaf == "b":
            t = torch.randn(shape, generator=g) * (1.5 if name.endswith(("i.b", "f.b")) else 0.3)
        elif name.endswith("mix.norm"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.1
        else:  # norm scales stored around zero
            t = torch.randn(shape, generator=g) * 0.1
        out[name] = t.to(torch.bfloat16).float()
    return out
