"""A plain, slow Zelasun decoder: one function per mechanism, whole sequences, no cache.

Written from the design's equations only; it shares no code with the engine.  A
sequence is run from its first token, token by token where the design has a
recurrence, so it is the oracle for every way of cutting and batching.

Notation: ``h`` is a mixer's input ``[T, width]``; weights are ``[out, in]`` and
applied as ``h @ W.T``; ``w`` maps a tensor name to its tensor.
"""

from __future__ import annotations

import math

import torch


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    centred = x - mean
    variance = (centred * centred).mean(-1, keepdim=True)
    return centred / torch.sqrt(variance + eps) * weight + bias


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def short_conv(x, taps_weight, bias=None):
    """Causal per-channel convolution over time: ``x [T, C]``, ``taps_weight [C, taps]`` whose last
    column multiplies the current token; zeros stand before the first token."""
    tokens, _ = x.shape
    taps = taps_weight.shape[1]
    out = torch.zeros_like(x)
    for t in range(tokens):
        for back in range(taps):
            if t - back >= 0:
                out[t] += taps_weight[:, taps - 1 - back] * x[t - back]
    if bias is not None:
        out = out + bias
    return out


def chunked_softmax(q, k, v, scale, size):
    """``q [T, heads, dim]``, ``k [T, kv_heads, dim]``, ``v [T, kv_heads, vdim]`` -> ``[T, heads, vdim]``:
    position i sees j <= i of its own chunk of ``size`` positions (chunks counted from position 0)."""
    tokens, heads, _ = q.shape
    rep = heads // k.shape[1]
    out = torch.zeros(tokens, heads, v.shape[2], dtype=q.dtype)
    for i in range(tokens):
        first = (i // size) * size
        for head in range(heads):
            kv = head // rep
            scores = (k[first : i + 1, kv] @ q[i, head]) * scale
            weights = torch.softmax(scores, 0)
            out[i, head] = (weights[:, None] * v[first : i + 1, kv]).sum(0)
    return out


def chunked_attention(h, w, p, prm):
    """Softmax attention without rotation over the token's own chunk, a sigmoid gate per head on the output."""
    heads, kv_heads, dim, vdim = prm["heads"], prm["kv_heads"], prm["dim"], prm["vdim"]
    tokens = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(tokens, heads, dim)
    k = (h @ w[p + "k"].T).reshape(tokens, kv_heads, dim)
    v = (h @ w[p + "v"].T).reshape(tokens, kv_heads, vdim)
    gate = torch.sigmoid(h @ w[p + "g"].T)  # [T, heads]
    out = chunked_softmax(q, k, v, prm["scale"], prm["mask"]["size"]) * gate[:, :, None]
    return out.reshape(tokens, heads * vdim) @ w[p + "o"].T


def delta_rule_scan(q, k, v, beta, decay):
    """``q, k [T, kv_heads, dim]`` (already unit vectors), ``v [T, heads, vdim]``, ``beta, decay [T, heads]``:
    per head ``S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``, S starting at zero."""
    tokens, heads, vdim = v.shape
    dim, rep = q.shape[2], heads // q.shape[1]
    out = torch.zeros(tokens, heads, vdim, dtype=v.dtype)
    for head in range(heads):
        state = torch.zeros(dim, vdim, dtype=v.dtype)
        kv = head // rep
        for t in range(tokens):
            state = decay[t, head] * state
            write = beta[t, head] * (v[t, head] - state.T @ k[t, kv])
            state = state + torch.outer(k[t, kv], write)
            out[t, head] = state.T @ q[t, kv]
    return out


def ssd_scan(x, b, c, dt, rate, skip):
    """``x [T, heads, vdim]``, ``b, c [T, groups, n]``, ``dt [T, heads]``, ``rate, skip [heads]``:
    ``S <- exp(-rate dt) S + dt b x^T; y = S^T c + skip x``, S ``[n, vdim]`` starting at zero."""
    tokens, heads, vdim = x.shape
    n, rep = b.shape[2], heads // b.shape[1]
    y = torch.zeros(tokens, heads, vdim, dtype=x.dtype)
    for head in range(heads):
        state = torch.zeros(n, vdim, dtype=x.dtype)
        grp = head // rep
        for t in range(tokens):
            state = torch.exp(-rate[head] * dt[t, head]) * state + dt[t, head] * torch.outer(b[t, grp], x[t, head])
            y[t, head] = state.T @ c[t, grp] + skip[head] * x[t, head]
    return y


def gated_delta_rule(h, w, p, prm, eps):
    """Per head a matrix state ``S [dim, vdim]``: decay, delta-rule write, read-out after the write."""
    heads, kv_heads, dim, vdim = prm["heads"], prm["kv_heads"], prm["dim"], prm["vdim"]
    tokens = h.shape[0]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(tokens, kv_heads, dim)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(tokens, kv_heads, dim)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(tokens, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)  # [T, heads]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))  # [T, heads]
    gate = silu(h @ w[p + "g"].T).reshape(tokens, heads, vdim)
    out = delta_rule_scan(q, k, v, beta, decay)
    out = rms_unit(out, eps) * w[p + "norm"] * gate
    return out.reshape(tokens, heads * vdim) @ w[p + "o"].T


def parallel_mixer(h, w, p, prm, eps):
    left = chunked_attention(h, w, p + "left.", prm["left"])
    right = gated_delta_rule(h, w, p + "right.", prm["right"], eps)
    return prm["left_scale"] * left + prm["right_scale"] * right


def mamba2(h, w, p, prm, eps):
    """State-space duality layer: per head ``S [state, vdim]``, scalar decay per head and token."""
    heads, vdim, n, groups = prm["heads"], prm["vdim"], prm["state"], prm["groups"]
    parts = prm["norm_groups"]
    inner = heads * vdim
    tokens = h.shape[0]
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner : 2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n :]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(tokens, heads, vdim)
    b = xbc[:, inner : inner + groups * n].reshape(tokens, groups, n)
    c = xbc[:, inner + groups * n :].reshape(tokens, groups, n)
    dt = softplus(dt + w[p + "dt_bias"])  # [T, heads]
    y = ssd_scan(x, b, c, dt, torch.exp(w[p + "A_log"]), w[p + "D"])
    y = y.reshape(tokens, inner) * silu(z)
    y = rms_unit(y.reshape(tokens, parts, inner // parts), eps).reshape(tokens, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def forward(config, w, token_ids, dtype=torch.float64):
    """``(logits [T, vocab], residual after every layer [L, T, width])`` of one whole sequence."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in w.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(token_ids, dtype=torch.long)]
    trail = []
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "parallel":
            delta = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "mamba2":
            delta = mamba2(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            delta = delta + dense_ff(h, w, p + "mlp.")
        x = x + delta
        trail.append(x)
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T
    return logits, torch.stack(trail)


# -- random models ---------------------------------------------------------------
def tensor_shapes(config):
    width, shapes = config["width"], {"embed": (config["vocab"], config["width"])}
    for index, layer in enumerate(config["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1.b"] = (width,)
        if layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            shapes.update({q + "q": (a["heads"] * a["dim"], width), q + "k": (a["kv_heads"] * a["dim"], width),
                           q + "v": (a["kv_heads"] * a["vdim"], width), q + "g": (a["heads"], width),
                           q + "o": (width, a["heads"] * a["vdim"])})
            q = p + "mix.right."
            qk, vv = r["kv_heads"] * r["dim"], r["heads"] * r["vdim"]
            shapes.update({q + "q": (qk, width), q + "q.conv": (qk, r["conv"]), q + "k": (qk, width),
                           q + "k.conv": (qk, r["conv"]), q + "v": (vv, width), q + "v.conv": (vv, r["conv"]),
                           q + "b": (r["heads"], width), q + "A_log": (r["heads"],), q + "norm": (r["vdim"],),
                           q + "a": (r["heads"], width), q + "dt_bias": (r["heads"],), q + "g": (vv, width),
                           q + "o": (width, vv)})
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            q = p + "mix."
            shapes.update({q + "in": (2 * inner + 2 * gn + m["heads"], width), q + "conv": (inner + 2 * gn, m["conv"]),
                           q + "conv.b": (inner + 2 * gn,), q + "dt_bias": (m["heads"],), q + "A_log": (m["heads"],),
                           q + "D": (m["heads"],), q + "norm": (inner,), q + "o": (width, inner)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "mlp.gate": (ff, width), p + "mlp.up": (ff, width), p + "mlp.down": (width, ff)})
    shapes["final.norm"] = shapes["final.norm.b"] = (width,)
    return shapes


def random_weights(config, seed, scale=1.0):
    """Weights rounded to bfloat16 (as checkpoints store them), sized so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.rsplit(".", 1)[-1]
        if len(shape) == 2 and not name.endswith(".conv"):
            t = torch.randn(shape, generator=g) * scale / math.sqrt(shape[1])
            if name == "embed":
                t = torch.randn(shape, generator=g)
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf == "A_log":
            t = torch.log(torch.rand(shape, generator=g) * 1.5 + 0.1)
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) * 0.5 - 1.0
        elif leaf == "D":
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf == "b":  # a bias of a norm or of a convolution
            t = torch.randn(shape, generator=g) * 0.1
        else:  # norm scales
            t = 1.0 + torch.randn(shape, generator=g) * 0.1
        out[name] = t.to(torch.bfloat16).float()
    return out
