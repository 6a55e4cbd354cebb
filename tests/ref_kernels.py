"""Plain tensor-op versions of every kernel, with the kernels' own signatures.

Two uses.  The ``-m gpu`` tests check each CUDA kernel against the function of the
same name here, at sizes the engine does not use.  And the CPU tests hand a
:class:`RefKernels` to the engine in place of the CUDA set, so that cache
bookkeeping, batching, scheduling and trace replay run end to end on a machine
without a GPU.  The product never imports this file.
"""

from __future__ import annotations

import torch

from distie_b200.kernels.interface import KernelSet, KvSlot, RotaryTable, StepTensors, Terms


def embed(ids, table):
    return table[ids.long()].float()


def add_rmsnorm(delta, residual, weight, eps, dtype, rows_index=None):
    """Returns (new residual, normed).  With rows_index only those rows are normed and the residual is unchanged."""
    if delta is not None and delta.dim() == 3:  # float32 slices of a split product
        delta = delta.float().sum(0)
    summed = residual if delta is None else residual + delta.float()
    source = summed if rows_index is None else summed[rows_index.long()]
    variance = (source * source).mean(dim=-1, keepdim=True)
    normed = (source * torch.rsqrt(variance + eps)).to(dtype)
    out = (weight.float() * normed.float()).to(dtype)
    return (summed if rows_index is None else residual), out


def swiglu(gate_up):
    inter = gate_up.shape[1] // 2
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    return (g / (1 + torch.exp(-g)) * u).to(gate_up.dtype)


def rotate(x, positions, rotary: RotaryTable | None):
    """x [T, heads, d] -> rotated, float32 arithmetic, stored back in x.dtype."""
    if rotary is None:
        return x.clone()
    rot = rotary.rotary_dim
    angles = positions.float()[:, None] * rotary.inv_freq.float()[None, :]
    factor = float(getattr(rotary, "factor", 1.0))
    cos, sin = angles.cos()[:, None, :] * factor, angles.sin()[:, None, :] * factor
    xf = x.float()
    out = xf.clone()
    if rotary.interleaved:
        a, b = xf[..., 0:rot:2], xf[..., 1:rot:2]
        out[..., 0:rot:2] = a * cos - b * sin
        out[..., 1:rot:2] = b * cos + a * sin
    else:
        a, b = xf[..., : rot // 2], xf[..., rot // 2 : rot]
        out[..., : rot // 2] = a * cos - b * sin
        out[..., rot // 2 : rot] = b * cos + a * sin
    return out.to(x.dtype)


def rope_kv_write(qkv, step: StepTensors, kv: KvSlot | None, rotary, num_heads, num_kv_heads, head_dim,
                  bias=None, q_out=None):
    if qkv.dim() == 3:  # float32 slices of the projection: sum, add the bias, then as below on a copy
        dense = qkv.float().sum(0)
        if bias is not None:
            dense = dense + bias.float()
        dense = dense.to(q_out.dtype)
        rope_kv_write(dense, step, kv, rotary, num_heads, num_kv_heads, head_dim)
        q_out.copy_(dense[:, : num_heads * head_dim])
        return
    tokens = step.num_tokens
    q_end, k_end = num_heads * head_dim, (num_heads + num_kv_heads) * head_dim
    positions = step.positions[:tokens]
    q = rotate(qkv[:tokens, :q_end].reshape(tokens, num_heads, head_dim), positions, rotary)
    qkv[:tokens, :q_end] = q.reshape(tokens, q_end)
    if q_out is not None:
        q_out.copy_(qkv[:tokens, :q_end])
    if kv is None:
        return
    k = rotate(qkv[:tokens, q_end:k_end].reshape(tokens, num_kv_heads, head_dim), positions, rotary)
    v = qkv[:tokens, k_end:].reshape(tokens, num_kv_heads, head_dim)
    seats = step.seq_seat[step.token_seq[:tokens].long()].long()
    pos = positions.long()
    pages = kv.block_table[seats, pos // kv.page_size].long()
    if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
        raise IndexError("a new token's page is missing from its block table")
    kv.k[pages, :, pos % kv.page_size, :] = k
    kv.v[pages, :, pos % kv.page_size, :] = v


def attention(qkv, step: StepTensors, kv: KvSlot, num_heads, num_kv_heads, head_dim, window, scale, chunk=None):
    """Token by token: gather the visible keys of the token's request from its pages, softmax in float32."""
    tokens = step.num_tokens
    out = torch.zeros((tokens, num_heads * kv.v.shape[-1]), dtype=qkv.dtype, device=qkv.device)
    rep = num_heads // num_kv_heads
    for t in range(tokens):
        pos = int(step.positions[t])
        seat = int(step.seq_seat[int(step.token_seq[t])])
        first = max(0, pos - int(window) + 1) if window else 0
        if chunk:
            first = max(first, pos // int(chunk) * int(chunk))
        keys = torch.arange(first, pos + 1, device=qkv.device)
        pages = kv.block_table[seat, keys // kv.page_size].long()
        if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
            raise IndexError("a block table does not cover the keys a token attends to")
        k = kv.k[pages, :, keys % kv.page_size, :].float()  # [n, kv_heads, d]
        v = kv.v[pages, :, keys % kv.page_size, :].float()
        q = qkv[t, : num_heads * head_dim].reshape(num_heads, head_dim).float()
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        scores = torch.einsum("hd,nhd->hn", q, k) * scale
        probs = torch.softmax(scores, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", probs, v).reshape(-1).to(qkv.dtype)
    return out


def add_layernorm(delta, residual, weight, bias, eps, dtype, rows_index=None):
    """Returns (new residual, normed), like add_rmsnorm."""
    if isinstance(delta, Terms):
        delta = delta.total()
    elif delta is not None and delta.dim() == 3:
        delta = delta.float().sum(0)
    summed = residual if delta is None else residual + delta.float()
    source = summed if rows_index is None else summed[rows_index.long()]
    centred = source - source.mean(dim=-1, keepdim=True)
    variance = (centred * centred).mean(dim=-1, keepdim=True)
    out = (centred / torch.sqrt(variance + eps) * weight.float() + bias.float()).to(dtype)
    return (summed if rows_index is None else residual), out


def token_seats(step: StepTensors):
    return step.seq_seat[step.token_seq[: step.num_tokens].long()].long()


def kv_write(k, v, step: StepTensors, kv: KvSlot):
    tokens = step.num_tokens
    pos = step.positions[:tokens].long()
    pages = kv.block_table[token_seats(step), pos // kv.page_size].long()
    if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
        raise IndexError("a new token's page is missing from its block table")
    kv.k[pages, :, pos % kv.page_size, :] = k[:tokens].reshape(tokens, kv.k.shape[1], kv.k.shape[3]).to(kv.k.dtype)
    kv.v[pages, :, pos % kv.page_size, :] = v[:tokens].reshape(tokens, kv.v.shape[1], kv.v.shape[3]).to(kv.v.dtype)


def whole(x):
    """A float32 matrix, or the sum of the slices ``[S, T, n]`` it was handed over as."""
    return x.float().sum(0) if x.dim() == 3 else x.float()


def head_gate(x, logits, num_heads):
    tokens = x.shape[0]
    logits = whole(logits)
    gated = x.float().reshape(tokens, num_heads, -1) * torch.sigmoid(logits.float())[:, :, None]
    return gated.reshape(tokens, -1).to(x.dtype)


def _silu(z):
    return z * torch.sigmoid(z)


def _softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def short_conv(x, weight, bias, state, step: StepTensors, activation="silu"):
    """Token by token in the step's order: the request's window of inputs lives in ``state[seat]``."""
    tokens, taps = step.num_tokens, weight.shape[1]
    x = whole(x)
    seats = token_seats(step)
    out = torch.zeros((tokens, x.shape[1]), dtype=torch.float32, device=x.device)
    for t in range(tokens):
        seat = int(seats[t])
        current = x[t].float()
        acc = weight[:, taps - 1].float() * current
        for back in range(1, taps):
            acc = acc + weight[:, taps - 1 - back].float() * state[seat, taps - 1 - back]
        if taps > 1:
            state[seat] = torch.cat([state[seat, 1:], current[None]], dim=0)
        if bias is not None:
            acc = acc + bias.float()
        out[t] = _silu(acc) if activation == "silu" else acc
    return out


def linear_recurrence(rule, q, k, v, decay, write, state, step: StepTensors, heads, groups, key_dim, value_dim,
                      decay_rate=None, decay_bias=None, skip=None):
    tokens = step.num_tokens
    decay, write = whole(decay), whole(write)
    seats = token_seats(step)
    out = torch.zeros((tokens, heads * value_dim), dtype=torch.float32, device=q.device)
    rep = heads // groups
    for t in range(tokens):
        seat = int(seats[t])
        for head in range(heads):
            grp = head // rep
            qt = q[t, grp * key_dim : (grp + 1) * key_dim].float()
            kt = k[t, grp * key_dim : (grp + 1) * key_dim].float()
            vt = v[t, head * value_dim : (head + 1) * value_dim].float()
            s = state[seat, head]  # [value_dim, key_dim]
            if rule == "delta":
                qt = qt / torch.sqrt((qt * qt).sum() + 1e-6) * key_dim ** -0.5
                kt = kt / torch.sqrt((kt * kt).sum() + 1e-6)
                g = torch.exp(-torch.exp(decay_rate[head].float()) * _softplus(decay[t, head].float() + decay_bias[head].float()))
                s = g * s
                u = torch.sigmoid(write[t, head].float()) * (vt - s @ kt)
            else:
                dt = _softplus(write[t, head].float() + decay_bias[head].float())
                g = torch.exp(-torch.exp(decay_rate[head].float()) * dt)
                s = g * s
                u = dt * vt
            s = s + torch.outer(u, kt)
            state[seat, head] = s
            read = s @ qt
            if skip is not None:
                read = read + skip[head].float() * vt
            out[t, head * value_dim : (head + 1) * value_dim] = read
    return out


def gated_rmsnorm(x, gate, weight, eps, group, gate_first, dtype):
    tokens, n = x.shape
    xf, gf = x.float(), _silu(whole(gate))
    w = weight.float().repeat(n // weight.numel())
    if gate_first:
        xf = xf * gf
    parts = xf.reshape(tokens, n // group, group)
    normed = (parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)).reshape(tokens, n) * w
    if not gate_first:
        normed = normed * gf
    return normed.to(dtype)


def sample(logits, temperatures, uniforms):
    picks = logits.float().argmax(dim=-1).to(torch.int32)
    if temperatures is None:
        return picks
    for row in range(logits.shape[0]):
        t = float(temperatures[row])
        if t > 0:
            z = logits[row].float() / t
            p = torch.exp(z - z.max())
            cdf = torch.cumsum(p.double(), dim=0)
            target = float(uniforms[row]) * float(cdf[-1])
            picks[row] = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True).clamp(max=logits.shape[1] - 1))
    return picks


class RefKernels(KernelSet):
    """The interface of the CUDA kernel sets, computed with the functions above."""

    def __init__(self, dtype=torch.float32, device="cpu") -> None:
        self.dtype = dtype
        self.device = torch.device(device)
        self.launches = 0

    def embed(self, step, table, residual):
        residual[: step.num_tokens] = embed(step.token_ids[: step.num_tokens], table)

    def add_rmsnorm(self, delta, residual, weight, eps, out, rows_index=None):
        new_residual, normed = add_rmsnorm(delta, residual, weight, eps, self.dtype, rows_index)
        if rows_index is None and delta is not None:
            residual.copy_(new_residual)
        out.copy_(normed)

    def linear(self, x, weight, bias=None, out_dtype=None):
        y = torch.nn.functional.linear(x.float(), weight.float(), bias.float() if bias is not None else None)
        return y.to(out_dtype or self.dtype)

    def swiglu(self, gate_up, out):
        out.copy_(swiglu(gate_up))

    def rope_kv_write(self, qkv, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias=None, q_out=None):
        rope_kv_write(qkv, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias, q_out)

    def attention(self, qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale, chunk=None):
        out.copy_(attention(qkv, step, kv, num_heads, num_kv_heads, head_dim, window, scale, chunk))

    def add_layernorm(self, delta, residual, weight, bias, eps, out, rows_index=None):
        new_residual, normed = add_layernorm(delta, residual, weight, bias, eps, self.dtype, rows_index)
        if rows_index is None and delta is not None:
            residual.copy_(new_residual)
        out.copy_(normed)

    def kv_write(self, k, v, step, kv):
        kv_write(k, v, step, kv)

    def head_gate(self, x, logits, num_heads):
        x.copy_(head_gate(x, logits, num_heads))

    def short_conv(self, x, weight, bias, state, step, activation="silu"):
        return short_conv(x, weight, bias, state, step, activation)

    def linear_recurrence(self, rule, q, k, v, decay, write, state, step, heads, groups, key_dim, value_dim,
                          decay_rate=None, decay_bias=None, skip=None):
        return linear_recurrence(rule, q, k, v, decay, write, state, step, heads, groups, key_dim, value_dim,
                                 decay_rate, decay_bias, skip)

    def gated_rmsnorm(self, x, gate, weight, eps, group, gate_first, out):
        out.copy_(gated_rmsnorm(x, gate, weight, eps, group, gate_first, out.dtype))

    def sample(self, logits, temperatures, uniforms, out_tokens):
        out_tokens.copy_(sample(logits, temperatures, uniforms))

    def check_errors(self):
        return None
