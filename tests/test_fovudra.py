"""The Fovudra decoder in the engine against the plain implementation (``plain_fovudra``).

Every test that needs a kernel set takes the fixture ``kit``: the plain tensor-op set on the CPU
(``ref_kernels.RefKernels``, which checks the engine's bookkeeping: cache, state slots, batching,
scheduling), and under ``-m gpu`` the CUDA sets in float32 and bfloat16.  Configurations are made
here, with random weights; they differ from one another in every size.
"""

from __future__ import annotations

import copy

import pytest
import torch

import helpers
import plain_fovudra as pf
from ref_kernels import RefKernels

from distie_b200.cache.manager import CacheManager, pages_needed
from distie_b200.config import ConfigError, EngineConfig, FovudraConfig, get_architecture
from distie_b200.engine.batch import BatchEntry, lay_out, views
from distie_b200.engine.engine import Engine, GenerateRequest
from distie_b200.engine.trace_replay import TraceSession
from distie_b200.kernels.interface import KvSlot, RotaryTable, Terms
from distie_b200.models.decoder import model_tensor_specs
from distie_b200.parts import CacheNeed


def _moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": None if shared is None else {"ff": shared}}


def _attention(heads, kv_heads, dim, window, keep, rot_dims, base, scaling, scale, mlp):
    rot = {"dims": rot_dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
                      "mask": {"size": window, "keep_first": keep}, "rot": rot}}


def _mlstm(heads, dim, vdim, cap, mlp):
    return {"type": "mlstm", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


# Small: every branch once; a window of 12 with 3 kept tokens over pages of 8, half of each head rotated.
SMALL = {
    "architecture": "Fovudra", "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _lightning(2, 16, 8, [0.9, 0.97], _moe(6, 2, 32, 48)),
        _attention(4, 2, 16, 12, 3, 8, 10000.0, (4.0, 1.0, 4.0, 32), 0.3, _moe(6, 2, 32, 48)),
        _mlstm(2, 16, 24, 10.0, _moe(6, 2, 32, 48)),
    ],
}
# Awkward: attention first with as many kv heads as heads, one kept token, whole heads rotated without scaling, a
# window of 7 over pages of 4; more kept tokens (9) than a page holds; no kept tokens; a window longer than any
# request; layers without a feed-forward; no shared expert; as many chosen experts as there are; a single head;
# sizes that are no powers of two.
AWKWARD = {
    "architecture": "Fovudra", "vocab": 101, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        _attention(3, 3, 24, 7, 1, 24, 500.0, None, 0.25, None),
        _mlstm(3, 20, 12, 4.0, _moe(5, 3, 40, None)),
        _attention(6, 1, 16, 10, 9, 4, 1e6, (8.0, 1.0, 2.0, 16), 0.2, _moe(2, 2, 24, 56)),
        _lightning(1, 40, 36, [0.6], None),
        _attention(2, 2, 32, 300, 2, 32, 100.0, (2.0, 0.5, 8.0, 64), 0.15, _moe(7, 1, 16, 16)),
        _attention(4, 2, 8, 5, 0, 8, 10000.0, None, 0.5, None),
    ],
}
# Head sizes of real models: in bfloat16 the tensor-core products and attention kernels take these.
WIDE = {
    "architecture": "Fovudra", "vocab": 500, "width": 256, "norm": {"eps": 1e-5},
    "layers": [
        _attention(4, 2, 64, 80, 5, 64, 50000.0, (8.0, 1.0, 4.0, 256), 0.125, _moe(8, 2, 64, 128)),
        _lightning(4, 64, 64, [0.5, 0.9, 0.99, 0.999], _moe(8, 2, 64, 128)),
        _attention(2, 1, 128, 150, 20, 32, 10000.0, None, 0.09, _moe(16, 4, 32, 64)),
        _mlstm(2, 128, 64, 15.0, _moe(8, 2, 64, 128)),
    ],
}
# Memories only: the model asks the cache manager for no pages at all.
NO_PAGES = {
    "architecture": "Fovudra", "vocab": 80, "width": 48, "norm": {"eps": 1e-5},
    "layers": [_mlstm(4, 12, 4, 20.0, _moe(3, 1, 20, None)), _lightning(3, 8, 12, [0.3, 0.8, 0.95], _moe(4, 2, 12, 12))],
}
CONFIGS = {"small": (SMALL, 8, 0), "awkward": (AWKWARD, 4, 1), "wide": (WIDE, 16, 2), "no_pages": (NO_PAGES, 8, 3)}

FP32_TOL = 1e-4    # rms over the vocabulary of the logits' difference, mean taken off, over the logit scale
BF16_TOL = 6e-2

KITS = ["cpu", pytest.param("gpu32", marks=pytest.mark.gpu), pytest.param("gpu16", marks=pytest.mark.gpu)]


ORACLE = {"stored": None}  # the type whose roundings the plain implementation takes on for the kit in use


@pytest.fixture(params=KITS)
def kit(request):
    ORACLE["stored"] = torch.bfloat16 if request.param == "gpu16" else None
    if request.param == "cpu":
        return RefKernels(torch.float32, "cpu")
    from distie_b200.kernels import make_kernels

    return make_kernels(torch.float32 if request.param == "gpu32" else torch.bfloat16, "cuda:0")


def tolerance(kit) -> float:
    return FP32_TOL if kit.dtype == torch.float32 else BF16_TOL


def every_expert(cfg: dict) -> dict:
    """``cfg`` with every router choosing all of its experts: the weights still vary with the token, but no choice can
    be turned around by rounding."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["mlp"] is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return out


def model(name: str, kit=None):
    """The configuration, its page size and random weights.  For the bfloat16 engine the routers choose every expert:
    over hundreds of tokens some choice of a few experts would hang on less than 16-bit activations can tell apart, and
    a choice turned around changes the tokens behind it through the recurrences.  The float32 engines run the choices
    everywhere, and ``test_clear_choices_in_sixteen_bits`` runs them in bfloat16 where they are clear."""
    cfg, page, seed = CONFIGS[name]
    cfg = every_expert(cfg) if kit is not None and kit.dtype != torch.float32 else copy.deepcopy(cfg)
    return cfg, page, pf.random_weights(cfg, seed)


def engine_of(cfg, weights, page, kit, num_blocks: int, max_seqs: int = 4, **knobs):
    arch = get_architecture(cfg["architecture"])
    dtype = "float32" if kit.dtype == torch.float32 else "bfloat16"
    config = EngineConfig(num_blocks=num_blocks, page_size=page, max_seqs=max_seqs, dtype=dtype, device=str(kit.device),
                          decode_graphs=kit.device.type == "cuda", **{"token_budget": 4096, **knobs})
    stored = {k: v.to(torch.bfloat16) for k, v in weights.items()}
    return Engine.assemble(arch, arch.config_cls.from_dict(cfg), stored, kit, config)


def engine_for(name: str, kit, num_blocks: int, max_seqs: int = 4, **knobs):
    cfg, page, weights = model(name, kit)
    return engine_of(cfg, weights, page, kit, num_blocks, max_seqs, **knobs), cfg, weights


def plain_logits(cfg, weights, ids, margins=None) -> torch.Tensor:
    """The oracle: the plain implementation in float64; for the bfloat16 engine with that type's roundings where an
    engine stores 16 bits between two products (and nowhere else), so that both read the same rounded activations."""
    with pf.stored_as(ORACLE["stored"]):
        return pf.forward(cfg, weights, ids, margins=margins).float()


def row_errors(have: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    diff = have.double() - want.double()
    diff = diff - diff.mean(-1, keepdim=True)
    return diff.pow(2).mean(-1).sqrt() / float(want.double().std())


CLOSE_CALL = 0.1  # a gap between router logits that the rounding left between engine and oracle may turn around


def close_calls(cfg, weights, requests, kit) -> dict:
    """Per request and position, the error the bfloat16 engine is allowed (nothing for the float32 engines, which are
    held to ``FP32_TOL`` everywhere): ``BF16_TOL``, and no limit where some router's choice hangs on less than
    ``CLOSE_CALL``."""
    if kit.dtype == torch.float32:
        return {}
    out = {}
    for rid, ids in requests.items():
        margins = []
        plain_logits(cfg, weights, ids, margins)
        allowed = torch.full((len(ids),), BF16_TOL, dtype=torch.float64)
        if margins:
            allowed[torch.stack(margins).min(0).values < CLOSE_CALL] = float("inf")
        out[rid] = allowed
    return out


def assert_close(got: dict, expected: dict, tol: float, what: str, close: dict | None = None) -> None:
    expected = helpers.expected_for(got, expected)
    for rid, want in expected.items():
        errors = row_errors(got[rid], want)
        allowed = (close or {}).get(rid.split("#")[0])
        if allowed is not None:
            assert allowed.numel() < 8 or float(torch.isinf(allowed).double().mean()) <= 0.5, f"{what}: request {rid} is mostly close calls"
            errors = errors / (allowed[: errors.shape[0]] / tol)
        at = int(errors.argmax())
        assert float(errors[at]) <= tol, f"{what}: request {rid}, position {at}: {float(errors[at]):.3e} of the logit scale"


def requests_of(cfg, lengths, seed=20):
    return {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


def step_for(kit, entries):
    layout = lay_out([BatchEntry(*e) for e in entries])
    return views(torch.from_numpy(layout.packed).to(kit.device), layout)[0], layout


def in_slices(x: torch.Tensor) -> torch.Tensor:
    """``x`` as three slices ``[3, T, n]`` whose sum it is exactly, as a split product leaves it."""
    return torch.stack([x * 0.5, x * 0.25, x * 0.25])


def _close(have, want, tol, what):
    scale = float(want.double().abs().max()) or 1.0
    err = float((have.double().cpu() - want.double()).abs().max()) / scale
    assert err <= tol, f"{what}: {err:.3e} of the largest value"


# -- configuration and weights -----------------------------------------------------------------------------
def test_config_reads_every_size_and_names_what_is_missing():
    cfg = FovudraConfig.from_dict(AWKWARD)
    assert (cfg.vocab, cfg.width, cfg.eps, len(cfg.layers)) == (101, 72, 1e-6, 6)
    first = cfg.layers[0].mixer
    assert (first.heads, first.kv_heads, first.dim, first.window, first.keep_first, first.rot_dims) == (3, 3, 24, 7, 1, 24)
    assert first.rot_scaling is None and cfg.layers[0].mlp is None
    assert cfg.layers[2].mixer.rot_scaling.original == 16 and cfg.layers[2].mlp.top == 2 and cfg.layers[2].mlp.shared_ff == 56
    assert cfg.layers[1].mixer.gate_cap == 4.0 and cfg.layers[1].mlp.shared_ff is None
    assert cfg.layers[3].mixer.decay == (0.6,)
    for path, match in (
        (("layers", 1, "mixer", "mask"), r"layers\[1\]\.mixer\.mask"),
        (("layers", 2, "mixer", "gate_cap"), r"layers\[2\]\.mixer\.gate_cap"),
        (("layers", 0, "mlp", "router"), r"layers\[0\]\.mlp\.router"),
        (("norm",), "norm"),
    ):
        broken = copy.deepcopy(SMALL)
        at = broken
        for key in path[:-1]:
            at = at[key]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=match):
            FovudraConfig.from_dict(broken)
    for change, match in (
        (lambda c: c["layers"][0].update(type="mamba"), "mamba"),
        (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "dense"),
        (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
        (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
        (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
        (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    ):
        broken = copy.deepcopy(SMALL)
        change(broken)
        with pytest.raises(ConfigError, match=match):
            FovudraConfig.from_dict(broken)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    cfg = CONFIGS[name][0]
    arch = get_architecture("Fovudra")
    specs = model_tensor_specs(arch.recipe(arch.config_cls.from_dict(cfg)))
    assert {s.name: tuple(s.shape) for s in specs} == {k: tuple(v) for k, v in pf.tensor_shapes(cfg).items()}


def test_random_model_folder_loads_by_its_config(tmp_path):
    from distie_b200.config import read_config
    from distie_b200.weights import write_random_model

    folder = write_random_model(str(tmp_path / "m"), SMALL, seed=3, std=0.1, norm_noise=0.05)
    arch, cfg = read_config(folder)
    assert arch.name == "Fovudra" and cfg.width == 64
    engine = Engine.assemble(arch, cfg, folder, RefKernels(torch.float32),
                             EngineConfig(num_blocks=8, page_size=16, max_seqs=2, dtype="float32", device="cpu", decode_graphs=False))
    out = engine.generate([[1, 2, 3]], max_new_tokens=3, ignore_eos=True)
    assert len(out[0].token_ids) == 3


def test_scaled_rotary_frequencies():
    from distie_b200.parts.position import scaled_frequencies

    for base, dims, scaling in ((10000.0, 32, (4.0, 1.0, 3.0, 64)), (5e5, 128, (8.0, 1.0, 4.0, 8192)), (100.0, 8, (2.0, 0.5, 8.0, 64))):
        want = pf.rotary_frequencies(dims, base, dict(zip(("factor", "low", "high", "original"), scaling)))
        have = scaled_frequencies(base, dims, *scaling)
        assert have.dtype == torch.float32 and float(((have.double() - want).abs() / want).max()) < 1e-7
        assert float((want / pf.rotary_frequencies(dims, base)).min()) < 0.999  # some wave was slowed down


# -- the cache manager: a window gives pages back but for the kept first tokens --------------------------------
class _Pool:
    def __init__(self, n):
        self.free_ids, self.num_free = list(range(n)), n

    def allocate(self, count):
        out, self.free_ids = self.free_ids[:count], self.free_ids[count:]
        self.num_free -= count
        return out

    def free(self, ids):
        self.free_ids += list(ids)
        self.num_free += len(ids)


def test_windowed_group_keeps_the_pages_of_the_first_tokens():
    cache = CacheManager({0: CacheNeed(1, 8, 10, keep_first=5), 1: CacheNeed(1, 8, 10)}, num_pages=16, page_size=4,
                         max_seats=2, max_tokens_per_request=64, pool_factory=_Pool)
    kept = next(g for g in cache.groups if g.need.keep_first)
    plain = next(g for g in cache.groups if not g.need.keep_first)
    seat = cache.open_seat()
    assert cache.grow(seat, 7)
    assert cache.trim(seat, 7) == 0  # nothing lies before the window yet
    assert cache.grow(seat, 30)
    cache.trim(seat, 30)  # positions >= 30 read keys >= 21 (pages 5..) and keys < 5 (pages 0, 1)
    assert kept.seats[seat].first == 5 and kept.pages_of(seat) == [0, 1, 5, 6, 7]
    assert list(kept.host_table[seat, :8]) == [0, 1, -1, -1, -1, 5, 6, 7]
    assert plain.pages_of(seat) == [5, 6, 7]
    assert cache.grow(seat, 41)  # the pages given back are handed out again
    assert kept.pages_of(seat)[-3:] == [2, 3, 4] or set(kept.pages_of(seat)[-3:]) <= set(range(16))
    cache.trim(seat, 41)
    assert kept.seats[seat].first == 8 and kept.pages_of(seat)[:2] == [0, 1]
    cache.close_seat(seat)
    assert kept.pool.num_free == 16 and plain.pool.num_free == 16 and (kept.host_table[seat] == -1).all()


# -- each mechanism alone: ops of the kernel set against the plain functions ------------------------------------
@pytest.mark.parametrize("width", [72, 201, 2304])
def test_norm_of_a_sum_joins_the_residual_and_is_normed_again(kit, width):
    g = torch.Generator().manual_seed(width)
    tokens = 7
    residual = torch.randn(tokens, width, generator=g) * 3 + 0.5
    a, b = torch.randn(2, tokens, width, generator=g), torch.randn(tokens, width, generator=g) * 4
    w_delta, w_out = 1 + torch.randn(width, generator=g) * 0.2, 1 + torch.randn(width, generator=g) * 0.2
    total = a.double().sum(0) + 0.5 * b.double()
    want_res = residual.double() + pf.rms_unit(total, 1e-5) * w_delta.double()
    want = pf.rms_unit(want_res, 1e-6) * w_out.double()
    dev = kit.device
    tol = 1e-5 if kit.dtype == torch.float32 else 2e-2
    res = residual.clone().to(dev)
    out = torch.empty(tokens, width, dtype=kit.dtype, device=dev)
    terms = Terms([(a.to(dev), 1.0), (b.to(dev), 0.5)])
    kit.norm_add_rmsnorm(terms, w_delta.to(dev), 1e-5, res, w_out.to(dev), 1e-6, out)
    _close(res, want_res, 2e-6, "residual")
    _close(out, want, tol, "norm")
    rows = torch.tensor([5, 1], dtype=torch.int32, device=dev)
    res2 = residual.clone().to(dev)
    picked = torch.empty(2, width, dtype=kit.dtype, device=dev)
    kit.norm_add_rmsnorm(terms, w_delta.to(dev), 1e-5, res2, w_out.to(dev), 1e-6, picked, rows)
    _close(res2, residual, 0.0, "residual kept")
    _close(picked, want[[5, 1]], tol, "picked rows")
    # nothing to add: a plain norm; a sum that joins as it is
    res3 = residual.clone().to(dev)
    kit.norm_add_rmsnorm(None, None, 0.0, res3, w_out.to(dev), 1e-6, out)
    _close(out, pf.rms_unit(residual.double(), 1e-6) * w_out.double(), tol, "plain norm")
    kit.norm_add_rmsnorm(b.to(dev), None, 0.0, res3, w_out.to(dev), 1e-6, out)
    _close(res3, residual.double() + b.double(), 2e-6, "plain sum")


def _paged(kit, kv_heads, dim, pages, page_size, table):
    dev = kit.device
    return KvSlot(torch.zeros(pages, kv_heads, page_size, dim, dtype=kit.dtype, device=dev),
                  torch.zeros(pages, kv_heads, page_size, dim, dtype=kit.dtype, device=dev),
                  torch.tensor(table, dtype=torch.int32, device=dev), page_size, pages)


@pytest.mark.parametrize("heads,kv_heads,dim,rot,interleaved,page", [(4, 2, 16, 8, False, 8), (3, 3, 24, 24, False, 4),
                                                                     (2, 1, 64, 32, True, 16), (2, 1, 128, 128, False, 16)])
def test_keys_kept_as_values_rotated_and_normed(kit, heads, kv_heads, dim, rot, interleaved, page):
    g = torch.Generator().manual_seed(dim + rot)
    n, past = 11, 37
    qk = torch.randn(n, (heads + kv_heads) * dim, generator=g) * 2
    bias = torch.randn((heads + kv_heads) * dim, generator=g)
    freqs = pf.rotary_frequencies(rot, 10000.0)
    full = (qk + bias).double()
    q, k = full[:, : heads * dim].reshape(n, heads, dim), full[:, heads * dim :].reshape(n, kv_heads, dim)
    positions = torch.arange(past, past + n)
    if interleaved:
        def turn(x):
            angles = positions.double()[:, None] * freqs[None, :]
            cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
            out = x.clone()
            out[..., 0:rot:2] = x[..., 0:rot:2] * cos - x[..., 1:rot:2] * sin
            out[..., 1:rot:2] = x[..., 1:rot:2] * cos + x[..., 0:rot:2] * sin
            return out
    else:
        def turn(x):
            return pf.rotate_half(x, positions, freqs, rot)
    want_q, want_k = pf.rms_unit(turn(q), 1e-5), pf.rms_unit(turn(k), 1e-5)
    dev = kit.device
    width = pages_needed(past + n, page)
    kv = _paged(kit, kv_heads, dim, width + 1, page, [[-1] * width, list(range(width - 1, -1, -1))])
    step, _ = step_for(kit, [(1, [0] * n, past, ())])
    table = RotaryTable(freqs.float().to(dev), rot, interleaved)
    q_out = torch.empty(n, heads * dim, dtype=kit.dtype, device=dev)
    kit.qk_rope_norm_write(in_slices(qk.to(dev)), bias.to(dev), step, kv, table, heads, kv_heads, dim, 1e-5, q_out)
    kit.check_errors()
    tol = 2e-5 if kit.dtype == torch.float32 else 1e-2
    _close(q_out, want_q.reshape(n, -1), tol, "q")
    pages = kv.block_table[1, (positions // page).to(dev)].long()
    _close(kv.k[pages, :, (positions % page).to(dev)], want_k, tol, "k in its pages")
    _close(kv.v[pages, :, (positions % page).to(dev)], k, tol, "the key as projected, kept as the value")
    # without a norm and without a cache: only q, rotated
    kit.qk_rope_norm_write(qk.to(dev), None, step, None, table, heads, kv_heads, dim, None, q_out)
    _close(q_out, turn(qk.double()[:, : heads * dim].reshape(n, heads, dim)).reshape(n, -1), tol, "q only")


@pytest.mark.parametrize("heads,kv_heads,dim,window,keep,page", [(4, 2, 16, 12, 3, 8), (3, 3, 24, 7, 1, 4), (2, 1, 64, 44, 6, 16),
                                                                 (4, 1, 128, 33, 17, 8), (2, 2, 32, 150, 2, 16), (2, 1, 64, 5, 0, 16)])
def test_window_with_kept_first_keys_that_stand_out(kit, heads, kv_heads, dim, window, keep, page):
    """Keys go through the paged write in portions; attention runs in portions and token by token.  Every query
    looks for one direction.  The last kept key and the first key that is not kept carry it, the latter more
    strongly, and so does every fifth key with a strength of its own: what a token sees just inside its window, just
    outside it and among the first keys decides nearly all of its output."""
    g = torch.Generator().manual_seed(window + keep)
    n = min(2 * window + keep + 9, window + 70)
    q = torch.randn(n, heads, dim, generator=g)
    k = torch.randn(n, kv_heads, dim, generator=g)
    anchor = torch.randn(dim, generator=g)
    anchor = anchor / anchor.norm()
    for j in range(0, n, 5):
        k[j] = (4.0 + (j * 7 % 11) * 0.5) * anchor
    if keep:
        k[keep - 1] = 7.0 * anchor
    k[keep] = 10.0 * anchor
    q = q + 3.0 * anchor
    if kit.dtype != torch.float32:
        q, k = (t.to(torch.bfloat16).float() for t in (q, k))
    scale = 0.7
    want = pf.windowed_softmax(q.double(), k.double(), k.double(), scale, window, keep).reshape(n, heads * dim)
    dev = kit.device
    width = pages_needed(n, page)
    kv = _paged(kit, kv_heads, dim, width + 1, page, [[-1] * width, list(range(width - 1, -1, -1))])
    got, at = [], 0
    cuts = [max(1, keep - 1), 2, 1, max(1, window - keep - 3), 1, 1, 1, 2, window + 1, 1, 1, 3]
    while at < n:
        count = min(cuts.pop(0) if cuts else 1, n - at)
        step, _ = step_for(kit, [(1, [0] * count, at, ())])
        rows = slice(at, at + count)
        qk = torch.cat([q[rows].reshape(count, -1), k[rows].reshape(count, -1)], 1).to(dev)
        q_out = torch.empty(count, heads * dim, dtype=kit.dtype, device=dev)
        kit.qk_rope_norm_write(qk, None, step, kv, None, heads, kv_heads, dim, None, q_out)
        out = torch.empty(count, heads * dim, dtype=kit.dtype, device=dev)
        kit.attention(q_out, out, step, kv, heads, kv_heads, dim, window, scale, None, keep)
        got.append(out.float().cpu())
        at += count
    kit.check_errors()
    _close(torch.cat(got), want, 2e-5 if kit.dtype == torch.float32 else 3e-2, "attention")


@pytest.mark.parametrize("heads,key_dim,value_dim,unit", [(2, 16, 8, False), (3, 20, 12, True), (1, 40, 36, False),
                                                          (2, 128, 64, True), (4, 64, 64, False), (12, 32, 65, True),
                                                          (48, 128, 128, False), (40, 256, 33, True)])
def test_gated_recurrence_in_portions_against_the_whole(kit, heads, key_dim, value_dim, unit):
    """``S <- g S + w k v^T``, ``o = S^T q`` with the decay and the write strength given per token (and a
    normaliser column fed the value 1), or a constant decay per head and no write strength."""
    g = torch.Generator().manual_seed(key_dim + value_dim)
    lengths = {1: 37, 3: 21}
    dev = kit.device
    width = value_dim + 1 if unit else value_dim
    rate = torch.rand(heads, generator=g) * 0.5 + 0.5
    data, want = {}, {}
    for s, n in lengths.items():
        data[s] = {"q": torch.randn(n, heads * key_dim, generator=g) * key_dim ** -0.5, "k": torch.randn(n, heads * key_dim, generator=g),
                   "v": torch.randn(n, heads * value_dim, generator=g), "d": torch.rand(n, heads, generator=g),
                   "w": torch.rand(n, heads, generator=g) * 2}
        d = {key: value.double() for key, value in data[s].items()}
        out = torch.zeros(n, heads, width, dtype=torch.float64)
        for h in range(heads):
            S = torch.zeros(key_dim, width, dtype=torch.float64)
            for t in range(n):
                v = d["v"][t, h * value_dim : (h + 1) * value_dim]
                if unit:
                    v = torch.cat([v, torch.ones(1, dtype=torch.float64)])
                decay, strength = (d["d"][t, h], d["w"][t, h]) if unit else (rate[h].double(), 1.0)
                S = decay * S + strength * torch.outer(d["k"][t, h * key_dim : (h + 1) * key_dim], v)
                out[t, h] = S.T @ d["q"][t, h * key_dim : (h + 1) * key_dim]
        want[s] = out.reshape(n, -1)
    state = torch.zeros(5, heads, width, key_dim, device=dev)
    done, got = {s: 0 for s in lengths}, {s: [] for s in lengths}
    for cut in ([(1, 19), (3, 2)], [(3, 1)], [(1, 1), (3, 17)], [(1, 17), (3, 1)]):
        step, layout = step_for(kit, [(s, [0] * n, done[s], ()) for s, n in cut])
        cat = {key: torch.cat([data[sl.seat][key][sl.past_len : sl.past_len + sl.q_len] for sl in layout.seqs]).to(dev)
               for key in "qkvdw"}
        if unit:
            both = in_slices(torch.cat([cat["d"], cat["w"]], dim=1)) if heads % 2 == 0 else torch.cat([cat["d"], cat["w"]], dim=1)
            decay, write = both[..., :heads], both[..., heads:]
            out = kit.linear_recurrence("gated", cat["q"], cat["k"], cat["v"], decay, write, state, step, heads, heads,
                                        key_dim, width, unit_column=True)
        else:
            out = kit.linear_recurrence("gated", cat["q"], cat["k"], cat["v"], None, None, state, step, heads, heads,
                                        key_dim, width, decay_rate=rate.to(dev))
        for sl in layout.seqs:
            got[sl.seat].append(out[sl.start : sl.start + sl.q_len].cpu())
            done[sl.seat] += sl.q_len
    for s in lengths:
        _close(torch.cat(got[s]), want[s], 2e-5, f"seat {s}")


def test_exponential_gates_under_a_running_maximum(kit):
    """The gates in portions against the whole; the maximum starts at 0, so a request whose first input gates are
    very negative keeps 0 for a while; the read-out's floor is ``exp(-m)``."""
    g = torch.Generator().manual_seed(11)
    heads, cap = 5, 6.0
    lengths = {0: 29, 2: 14}
    raw = {s: (torch.randn(n, heads, generator=g) * 4 - (6.0 if s == 0 else 0.0), torch.randn(n, heads, generator=g) * 4 + 2)
           for s, n in lengths.items()}
    in_bias, forget_bias = torch.randn(heads, generator=g), torch.randn(heads, generator=g) + 1
    want = {}
    for s, (a, b) in raw.items():
        i = pf.soft_cap(a.double() + in_bias.double(), cap)
        f = torch.nn.functional.logsigmoid(pf.soft_cap(b.double() + forget_bias.double(), cap))
        m, rows = torch.zeros(heads, dtype=torch.float64), []
        for t in range(a.shape[0]):
            new = torch.maximum(f[t] + m, i[t])
            rows.append(torch.stack([torch.exp(f[t] + m - new), torch.exp(i[t] - new), torch.exp(-new)]))
            m = new
        want[s] = torch.stack(rows, 1)  # [3, n, heads]
    first_in = pf.soft_cap(raw[0][0][0].double() + in_bias.double(), cap)
    assert float((torch.exp(-first_in) / want[0][2, 0]).max()) > 20  # the 0 the maximum starts from decided the first floor
    dev = kit.device
    state = torch.zeros(4, heads, device=dev)
    done, got = {s: 0 for s in lengths}, {s: [] for s in lengths}
    for cut in ([(0, 3), (2, 1)], [(2, 2)], [(0, 1), (2, 1)], [(0, 25), (2, 10)]):
        step, layout = step_for(kit, [(s, [0] * n, done[s], ()) for s, n in cut])
        both = torch.cat([torch.cat([raw[sl.seat][j][sl.past_len : sl.past_len + sl.q_len] for sl in layout.seqs]) for j in (0, 1)], 1)
        both = in_slices(both.to(dev))
        keep, take, floor = kit.exp_gate_scan(both[:, :, :heads], both[:, :, heads:], in_bias.to(dev), forget_bias.to(dev), cap,
                                              state, step)
        for sl in layout.seqs:
            got[sl.seat].append(torch.stack([t[sl.start : sl.start + sl.q_len].cpu() for t in (keep, take, floor)]))
            done[sl.seat] += sl.q_len
    for s in lengths:
        _close(torch.cat(got[s], 1), want[s], 1e-5, f"gates of seat {s}")
    read = torch.randn(6, 3 * 5, generator=g)
    read[:, 4] *= 1e-3  # a normaliser far below the floor
    floor = torch.rand(6, 3, generator=g) + 0.1
    parts = read.double().reshape(6, 3, 5)
    want_read = parts[:, :, :4] / (torch.maximum(parts[:, :, 4].abs(), floor.double())[:, :, None] + 1e-6)
    _close(kit.stabilized_readout(read.to(dev), floor.to(dev), 3, 4), want_read.reshape(6, 12), 1e-6, "read-out")


@pytest.mark.parametrize("group,sigmoid", [(8, True), (72, True), (640, True), (24, False)])
def test_gated_rmsnorm_with_either_gate(kit, group, sigmoid):
    g = torch.Generator().manual_seed(group)
    tokens, n = 5, 2 * group
    x, gate, weight = torch.randn(tokens, n, generator=g) * 2, torch.randn(tokens, n, generator=g), torch.randn(n, generator=g)
    act = torch.sigmoid(gate.double()) if sigmoid else pf.silu(gate.double())
    want = pf.rms_unit(x.double().reshape(tokens, 2, group), 1e-5).reshape(tokens, n) * weight.double() * act
    dev = kit.device
    out = torch.empty(tokens, n, dtype=kit.dtype, device=dev)
    kit.gated_rmsnorm(x.to(dev), in_slices(gate.to(dev)), weight.to(dev), 1e-5, group, False, out,
                      activation="sigmoid" if sigmoid else "silu")
    _close(out, want, 1e-5 if kit.dtype == torch.float32 else 2e-2, "gated norm")
    act_out = kit.activation(in_slices(x.to(dev))[:, :, 1 : n - 1], "silu" if sigmoid else "none", scale=0.25, scaled_columns=group)
    want_act = pf.silu(x.double()) if sigmoid else x.double().clone()
    want_act = want_act[:, 1 : n - 1]
    want_act[:, :group] *= 0.25
    _close(act_out, want_act, 1e-6, "activation")


@pytest.mark.parametrize("experts,top,width,ff,on_input", [(6, 2, 64, 32, True), (5, 3, 72, 40, True), (2, 2, 48, 24, False),
                                                           (16, 4, 256, 96, True), (7, 1, 40, 12, True), (64, 8, 128, 64, True)])
def test_routed_experts_against_the_plain_loop(kit, experts, top, width, ff, on_input):
    g = torch.Generator().manual_seed(experts * 10 + top)
    tokens = 70 if experts < 64 else 150
    x = torch.randn(tokens, width, generator=g)
    w = {"router": torch.randn(experts, width, generator=g) * 2 / width ** 0.5}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"] = (torch.randn(ff, width, generator=g) / width ** 0.5 for _ in range(2))
        w[f"e{e}.down"] = torch.randn(width, ff, generator=g) / ff ** 0.5
    x, w = x.to(torch.bfloat16).float(), {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    x[3] = x[2]  # equal tokens choose equal experts and give equal rows, wherever they lie in the sorted order
    scores = torch.sigmoid(x.double() @ w["router"].double().T)
    want_weights, want_ids = torch.topk(scores, top)
    wd = {k: v.double() for k, v in w.items()}
    want = torch.zeros(tokens, width, dtype=torch.float64)
    for t in range(tokens):
        for e, s in zip(want_ids[t].tolist(), want_weights[t]):
            want[t] += pf.expert(s * x[t : t + 1].double(), wd, f"e{e}.")[0] if on_input else s * pf.expert(x[t : t + 1].double(), wd, f"e{e}.")[0]
    dev = kit.device
    xd = x.to(dev, kit.dtype)
    ids, weights = kit.route_top(xd, w["router"].to(dev, kit.dtype), top)
    assert ids.dtype == torch.int32 and ids.cpu().tolist() == want_ids.tolist()
    _close(weights, want_weights, 1e-5, "scores of the chosen experts")
    gate_up = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]).to(dev, kit.dtype)
    down = torch.stack([w[f"e{e}.down"] for e in range(experts)]).to(dev, kit.dtype)
    out = kit.routed_swiglu(xd, ids, weights, gate_up, down, on_input)
    assert out.shape == (top, tokens, width) and out.dtype == torch.float32
    total = out.sum(0)
    _close(total, want, 2e-5 if kit.dtype == torch.float32 else 2e-2, "routed output")
    assert torch.equal(total[3], total[2])
    few = kit.routed_swiglu(xd[:3], ids[:3].contiguous(), weights[:3].contiguous(), gate_up, down, on_input)
    # a row does not depend on what else was routed, beyond the rounding of the kernel that serves the step's size
    _close(few.sum(0), total[:3].double().cpu(), 1e-5 if kit.dtype == torch.float32 else 1e-2, "few rows against many")


# -- each kind of layer alone in a model, then all of them ---------------------------------------------------
ALONE = {
    "attention": _attention(4, 2, 16, 9, 2, 12, 3000.0, (4.0, 1.0, 4.0, 16), 0.4, None),
    "mlstm": _mlstm(3, 12, 20, 8.0, None),
    "lightning": _lightning(2, 24, 10, [0.7, 0.99], None),
    "routed": _lightning(1, 8, 8, [0.5], _moe(9, 3, 20, 28)),
}


@pytest.mark.parametrize("kind", list(ALONE))
def test_one_layer_of_a_kind_prefill_against_single_tokens(kit, kind):
    cfg = {"architecture": "Fovudra", "vocab": 60, "width": 56, "norm": {"eps": 1e-5}, "layers": [copy.deepcopy(ALONE[kind])]}
    if kit.dtype != torch.float32:
        cfg = every_expert(cfg)
    weights = pf.random_weights(cfg, 40)
    requests = requests_of(cfg, [41, 6], seed=70)
    expected = {rid: plain_logits(cfg, weights, ids) for rid, ids in requests.items()}
    close = close_calls(cfg, weights, requests, kit)
    for schedule in (helpers.schedule_whole, lambda r: helpers.schedule_tail(r, tail=25)):
        steps = schedule(requests)
        engine = engine_of(cfg, weights, 4, kit, num_blocks=pages_needed(41, 4) + 2, max_seqs=2)
        got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
        assert_close(got, expected, tolerance(kit), kind, close)


@pytest.mark.gpu
def test_clear_choices_in_sixteen_bits():
    """The bfloat16 engine with routers that choose a few experts, on prompts whose every choice is clear (found by
    trying seeds against the plain implementation): whole prompts, then prefill against single tokens."""
    from distie_b200.kernels import make_kernels

    kit = make_kernels(torch.bfloat16, "cuda:0")
    ORACLE["stored"] = torch.bfloat16
    cfg, page, weights = copy.deepcopy(SMALL), 8, pf.random_weights(SMALL, 0)
    requests = {}
    for seed in range(400, 1400):
        ids = helpers.random_ids(cfg["vocab"], 14, seed)
        margins = []
        plain_logits(cfg, weights, ids, margins)
        if float(torch.stack(margins).min()) >= 0.4:
            requests[f"c{len(requests)}"] = ids
            if len(requests) == 3:
                break
    assert len(requests) == 3, "no prompts with clear choices among the seeds tried"
    expected = {rid: plain_logits(cfg, weights, ids) for rid, ids in requests.items()}
    for schedule in (helpers.schedule_whole, lambda r: helpers.schedule_tail(r, tail=9), helpers.schedule_portions):
        steps = schedule(requests)
        engine = engine_of(cfg, weights, page, kit, num_blocks=8, max_seqs=2)
        got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
        assert_close(got, expected, BF16_TOL, "clear choices")
    assert kit.kernel_counts.get("routed_swiglu") and kit.kernel_counts.get("route_top")


LENGTHS = {"small": [70, 1, 29, 51], "awkward": [45, 3, 23, 38], "wide": [230, 97, 2, 140], "no_pages": [33, 5, 18]}
SCHEDULES = {
    "whole": helpers.schedule_whole,
    "tail": lambda r: helpers.schedule_tail(r, tail=30),
    "portions": helpers.schedule_portions,
    "mixed": lambda r: helpers.schedule_mixed(r, seed=5, live_max=3, refeed=1),
}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("mode", list(SCHEDULES))
def test_replay_against_plain(kit, name, mode):
    """Whole prompts, prefill against token-by-token decoding, portions down to two tokens, and batches of unequal
    requests (portions beside single tokens, a request given up and fed again) in a pool made for the schedule's
    peak and three seats, so that pages, seats and state slots are used again."""
    if name == "wide" and kit.device.type == "cpu" and mode != "mixed":
        pytest.skip("the wide configuration runs on the CPU in one mode only: it is slow there")
    cfg, page, weights = model(name, kit)
    requests = requests_of(cfg, LENGTHS[name])
    steps = SCHEDULES[mode](requests)
    peak = helpers.peak_tokens(steps, granule=page)
    engine, _, _ = engine_for(name, kit, num_blocks=pages_needed(peak, page), max_seqs=3)
    session = TraceSession(engine)
    got = helpers.collect(steps, helpers.run_schedule(session, steps))
    expected = {rid: plain_logits(cfg, weights, ids) for rid, ids in requests.items()}
    assert_close(got, expected, tolerance(kit), f"{name}/{mode}", close_calls(cfg, weights, requests, kit))
    assert engine.cache.free_seats == 3 and all(g.pool.num_free == g.num_pages for g in engine.cache.groups)
    if kit.device.type == "cuda":
        ran = kit.kernel_counts
        assert ran.get("linear_recurrence") and ran.get("norm_add_rmsnorm") and ran.get("routed_swiglu") and ran.get("exp_gate_scan")
        if name != "no_pages":
            assert ran.get("qk_rope_norm_write")
        if name == "wide" and kit.dtype == torch.bfloat16 and mode != "tail":
            # head sizes 64 and 128 in bfloat16: prompt portions on the tcgen05 attention, single tokens on the
            # tensor-core decode attention, kept first keys and all
            assert ran.get("attention_prefill_tcgen05") and not ran.get("attention_generic"), ran
            if mode == "mixed":
                assert ran.get("attention_decode_mma"), ran


@pytest.mark.parametrize("name", ["small", "awkward"])
def test_cuts_at_around_and_across_every_edge(kit, name):
    """The first tokens one by one; portions that end just before, at and just after the last kept token, the
    window's first slide and page edges; then single tokens across the next edges."""
    cfg, page, weights = model(name, kit)
    mask = cfg["layers"][1 if name == "small" else 2]["mixer"]["mask"]
    window, keep = mask["size"], mask["keep_first"]
    ids = helpers.random_ids(cfg["vocab"], 3 * window + keep + 11, 77)
    cuts = [max(1, c) for c in (1, 1, 1, keep, 2, window - keep - 4, 2, 1, 1, 1, page - 1, 2, window, 1, 1, window + 1)]
    steps, at = [], 0
    while at < len(ids):
        size = min(cuts.pop(0) if cuts else 1, len(ids) - at)
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": ids[at : at + size], "want": list(range(size))}],
                      "end": ["a"] if at + size == len(ids) else []})
        at += size
    engine, _, _ = engine_for(name, kit, num_blocks=pages_needed(len(ids), page) + 1)
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    assert_close(got, {"a": plain_logits(cfg, weights, ids)}, tolerance(kit), name, close_calls(cfg, weights, {"a": ids}, kit))


def test_long_decoding_keeps_the_state(kit):
    """Two tokens of prompt, then 150 tokens one by one beside another request that comes and goes: the window
    passes over decoded tokens many times and its pages go back to the pool while the first tokens' page stays."""
    cfg, page, weights = model("small", kit)
    long_ids = helpers.random_ids(cfg["vocab"], 152, 5)
    other = helpers.random_ids(cfg["vocab"], 40, 6)
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": long_ids[:2], "want": [0, 1]}], "end": []}]
    for at in range(2, len(long_ids)):
        entries = [{"id": "long", "tokens": [long_ids[at]], "want": [0]}]
        end = ["long"] if at == len(long_ids) - 1 else []
        if 40 <= at < 60:  # another request, four tokens a step, twice over (its seat and pages are used again)
            part = (at - 40) % 10
            entries.append({"id": f"o{(at - 40) // 10}", "tokens": other[4 * part : 4 * part + 4], "want": [3]})
            if part == 9:
                end.append(f"o{(at - 40) // 10}")
        steps.append({"step": at - 1, "entries": entries, "end": end})
    # a pool far smaller than the request: only the window's pages and the first tokens' page are ever held
    engine, _, _ = engine_for("small", kit, num_blocks=pages_needed(40, page) + 6, max_seqs=2, max_model_len=160)
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    want_other = plain_logits(cfg, weights, other)[3::4]
    close = close_calls(cfg, weights, {"long": long_ids, "o0": other}, kit)
    if close:
        close["o0"] = close["o1"] = close["o0"][3::4]
    assert_close(got, {"long": plain_logits(cfg, weights, long_ids), "o0": want_other, "o1": want_other}, tolerance(kit), "long", close)
    if kit.device.type == "cuda":  # steps of single tokens replayed the captured decode step, state and all
        assert engine.runner.use_graphs and engine.runner.graph_replays >= 100


@pytest.mark.parametrize("name", ["small", "awkward", "no_pages"])
def test_greedy_generation_through_the_scheduler(kit, name):
    """``Engine.run``: prompts cut into portions of five beside decoding requests, two seats for three requests, and
    one request sent back and recomputed; every token must be the plain implementation's arg-max (or a near tie)."""
    cfg, page, weights = model(name, kit)
    prompts = [helpers.random_ids(cfg["vocab"], n, 300 + n) for n in (17, 4, 26)]
    new_tokens = 12
    pool = pages_needed(max(len(p) for p in prompts) + new_tokens, page) * 2 + 1
    engine, _, _ = engine_for(name, kit, num_blocks=pool, max_seqs=2, prefill_chunk=5)
    sent_back, seen = [], []

    def on_token(request_id, token, finished):
        if request_id == "g0":
            seen.append(token)
            if len(seen) == 4:
                sent_back.append(engine.scheduler.force_preempt("g0"))

    results = engine.run([GenerateRequest(f"g{i}", p, new_tokens) for i, p in enumerate(prompts)], ignore_eos=True, on_token=on_token)
    assert sent_back == [True] and results[0].preemptions == 1
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == new_tokens
        whole = prompt + result.token_ids[:-1]
        logits = plain_logits(cfg, weights, whole)[len(prompt) - 1 :]
        allowed = close_calls(cfg, weights, {"g": whole}, kit).get("g")
        for index, token in enumerate(result.token_ids):
            best = float(logits[index].max())
            slack = (2e-4 if kit.dtype == torch.float32 else 8e-2) * float(logits[index].std())
            if allowed is not None and bool(torch.isinf(allowed[: len(prompt) + index]).any()):
                break  # a router's close call: from here on the engine may have gone another way
            assert float(logits[index, token]) >= best - slack, f"{result.request_id}: output {index} is no arg-max"


# -- the command line and the trace runner, as a user runs them ---------------------------------------------
@pytest.mark.gpu
def test_command_line_and_trace_runner(tmp_path):
    """``init-random`` writes a Fovudra folder from its configuration file, ``generate`` decodes greedily from it and
    ``bin/trace_run`` replays steps against it (a portion, then portions beside single tokens, then an ended request's
    seat used again): tokens and logits are the plain implementation's."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    from distie_b200.weights import ModelTensors

    ORACLE["stored"] = None  # both child processes run the float32 engine
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    config_file = tmp_path / "cfg.json"
    config_file.write_text(json.dumps(SMALL))
    folder = tmp_path / "model"
    subprocess.run([sys.executable, "-m", "distie_b200", "init-random", "--config", str(config_file), "--out", str(folder),
                    "--seed", "9", "--std", "0.3", "--dtype", "bfloat16"], check=True, env=env, cwd=root, timeout=600)
    stored = ModelTensors(str(folder))
    weights = {name: stored.tensor(name).float() for name in stored.keys()}
    prompt = helpers.random_ids(SMALL["vocab"], 19, 41)
    proc = subprocess.run([sys.executable, "-m", "distie_b200", "generate", "--model", str(folder), "--dtype", "fp32",
                           "--prompt", " ".join(map(str, prompt)), "--max-new-tokens", "8", "--num-blocks", "8",
                           "--ignore-eos"], capture_output=True, text=True, env=env, cwd=root, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    tokens = json.loads(proc.stdout)[0]["token_ids"]
    logits = plain_logits(SMALL, weights, prompt + tokens[:-1])[len(prompt) - 1 :]
    for index, token in enumerate(tokens):
        assert float(logits[index, token]) >= float(logits[index].max()) - 2e-4 * float(logits[index].std())

    a, b = helpers.random_ids(SMALL["vocab"], 40, 42), helpers.random_ids(SMALL["vocab"], 30, 43)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [0, 24]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[25:26], "want": [0]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [22]}, {"id": "a", "tokens": a[26:], "want": [13]}], "end": ["a", "b"]},
        {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [29]}], "end": ["c"]},
    ]
    out = tmp_path / "out"
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                          text=True, env=env, cwd=root, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(4)]
    full_a, full_b = plain_logits(SMALL, weights, a), plain_logits(SMALL, weights, b)
    want = {0: full_a[[0, 24]], 1: torch.stack([full_a[25], full_b[6]]), 2: torch.stack([full_b[29], full_a[39]]), 3: full_b[[29]]}
    for step, rows in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(rows.shape))
        assert float(row_errors(got, rows).max()) <= FP32_TOL, f"step {step}"
