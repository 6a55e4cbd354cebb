"""The Zelasun decoder in the engine against the plain implementation (``plain_zelasun``).

Every test that needs a kernel set takes the fixture ``kit``: the plain tensor-op set on the CPU
(``ref_kernels.RefKernels``, which checks the engine's bookkeeping: cache, state slots, batching,
scheduling), and under ``-m gpu`` the CUDA sets in float32 and bfloat16.  Configurations are
made here, with random weights; they differ from one another in every size.
"""

from __future__ import annotations

import copy

import pytest
import torch

import helpers
import plain_zelasun as pz
from ref_kernels import RefKernels

from distie_b200.cache.manager import CacheManager, pages_needed
from distie_b200.config import ConfigError, EngineConfig, ZelasunConfig, get_architecture
from distie_b200.engine.batch import BatchEntry, lay_out, views
from distie_b200.engine.engine import Engine, GenerateRequest
from distie_b200.engine.trace_replay import TraceSession
from distie_b200.kernels.interface import KvSlot, Terms
from distie_b200.models.decoder import model_tensor_specs
from distie_b200.parts import CacheNeed


def _parallel(left, right, left_scale, right_scale, ff):
    return {"type": "parallel", "mlp": None if ff is None else {"kind": "dense", "ff": ff},
            "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def _mamba(sizes, ff):
    return {"type": "mamba2", "mlp": None if ff is None else {"kind": "dense", "ff": ff}, "mixer": sizes}


# Small: every branch once, chunk of 24 over pages of 16.
SMALL = {
    "architecture": "Zelasun", "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _parallel({"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3, "mask": {"size": 24}},
                  {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "conv": 4}, 0.7, 0.4, 96),
        _mamba({"heads": 4, "vdim": 8, "state": 16, "groups": 2, "norm_groups": 2, "conv": 4}, 96),
    ],
}
# Awkward: values of another size than keys, as many kv heads as heads and a single one, a layer without
# feed-forward, one norm group and one B/C group, 2 and 3 taps, a chunk of 7 over pages of 4, sizes that are
# no powers of two, a mamba2 layer first.
AWKWARD = {
    "architecture": "Zelasun", "vocab": 101, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        _mamba({"heads": 3, "vdim": 12, "state": 20, "groups": 1, "norm_groups": 1, "conv": 2}, None),
        _parallel({"heads": 3, "kv_heads": 3, "dim": 24, "vdim": 40, "scale": 0.25, "mask": {"size": 7}},
                  {"heads": 2, "kv_heads": 2, "dim": 40, "vdim": 20, "conv": 3}, 1.25, 0.75, 50),
        _parallel({"heads": 6, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2, "mask": {"size": 10}},
                  {"heads": 6, "kv_heads": 1, "dim": 8, "vdim": 4, "conv": 5}, 0.5, 1.0, None),
        _mamba({"heads": 4, "vdim": 6, "state": 36, "groups": 4, "norm_groups": 3, "conv": 4}, 40),
    ],
}
# Head sizes of real models: in bfloat16 the tensor-core attention kernels and products take these.
WIDE = {
    "architecture": "Zelasun", "vocab": 500, "width": 256, "norm": {"eps": 1e-5},
    "layers": [
        _parallel({"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 80}},
                  {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 64, "conv": 4}, 0.8, 0.6, 320),
        _mamba({"heads": 8, "vdim": 32, "state": 64, "groups": 2, "norm_groups": 4, "conv": 4}, 320),
        _parallel({"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.09, "mask": {"size": 200}},
                  {"heads": 2, "kv_heads": 1, "dim": 160, "vdim": 48, "conv": 4}, 0.5, 0.5, 320),
    ],
}
# Recurrences only: the model asks the cache manager for no pages at all.
NO_PAGES = {
    "architecture": "Zelasun", "vocab": 80, "width": 48, "norm": {"eps": 1e-5},
    "layers": [_mamba({"heads": 2, "vdim": 16, "state": 8, "groups": 2, "norm_groups": 1, "conv": 3}, 64),
               _mamba({"heads": 4, "vdim": 4, "state": 12, "groups": 1, "norm_groups": 2, "conv": 4}, None)],
}
CONFIGS = {"small": (SMALL, 16, 0), "awkward": (AWKWARD, 4, 1), "wide": (WIDE, 16, 2), "no_pages": (NO_PAGES, 8, 3)}

FP32_TOL = 1e-4    # rms over the vocabulary of the logits' difference, mean taken off, over the logit scale
BF16_TOL = 6e-2


# -- kernel sets ---------------------------------------------------------------------------------------
KITS = ["cpu", pytest.param("gpu32", marks=pytest.mark.gpu), pytest.param("gpu16", marks=pytest.mark.gpu)]


@pytest.fixture(params=KITS)
def kit(request):
    if request.param == "cpu":
        return RefKernels(torch.float32, "cpu")
    from distie_b200.kernels import make_kernels

    return make_kernels(torch.float32 if request.param == "gpu32" else torch.bfloat16, "cuda:0")


def tolerance(kit) -> float:
    return FP32_TOL if kit.dtype == torch.float32 else BF16_TOL


def model(name: str):
    cfg, page, seed = CONFIGS[name]
    return copy.deepcopy(cfg), page, pz.random_weights(cfg, seed)


def engine_for(name: str, kit, num_blocks: int, max_seqs: int = 4, **knobs):
    cfg, page, weights = model(name)
    arch = get_architecture(cfg["architecture"])
    dtype = "float32" if kit.dtype == torch.float32 else "bfloat16"
    config = EngineConfig(num_blocks=num_blocks, page_size=page, max_seqs=max_seqs, dtype=dtype, device=str(kit.device),
                          decode_graphs=kit.device.type == "cuda", **{"token_budget": 4096, **knobs})
    stored = {k: v.to(torch.bfloat16) for k, v in weights.items()}
    return Engine.assemble(arch, arch.config_cls.from_dict(cfg), stored, kit, config), cfg, weights


def plain_logits(cfg, weights, ids) -> torch.Tensor:
    return pz.forward(cfg, weights, ids)[0].float()


def row_errors(have: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    diff = have.double() - want.double()
    diff = diff - diff.mean(-1, keepdim=True)
    return diff.pow(2).mean(-1).sqrt() / float(want.double().std())


def assert_close(got: dict, expected: dict, tol: float, what: str) -> None:
    expected = helpers.expected_for(got, expected)
    for rid, want in expected.items():
        errors = row_errors(got[rid], want)
        at = int(errors.argmax())
        assert float(errors[at]) <= tol, f"{what}: request {rid}, position {at}: {float(errors[at]):.3e} of the logit scale"


def requests_of(cfg, lengths, seed=20):
    return {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


# -- configuration and weights -----------------------------------------------------------------------------
def test_config_reads_every_size_and_names_what_is_missing():
    cfg = ZelasunConfig.from_dict(AWKWARD)
    assert (cfg.vocab, cfg.width, cfg.eps, len(cfg.layers)) == (101, 72, 1e-6, 4)
    assert cfg.layers[0].type == "mamba2" and cfg.layers[0].ff is None and cfg.layers[0].mixer.conv == 2
    left = cfg.layers[1].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.scale, left.chunk) == (3, 3, 24, 40, 0.25, 7)
    assert cfg.layers[2].mixer.right_scale == 1.0 and cfg.layers[3].mixer.norm_groups == 3
    broken = copy.deepcopy(SMALL)
    del broken["layers"][0]["mixer"]["left"]["mask"]
    with pytest.raises(ConfigError, match=r"layers\[0\]\.mixer\.left\.mask"):
        ZelasunConfig.from_dict(broken)
    broken = copy.deepcopy(SMALL)
    broken["layers"][1]["type"] = "lstm"
    with pytest.raises(ConfigError, match="lstm"):
        ZelasunConfig.from_dict(broken)
    broken = copy.deepcopy(SMALL)
    broken["layers"][1]["mlp"] = {"kind": "routed", "ff": 8}
    with pytest.raises(ConfigError, match="routed"):
        ZelasunConfig.from_dict(broken)
    broken = copy.deepcopy(SMALL)
    broken["layers"][0]["mixer"]["right"]["kv_heads"] = 3
    with pytest.raises(ConfigError, match="kv_heads"):
        ZelasunConfig.from_dict(broken)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    cfg = CONFIGS[name][0]
    arch = get_architecture("Zelasun")
    specs = model_tensor_specs(arch.recipe(arch.config_cls.from_dict(cfg)))
    assert {s.name: tuple(s.shape) for s in specs} == {k: tuple(v) for k, v in pz.tensor_shapes(cfg).items()}


def test_random_model_folder_loads_by_its_config(tmp_path):
    from distie_b200.config import read_config
    from distie_b200.weights import write_random_model

    folder = write_random_model(str(tmp_path / "m"), SMALL, seed=3, std=0.1)
    arch, cfg = read_config(folder)
    assert arch.name == "Zelasun" and cfg.width == 64
    engine = Engine.assemble(arch, cfg, folder, RefKernels(torch.float32),
                             EngineConfig(num_blocks=8, page_size=16, max_seqs=2, dtype="float32", device="cpu", decode_graphs=False))
    out = engine.generate([[1, 2, 3]], max_new_tokens=3, ignore_eos=True)
    assert len(out[0].token_ids) == 3


# -- the cache manager: chunks give pages back, values of another size, state by name -------------------------
def test_chunked_group_gives_back_the_pages_before_the_chunk():
    class Pool:
        def __init__(self, n):
            self.free_ids, self.num_free = list(range(n)), n

        def allocate(self, count):
            out, self.free_ids = self.free_ids[:count], self.free_ids[count:]
            self.num_free -= count
            return out

        def free(self, ids):
            self.free_ids += list(ids)
            self.num_free += len(ids)

    cache = CacheManager({0: CacheNeed(1, 8, None, chunk=10), 1: CacheNeed(1, 8)}, num_pages=16, page_size=4,
                         max_seats=2, max_tokens_per_request=64, pool_factory=Pool)
    chunked = next(g for g in cache.groups if g.need.chunk)
    full = next(g for g in cache.groups if not g.need.chunk)
    seat = cache.open_seat()
    assert cache.grow(seat, 23)
    cache.trim(seat, 23)        # positions >= 23 read keys >= 20: pages 0..4 (keys 0..19) go back
    assert chunked.seats[seat].first == 5 and len(chunked.pages_of(seat)) == 1 and len(full.pages_of(seat)) == 6
    cache.trim(seat, 19)        # an earlier count never brings pages back or drops more
    assert chunked.seats[seat].first == 5
    assert chunked.first_needed_page(9) == 0 and chunked.first_needed_page(10) == 2 and chunked.first_needed_page(30) == 7


def test_values_of_another_size_and_named_state_slots():
    from distie_b200.parts import StateNeed

    need = CacheNeed(2, 8, None, None, 12)
    cache = CacheManager({0: need}, {0: {"matrix": StateNeed((2, 3)), "conv": StateNeed((1, 5))}, 1: StateNeed((4,))},
                         num_pages=4, page_size=4, max_seats=2, max_tokens_per_request=16, device="cpu", dtype=torch.float32)
    slot = cache.kv_slot(0)
    assert slot.k.shape == (5, 2, 4, 8) and slot.v.shape == (5, 2, 4, 12)
    assert set(cache.state_slot(0)) == {"matrix", "conv"} and cache.state_slot(1).shape == (3, 4)
    seat = cache.open_seat()
    for t in cache.state_tensors():
        t[seat] += 1
    cache.reset_seat(seat)
    assert all(float(t[seat].abs().sum()) == 0 for t in cache.state_tensors())
    assert cache.state_bytes_per_seat() == 4 * (6 + 5 + 4)


# -- each mechanism alone: an op of the kernel set against the plain function ---------------------------------
def step_for(kit, entries):
    layout = lay_out([BatchEntry(*e) for e in entries])
    return views(torch.from_numpy(layout.packed).to(kit.device), layout)[0], layout


def in_slices(x: torch.Tensor) -> torch.Tensor:
    """``x`` as three slices ``[3, T, n]`` whose sum it is exactly (halves and quarters), as a split product leaves it."""
    return torch.stack([x * 0.5, x * 0.25, x * 0.25])


def _close(have, want, tol, what):
    scale = float(want.double().abs().max()) or 1.0
    err = float((have.double().cpu() - want.double()).abs().max()) / scale
    assert err <= tol, f"{what}: {err:.3e} of the largest value"


@pytest.mark.parametrize("width", [200, 201, 2304])
def test_layernorm_adds_a_weighted_sum_and_norms(kit, width):
    g = torch.Generator().manual_seed(0)
    tokens = 9
    residual = torch.randn(tokens, width, generator=g) * 3 + 1.5
    a, b = torch.randn(2, tokens, width, generator=g), torch.randn(tokens, width, generator=g)
    weight, bias = torch.randn(width, generator=g), torch.randn(width, generator=g)
    want_res = residual.double() + 0.6 * a.double().sum(0) + 0.5 * b.double()
    want = pz.layer_norm(want_res, weight.double(), bias.double(), 1e-5)
    dev = kit.device
    res = residual.clone().to(dev)
    out = torch.empty(tokens, width, dtype=kit.dtype, device=dev)
    kit.add_layernorm(Terms([(a.to(dev), 0.6), (b.to(dev), 0.5)]), res, weight.to(dev), bias.to(dev), 1e-5, out)
    _close(res, want_res, 1e-6, "residual")
    _close(out, want, 1e-5 if kit.dtype == torch.float32 else 2e-2, "norm")
    rows = torch.tensor([7, 2], dtype=torch.int32, device=dev)
    res2 = residual.clone().to(dev)
    picked = torch.empty(2, width, dtype=kit.dtype, device=dev)
    kit.add_layernorm(Terms([(a.to(dev), 0.6), (b.to(dev), 0.5)]), res2, weight.to(dev), bias.to(dev), 1e-5, picked, rows)
    _close(res2, residual, 0.0, "residual kept")
    _close(picked, want[[7, 2]], 1e-5 if kit.dtype == torch.float32 else 2e-2, "picked rows")
    # more terms than the kernel's argument list holds: the slices of three deep products
    many = [torch.randn(11, tokens, width, generator=g) for _ in range(3)]
    want_res = residual.double() + sum(scale * m.double().sum(0) for scale, m in zip((0.5, 1.0, -0.25), many))
    res3 = residual.clone().to(dev)
    kit.add_layernorm(Terms([(m.to(dev), scale) for scale, m in zip((0.5, 1.0, -0.25), many)]), res3, weight.to(dev),
                      bias.to(dev), 1e-5, out)
    _close(res3, want_res, 2e-6, "residual after 33 terms")
    _close(out, pz.layer_norm(want_res, weight.double(), bias.double(), 1e-5), 1e-5 if kit.dtype == torch.float32 else 2e-2,
           "norm after 33 terms")


@pytest.mark.parametrize("taps,channels", [(4, 37), (2, 130), (1, 8), (7, 16), (4, 64), (3, 260)])
def test_short_conv_in_portions_against_the_whole(kit, taps, channels):
    g = torch.Generator().manual_seed(taps)
    lengths = {0: 23, 2: 9}  # seat -> tokens
    x = {s: torch.randn(n, channels, generator=g) for s, n in lengths.items()}
    weight, bias = torch.randn(channels, taps, generator=g), torch.randn(channels, generator=g)
    want = {s: pz.silu(pz.short_conv(x[s].double(), weight.double(), bias.double())) for s in x}
    dev = kit.device
    state = torch.zeros(4, taps - 1, channels, device=dev) if taps > 1 else None
    done = {s: 0 for s in x}
    got = {s: [] for s in x}
    for cut in ([(0, 1), (2, 2)], [(0, 2)], [(2, 1), (0, 5)], [(0, 1)], [(0, 14), (2, 6)]):  # (seat, tokens) per step
        entries = [(s, [0] * n, done[s], ()) for s, n in cut]
        step, layout = step_for(kit, entries)
        rows = torch.cat([x[sl.seat][sl.past_len : sl.past_len + sl.q_len] for sl in layout.seqs])
        padded = torch.cat([rows, torch.zeros(rows.shape[0], 4)], dim=1).to(dev)  # a view with a row stride
        given = padded[:, :channels] if taps != 4 else in_slices(padded)[:, :, :channels]  # a matrix, or slices of one
        out = kit.short_conv(given, weight.to(dev), bias.to(dev), state, step, "silu")
        for sl in layout.seqs:
            got[sl.seat].append(out[sl.start : sl.start + sl.q_len].cpu())
            done[sl.seat] += sl.q_len
    for s in x:
        assert done[s] == lengths[s]
        _close(torch.cat(got[s]), want[s], 1e-5, f"seat {s}")


@pytest.mark.parametrize("rule,heads,groups,key_dim,value_dim", [
    ("delta", 4, 2, 16, 8), ("delta", 2, 2, 40, 20), ("delta", 3, 1, 160, 18), ("delta", 1, 1, 128, 33),
    ("ssd", 4, 2, 16, 8), ("ssd", 3, 1, 20, 12), ("ssd", 2, 2, 64, 40), ("ssd", 1, 1, 200, 5),
    # many columns: the kernel then gives a column fewer lanes
    ("delta", 48, 2, 128, 128), ("ssd", 12, 1, 100, 64), ("delta", 12, 4, 256, 64), ("ssd", 64, 1, 64, 64),
    ("ssd", 48, 2, 256, 128),
])
def test_linear_recurrence_in_portions_against_the_whole(kit, rule, heads, groups, key_dim, value_dim):
    g = torch.Generator().manual_seed(key_dim)
    lengths = {1: 37, 3: 21}
    dev = kit.device
    data = {}
    for s, n in lengths.items():
        data[s] = {"q": torch.randn(n, groups * key_dim, generator=g), "k": torch.randn(n, groups * key_dim, generator=g),
                   "v": torch.randn(n, heads * value_dim, generator=g), "d": torch.randn(n, heads, generator=g),
                   "w": torch.randn(n, heads, generator=g)}
    rate, bias, skip = torch.randn(heads, generator=g) * 0.5, torch.randn(heads, generator=g), torch.randn(heads, generator=g)
    want = {}
    for s, n in lengths.items():
        d = {k: v.double() for k, v in data[s].items()}
        q, k = d["q"].reshape(n, groups, key_dim), d["k"].reshape(n, groups, key_dim)
        v = d["v"].reshape(n, heads, value_dim)
        if rule == "delta":
            q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * key_dim ** -0.5
            k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            decay = torch.exp(-torch.exp(rate.double()) * pz.softplus(d["d"] + bias.double()))
            want[s] = pz.delta_rule_scan(q, k, v, torch.sigmoid(d["w"]), decay).reshape(n, -1)
        else:
            dt = pz.softplus(d["w"] + bias.double())
            want[s] = pz.ssd_scan(v, k, q, dt, torch.exp(rate.double()), skip.double()).reshape(n, -1)
    state = torch.zeros(5, heads, value_dim, key_dim, device=dev)
    done, got = {s: 0 for s in lengths}, {s: [] for s in lengths}
    for cut in ([(1, 19), (3, 2)], [(3, 1)], [(1, 1), (3, 17)], [(1, 17), (3, 1)]):
        step, layout = step_for(kit, [(s, [0] * n, done[s], ()) for s, n in cut])
        cat = {key: torch.cat([data[sl.seat][key][sl.past_len : sl.past_len + sl.q_len] for sl in layout.seqs]).to(dev)
               for key in "qkvdw"}
        if value_dim % 2 == 0:  # decay and write as slices of a split product
            both = in_slices(torch.cat([cat["d"], cat["w"]], dim=1))
            cat["d"], cat["w"] = both[:, :, :heads], both[:, :, heads:]
        out = kit.linear_recurrence(rule, cat["q"], cat["k"], cat["v"], cat["d"], cat["w"], state, step, heads, groups,
                                    key_dim, value_dim, decay_rate=rate.to(dev), decay_bias=bias.to(dev),
                                    skip=skip.to(dev) if rule == "ssd" else None)
        for sl in layout.seqs:
            got[sl.seat].append(out[sl.start : sl.start + sl.q_len].cpu())
            done[sl.seat] += sl.q_len
    for s in lengths:
        _close(torch.cat(got[s]), want[s], 2e-5, f"{rule} seat {s}")


@pytest.mark.parametrize("gate_first,group,weight_len", [(False, 8, 8), (True, 24, 48), (True, 48, 48), (False, 33, 33),
                                                         (True, 640, 640), (False, 300, 300), (True, 2052, 2052)])
def test_gated_rmsnorm(kit, gate_first, group, weight_len):
    g = torch.Generator().manual_seed(group)
    tokens, n = 5, 2 * group * (2 if weight_len == group else 1)
    n = max(n, weight_len)
    x, gate = torch.randn(tokens, n, generator=g) * 2, torch.randn(tokens, n, generator=g)
    weight = torch.randn(weight_len, generator=g)
    xd, gd = x.double(), pz.silu(gate.double())
    full = weight.double().repeat(n // weight_len)
    if gate_first:
        want = pz.rms_unit((xd * gd).reshape(tokens, n // group, group), 1e-5).reshape(tokens, n) * full
    else:
        want = pz.rms_unit(xd.reshape(tokens, n // group, group), 1e-5).reshape(tokens, n) * full * gd
    dev = kit.device
    out = torch.empty(tokens, n, dtype=kit.dtype, device=dev)
    kit.gated_rmsnorm(x.to(dev), in_slices(gate.to(dev)) if gate_first else gate.to(dev), weight.to(dev), 1e-5, group,
                      gate_first, out)
    _close(out, want, 1e-5 if kit.dtype == torch.float32 else 2e-2, "gated norm")


def _paged(kit, kv_heads, dim, vdim, pages, page_size, table):
    dev = kit.device
    return KvSlot(torch.zeros(pages, kv_heads, page_size, dim, dtype=kit.dtype, device=dev),
                  torch.zeros(pages, kv_heads, page_size, vdim, dtype=kit.dtype, device=dev),
                  torch.tensor(table, dtype=torch.int32, device=dev), page_size, pages)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,size,page", [(4, 2, 16, 16, 24, 16), (3, 3, 24, 40, 7, 4), (2, 1, 64, 64, 50, 16),
                                                                (6, 1, 128, 128, 33, 8), (2, 2, 48, 8, 300, 16)])
def test_chunked_attention_with_a_key_that_stands_out(kit, heads, kv_heads, dim, vdim, size, page):
    """Keys written through the paged write in portions, attention in portions and token by token.  One key per chunk
    (its first) is made to match every later query of the chunk, so that nearly all weight sits on the oldest key a
    token may see: dropping it, or seeing the key one place before the chunk, changes everything."""
    g = torch.Generator().manual_seed(size)
    n = max(2 * size + 5, 40) if size < 200 else size + 40
    q = torch.randn(n, heads, dim, generator=g)
    k = torch.randn(n, kv_heads, dim, generator=g)
    v = torch.randn(n, kv_heads, vdim, generator=g)
    anchor = torch.randn(dim, generator=g)
    anchor = anchor / anchor.norm()
    for start in range(0, n, size):
        k[start] = 6.0 * anchor            # the first key of a chunk
        if start:
            k[start - 1] = 9.0 * anchor    # the key just outside: larger still, and never to be seen
    q = q + 3.0 * anchor                   # every query looks for the anchor
    if kit.dtype != torch.float32:
        q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    scale = 0.7
    want = pz.chunked_softmax(q.double(), k.double(), v.double(), scale, size).reshape(n, heads * vdim)
    dev = kit.device
    width = pages_needed(n, page)
    table = [[-1] * width, list(range(width - 1, -1, -1))]  # seat 1, pages handed out backwards
    kv = _paged(kit, kv_heads, dim, vdim, width + 1, page, table)
    got, at = [], 0
    cuts = [size - 1, 2, 1, 1, size, 1, 1, 3, 1]
    while at < n:
        count = min(cuts.pop(0) if cuts else 5, n - at)
        step, _ = step_for(kit, [(1, [0] * count, at, ())])
        rows = slice(at, at + count)
        qkv = torch.cat([q[rows].reshape(count, -1), k[rows].reshape(count, -1), v[rows].reshape(count, -1)], 1).to(dev, kit.dtype)
        q_end, k_end = heads * dim, (heads + kv_heads) * dim
        kit.kv_write(qkv[:, q_end:k_end], qkv[:, k_end:], step, kv)
        out = torch.empty(count, heads * vdim, dtype=kit.dtype, device=dev)
        kit.attention(qkv, out, step, kv, heads, kv_heads, dim, None, scale, size)
        got.append(out.float().cpu())
        at += count
    kit.check_errors()
    _close(torch.cat(got), want, 2e-5 if kit.dtype == torch.float32 else 3e-2, "attention")


def test_head_gate(kit):
    g = torch.Generator().manual_seed(5)
    x, logits = torch.randn(7, 6 * 10, generator=g), torch.randn(7, 9, generator=g) * 3
    want = (x.double().reshape(7, 6, 10) * torch.sigmoid(logits.double()[:, 2:8, None])).reshape(7, 60)
    dev = kit.device
    have = x.clone().to(dev, kit.dtype).contiguous()
    kit.head_gate(have, logits.to(dev)[:, 2:8], 6)
    _close(have, want, 1e-6 if kit.dtype == torch.float32 else 1e-2, "head gate")
    again = x.clone().to(dev, kit.dtype).contiguous()
    kit.head_gate(again, in_slices(logits.to(dev))[:, :, 2:8], 6)
    _close(again, want, 1e-6 if kit.dtype == torch.float32 else 1e-2, "head gate from slices")


# -- the whole model through the engine's step function -----------------------------------------------------
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
    cfg, page, weights = model(name)
    requests = requests_of(cfg, LENGTHS[name])
    steps = SCHEDULES[mode](requests)
    peak = helpers.peak_tokens(steps, granule=page)
    engine, _, _ = engine_for(name, kit, num_blocks=pages_needed(peak, page), max_seqs=3)
    session = TraceSession(engine)
    got = helpers.collect(steps, helpers.run_schedule(session, steps))
    expected = {rid: plain_logits(cfg, weights, ids) for rid, ids in requests.items()}
    assert_close(got, expected, tolerance(kit), f"{name}/{mode}")
    assert engine.cache.free_seats == 3 and all(g.pool.num_free == g.num_pages for g in engine.cache.groups)
    if kit.device.type == "cuda":
        ran = kit.kernel_counts
        assert ran.get("linear_recurrence") and ran.get("short_conv") and ran.get("add_layernorm") and ran.get("gated_rmsnorm")
        if name == "wide" and kit.dtype == torch.bfloat16 and mode != "tail":
            # head sizes 64 and 128 in bfloat16: prompt portions on the tcgen05 attention, single tokens on the
            # tensor-core decode attention that starts from the projection's slices
            assert ran.get("attention_prefill_tcgen05") and not ran.get("attention_generic"), ran
            if mode == "mixed":
                assert ran.get("attention_decode_mma"), ran


@pytest.mark.parametrize("name", ["small", "awkward"])
def test_cuts_at_around_and_across_every_edge(kit, name):
    """Portions that end just before, at and just after the edges of chunks and pages, then single tokens across the
    next edges; the first tokens of the sequence one by one."""
    cfg, page, weights = model(name)
    chunk = cfg["layers"][0 if name == "small" else 1]["mixer"]["left"]["mask"]["size"]
    ids = helpers.random_ids(cfg["vocab"], 4 * chunk + 9, 77)
    cuts = [1, 1, 1, chunk - 4, 2, chunk - 1, 2, chunk, 1, 1]
    steps, at = [], 0
    while at < len(ids):
        size = min(cuts.pop(0) if cuts else 1, len(ids) - at)
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": ids[at : at + size], "want": list(range(size))}],
                      "end": ["a"] if at + size == len(ids) else []})
        at += size
    engine, _, _ = engine_for(name, kit, num_blocks=pages_needed(len(ids), page) + 1)
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    assert_close(got, {"a": plain_logits(cfg, weights, ids)}, tolerance(kit), name)


def test_long_decoding_keeps_the_state(kit):
    """Two tokens of prompt, then 150 tokens one by one beside another request that comes and goes."""
    cfg, page, weights = model("small")
    long_ids = helpers.random_ids(cfg["vocab"], 152, 5)
    other = helpers.random_ids(cfg["vocab"], 40, 6)
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": long_ids[:2], "want": [0, 1]}], "end": []}]
    for at in range(2, len(long_ids)):
        entries = [{"id": "long", "tokens": [long_ids[at]], "want": [0]}]
        end = ["long"] if at == len(long_ids) - 1 else []
        if 40 <= at < 60:  # another request, two tokens a step, twice over (its seat and pages are used again)
            part = (at - 40) % 10
            entries.append({"id": f"o{(at - 40) // 10}", "tokens": other[4 * part : 4 * part + 4], "want": [3]})
            if part == 9:
                end.append(f"o{(at - 40) // 10}")
        steps.append({"step": at - 1, "entries": entries, "end": end})
    engine, _, _ = engine_for("small", kit, num_blocks=pages_needed(152, page) + 3, max_seqs=2)
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    want_other = plain_logits(cfg, weights, other)[3::4]
    assert_close(got, {"long": plain_logits(cfg, weights, long_ids), "o0": want_other, "o1": want_other}, tolerance(kit), "long")
    if kit.device.type == "cuda":  # steps of single tokens replayed the captured decode step, state and all
        assert engine.runner.use_graphs and engine.runner.graph_replays >= 100


@pytest.mark.parametrize("name", ["small", "awkward", "no_pages"])
def test_greedy_generation_through_the_scheduler(kit, name):
    """``Engine.run``: prompts cut into portions of five beside decoding requests, two seats for three requests, and
    one request sent back and recomputed; every token must be the plain implementation's arg-max (or a near tie)."""
    cfg, page, weights = model(name)
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
        logits = plain_logits(cfg, weights, prompt + result.token_ids[:-1])[len(prompt) - 1 :]
        for index, token in enumerate(result.token_ids):
            best = float(logits[index].max())
            slack = (2e-4 if kit.dtype == torch.float32 else 8e-2) * float(logits[index].std())
            assert float(logits[index, token]) >= best - slack, f"{result.request_id}: output {index} is no arg-max"


# -- the command line and the trace runner, as a user runs them ---------------------------------------------
@pytest.mark.gpu
def test_command_line_and_trace_runner(tmp_path):
    """``init-random`` writes a Zelasun folder from its configuration file, ``generate`` decodes greedily from it and
    ``bin/trace_run`` replays steps against it (a portion, then portions beside single tokens, then an ended request's
    seat used again): tokens and logits are the plain implementation's."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    from distie_b200.weights import ModelTensors

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
