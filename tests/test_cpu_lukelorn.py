"""Lukelorn without a GPU: configuration, tensor names, lanes and state, the cache's kept pages, identities of the
plain mechanisms."""
from __future__ import annotations

import copy
import math

import pytest
import torch

from tests import lukelorn_cases as cases
from tests.plain import lukelorn_plain as plain

F64 = torch.float64


@pytest.mark.parametrize("name", sorted(cases.CONFIGS))
def test_config_round_trip_declared_tensors_and_lanes(name, tmp_path):
    from cpmcu_b200.models.model import Model
    from cpmcu_b200.registry import architecture, load_config

    cfg = cases.CONFIGS[name]()
    folder = cases.write_folder(cfg, cases.random_weights(cfg, 1), str(tmp_path / name))
    arch, typed = load_config(folder)
    assert arch is architecture("Lukelorn")
    assert arch.config_class.from_dict(typed.to_dict()) == typed
    model = Model(arch.model_spec(typed), None)
    specs = model.weight_specs()
    shapes = cases.tensor_shapes(cfg)
    assert set(specs) == set(shapes)
    assert all(tuple(specs[k].shape) == tuple(shapes[k]) for k in shapes)
    # every layer of the configuration is one run with a lane of its own; a layer that names another runs that one's parts
    assert [run.lane for run in model.schedule] == list(range(len(cfg["layers"])))
    assert all(run.writes_cache for run in model.schedule)
    own = [i for i, layer in enumerate(cfg["layers"]) if "weights_of" not in layer]
    for i, (layer, run) in enumerate(zip(cfg["layers"], model.schedule)):
        assert run.layer == own.index(layer.get("weights_of", i))
    needs = model.cache_needs()
    for layer, n in zip(cfg["layers"], needs):
        m = layer["mixer"]
        mask = m.get("mask") or {}
        if layer["type"] == "channel_delta":
            assert n.kv_heads == 0 and n.state["matrix_state"][0] == (m["heads"], m["dim"], m["vdim"])
            channels = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
            assert n.state["conv_inputs"][0] == (max(m["conv"] - 1, 1), channels)
        elif layer["type"] == "latent_attention":
            assert (n.kv_heads, n.head_dim, n.values, n.window) == (1, m["kv_rank"] + m["rot_dim"], False, mask.get("size"))
        else:
            assert (n.kv_heads, n.head_dim, n.value_dim or n.head_dim) == (m["kv_heads"], m["dim"], m["vdim"])
            assert n.window == mask.get("size") and n.keep_first == (mask.get("keep_first", 0) if mask.get("size") else 0)


def test_config_errors_are_collected():
    from cpmcu_b200.config.base import ConfigError
    from cpmcu_b200.config.lukelorn import LukelornConfig

    bad = copy.deepcopy(cases.config_a())
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    bad["layers"][1]["mixer"]["conv"] = 9
    bad["layers"][2]["mlp"]["router"]["top"] = 7
    bad["layers"][2]["mixer"]["rot"]["dims"] = 6                 # the rotated part of a latent layer is all of rot_dim
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        LukelornConfig.from_dict(bad)
    text = str(e.value)
    assert all(word in text for word in ("kv_heads", "conv", "top", "norm", "rot_dim"))
    for j in (3, 0, 9):                                          # a layer without tensors of its own, the layer itself, none
        bad = copy.deepcopy(cases.config_a())
        bad["layers"][4]["weights_of"] = j if j != 0 else 4
        with pytest.raises(ConfigError) as e:
            LukelornConfig.from_dict(bad)
        assert "weights_of" in str(e.value)
    bad = copy.deepcopy(cases.config_a())
    bad["layers"][3]["mixer"] = copy.deepcopy(bad["layers"][3]["mixer"])
    bad["layers"][3]["mixer"]["mask"]["size"] = 21               # the rest of the entry must equal the named layer's
    with pytest.raises(ConfigError) as e:
        LukelornConfig.from_dict(bad)
    assert "differs" in str(e.value)


def test_ranks_come_from_the_checkpoint(tmp_path):
    from cpmcu_b200.registry import load_config

    cfg = cases.config_c()
    folder = cases.write_folder(cfg, cases.random_weights(cfg, 2), str(tmp_path / "c"))
    _, typed = load_config(folder)
    assert (typed.layers[0].mixer.decay_rank, typed.layers[0].mixer.gate_rank) == (5, 9)
    cfg = cases.config_a()
    folder = cases.write_folder(cfg, cases.random_weights(cfg, 2), str(tmp_path / "a"))
    _, typed = load_config(folder)
    assert typed.layers[4].mixer == typed.layers[1].mixer and typed.layers[4].mixer.decay_rank == 12


def test_cache_keeps_the_pages_of_the_first_tokens():
    """A windowed group gives back the pages behind the window but never those that hold kept first tokens."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.cache.cache import RELEASED
    from cpmcu_b200.parts.base import CacheNeeds

    needs = [CacheNeeds(kv_heads=1, head_dim=8, window=70, keep_first=65), CacheNeeds(kv_heads=1, head_dim=8, window=70),
             CacheNeeds(kv_heads=1, head_dim=8, window=70, keep_first=64)]
    cache = Cache(needs, max_tokens=64 * 40, dtype=torch.float32, device="cpu", n_slots=2, max_step_tokens=64)
    assert len(cache.groups) == 3
    slot = cache.open_sequence()
    length = 0
    for step in [64] * 6 + [1] * 130:
        cache.check_room([(slot, length + step)], 64)
        cache.reserve(slot, length + step)
        cache.sync()
        length += step
        cache.set_length(slot, length)
        cache.check_consistent()
        for g, kept in zip(cache.groups, (2, 0, 1)):
            pages = g.pages_of_slot[slot]
            dead = max(0, length - 70 + 1) // 64
            for i, p in enumerate(pages):
                assert (p == RELEASED) == (kept <= i < dead), (length, kept, i, pages)
            table = g.page_table[slot, :len(pages)].tolist()
            assert all(table[i] == p for i, p in enumerate(pages) if p != RELEASED)
    cache.close_sequence(slot)
    assert all(g.pages.n_held == 0 for g in cache.groups)


def test_plain_softmax_with_a_sink_and_visible_keys():
    s = torch.tensor([[0.0, math.log(3.0), 5.0]], dtype=F64)
    visible = torch.tensor([[True, True, False]])
    p = plain.softmax_with_sink(s, visible, math.log(4.0))
    assert torch.allclose(p, torch.tensor([[1 / 8, 3 / 8, 0.0]], dtype=F64))
    assert torch.allclose(plain.softmax_with_sink(s, visible, None), torch.tensor([[0.25, 0.75, 0.0]], dtype=F64))
    far = plain.softmax_with_sink(torch.tensor([[-800.0, -801.0]], dtype=F64), torch.tensor([[True, True]]), -900.0)
    assert torch.isfinite(far).all() and abs(float(far.sum()) - 1.0) < 1e-12          # the sink far below the scores
    seen = plain.visible_keys(8, 3, 2)
    assert seen[7].tolist() == [True, True, False, False, False, True, True, True]
    assert seen[3].tolist() == [True, True, True, True, False, False, False, False]
    assert plain.visible_keys(4, None, 2).tolist() == torch.tril(torch.ones(4, 4, dtype=torch.bool)).tolist()


def test_plain_rotation_turns_adjacent_pairs_and_stretches_long_waves():
    rot = {"dims": 4, "base": 100.0}
    x = torch.zeros(3, 1, 6, dtype=F64)
    x[:, 0, 0] = 1.0                 # the first member of pair 0
    x[:, 0, 3] = 2.0                 # the second member of pair 1
    x[:, 0, 5] = 7.0                 # beyond the rotated part
    y = plain.rotate_pairs(x, rot)
    f = [1.0, 100.0 ** -0.5]
    for p in range(3):
        assert torch.allclose(y[p, 0, :2], torch.tensor([math.cos(p * f[0]), math.sin(p * f[0])], dtype=F64))
        assert torch.allclose(y[p, 0, 2:4], torch.tensor([-2 * math.sin(p * f[1]), 2 * math.cos(p * f[1])], dtype=F64))
        assert float(y[p, 0, 5]) == 7.0 and float(y[p, 0, 4]) == 0.0
    # wavelengths 2 pi / f: short ones stay, long ones are divided by the factor, those between are blended
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    plain_f = plain.frequencies({"dims": 16, "base": 5000.0})
    stretched = plain.frequencies({"dims": 16, "base": 5000.0, "scaling": sc})
    wave = 2 * math.pi / plain_f
    kinds = set()
    for i in range(8):
        if wave[i] < 64 / 4.0:
            kinds.add("short")
            assert stretched[i] == plain_f[i]
        elif wave[i] > 64 / 1.0:
            kinds.add("long")
            assert torch.isclose(stretched[i], plain_f[i] / 4.0)
        else:
            kinds.add("between")
            assert plain_f[i] / 4.0 < stretched[i] < plain_f[i]
    assert kinds == {"short", "long", "between"}


def test_plain_delta_rule_in_pieces_and_against_its_definition():
    g = torch.Generator().manual_seed(3)
    T, H, d, dv = 9, 2, 5, 3
    q, k = torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, d, generator=g, dtype=F64)
    v = torch.randn(T, H, dv, generator=g, dtype=F64)
    beta, decay = torch.rand(T, H, generator=g, dtype=F64), torch.rand(T, H, d, generator=g, dtype=F64)
    whole, S = plain.delta_recurrence(q, k, v, beta, decay)
    first, S1 = plain.delta_recurrence(q[:4], k[:4], v[:4], beta[:4], decay[:4])
    rest, S2 = plain.delta_recurrence(q[4:], k[4:], v[4:], beta[4:], decay[4:], state=S1)
    assert torch.allclose(torch.cat([first, rest]), whole) and torch.allclose(S2, S)
    # one token from an empty state: S = k (beta v)^T, o = (q . k) beta v, whatever the decay
    one, _ = plain.delta_recurrence(q[:1], k[:1], v[:1], beta[:1], decay[:1])
    want = (q[0] * k[0]).sum(-1, keepdim=True) * beta[0][:, None] * v[0]
    assert torch.allclose(one[0], want)
    # with beta = 1 and a unit key, the value stored under the key is replaced: reading with the same key gives v
    kk = k / k.norm(dim=-1, keepdim=True)
    out, _ = plain.delta_recurrence(kk, kk, v, torch.ones(T, H, dtype=F64), decay)
    assert torch.allclose(out, v)


def test_plain_convolution_and_routing():
    x = torch.arange(12, dtype=F64).view(6, 2)
    taps = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]], dtype=F64)
    y = plain.short_convolution(x, taps)
    assert y[0].tolist() == [0.0, 2.0] and y[1].tolist() == [200.0, 6.0] and y[2].tolist() == [100 * 4 + 10 * 2 + 0, 10.0]
    W = 6
    g = torch.Generator().manual_seed(1)
    w = {"r.router": torch.randn(5, W, generator=g, dtype=F64)}
    for e in range(5):
        w[f"r.e{e}.up"] = torch.randn(4, W, generator=g, dtype=F64)
        w[f"r.e{e}.down"] = torch.randn(W, 4, generator=g, dtype=F64)
    h = torch.randn(7, W, generator=g, dtype=F64)
    m = {"router": {"experts": 5, "top": 2}}
    out, s, idx = plain.mixture_of_experts(h, w, "r.", m)
    assert torch.equal(idx, torch.topk(torch.sigmoid(h @ w["r.router"].T), 2).indices)
    t = 3
    want = sum(plain.expert((s[t, e] * h[t])[None], w, f"r.e{int(e)}.")[0] for e in idx[t])
    assert torch.allclose(out[t], want)
    # the weight on the input of an expert whose activation is a square counts twice
    assert torch.allclose(plain.expert(0.5 * h, w, "r.e0."), 0.25 * plain.expert(h, w, "r.e0."))
