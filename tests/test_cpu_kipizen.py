"""Kipizen without a GPU: configuration, tensor names, lanes and state, identities of the plain mechanisms."""
from __future__ import annotations

import math

import pytest
import torch

from tests import kipizen_cases as cases
from tests.plain import kipizen_plain as plain

F64 = torch.float64


@pytest.mark.parametrize("name", sorted(cases.CONFIGS))
def test_config_round_trip_declared_tensors_and_lanes(name, tmp_path):
    from cpmcu_b200.models.model import Model
    from cpmcu_b200.registry import architecture, load_config

    cfg = cases.CONFIGS[name]()
    folder = cases.write_folder(cfg, cases.random_weights(cfg, 1), str(tmp_path / name))
    arch, typed = load_config(folder)
    assert arch is architecture("Kipizen")
    assert arch.config_class.from_dict(typed.to_dict()) == typed
    model = Model(arch.model_spec(typed), None)
    specs = model.weight_specs()
    shapes = cases.tensor_shapes(cfg)
    assert set(specs) == set(shapes)
    assert all(tuple(specs[k].shape) == tuple(shapes[k]) for k in shapes)
    # a layer with keys and values of its own has a lane of its own; a reader runs on its writer's lane and never writes
    lane_of, readers = {}, {}
    for i, (layer, run) in enumerate(zip(cfg["layers"], model.schedule)):
        src = layer["mixer"].get("kv_from")
        if src is None:
            lane_of[i] = run.lane
            assert run.writes_cache
        else:
            assert run.lane == lane_of[src] and not run.writes_cache
            readers.setdefault(src, []).append(layer["mixer"].get("mask", {}).get("size"))
    assert sorted(lane_of.values()) == list(range(len(lane_of)))
    needs = model.cache_needs()
    for i, lane in lane_of.items():
        m, n = cfg["layers"][i]["mixer"], needs[lane]
        if cfg["layers"][i]["type"] == "lightning":
            assert n.kv_heads == 0 and n.state["matrix_state"][0] == (m["heads"], m["dim"], m["vdim"])
            continue
        assert (n.kv_heads, n.head_dim, n.value_dim or n.head_dim) == (m["kv_heads"], m["dim"], m["vdim"])
        # the lane keeps what its widest reader sees (None: every key)
        windows = [m.get("mask", {}).get("size")] + readers.get(i, [])
        assert n.window == (None if None in windows else max(windows))


def test_config_errors_are_collected():
    from cpmcu_b200.config.base import ConfigError
    from cpmcu_b200.config.kipizen import KipizenConfig

    bad = cases.config_a()
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    bad["layers"][1]["mixer"]["decay"] = [0.5]
    bad["layers"][1]["mlp"]["router"]["top"] = 7
    bad["layers"][2]["mixer"]["kv_from"] = 1                  # a lightning layer has no keys
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        KipizenConfig.from_dict(bad)
    text = str(e.value)
    assert all(word in text for word in ("kv_heads", "decay", "top", "norm"))
    bad = cases.config_a()
    bad["layers"][2]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError) as e:
        KipizenConfig.from_dict(bad)
    assert "kv_from" in str(e.value)
    bad = cases.config_a()
    bad["layers"][2]["mixer"]["rot"]["base"] = 123.0           # the reader's rotation must be the writer's
    with pytest.raises(ConfigError):
        KipizenConfig.from_dict(bad)


def test_plain_sink_softmax_and_window():
    s = torch.tensor([[0.0, math.log(3.0), 5.0]], dtype=F64)
    visible = torch.tensor([[True, True, False]])
    p = plain.sink_softmax(s, visible)
    assert torch.allclose(p, torch.tensor([[1 / 5, 3 / 5, 0.0]], dtype=F64), atol=1e-12)       # 1 / (1 + 1 + 3): the sink's share is lost
    # very negative scores: the sink takes everything, the output goes to zero instead of an average of the values
    q = torch.full((4, 1, 2), -30.0, dtype=F64)
    k = torch.ones(4, 1, 2, dtype=F64)
    v = torch.ones(4, 1, 3, dtype=F64)
    assert float(plain.window_attention_core(q, k, v, 1.0, 0.0, None).abs().max()) < 1e-20
    assert torch.allclose(plain.window_attention_core(q, k, v, 1.0, 0.0, None, sink=False), torch.ones(4, 1, 3, dtype=F64))
    # a window of two: token 3 sees keys 2 and 3 only; the cap bounds a huge score
    q = torch.zeros(4, 1, 2, dtype=F64)
    v = torch.arange(4, dtype=F64).view(4, 1, 1)
    o = plain.window_attention_core(q, k, v, 1.0, 0.0, 2)
    assert abs(float(o[3, 0, 0]) - (2 + 3) / 3) < 1e-12 and abs(float(o[0, 0, 0])) < 1e-12
    q = torch.full((1, 1, 1), 1000.0, dtype=F64)
    o = plain.window_attention_core(q, torch.ones(1, 1, 1, dtype=F64), torch.ones(1, 1, 1, dtype=F64), 1.0, 2.0, None)
    assert abs(float(o) - math.exp(2.0) / (1 + math.exp(2.0))) < 1e-9


def test_plain_rotation_pairs_halves_and_stretches_positions():
    x = torch.zeros(3, 1, 6, dtype=F64)
    x[:, 0, 0] = 1.0                                           # pair (0, 2) of four rotated channels
    x[:, 0, 5] = 7.0
    y = plain.rotate_half(x, 4, 100.0, 2.0)
    for p in range(3):
        a = p / 2.0
        assert torch.allclose(y[p, 0], torch.tensor([math.cos(a), 0.0, math.sin(a), 0.0, 0.0, 7.0], dtype=F64), atol=1e-12)
    later = plain.rotate_half(x[1:], 4, 100.0, 2.0, first=1)
    assert torch.allclose(later, y[1:], atol=1e-12)


def test_plain_lightning_recurrence_in_pieces_and_in_closed_form():
    g = torch.Generator().manual_seed(3)
    T, H, d, dv = 9, 2, 5, 4
    q, k, v = (torch.randn(T, H, n, generator=g, dtype=F64) for n in (d, d, dv))
    decay = torch.tensor([0.5, 1.0], dtype=F64)
    whole, _ = plain.lightning_recurrence(q, k, v, decay)
    first, S = plain.lightning_recurrence(q[:4], k[:4], v[:4], decay)
    rest, _ = plain.lightning_recurrence(q[4:], k[4:], v[4:], decay, S)
    assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-12)
    # o_t = sum_{j <= t} decay^(t-j) (q_t . k_j) v_j
    t = T - 1
    for h in range(H):
        want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(T))
        assert torch.allclose(whole[t, h], want, atol=1e-10)


def test_plain_routing_chooses_by_logit_and_weighs_the_chosen_only():
    w = {"router": torch.eye(4, dtype=F64), "router.b": torch.tensor([0.0, 0.0, 0.0, 2.5], dtype=F64)}
    h = torch.tensor([[-1.0, -3.0, -2.0, -4.0]], dtype=F64)    # all logits negative; the bias lifts the last to -1.5
    z, idx, wt = plain.route(h, w, "", {"router": {"experts": 4, "top": 2}})
    assert sorted(idx[0].tolist()) == [0, 3]
    assert abs(float(wt.sum()) - 1.0) < 1e-12
    a, b = math.exp(-1.0), math.exp(-1.5)
    assert torch.allclose(wt[0].sort().values, torch.tensor(sorted([a / (a + b), b / (a + b)]), dtype=F64), atol=1e-12)
