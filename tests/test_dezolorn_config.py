"""Without a GPU: the Dezolorn configuration and recipe, its tensor names, the plain statement against itself (a prompt
whole equals its prefixes), and the cache manager's kept first pages behind a window."""

from __future__ import annotations

import json

import pytest
import torch

import plain_dezolorn as plain
from test_dezolorn_gpu import attention_layer, config, delta_layer, mixed_config, random_weights, retention_layer, tokens, write_folder


def test_order_of_runs_and_lanes():
    from nanospec_b200.config import DezolornConfig
    from nanospec_b200.architectures.dezolorn import dezolorn_recipe

    cfg = DezolornConfig.from_hf(mixed_config())
    assert cfg.runs() == plain.layer_schedule(mixed_config())
    assert [r[0] for r in cfg.runs()] == [0, 1, 2, 1, 2, 1, 2, 3] and [r[1] for r in cfg.runs()] == [False, False, False, True, False, True, False, False]
    recipe = dezolorn_recipe(cfg)
    assert [run.lane for run in recipe.order] == list(range(8))          # every pass has a cache or state of its own
    assert [run.add_input for run in recipe.order] == [r[1] for r in cfg.runs()]
    assert DezolornConfig.from_hf(cfg.to_hf()) == cfg
    once = mixed_config()
    once["loop"] = {"start": 2, "stop": 2, "times": 5}
    assert [r[0] for r in DezolornConfig.from_hf(once).runs()] == [0, 1, 2, 3]


def test_refusals():
    from nanospec_b200.config import ConfigError, DezolornConfig, resolve_architecture

    assert resolve_architecture(mixed_config()).name == "Dezolorn"
    bad = mixed_config()
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError, match="unknown mixer type"):
        DezolornConfig.from_hf(bad)
    bad = mixed_config()
    del bad["layers"][1]["mixer"]["mask"]["size"]
    with pytest.raises(ConfigError, match="size"):
        DezolornConfig.from_hf(bad)
    bad = mixed_config()
    bad["loop"] = {"start": 3, "stop": 1, "times": 2}
    with pytest.raises(ConfigError, match="loop"):
        DezolornConfig.from_hf(bad)
    bad = config([retention_layer(heads=3, decay=[0.5, 0.5])])
    with pytest.raises(ConfigError, match="decays"):
        DezolornConfig.from_hf(bad)


def test_tensor_names_and_loading(tmp_path):
    from nanospec_b200.weights import WeightError, load_model

    cfg = config([attention_layer(ff=20), retention_layer(), delta_layer()])
    w = random_weights(cfg, 1)
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.o", "l0.mlp.gate",
            "l0.mlp.up", "l0.mlp.down", "l1.norm1", "l1.mix.g", "l2.mix.q.conv", "l2.mix.v.conv", "l2.mix.A_log", "l2.mix.dt_bias",
            "l2.mix.norm", "l2.mix.a", "l2.mix.b"} <= set(w)
    assert "l1.norm2" not in w and "l1.mlp.gate" not in w
    assert w["l0.mix.v"].shape == (2 * 16, 48) and w["l2.mix.v.conv"].shape == (4 * 12, 3) and w["l2.mix.q"].shape == (2 * 8, 48)
    model = load_model(write_folder(tmp_path / "ok", cfg, w), device="cpu", dtype=torch.float32)
    needs = model.lane_needs()
    assert needs[0][0].window == 6 and needs[0][0].keep_first == 2 and needs[0][1] is None
    assert needs[1][0] is None and needs[1][1].shape == (3 * 16 * 8,)
    assert needs[2][1].shape == (4 * 8 * 12 + 2 * (2 * 2 * 8 + 4 * 12),)
    del w["l2.mix.dt_bias"]
    w["l2.mix.extra"] = torch.zeros(2)
    with pytest.raises(WeightError) as e:
        load_model(write_folder(tmp_path / "bad", cfg, w), device="cpu", dtype=torch.float32)
    assert "l2.mix.dt_bias" in e.value.missing and "l2.mix.extra" in e.value.unexpected


def test_plain_statement_is_causal_and_feels_every_mechanism():
    cfg = mixed_config()
    w = random_weights(cfg, 2)
    ids = tokens(30, cfg["vocab"], 3)
    whole = plain.forward(cfg, w, ids)
    assert (plain.forward(cfg, w, ids[:17]) - whole[:17]).abs().max() < 1e-9
    for change in ("loop", "keep", "decay", "conv"):
        other = json.loads(json.dumps(cfg))
        w2 = dict(w)
        if change == "loop":
            other["loop"]["times"] = 2
        elif change == "keep":
            other["layers"][1]["mixer"]["mask"]["keep_first"] = 0
        elif change == "decay":
            other["layers"][2]["mixer"]["decay"][0] = 0.5
        else:
            w2["l0.mix.k.conv"] = w["l0.mix.k.conv"].flip(1)
        assert (plain.forward(other, w2, ids) - whole)[-1].abs().max() > 1e-3, change


def test_kept_first_pages_stay_behind_a_window():
    from nanospec_b200.cache import CacheManager
    from nanospec_b200.parts.base import CacheNeed

    m = CacheManager([(CacheNeed(2, 8, window=6, keep_first=5), None), (CacheNeed(2, 8, window=6), None)], num_blocks=12,
                     block_size=4, num_state_slots=2)
    assert len(m.groups) == 2
    m.begin(7)
    held = []
    for _ in range(10):
        m.extend(7, 4)
        m.trim(7)
        m.check()
        held.append(m.held_pages(7))
    # positions 0..4 live in blocks 0 and 1, which the first group never gives back; the window needs two or three more
    assert held[-1][0] == held[-1][1] + 2
    table = m.table(0, 7)
    assert table[0] >= 0 and table[1] >= 0 and table[2] == -1 and table[-1] >= 0
    assert m.table(1, 7)[0] == -1
    m.end(7)
    m.check()
    assert m.free_pages() == [12, 12]
    # a sequence shorter than what is kept gives nothing back
    m.begin(8)
    m.extend(8, 3)
    m.trim(8)
    assert m.held_pages(8) == [1, 1]
    m.end(8)
