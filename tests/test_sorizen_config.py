"""The Sorizen configuration, its recipe and its tensor names, and the plain statement against itself; no GPU."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_sorizen as plain
import nanospec_b200.architectures  # noqa: F401  (registers the architectures)
from nanospec_b200.config import ConfigError, SorizenConfig, resolve_architecture
from nanospec_b200.weights import build_model


def _mixer(**kw):
    m = {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 12, "scale": 0.3, "mask": {"size": 5},
         "rot": {"dims": 4, "base": 1000.0, "scaling": {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0}}}
    m.update(kw)
    return m


def _cfg():
    moe = {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}}
    layers = [{"type": "latent_attention_2", "mixer": _mixer(), "mlp": {"kind": "dense", "ff": 20}},
              {"type": "latent_attention", "mixer": _mixer(heads=3), "mlp": moe},
              {"type": "latent_attention", "mixer": _mixer(rot_dim=0, rot=None), "mlp": None},
              {"type": "latent_attention", "mixer": _mixer(heads=3), "mlp": moe, "weights_of": 1}]
    return {"architecture": "Sorizen", "vocab": 61, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5}, "streams": 2,
            "layers": layers}


def test_round_trip_and_registry():
    cfg = SorizenConfig.from_hf(_cfg())
    assert SorizenConfig.from_hf(cfg.to_hf()) == cfg
    assert resolve_architecture(_cfg()).name == "Sorizen"
    assert cfg.streams == 2 and cfg.embedding_scale == 2.5 and cfg.layers[3].weights_of == 1
    plain_stream = _cfg()
    del plain_stream["streams"]
    assert SorizenConfig.from_hf(plain_stream).streams is None


def test_recipe_order_lanes_and_names():
    model, _ = build_model(_cfg(), None, torch.float32, "cpu")
    order = model.recipe.order
    assert [(r.layer, r.lane) for r in order] == [(0, 0), (1, 1), (2, 2), (1, 3)]  # the fourth layer runs the second's parts on a lane of its own
    names = set(model.weight_specs())
    assert {"embed", "head", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.mix.g", "l0.mix.dkv.norm", "l0.mlp.up",
            "l0.hc1.mix", "l0.hc2.in", "l1.mix.sink", "l1.mlp.router", "l1.mlp.e5.down", "l2.hc1.out"} <= names
    assert not any(n.startswith("l3.") for n in names)          # no tensors of its own
    assert "l2.norm2" not in names and "l2.hc2.in" not in names  # no feed-forward, none of its tensors
    assert "l0.mix.sink" not in names and "l1.mix.g" not in names
    needs = model.lane_needs()
    assert needs[0][0].head_dim == 16 and needs[2][0].head_dim == 12 and all(n[0].v_dim == 0 and n[0].kv_heads == 1 for n in needs)
    del_streams = _cfg()
    del del_streams["streams"]
    model, _ = build_model(del_streams, None, torch.float32, "cpu")
    assert not any(".hc" in n for n in model.weight_specs())


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][0].update(type="attention"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "chosen"),
    (lambda c: c["layers"][3].update(weights_of=3), "weights of"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "feed-forward kind"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "pairs"),
    (lambda c: c.update(streams=0), "streams"),
])
def test_refusals(edit, text):
    cfg = _cfg()
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        SorizenConfig.from_hf(cfg)


def test_plain_statement_against_itself():
    """The plain statement's own consistency: a token's logits do not depend on what follows it, and a window longer than
    the sequence is no window."""
    cfg = _cfg()
    model, _ = build_model(cfg, None, torch.float32, "cpu")
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.randn(s.shape, generator=g) * (0.3 if len(s.shape) == 2 else 0.2) + (1.0 if n.endswith(("norm", "norm1", "norm2", ".in", ".out")) else 0.0))
         for n, s in model.weight_specs().items()}
    ids = torch.randint(0, cfg["vocab"], (19,), generator=g).tolist()
    whole = plain.forward(cfg, w, ids)
    assert torch.allclose(plain.forward(cfg, w, ids[:11]), whole[:11], atol=1e-9)
    wide = copy.deepcopy(cfg)
    for layer in wide["layers"]:
        layer["mixer"]["mask"]["size"] = 19
    wider = copy.deepcopy(wide)
    for layer in wider["layers"]:
        layer["mixer"]["mask"]["size"] = 500
    assert torch.allclose(plain.forward(wide, w, ids), plain.forward(wider, w, ids), atol=1e-9)
    assert not torch.allclose(plain.forward(wide, w, ids), whole, atol=1e-6)
