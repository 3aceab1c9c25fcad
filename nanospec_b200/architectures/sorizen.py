"""The Sorizen decoder as a recipe: pre-norm layers (a layer norm with gain and bias) over attention on a cached latent -
with a sink in the softmax or a gate on the heads' outputs - and a dense gelu feed-forward, routed experts or none; the
stream as one residual or as several copies joined by hyper-connections; layers that run on another layer's weights with a
lane of their own; a scaled embedding, a final layer norm and a head.  Tensor names: `embed`, `l<i>.norm1` (+ `.b`),
`l<i>.mix.<name>`, `l<i>.hc1.<name>`, `l<i>.norm2` (+ `.b`), `l<i>.mlp.<name>`, `l<i>.hc2.<name>`, `final.norm` (+ `.b`), `head`."""

from __future__ import annotations

from ..config.recipe import LayerSpec, ModelRecipe, PartSpec, Run
from ..config.registry import Architecture, register_architecture
from ..config.sorizen import MAX_POSITIONS, SorizenConfig


def _mixer(kind: str, m: dict, width: int, eps: float) -> PartSpec:
    rot_dim = int(m["rot_dim"])
    position = None
    if rot_dim > 0:
        rot = m["rot"]
        position = PartSpec("rotary", {"head_dim": rot_dim, "dims": int(rot["dims"]), "base": float(rot["base"]),
                                       "layout": "interleaved", "scaling": rot.get("scaling") or None})
    return PartSpec("latent_attention", {
        "hidden": width, "heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": rot_dim, "v_dim": int(m["vdim"]),
        "rank": int(m["kv_rank"]), "scale": float(m["scale"]), "window": int((m.get("mask") or {}).get("size") or 0), "eps": eps,
        "sink": kind == "latent_attention", "gate": kind == "latent_attention_2", "position": position})


def _feed_forward(mlp: dict | None, width: int) -> PartSpec | None:
    if mlp is None:
        return None
    if mlp.get("kind", "dense") == "dense":
        return PartSpec("dense_act", {"hidden": width, "intermediate": int(mlp["ff"]), "activation": "gelu_erf"})
    r = mlp["router"]
    g = r.get("groups") or {}
    return PartSpec("routed_experts", {
        "hidden": width, "experts": int(r["experts"]), "top": int(r["top"]), "intermediate": int(mlp["expert"]["ff"]),
        "groups": int(g.get("count") or 1), "keep": int(g.get("keep") or 1),
        "scale": float(r["scale"]) if r.get("scale") is not None else 1.0, "score": "sigmoid"})


def sorizen_recipe(cfg: SorizenConfig) -> ModelRecipe:
    norm = PartSpec("layernorm", {"hidden": cfg.width, "eps": cfg.eps, "weight_name": "", "bias_name": ".b"})
    hyper = cfg.streams is not None
    names = {"mixer": "mix.", "feed_forward": "mlp.", "norm_mixer": "norm1", "norm_feed_forward": "norm2",
             "hc_mixer": "hc1.", "hc_feed_forward": "hc2."}
    layers, spec_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        spec_of[i] = len(layers)
        layers.append(LayerSpec(block="hyper" if hyper else "prenorm", prefix=f"l{i}.",
                                mixer=_mixer(layer.type, layer.mixer, cfg.width, cfg.eps),
                                feed_forward=_feed_forward(layer.mlp, cfg.width), norm=norm, names=names,
                                params={"streams": cfg.streams} if hyper else {}))
    # every layer of the file is a run on a lane of its own; one that names another layer's weights runs that layer's parts
    order = tuple(Run(layer=spec_of[i if layer.weights_of is None else layer.weights_of], lane=i)
                  for i, layer in enumerate(cfg.layers))
    return ModelRecipe(
        architecture=cfg.architecture,
        embedding=PartSpec("table", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "", "weight_name": "embed",
                                     "scale": cfg.embedding_scale, "copies": cfg.streams or 1}),
        layers=tuple(layers), order=order, final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "", "weight_name": "head", "tied_to": None}),
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS, eos_token_ids=cfg.eos_token_ids)


SORIZEN = register_architecture(Architecture(
    name="Sorizen", model_type="sorizen", config_from_hf=SorizenConfig.from_hf, recipe=sorizen_recipe))
