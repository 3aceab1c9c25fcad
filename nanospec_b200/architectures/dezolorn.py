"""The Dezolorn decoder as a recipe: pre-norm layers (a bias-free layer norm) whose mixer is windowed attention with kept
first keys, retention or the gated delta rule, an optional SwiGLU feed-forward, a span of layers that runs several times
(every pass on cache lanes and state of its own, the embedding's output added at the start of each pass but the first), a
final layer norm and a head with scaled, soft-capped logits.  Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.<name>`,
`l<i>.norm2`, `l<i>.mlp.<name>`, `final.norm`, `head`."""

from __future__ import annotations

from ..config.dezolorn import DezolornConfig, MAX_POSITIONS
from ..config.recipe import LayerSpec, ModelRecipe, PartSpec, Run
from ..config.registry import Architecture, register_architecture


def _mixer(kind: str, m: dict, width: int, eps: float) -> PartSpec:
    if kind == "attention":
        rot = m["rot"]
        position = PartSpec("rotary", {"head_dim": int(m["dim"]), "dims": int(rot["dims"]), "base": float(rot["base"]),
                                       "layout": "interleaved", "scaling": rot.get("scaling") or None})
        return PartSpec("gqa_attention", {
            "hidden": width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
            "v_dim": int(m["vdim"]), "window": int(m["mask"]["size"]), "keep_first": int(m["mask"]["keep_first"]),
            "scale": float(m["scale"]), "qk_norm": {"eps": eps}, "position": position, "wide_weights": True,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}})
    if kind == "retention":
        rot = m["rot"]
        position = PartSpec("rotary", {"head_dim": int(m["dim"]), "dims": int(rot["dims"]), "base": float(rot["base"]),
                                       "layout": "half", "scaling": rot.get("scaling") or None})
        return PartSpec("retention", {
            "hidden": width, "heads": int(m["heads"]), "head_dim": int(m["dim"]), "v_dim": int(m["vdim"]),
            "decay": tuple(float(d) for d in m["decay"]), "eps": eps, "position": position,
            "names": {k: k for k in ("q", "k", "v", "g", "o")}})
    return PartSpec("gated_delta", {
        "hidden": width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
        "v_dim": int(m["vdim"]), "conv": int(m["conv"]), "eps": eps, "unit_eps": 1e-6,
        "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a": "a", "b": "b", "q_conv": "q.conv", "k_conv": "k.conv",
                  "v_conv": "v.conv", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm"}})


def dezolorn_recipe(cfg: DezolornConfig) -> ModelRecipe:
    norm = PartSpec("layernorm", {"hidden": cfg.width, "eps": cfg.eps, "weight_name": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        ff = None if layer.ff is None else PartSpec("swiglu", {"hidden": cfg.width, "intermediate": layer.ff,
                                                                "names": {"gate": "gate", "up": "up", "down": "down"}})
        layers.append(LayerSpec(block="prenorm", prefix=f"l{i}.", mixer=_mixer(layer.type, layer.mixer, cfg.width, cfg.eps),
                                feed_forward=ff, norm=norm,
                                names={"mixer": "mix.", "feed_forward": "mlp.", "norm_mixer": "norm1", "norm_feed_forward": "norm2"}))
    # every run has a lane of its own: a layer that runs again keeps another cache or state for each pass
    order = tuple(Run(layer=i, lane=n, add_input=add) for n, (i, add) in enumerate(cfg.runs()))
    return ModelRecipe(
        architecture=cfg.architecture,
        embedding=PartSpec("table", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "", "weight_name": "embed"}),
        layers=tuple(layers), order=order, final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "", "weight_name": "head", "tied_to": None,
                                 "scale": cfg.logit_scale, "softcap": cfg.logit_softcap}),
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS, eos_token_ids=cfg.eos_token_ids)


DEZOLORN = register_architecture(Architecture(
    name="Dezolorn", model_type="dezolorn", config_from_hf=DezolornConfig.from_hf, recipe=dezolorn_recipe))
