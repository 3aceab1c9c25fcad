"""Typed configuration of the Sorizen decoder, read from its own config.json.

A Sorizen model is a list of pre-norm layers (a layer norm with gain and bias) whose mixer is attention over a cached
latent, inside a sliding window, in one of two kinds - with a learned sink in the softmax, or with a sigmoid gate on each
head's output - and whose feed-forward is dense (exact gelu), a set of routed experts, or absent.  The residual stream may
be kept as several copies joined by hyper-connections, a layer may run on another layer's weights with a cache of its
own, and the embedding's output is scaled.  Every size and every constant that can differ between models comes from the file:

    architecture "Sorizen";  vocab, width;  norm.eps;  embedding.scale;  streams (absent: one plain stream)
    layers[i]: type ("latent_attention" | "latent_attention_2"), mixer {...}, mlp {...} or null, weights_of (optional)
      mixer: heads, dim, rot_dim, vdim, kv_rank, scale, mask {size}, rot {dims, base, scaling {factor, original, fast, slow}}
      mlp:   {kind "dense", ff}  or  {kind "moe", expert {ff}, router {experts, top, scale, groups {count, keep}}}
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .files import ConfigError

MIXER_TYPES = ("latent_attention", "latent_attention_2")
MAX_POSITIONS = 1 << 20  # the file gives no limit; positions are 32-bit and angles float32


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Sorizen config: {where} lacks {key!r}")
    return d[key]


@dataclass(frozen=True)
class SorizenLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None      # None: no feed-forward
    weights_of: int | None = None   # the layer whose tensors this one runs on (with a cache of its own)

    def to_hf(self) -> dict[str, Any]:
        out = {"type": self.type, "mixer": self.mixer, "mlp": self.mlp}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


@dataclass(frozen=True)
class SorizenConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[SorizenLayer, ...]
    embedding_scale: float = 1.0
    streams: int | None = None      # None: a plain residual stream; S >= 1: hyper-connections over S copies
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = "Sorizen"

    @classmethod
    def from_hf(cls, cfg: dict[str, Any], generation: dict[str, Any] | None = None) -> "SorizenConfig":
        if cfg.get("architecture") != "Sorizen" and "Sorizen" not in (cfg.get("architectures") or []):
            raise ConfigError(f"not a Sorizen config: architecture={cfg.get('architecture')!r}")
        entries = _need(cfg, "layers", "config.json")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"Sorizen config: {where} has the unknown mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            m = dict(_need(entry, "mixer", where))
            for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"):
                _need(m, key, where + ".mixer")
            if m.get("mask") is not None:
                m["mask"] = {"size": int(_need(m["mask"], "size", where + ".mixer.mask"))}
            rot = m.get("rot")
            if int(m["rot_dim"]) > 0:
                rot = dict(_need(m, "rot", where + ".mixer"))
                for key in ("dims", "base"):
                    _need(rot, key, where + ".mixer.rot")
                if int(rot["dims"]) % 2 or int(rot["dims"]) > int(m["rot_dim"]):
                    raise ConfigError(f"Sorizen config: {where}: {rot['dims']} of {m['rot_dim']} features cannot turn in pairs")
                if rot.get("scaling"):
                    for key in ("factor", "original", "fast", "slow"):
                        _need(rot["scaling"], key, where + ".mixer.rot.scaling")
                m["rot"] = rot
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                k = mlp.get("kind", "dense")
                if k == "dense":
                    _need(mlp, "ff", where + ".mlp")
                elif k == "moe":
                    _need(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                    r = _need(mlp, "router", where + ".mlp")
                    for key in ("experts", "top"):
                        _need(r, key, where + ".mlp.router")
                    g = r.get("groups")
                    if g:
                        count, keep = int(_need(g, "count", where + ".mlp.router.groups")), int(_need(g, "keep", where + ".mlp.router.groups"))
                        per = int(r["experts"]) // max(count, 1)
                        if count < 1 or int(r["experts"]) % count or not 1 <= keep <= count or keep * per < int(r["top"]):
                            raise ConfigError(f"Sorizen config: {where}: {r['experts']} experts in {count} groups, {keep} kept, {r['top']} chosen")
                    if int(r["top"]) > int(r["experts"]):
                        raise ConfigError(f"Sorizen config: {where}: {r['top']} of {r['experts']} experts")
                else:
                    raise ConfigError(f"Sorizen config: {where} has the unknown feed-forward kind {k!r}")
            of = entry.get("weights_of")
            if of is not None:
                of = int(of)
                if not 0 <= of < len(entries) or of == i or entries[of].get("weights_of") is not None:
                    raise ConfigError(f"Sorizen config: {where} runs on the weights of layer {of}, which has none of its own")
            layers.append(SorizenLayer(kind, m, mlp, of))
        streams = cfg.get("streams")
        if streams is not None and int(streams) < 1:
            raise ConfigError(f"Sorizen config: streams={streams}")
        eos = (generation or {}).get("eos_token_id", cfg.get("eos_token_id"))
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        emb = cfg.get("embedding") or {}
        return cls(vocab=int(_need(cfg, "vocab", "config.json")), width=int(_need(cfg, "width", "config.json")),
                   eps=float(_need(_need(cfg, "norm", "config.json"), "eps", "norm")), layers=tuple(layers),
                   embedding_scale=float(emb["scale"]) if emb.get("scale") is not None else 1.0,
                   streams=None if streams is None else int(streams), eos_token_ids=eos_ids)

    def to_hf(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
                               "layers": [layer.to_hf() for layer in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
