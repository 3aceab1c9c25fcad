"""Typed configuration of the Dezolorn decoder, read from its own config.json.

A Dezolorn model is a list of pre-norm layers, each with one of three mixers - windowed softmax attention that keeps a
sequence's first keys, retention, or the gated delta rule - and an optional gated feed-forward; a span of the layers may be
run several times in a row with the same weights.  Every size and every constant that can differ between models comes from
the file:

    architecture "Dezolorn";  vocab, width;  norm.eps;  logit_scale, logit_softcap
    loop {start, stop, times}: layers start .. stop - 1 run `times` times in a row
    layers[i]: type ("attention" | "retention" | "delta"), mixer {...}, mlp {kind "dense", ff} or null
      attention: heads, kv_heads, dim, vdim, scale, mask {size, keep_first}, rot {dims, base, scaling {factor, original, fast, slow}}
      retention: heads, dim, vdim, decay [per head], rot {dims, base}
      delta:     heads, kv_heads, dim, vdim, conv
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .files import ConfigError

MIXER_TYPES = ("attention", "retention", "delta")
MAX_POSITIONS = 1 << 20  # the file gives no limit; positions are 32-bit and angles float32


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Dezolorn config: {where} lacks {key!r}")
    return d[key]


@dataclass(frozen=True)
class DezolornLayer:
    type: str
    mixer: dict[str, Any]
    ff: int | None  # None: no feed-forward

    def to_hf(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer, "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class DezolornConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[DezolornLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = "Dezolorn"

    @classmethod
    def from_hf(cls, cfg: dict[str, Any], generation: dict[str, Any] | None = None) -> "DezolornConfig":
        if cfg.get("architecture") != "Dezolorn" and "Dezolorn" not in (cfg.get("architectures") or []):
            raise ConfigError(f"not a Dezolorn config: architecture={cfg.get('architecture')!r}")
        layers = []
        for i, entry in enumerate(_need(cfg, "layers", "config.json")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"Dezolorn config: {where} has the unknown mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            m = dict(_need(entry, "mixer", where))
            if m.get("heads") is not None and m.get("kv_heads") is None and kind != "retention":
                m["kv_heads"] = m["heads"]      # a file that leaves it out means one key head per head
            if m.get("dim") is not None and m.get("vdim") is None:
                m["vdim"] = m["dim"]            # ... and values as wide as keys
            for key in {"attention": ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"),
                        "retention": ("heads", "dim", "vdim", "decay", "rot"),
                        "delta": ("heads", "kv_heads", "dim", "vdim", "conv")}[kind]:
                _need(m, key, where + ".mixer")
            if kind == "attention":
                _need(m["mask"], "size", where + ".mixer.mask")
                m["mask"] = {"size": int(m["mask"]["size"]), "keep_first": int(m["mask"].get("keep_first") or 0)}
            if kind in ("attention", "retention"):
                for key in ("dims", "base"):
                    _need(m["rot"], key, where + ".mixer.rot")
                sc = m["rot"].get("scaling")
                if sc:
                    for key in ("factor", "original", "fast", "slow"):
                        _need(sc, key, where + ".mixer.rot.scaling")
            if kind == "retention" and len(m["decay"]) != int(m["heads"]):
                raise ConfigError(f"Dezolorn config: {where} gives {len(m['decay'])} decays for {m['heads']} heads")
            if kind != "retention" and int(m["heads"]) % int(m["kv_heads"]):
                raise ConfigError(f"Dezolorn config: {where}: {m['heads']} heads over {m['kv_heads']} key heads")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"Dezolorn config: {where} has the unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append(DezolornLayer(kind, m, None if mlp is None else int(_need(mlp, "ff", where + ".mlp"))))
        loop = cfg.get("loop") or {}
        start, stop, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
        if not (0 <= start <= stop <= len(layers)) or times < 1:
            raise ConfigError(f"Dezolorn config: loop {loop} does not fit {len(layers)} layers")
        eos = (generation or {}).get("eos_token_id", cfg.get("eos_token_id"))
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab=int(_need(cfg, "vocab", "config.json")), width=int(_need(cfg, "width", "config.json")),
                   eps=float(_need(_need(cfg, "norm", "config.json"), "eps", "norm")), layers=tuple(layers),
                   loop_start=start, loop_stop=stop, loop_times=times, logit_scale=float(cfg.get("logit_scale") or 1.0),
                   logit_softcap=float(cfg.get("logit_softcap") or 0.0), eos_token_ids=eos_ids)

    def to_hf(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
            "layers": [layer.to_hf() for layer in self.layers],
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
            "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def runs(self) -> list[tuple[int, bool]]:
        """(layer, whether the embedding's output is added before it) in the order of execution."""
        out = [(i, False) for i in range(self.loop_start)]
        for t in range(self.loop_times if self.loop_stop > self.loop_start else 0):
            out += [(i, t > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        out += [(i, False) for i in range(self.loop_stop, len(self.layers))]
        return out
