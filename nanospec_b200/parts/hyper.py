"""Hyper-connections: the residual stream kept as `streams` copies that every sublayer reads and rewrites through
small learned coefficients.

The stream of a step is one float32 tensor [N, streams * hidden] (a token's copies side by side); the embedding opens it
with every copy equal (`copies` of the "table" embedding).  Sublayer q of a layer, with coefficients in[S], out[S] and
mix[S, S] (first index: the copy read; second: the copy written):

    u   = sum_s in[s] x_s
    y   = sublayer(norm(u))
    x_t = sum_s mix[s, t] x_s + out[t] y        every t at once, from the old copies

and at the end the copies are added up.  This takes the place of the residual sum of "prenorm".  As there, a sublayer's
output stays pending: one kernel (`ops.stream_mix_norm`) rewrites the copies with the pending output, forms the next
sublayer's u and norms it, so the copies are read and written once per sublayer.  The same kernel closes the model (every
copy counted once, the final norm, only the wanted rows).

"hyper" is a block arrangement like "prenorm": mixer first, then an optional feed-forward, each behind its norm.  Slots
beside those of "prenorm": "hc_mixer" and "hc_feed_forward", the coefficients of the two sublayers (tensors `in`, `out`,
`mix` under the slot's sub-prefix).  `LayerSpec.params`: {"streams": S}.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..config.recipe import LayerSpec, PartSpec
from .base import Part, WeightSpec
from .context import LaneView, StepContext
from .registry import build_part, register_part


class StreamCoefficients(Part):
    """The coefficients of one sublayer: `in` [S], `out` [S], `mix` [S, S]; float32 in every mode."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.streams = int(spec["streams"])
        self.w_in = self.w_out = self.w_mix = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        s = self.streams
        return {"in": WeightSpec((s,), rule="float32", init="gain"), "out": WeightSpec((s,), rule="float32", init="gain"),
                "mix": WeightSpec((s, s), rule="float32", init="normal", std=0.5)}

    def bind(self, tensors) -> None:
        self.w_in, self.w_out, self.w_mix = (tensors[k].contiguous() for k in ("in", "out", "mix"))


@dataclass
class PendingWrite:
    """A sublayer's output that the copies have not taken yet, with the coefficients that say how they take it."""

    y: torch.Tensor
    coef: StreamCoefficients


@register_part("block", "hyper")
class HyperBlock:
    slots = ("norm_mixer", "mixer", "hc_mixer", "norm_feed_forward", "feed_forward", "hc_feed_forward")

    def __init__(self, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.layer = layer
        self.streams = int(layer.params["streams"])
        coef = PartSpec("stream_coefficients", {"streams": self.streams})
        self.mixer = build_part("mixer", layer.mixer, dtype, device)
        self.norm_mixer = build_part("norm", layer.norm, dtype, device)
        self.hc_mixer = StreamCoefficients(coef, dtype, device)
        has_ff = layer.feed_forward is not None
        self.feed_forward = build_part("feed_forward", layer.feed_forward, dtype, device) if has_ff else None
        self.norm_feed_forward = build_part("norm", layer.norm, dtype, device) if has_ff else None
        self.hc_feed_forward = StreamCoefficients(coef, dtype, device) if has_ff else None
        for norm in (self.norm_mixer, self.norm_feed_forward):
            if norm is not None and not hasattr(norm, "gain"):
                raise ValueError("the hyper arrangement folds its norms into the streams' kernel: a norm part with `gain`, `eps`, "
                                 "`centered` and `bias` is needed")

    def parts(self) -> dict:
        return {s: getattr(self, s) for s in self.slots if getattr(self, s) is not None}

    def _read(self, streams: torch.Tensor, pending: PendingWrite | None, coef: StreamCoefficients | None, norm, ctx: StepContext,
              rows: torch.Tensor | None = None, out_name: str = "normed") -> torch.Tensor:
        if pending is not None and not isinstance(pending, PendingWrite):
            raise ValueError("the hyper arrangement follows a block of its own kind (or opens the model)")
        n = streams.shape[0] if rows is None else rows.numel()
        out = ctx.buffer(out_name, norm.hidden, rows=n)
        pc = pending.coef if pending is not None else None
        return ops.stream_mix_norm(streams, self.streams, pending.y if pending is not None else None,
                                   pc.w_mix if pc is not None else None, pc.w_out if pc is not None else None,
                                   coef.w_in if coef is not None else None, norm.gain, norm.bias, norm.eps, norm.centered, out, rows=rows)

    def forward(self, streams: torch.Tensor, pending, ctx: StepContext, lane: LaneView, writes: bool = True):
        x = self._read(streams, pending, self.hc_mixer, self.norm_mixer, ctx)
        y = self.mixer.forward(x, ctx, lane, writes)
        pending = PendingWrite(y, self.hc_mixer)
        if self.feed_forward is None:
            return streams, pending
        x = self._read(streams, pending, self.hc_feed_forward, self.norm_feed_forward, ctx)
        return streams, PendingWrite(self.feed_forward.forward(x, ctx), self.hc_feed_forward)

    def close(self, streams: torch.Tensor, pending, norm, ctx: StepContext, rows: torch.Tensor | None = None,
              out_name: str = "final_normed") -> torch.Tensor:
        """The model's end: the pending output taken, the copies added up, the final norm; only `rows` when given."""
        return self._read(streams, pending, None, norm, ctx, rows=rows, out_name=out_name)

    def stream_sum(self, streams: torch.Tensor, pending, ctx: StepContext) -> torch.Tensor:
        """The sum of the copies as it stands after `pending` (float32 [N, hidden]); nothing is rewritten.  For probes."""
        out = ctx.buffer("stream_sum", streams.shape[1] // self.streams, torch.float32)
        pc = pending.coef if pending is not None else None
        return ops.stream_read(streams, self.streams, pending.y if pending is not None else None,
                               pc.w_mix if pc is not None else None, pc.w_out if pc is not None else None, None, out)
