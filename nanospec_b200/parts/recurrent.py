"""Mixers whose memory is a matrix per head instead of a growing cache: retention (linear attention with a fixed decay
per head) and the gated delta rule.  Both keep S [heads, head_dim, v_dim] in float32 in the request's state slot and walk
a step's tokens in order (csrc/recurrent.cu), so portions of a prompt, single decoded tokens and whole prompts give the
same numbers; under CUDA graphs they address the state through the device's `qo_indptr` and `state_slot`.

    retention   S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t;  q and k rotated by position, k times head_dim^-1/2;
                per head o / rms(o), all heads times silu(gate), output projection.
    delta       q, k, v pass a short causal convolution per channel and silu; q and k become unit vectors, q times
                head_dim^-1/2; beta = sigmoid(b h), g = exp(-exp(A_log) softplus(a h + dt_bias));
                S = g S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q;  per head o / rms(o) times a gain shared by the
                heads, times silu(gate), output projection.  The last taps - 1 inputs of the convolution are state as well.

The projections are one packed product; the convolution, the rotation, the unit norms, the decay and the read-out's norm are
float32.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Part, StateNeed, WeightSpec
from .context import LaneView, StepContext
from .registry import build_part, register_part


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """A packed projection whose row count is a multiple of 8: rows of its output are then 16-byte aligned in bfloat16."""
    extra = -w.shape[0] % multiple
    if extra:
        w = torch.cat([w, torch.zeros((extra, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
    return w.contiguous()


@register_part("mixer", "retention")
class Retention(Part):
    """params: hidden, heads, head_dim, v_dim, decay (one per head), eps (of the read-out's norm), position (PartSpec of kind
    "rotary", or None), names (optional: keys "q", "k", "v", "g", "o")."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.head_dim, self.v_dim = int(p["head_dim"]), int(p["v_dim"])
        self.eps = float(p["eps"])
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"retention: {len(decay)} decays for {self.heads} heads")
        self.decay_host = torch.tensor(decay, dtype=torch.float32)
        self._decay: torch.Tensor | None = None
        self.position = build_part("position", p["position"], dtype, device) if p.get("position") is not None else None
        names = dict(p.get("names") or {})
        self.names = {k: names.get(k, k + "_proj.weight") for k in ("q", "k", "v", "g", "o")}
        self.qk_size, self.v_size = self.heads * self.head_dim, self.heads * self.v_dim
        self.dp = ops.scan_padded_dim(self.head_dim)
        self.rec_cols = -(-(2 * self.heads * self.dp + self.v_size + self.heads) // 4) * 4  # q, k, v, k . q
        self.w_in: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        n = self.names
        return {n["q"]: WeightSpec((self.qk_size, self.hidden)), n["k"]: WeightSpec((self.qk_size, self.hidden)),
                n["v"]: WeightSpec((self.v_size, self.hidden)), n["g"]: WeightSpec((self.v_size, self.hidden)),
                n["o"]: WeightSpec((self.hidden, self.v_size))}

    def bind(self, tensors) -> None:
        n = self.names
        self.w_in = _pad_rows(torch.cat([tensors[n[k]] for k in ("q", "k", "v", "g")], dim=0))
        self.w_o = tensors[n["o"]].contiguous()

    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return StateNeed((self.heads * self.head_dim * self.v_dim,), torch.float32)

    def forward(self, x, ctx: StepContext, lane: LaneView, writes: bool = True):
        if not writes:
            raise ValueError("a retention mixer owns its state: its lane cannot be shared")
        if self._decay is None:
            self._decay = self.decay_host.to(self.device)
        proj = ops.linear(x, self.w_in, ctx.buffer("rec_proj", self.w_in.shape[0]))
        rec = ctx.buffer("rec_in", self.rec_cols, torch.float32)
        pos = self.position
        ops.rotary_prepare(proj, ctx, pos.inv_freq if pos is not None and pos.dims else None, pos.magnitude if pos is not None else 1.0,
                           pos.interleaved if pos is not None else False, rec, self.heads, self.head_dim, self.v_dim,
                           1.0, self.head_dim ** -0.5)
        read = ops.linear_scan(rec, lane.state, ctx, ctx.buffer("rec_out", self.v_size, torch.float32), self.heads, self.heads,
                               self.head_dim, self.v_dim, decay=self._decay)
        gate = proj[:, 2 * self.qk_size + self.v_size: 2 * self.qk_size + 2 * self.v_size]
        y = ops.head_norm_gate(read, gate, None, self.eps, ctx.buffer("rec_y", self.v_size), ctx, self.heads, self.v_dim)
        return ops.linear(y, self.w_o, ctx.buffer("branch", self.hidden))


@register_part("mixer", "gated_delta")
class GatedDeltaRule(Part):
    """params: hidden, heads, kv_heads (q and k heads; head h reads q/k head h // (heads / kv_heads)), head_dim, v_dim, conv
    (taps of the short convolution), eps (of the read-out's norm), unit_eps (inside the root of the unit norms; default 1e-6),
    names (optional: keys "q", "k", "v", "g", "o", "a", "b", "q_conv", "k_conv", "v_conv", "A_log", "dt_bias", "norm")."""

    DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight", "o": "o_proj.weight",
                     "a": "a_proj.weight", "b": "b_proj.weight", "q_conv": "q_conv.weight", "k_conv": "k_conv.weight",
                     "v_conv": "v_conv.weight", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "o_norm.weight"}

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.head_dim, self.v_dim, self.taps = int(p["head_dim"]), int(p["v_dim"]), int(p["conv"])
        self.eps = float(p["eps"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        if self.heads % self.kv_heads or self.taps < 1:
            raise ValueError(f"gated_delta: {self.heads} heads over {self.kv_heads} key heads, {self.taps} taps")
        names = dict(p.get("names") or {})
        self.names = {k: names.get(k, d) for k, d in self.DEFAULT_NAMES.items()}
        self.qk_size, self.v_size = self.kv_heads * self.head_dim, self.heads * self.v_dim
        self.channels = 2 * self.qk_size + self.v_size
        self.dp = ops.scan_padded_dim(self.head_dim)
        self.rec_cols = -(-(2 * self.kv_heads * self.dp + self.v_size + 2 * self.heads + self.kv_heads) // 4) * 4  # q, k, v, g, beta, k . q
        self.s_floats = self.heads * self.head_dim * self.v_dim
        self.off_g = self.channels
        self.off_b = self.channels + self.v_size
        self.off_a = self.off_b + self.heads
        self.w_in = self.w_o = self.conv_taps = self.a_log = self.dt_bias = self.gain = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        n = self.names
        small = dict(rule="float32")
        return {
            n["q"]: WeightSpec((self.qk_size, self.hidden)), n["k"]: WeightSpec((self.qk_size, self.hidden)),
            n["v"]: WeightSpec((self.v_size, self.hidden)), n["g"]: WeightSpec((self.v_size, self.hidden)),
            n["b"]: WeightSpec((self.heads, self.hidden)), n["a"]: WeightSpec((self.heads, self.hidden)),
            n["o"]: WeightSpec((self.hidden, self.v_size)),
            n["q_conv"]: WeightSpec((self.qk_size, self.taps), std=0.5, **small),
            n["k_conv"]: WeightSpec((self.qk_size, self.taps), std=0.5, **small),
            n["v_conv"]: WeightSpec((self.v_size, self.taps), std=0.5, **small),
            n["A_log"]: WeightSpec((self.heads,), std=0.5, **small), n["dt_bias"]: WeightSpec((self.heads,), std=0.5, **small),
            n["norm"]: WeightSpec((self.v_dim,), init="gain", **small),
        }

    def bind(self, tensors) -> None:
        n = self.names
        self.w_in = _pad_rows(torch.cat([tensors[n[k]] for k in ("q", "k", "v", "g", "b", "a")], dim=0))
        self.w_o = tensors[n["o"]].contiguous()
        self.conv_taps = torch.cat([tensors[n[k]] for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias = tensors[n["A_log"]].contiguous(), tensors[n["dt_bias"]].contiguous()
        self.gain = tensors[n["norm"]].contiguous()

    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        # S, then the convolution's last taps - 1 inputs [taps - 1, channels]
        return StateNeed((self.s_floats + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, ctx: StepContext, lane: LaneView, writes: bool = True):
        if not writes:
            raise ValueError("a delta-rule mixer owns its state: its lane cannot be shared")
        proj = ops.linear(x, self.w_in, ctx.buffer("rec_proj", self.w_in.shape[0]))
        rec = ctx.buffer("rec_in", self.rec_cols, torch.float32)
        ops.delta_prepare(proj, self.conv_taps, self.a_log, self.dt_bias, lane.state, self.s_floats, ctx, rec, self.kv_heads,
                          self.heads, self.head_dim, self.v_dim, self.off_b, self.off_a, self.head_dim ** -0.5, self.unit_eps)
        read = ops.linear_scan(rec, lane.state, ctx, ctx.buffer("rec_out", self.v_size, torch.float32), self.heads, self.kv_heads,
                               self.head_dim, self.v_dim, gated=True)
        gate = proj[:, self.off_g: self.off_g + self.v_size]
        y = ops.head_norm_gate(read, gate, self.gain, self.eps, ctx.buffer("rec_y", self.v_size), ctx, self.heads, self.v_dim)
        return ops.linear(y, self.w_o, ctx.buffer("branch", self.hidden))
