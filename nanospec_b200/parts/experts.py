"""A feed-forward of routed experts: every token runs `top` of `experts` small gated feed-forwards and adds their outputs
up with weights from a router.

    z = W_router h   (a float32 product in every mode)          s = sigmoid(z)   ("score": "softmax" for a softmax over z)
    experts e * per .. (e + 1) * per - 1 form group e (`groups` of them, per = experts / groups); group score = top-2 sum of its s
    (its one s when per is 1); the `keep` groups of highest score stay eligible, the rest are barred (groups <= 1: none barred)
    the `top` eligible experts of largest s are chosen; weight_k = s_k / (sum of the chosen s + 1e-20) * scale
    y = sum_k weight_k * down_k(silu(gate_k h) * (up_k h))

Four routes, the same numbers up to rounding.  A bfloat16 step (of up to `GROUPED_MAX` tokens when that is set, and every step that a CUDA
graph captures) lays the (token, choice) pairs out by expert on the device (`ops.moe_plan`) and runs every expert over its
rows in one tensor-core kernel that reads the counts on the device (`ops.moe_grouped`): each chosen expert's weights are
read once, nothing comes back to the host.  float32 steps of a few tokens (`ROWS_MAX` or fewer, or captured) run
`ops.moe_expert_rows`: the chosen experts' rows are streamed per (token, choice).  A longer step brings every expert's tokens side by side (`ops.moe_plan`, `ops.moe_gather`) and reads the counts
on the host; in bfloat16 every expert then owns the same number of rows (`ops.moe_pad_rows`) and all experts run as one batched
library product for gate/up and one for down; in float32 each expert that has tokens runs as the framework's gated product and down
product over its run of rows.  `ops.moe_combine` adds the results per token in the order of the choice (float32 sums, one rounding).

params: hidden, experts, top, intermediate (an expert's width), groups, keep, scale, score, names (optional: "router";
the experts' tensors are e<k>.gate, e<k>.up, e<k>.down).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec
from .context import StepContext
from .registry import register_part

ROWS_MAX = 16      # steps of up to this many tokens stream the chosen experts' rows (float32, or widths that are no multiple of 8)
# bfloat16 steps of up to this many tokens run every expert over its tokens in one tensor-core kernel that reads the counts on the
# device (None: every step).  Longer steps read the counts on the host and run all experts as ONE batched library product over a
# layout in which every expert owns the same number of rows (the largest count, rounded up to 64): a product per expert would change
# shape with every step's counts, and the library's choice of a kernel for a shape it has not seen costs the host about a
# millisecond a call (a prompt of 2,048 tokens over 32 experts spent 75 ms there); the batched shapes are few and come again.
GROUPED_MAX: int | None = 512
PAD_WASTE_MAX = 4.0  # the batched layout is used while it holds at most this many times the step's rows (else: the grouped kernel)


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden, self.experts, self.top, self.inter = int(p["hidden"]), int(p["experts"]), int(p["top"]), int(p["intermediate"])
        self.groups, self.keep = int(p.get("groups") or 1), int(p.get("keep") or 1)
        self.scale = float(p.get("scale") if p.get("scale") is not None else 1.0)
        self.softmax = p.get("score", "sigmoid") == "softmax"
        if p.get("score", "sigmoid") not in ("sigmoid", "softmax"):
            raise ValueError(f"routed_experts: unknown score {p.get('score')!r}")
        if self.top > self.experts or (self.groups > 1 and (self.experts % self.groups or not 1 <= self.keep <= self.groups
                                                             or self.keep * (self.experts // self.groups) < self.top)):
            raise ValueError(f"routed_experts: {self.top} of {self.experts} experts in {self.groups} groups of which {self.keep} stay")
        self.n_router = dict(p.get("names") or {}).get("router", "router")
        self.w_router = self.w_gate = self.w_up = self.w_down = self.w_gate_up = None
        self.gate_block = 0

    def weight_specs(self) -> dict[str, WeightSpec]:
        specs = {self.n_router: WeightSpec((self.experts, self.hidden), rule="float32", init="normal", std=0.1)}
        for e in range(self.experts):
            specs[f"e{e}.gate"] = WeightSpec((self.inter, self.hidden))
            specs[f"e{e}.up"] = WeightSpec((self.inter, self.hidden))
            specs[f"e{e}.down"] = WeightSpec((self.hidden, self.inter))
        return specs

    def bind(self, tensors) -> None:
        E = self.experts
        self.w_router = tensors[self.n_router].contiguous()
        self.w_gate = torch.stack([tensors[f"e{e}.gate"] for e in range(E)]).contiguous()   # [E, ff, width]
        self.w_up = torch.stack([tensors[f"e{e}.up"] for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()   # [E, width, ff]
        # per expert the packed projection that the gated product takes (see parts/feed_forward.py)
        self.gate_block = ops.GATE_BLOCK if self.inter % ops.GATE_BLOCK == 0 else 0
        if self.gate_block:
            b = self.gate_block
            packed = torch.stack([self.w_gate.view(E, self.inter // b, b, self.hidden), self.w_up.view(E, self.inter // b, b, self.hidden)], dim=2)
            self.w_gate_up = packed.reshape(E, 2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([self.w_gate, self.w_up], dim=1).contiguous()

    def route(self, x, ctx: StepContext) -> tuple[torch.Tensor, torch.Tensor]:
        """(chosen experts int32 [N, top], their weights float32 [N, top])"""
        n = x.shape[0]
        logits = ops.router_logits(x, self.w_router, ctx.buffer("router_logits", self.experts, torch.float32),
                                   scratch=lambda rows, cols: ctx.buffer("router_in", cols, torch.float32, rows=rows))
        ids = ctx.buffer("expert_ids", self.top, torch.int32)
        weights = ctx.buffer("expert_weights", self.top, torch.float32)
        ops.moe_route(logits, self.groups, self.keep, self.top, self.scale, ids, weights, self.softmax)
        return ids, weights

    def _grouped(self, x, ids, weights, offsets, row_of, out, ctx: StepContext):
        n = x.shape[0]
        pair_of = ctx.buffer("expert_pairs", self.top, torch.int32)
        ops.moe_plan(ids, self.experts, offsets, row_of, pair_of)
        act = ctx.buffer("expert_act", self.inter, rows=n * self.top)
        ys = ctx.buffer("expert_out", self.hidden, rows=n * self.top)
        ops.moe_grouped(x, pair_of, offsets, self.w_gate, self.w_up, self.w_down, act, ys, self.top)
        return ops.moe_combine(ys, row_of, weights, out, self.top)

    def forward(self, x, ctx: StepContext):
        n = x.shape[0]
        ids, weights = self.route(x, ctx)
        out = ctx.buffer("branch", self.hidden)
        captured = bool(ctx.extras.get("graph")) or torch.cuda.is_current_stream_capturing()
        offsets = ctx.buffer("expert_offsets", 1, torch.int32, rows=self.experts + 1).view(-1)
        row_of = ctx.buffer("expert_rows", self.top, torch.int32)
        grouped_ok = ops.moe_grouped_ok(x, self.hidden, self.inter)
        if grouped_ok and (GROUPED_MAX is None or n <= GROUPED_MAX or captured):
            return self._grouped(x, ids, weights, offsets, row_of, out, ctx)
        if n <= ROWS_MAX or captured:
            act = ctx.buffer("expert_act", self.inter, rows=n * self.top)
            return ops.moe_expert_rows(x, ids, weights, self.w_gate, self.w_up, self.w_down, act, out)
        ops.moe_plan(ids, self.experts, offsets, row_of)
        bounds = offsets.tolist()  # the one host round trip of the step's experts
        if grouped_ok:
            # bfloat16: every expert owns `cap` rows and all run as one batched product each for gate/up and down
            cap = -(-max(b - a for a, b in zip(bounds, bounds[1:])) // 64) * 64
            rows = self.experts * cap
            if rows > PAD_WASTE_MAX * n * self.top:  # the tokens crowd a few experts: no layout of equal shares for them
                return self._grouped(x, ids, weights, offsets, row_of, out, ctx)
            ops.moe_pad_rows(ids, offsets, row_of, cap)
            xs = ops.moe_gather(x, row_of, ctx.buffer("expert_in", self.hidden, rows=rows), self.top)
            gu = ctx.buffer("expert_gate_up", 2 * self.inter, rows=rows)
            torch.bmm(xs.view(self.experts, cap, self.hidden), self.w_gate_up.transpose(1, 2), out=gu.view(self.experts, cap, 2 * self.inter))
            act = ops.swiglu(gu, ctx.buffer("expert_act", self.inter, rows=rows), self.gate_block)
            ys = ctx.buffer("expert_out", self.hidden, rows=rows)
            torch.bmm(act.view(self.experts, cap, self.inter), self.w_down.transpose(1, 2), out=ys.view(self.experts, cap, self.hidden))
            return ops.moe_combine(ys, row_of, weights, out, self.top)
        xs = ops.moe_gather(x, row_of, ctx.buffer("expert_in", self.hidden, rows=n * self.top), self.top)
        ys = ctx.buffer("expert_out", self.hidden, rows=n * self.top)
        act = ctx.buffer("expert_act", self.inter, rows=n * self.top)
        scratch = ctx.buffer("expert_gate_up", 2 * self.inter, rows=n * self.top)
        for e in range(self.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                ops.gated_linear(xs[lo:hi], self.w_gate_up[e], act[lo:hi], scratch[lo:hi], self.gate_block)
                ops.linear(act[lo:hi], self.w_down[e], ys[lo:hi])
        return ops.moe_combine(ys, row_of, weights, out, self.top)
