"""A mixture-of-experts feed-forward.

    z = W_router h (float32);  s = softmax(z) over all experts;  the `top` experts with the largest s are
    chosen (the lowest index wins a tie);  weight_e = s_e * router_scale, not renormalised;
    out = sum over the chosen e of weight_e * W_down,e (silu(W_gate,e h) * (W_up,e h));
    with a shared expert (same form, its own size):  out += sigmoid(w_sg . h) * shared(h), one gate per token.

The experts' matrices are stacked ([experts, 2 * ff, hidden] with an expert's gate rows before its up
rows, and [experts, hidden, ff]); a step's (token, choice) slots are grouped by expert on the device, and
two grouped products walk the groups, so no host decision depends on the router and a step is captured
in a CUDA graph like any other.  bfloat16 steps run both on the tensor cores (the dense product's kernel,
given the list of row tiles: a tile's rows are one expert's, its weight rows that expert's); float32 steps
run them in plain arithmetic.  A row of a product depends on that row alone, and a token's slots are added
in the order of the choice, so a token's result does not depend on what else is in the step.  The
shared expert runs on the engine's dense products.

Options beside that form (each off unless its parameter is given):

* `expert_form` "relu2": an expert is W_down relu(W_up h)^2, with no gate matrix;
* `identity` n: the router has n more outputs behind the experts' own, identity experts without tensors
  whose result is h itself (times the weight);
* `correction`: a tensor with one number per router output that is added to the score for the choice
  only; the weight stays the score;
* `groups`, `keep`: the router's outputs (identity experts included) form `groups` equal groups of
  neighbours, a group counts by its largest choice value, and only experts of the `keep` best groups can
  be chosen.

params: `hidden`, `experts`, `top`, `router_scale`, `intermediate`, `shared_intermediate` (None: no shared
expert), `shared_gate` (bool), `expert_form`, `identity`, `correction` (bool), `groups`, `keep`.
tensors: `router` [experts + identity, hidden], `correction` [experts + identity], `e<j>.gate|up`
[intermediate, hidden] (relu2: `e<j>.up` only), `e<j>.down` [hidden, intermediate], `shared.gate|up|down`,
`shared.sg` [1, hidden].
"""

from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import lib as K
from .base import Part
from .linear import Linear
from .registry import register_feed_forward
from ..weights.loader import fused_rows


@register_feed_forward("moe")
class MixtureOfExperts(Part):
    takes_lazy_input = False

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.experts, self.top, self.ff = int(p["hidden"]), int(p["experts"]), int(p["top"]), int(p["intermediate"])
        self.router_scale = float(p.get("router_scale", 1.0))
        self.shared_ff = int(p["shared_intermediate"]) if p.get("shared_intermediate") else 0
        self.has_shared_gate = bool(p.get("shared_gate")) and self.shared_ff > 0
        self.gated = p.get("expert_form", "glu_silu") != "relu2"
        if p.get("expert_form", "glu_silu") not in ("glu_silu", "relu2"):
            raise ConfigError(f"moe: expert_form '{p.get('expert_form')}' is not one of ['glu_silu', 'relu2']")
        self.identity = int(p.get("identity") or 0)
        self.outputs = self.experts + self.identity          # what the router scores
        self.has_correction = bool(p.get("correction"))
        self.groups, self.keep = int(p.get("groups") or 1), int(p.get("keep") or p.get("groups") or 1)
        from ..kernels.moe import MAX_EXPERTS
        if not (1 <= self.top <= self.outputs <= MAX_EXPERTS) or self.experts < 1:
            raise ConfigError(f"moe: {self.top} of {self.outputs} experts (at most {MAX_EXPERTS}) cannot be chosen")
        if self.groups > 1 and (self.outputs % self.groups or not (1 <= self.keep <= self.groups)
                                or self.top > self.keep * (self.outputs // self.groups)):
            raise ConfigError(f"moe: {self.outputs} router outputs in {self.groups} groups of which {self.keep} stay "
                              f"cannot give {self.top} choices")

    def _matrices(self):
        return ("gate", "up") if self.gated else ("up",)

    def local_weights(self):
        out = {"router": ((self.outputs, self.hidden), "matrix")}
        if self.has_correction:
            out["correction"] = ((self.outputs,), "zero")
        for e in range(self.experts):
            for n in self._matrices():
                out[f"e{e}.{n}"] = ((self.ff, self.hidden), "matrix")
            out[f"e{e}.down"] = ((self.hidden, self.ff), "matrix")
        if self.shared_ff:
            out["shared.gate"] = ((self.shared_ff, self.hidden), "matrix")
            out["shared.up"] = ((self.shared_ff, self.hidden), "matrix")
            out["shared.down"] = ((self.hidden, self.shared_ff), "matrix")
            if self.has_shared_gate:
                out["shared.sg"] = ((1, self.hidden), "matrix")
        return out

    def adjacent_weights(self):
        groups = [tuple(f"e{e}.{t}" for e in range(self.experts) for t in self._matrices()),
                  tuple(f"e{e}.down" for e in range(self.experts))]
        if self.shared_ff:
            groups.append(("shared.gate", "shared.up"))
        return groups

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        E = self.experts
        self.w_up = fused_rows([t[f"e{e}.{n}"] for e in range(E) for n in self._matrices()]).to(dtype).contiguous()
        self.correction = t["correction"].to(torch.float32).contiguous() if self.has_correction else None
        self.w_down = fused_rows([t[f"e{e}.down"] for e in range(E)]).to(dtype).contiguous()
        self.w_router = t["router"].contiguous()
        self.w_sg = t["shared.sg"].to(self.w_router.dtype).reshape(-1).contiguous() if self.has_shared_gate else None
        if self.shared_ff:
            self.shared_gate_up = Linear(fused_rows([t["shared.gate"], t["shared.up"]]), "moe.shared.gate_up")
            self.shared_down = Linear(t["shared.down"], "moe.shared.down")
            self.shared_gate_up.prepare(dtype)
            self.shared_down.prepare(dtype)
        from ..kernels.moe import GroupedPlan
        # bfloat16 experts whose rows the copy engine can fetch run on the tensor cores
        self.plan = (GroupedPlan(self.w_up, self.w_down, E, self.gated)
                     if self.w_up.is_cuda and self.ff % 8 == 0 and GroupedPlan.takes(self.w_up, self.w_down) else None)
        for e in range(E):      # the stacked matrices stand for them from here on
            for n in self._matrices() + ("down",):
                t.pop(f"e{e}.{n}")
        t["experts.up"], t["experts.down"] = self.w_up, self.w_down

    def forward(self, ctx, h):
        from ..kernels import moe as M
        n, top, E = ctx.n_tokens, self.top, self.experts
        slots = n * top
        i32, f32 = torch.int32, torch.float32
        ids = ctx.ws.get("moe_ids", (n, top), i32)
        weights = ctx.ws.get("moe_weights", (n, top), f32)
        gate = ctx.ws.get("moe_shared_gate", (n, 1), f32) if self.has_shared_gate else None
        sorted_slots = ctx.ws.get("moe_sorted", (n, top), i32)
        # room for every tile a step of this shape can make, three numbers each, and their count
        tiles = ctx.ws.get("moe_tiles", (n, 3 * (top + E) + 1), i32)
        tc = self.plan is not None and ctx.dtype == torch.bfloat16 and h.dtype == torch.bfloat16
        n_tiles = tiles.view(-1)[3 * M.max_tiles(slots, E, tc):]
        M.route(ctx, h, self.w_router, self.w_sg, top, self.router_scale, ids, weights, gate, n, self.correction,
                self.groups, self.keep)
        M.sort(ctx, ids, slots, E, sorted_slots, tiles, n_tiles, tc)
        act = ctx.ws.get("moe_act", (n, top * self.ff), ctx.dtype)
        act_rows = act.view(-1)[: slots * self.ff].view(slots, self.ff)
        y = ctx.ws.get("moe_y", (n, top * self.hidden), f32)
        if tc:
            # the tokens' rows in the order of the list, so that a tile's rows lie together for the copy engine
            rows_in = ctx.ws.get("moe_rows", (n, top * self.hidden), ctx.dtype)
            rows_in = rows_in.view(-1)[: slots * self.hidden].view(slots, self.hidden)
            M.gather_rows(ctx, h, sorted_slots, top, rows_in, slots)
            M.grouped_tensor(ctx, self.plan, rows_in, act_rows, False, sorted_slots, tiles, n_tiles, weights, slots)
            M.grouped_tensor(ctx, self.plan, act_rows, y.view(-1)[: slots * self.hidden].view(slots, self.hidden), True,
                             sorted_slots, tiles, n_tiles, weights, slots)
        else:
            M.grouped(ctx, h, self.w_up, act, False, sorted_slots, tiles, n_tiles, weights, top, self.ff, self.hidden,
                      slots, E, self.gated)
            M.grouped(ctx, act_rows, self.w_down, y, True, sorted_slots, tiles, n_tiles, weights, top, self.hidden, self.ff,
                      slots, E)
        shared = None
        if self.shared_ff:
            a = self.shared_gate_up.forward(ctx, h, n, ctx.dtype, "moe_shared_act", glu="silu")
            shared = self.shared_down.forward(ctx, a.tensor, n, f32, "moe_shared_out", allow_partials=True)
        out = ctx.ws.get("ffn_out", (n, self.hidden), f32)
        if self.identity:
            M.combine(ctx, y, top, shared, gate, out, n, self.hidden, ids, weights, E, h)
        else:
            M.combine(ctx, y, top, shared, gate, out, n, self.hidden)
        return K.Partials(out)
