"""A layer arrangement with norms on both sides of every sublayer, a sigmoid gate on every sublayer's
result, and a weighted sum over the depth of the model at every layer's end:

    h = norm1(x);  x <- x + norm1b(mixer(h) * sigmoid(W_g1 h + b_g1))
    h = norm2(x);  x <- x + norm2b(ff(h) * sigmoid(W_g2 h + b_g2))          (where the layer has a feed-forward)
    X_(i+1) <- x;  x <- sum_{j = 0 .. i+1} a_i[j] X_j                       (X_0: the embedding's output)

The gate, the norm behind a sublayer, the add, the weighted sum and the next sublayer's norm are one
kernel (`kernels.gated_sandwich`): a sublayer's result is handed on as a `GatedDelta`, and the norm
that reads the stream next carries it out first.  Every X_j of the step's rows is kept in one float32
workspace buffer [layers + 1, rows, width]; nothing of it outlives the step.

Block "gated_sandwich": `layer_spec.extras` names "post1", "post2" (norms behind the sublayers), and
optionally "gate1", "gate2" (`ResidualGate`) and "depth" (`DepthAverage`); a part left out is a step
left out, so the arrangement also serves designs with only some of the three.
"""

from __future__ import annotations

import torch

from ..kernels.gated_sandwich import DepthMix, GatedDelta
from .base import Part
from .linear import Linear
from .registry import build_part, register_block


class ResidualGate(Part):
    """sigmoid(W h + b) on a sublayer's result, from the sublayer's own input h.  The projection runs
    here; the bias, the sigmoid and the product ride in the kernel that norms and adds the result.

    params: `size`.  tensors: `weight` [size, size], `bias` [size]."""

    def local_weights(self):
        n = int(self.params["size"])
        return {"weight": ((n, n), "matrix"), "bias": ((n,), "zero")}

    def prepare(self, dtype, device) -> None:
        self.proj = Linear(self.tensors["weight"], "residual_gate")
        self.proj.prepare(dtype)
        self.bias = self.tensors["bias"].to(torch.float32).contiguous()

    def forward(self, ctx, h, buffer: str):
        return self.proj.forward(ctx, h, ctx.n_tokens, ctx.dtype, buffer).tensor


class DepthAverage(Part):
    """Layer `index` keeps its result as entry index + 1 and hands sum_j weights[j] * entry j on.

    params: `index`, `entries` (layers + 1), `size`.  tensors: `weights` [index + 2]."""

    def local_weights(self):
        return {"weights": ((int(self.params["index"]) + 2,), "norm")}

    def prepare(self, dtype, device) -> None:
        self.weights = self.tensors["weights"].to(torch.float32).contiguous()
        self.index, self.entries, self.size = int(self.params["index"]), int(self.params["entries"]), int(self.params["size"])

    def history(self, ctx) -> torch.Tensor:
        return ctx.ws.get("depth_history", (self.entries, ctx.n_tokens, self.size), torch.float32, max_lead=self.entries)


@register_block("gated_sandwich")
class GatedSandwichBlock:
    def __init__(self, layer_spec):
        ex = layer_spec.extras
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.post1 = build_part("norm", ex["post1"])
        self.gate1 = ResidualGate(ex["gate1"]) if "gate1" in ex else None
        self.has_ffn = layer_spec.ffn is not None
        self.gate2 = None
        if self.has_ffn:
            self.ffn_norm = build_part("norm", layer_spec.ffn_norm)
            self.ffn = build_part("feed_forward", layer_spec.ffn)
            self.post2 = build_part("norm", ex["post2"])
            self.gate2 = ResidualGate(ex["gate2"]) if "gate2" in ex else None
        self.depth = DepthAverage(ex["depth"]) if "depth" in ex else None

    def parts(self):
        out = [self.mixer_norm, self.mixer, self.post1, self.gate1]
        if self.has_ffn:
            out += [self.ffn_norm, self.ffn, self.post2, self.gate2]
        return [p for p in out + [self.depth] if p is not None]

    def cache_demands(self):
        many = getattr(self.mixer, "cache_demands", None)
        return many() if many else [(self.mixer.cache_request(), self.mixer.state_request())]

    def entry_norm(self):
        return self.mixer_norm

    def _pending(self, ctx, post, gate, h, y, buffer, last: bool):
        depth = DepthMix(self.depth.history(ctx), self.depth.index + 1, self.depth.weights) if last and self.depth else None
        g = gate.forward(ctx, h, buffer) if gate is not None else None
        return GatedDelta(y, g, gate.bias if gate is not None else None, post.factor, float(post.params["eps"]), depth)

    def forward(self, ctx, call, residual, pending):
        n = ctx.n_tokens
        ctx.residual = None          # sublayers hand their result back: it is gated and normed before it is added
        ctx.following_norm = None
        if self.depth is not None and self.depth.index == 0 and pending is None:
            pending = GatedDelta(None, None, None, None, 0.0, DepthMix(self.depth.history(ctx), 0, None))   # entry 0
        h = self.mixer_norm.forward(ctx, residual, pending, n)
        pending = self._pending(ctx, self.post1, self.gate1, h, self.mixer.forward(ctx, call, h), "residual_gate1",
                                not self.has_ffn)
        if self.has_ffn:
            h = self.ffn_norm.forward(ctx, residual, pending, n)
            pending = self._pending(ctx, self.post2, self.gate2, h, self.ffn.forward(ctx, h), "residual_gate2", True)
        return pending
