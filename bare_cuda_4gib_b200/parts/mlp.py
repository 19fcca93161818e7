"""Dense SwiGLU feed-forward: down(silu(gate(h)) * up(h)), no biases, silu(g) = g / (1 + exp(-g))
(cuongvng/bare-cuda-4gib engine/src/model.cpp:589-598, engine/kernels/swiglu.cu:22-23).
gate and up are one matrix product against [Wgate; Wup], fused at load; where the fast kernel
runs, silu(gate) * up is its epilogue.

params: `hidden`, `intermediate`.  tensors: `gate`, `up`, `down`.
"""

from __future__ import annotations

import torch

from ..kernels import lib as K
from .base import Part
from .linear import Linear
from .registry import register_feed_forward
from ..weights.loader import fused_rows


@register_feed_forward("swiglu")
class SwiGLUFeedForward(Part):
    def local_weights(self):
        h, i = int(self.params["hidden"]), int(self.params["intermediate"])
        return {"gate": ((i, h), "matrix"), "up": ((i, h), "matrix"), "down": ((h, i), "matrix")}

    def adjacent_weights(self):
        return [("gate", "up")]

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.gate_up = Linear(fused_rows([t.pop("gate"), t.pop("up")]), "gate_up")
        self.down = Linear(t.pop("down"), "down")
        self.gate_up.prepare(dtype)
        self.down.prepare(dtype)

    takes_lazy_input = True

    def forward(self, ctx, h):
        n = ctx.n_tokens
        act = self.gate_up.forward(ctx, h, n, ctx.dtype, "ffn_act", swiglu=True)
        residual = getattr(ctx, "residual", None)
        return self.down.forward(ctx, act.tensor, n, torch.float32, "ffn_out", allow_partials=True,
                                 epilogue=K.AddTo(residual, getattr(ctx, "following_norm", None)) if residual is not None else None)


@register_feed_forward("dense")
class DenseFeedForward(Part):
    """down(act(up(h))), no gate and no biases; `activation` is "relu2" (the square of relu),
    "gelu_tanh", "silu" or "relu".

    params: `hidden`, `intermediate`, `activation`.  tensors: `up`, `down`."""

    takes_lazy_input = False

    def local_weights(self):
        h, i = int(self.params["hidden"]), int(self.params["intermediate"])
        return {"up": ((i, h), "matrix"), "down": ((h, i), "matrix")}

    def prepare(self, dtype, device) -> None:
        from ..kernels.streams import ACTIVATIONS
        if self.params.get("activation", "relu2") not in ACTIVATIONS:
            raise KeyError(f"dense feed-forward: activation '{self.params.get('activation')}' is not one of {sorted(ACTIVATIONS)}")
        t = self.tensors
        self.up = Linear(t.pop("up"), "up")
        self.down = Linear(t.pop("down"), "down")
        self.up.prepare(dtype)
        self.down.prepare(dtype)

    def forward(self, ctx, h):
        from ..kernels import streams as SK
        n = ctx.n_tokens
        z = self.up.forward(ctx, h, n, ctx.dtype, "ffn_up")
        act = ctx.ws.get("ffn_act", (n, int(self.params["intermediate"])), ctx.dtype)
        SK.activation(z, act, n, self.params.get("activation", "relu2"), ctx.stream)
        return self.down.forward(ctx, act, n, torch.float32, "ffn_out", allow_partials=True)


@register_feed_forward("glu")
class GatedFeedForward(Part):
    """down(act(gate(h)) * up(h)), no biases; `activation` is "silu" or "gelu_tanh" (the tanh form of
    gelu).  gate and up are one matrix product against [Wgate; Wup]; the kernels that fuse the
    activation into that product do so for both activations.  A third form, "clamped_swish", bounds
    both factors first: g = min(gate(h), limit), u = clamp(up(h), -limit, limit), and the product is
    g sigmoid(alpha g) (u + 1); the products fuse it from a library built with the two constants.

    params: `hidden`, `intermediate`, `activation` (, `limit`, `alpha`).  tensors: `gate`, `up`, `down`."""

    takes_lazy_input = False

    def local_weights(self):
        h, i = int(self.params["hidden"]), int(self.params["intermediate"])
        return {"gate": ((i, h), "matrix"), "up": ((i, h), "matrix"), "down": ((h, i), "matrix")}

    def adjacent_weights(self):
        return [("gate", "up")]

    def prepare(self, dtype, device) -> None:
        self.activation = self.params.get("activation", "silu")
        self.clamped = self.activation == "clamped_swish"
        if self.clamped:
            # the gated products take the form with its two constants like any other activation
            self.activation = K.clamped_swish(float(self.params["limit"]), float(self.params.get("alpha", 1.0)))
        elif self.activation not in K.GLU_ACTIVATIONS:
            raise KeyError(f"glu feed-forward: activation '{self.activation}' is not one of "
                           f"{sorted(K.GLU_ACTIVATIONS) + ['clamped_swish']}")
        t = self.tensors
        self.gate_up = Linear(fused_rows([t.pop("gate"), t.pop("up")]), "gate_up")
        self.down = Linear(t.pop("down"), "down")
        self.gate_up.prepare(dtype)
        self.down.prepare(dtype)

    def forward(self, ctx, h):
        n = ctx.n_tokens
        act = self.gate_up.forward(ctx, h, n, ctx.dtype, "ffn_act", glu=self.activation)
        return self.down.forward(ctx, act.tensor, n, torch.float32, "ffn_out", allow_partials=True)
