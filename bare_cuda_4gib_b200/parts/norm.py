"""RMSNorm, fused with the residual add that precedes it.

out = x * rsqrt(mean(x^2) + eps) * w with eps inside the root, on the mean, and the weight
multiplied last (cuongvng/bare-cuda-4gib engine/kernels/rmsnorm.cu:26-40).  The reference adds
the residual in a kernel of its own (engine/kernels/residual_add.cu:20); here the add of the
previous part's contribution and the norm are one kernel, and the residual stream stays float32.

params: `size` (width), `eps`, `one_plus` (optional: the weight is stored around zero and the factor
is 1 + w, formed once in float32).  tensors: `weight` [size].
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import lib as K
from .base import Part
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    prenormable = True      # the norm's factor is one number per row (see kernels.lib.AddTo)

    def __init__(self, spec):
        super().__init__(spec)
        if self.params.get("one_plus"):
            # 1 + w needs more digits than a 16-bit weight has: it stays float32, and the products that
            # norm their own input (which take the weight in the step's type) are not offered this norm
            self.prenormable = False

    def local_weights(self):
        return {"weight": ((self.params["size"],), "zero" if self.params.get("one_plus") else "norm")}

    def prepare(self, dtype, device) -> None:
        if self.params.get("one_plus"):
            self.tensors["weight"] = (1.0 + self.tensors["weight"].to(torch.float32)).contiguous()

    def forward(self, ctx, residual: torch.Tensor, delta: Optional[K.Partials], rows: int,
                row_index: Optional[torch.Tensor] = None, buffer: str = "normed", lazy: bool = False):
        """With `lazy` (the consumer takes a `LazyNorm`) and nothing to add, a few-token bfloat16
        step gets the norm as a description that the consuming product computes in its own kernel."""
        left = getattr(ctx, "prenormed", None)       # what the last adding product may have left for this norm
        ctx.prenormed = None
        if lazy and delta is None and ctx.dtype == torch.bfloat16 and ctx.use_fast_gemm and self.prenormable:
            from ..kernels import gemv
            mine = left if left is not None and left.norm is self else None
            # a few-token step norms inside the consuming product; a many-token step only where the
            # product before this norm has prepared it
            if (gemv.takes(rows, int(self.params["size"])) or mine is not None) and self.tensors["weight"].is_cuda:
                return K.LazyNorm(ctx, residual, self.tensors["weight"], float(self.params["eps"]), rows,
                                  row_index, buffer, mine)
        out = ctx.ws.get(buffer, (rows, self.params["size"]), ctx.dtype)
        K.add_rmsnorm(residual, delta, self.tensors["weight"], out, float(self.params["eps"]), rows,
                      row_index, ctx.stream)
        return out


@register_norm("sandwich_rmsnorm")
class SandwichRMSNorm(Part):
    """RMS norm of a stream whose sublayers are normed on both sides, x <- x + norm_b(f(norm(x))).
    As the norm before a sublayer it first adds what is pending, a `NormedDelta` (the previous
    sublayer's result with the weight of its norm behind), in the same kernel; as the norm behind a
    sublayer it only lends its weight (`pending`).

    params: `size`, `eps`.  tensors: `weight` [size]."""

    def local_weights(self):
        return {"weight": ((self.params["size"],), "norm")}

    def prepare(self, dtype, device) -> None:
        self.weight = self.tensors["weight"].to(dtype).contiguous()

    def pending(self, y):
        from ..kernels.sandwich import NormedDelta
        return NormedDelta(y, self.weight, float(self.params["eps"]))

    def forward(self, ctx, residual: torch.Tensor, delta, rows: int, row_index: Optional[torch.Tensor] = None,
                buffer: str = "normed", lazy: bool = False):
        from ..kernels import sandwich as SW
        out = ctx.ws.get(buffer, (rows, self.params["size"]), ctx.dtype)
        SW.postnorm_add_rmsnorm(residual, delta, self.weight, out, float(self.params["eps"]), rows, row_index, ctx.stream)
        return out


@register_norm("gated_sandwich_rmsnorm")
class GatedSandwichRMSNorm(Part):
    """RMS norm of a stream whose sublayers are normed on both sides and gated, x <- x + norm_b(gate *
    f(norm(x))), with float32 factors.  As the norm before a sublayer it first does what is pending (a
    `kernels.gated_sandwich.GatedDelta`: gate, norm behind the sublayer, add, and at a layer's end the
    weighted sum over the layers so far), in the same kernel; as the norm behind a sublayer it only
    lends its factor (`factor`).

    params: `size`, `eps`, `one_plus` (the weight is stored around zero and the factor is 1 + w).
    tensors: `weight` [size]."""

    def local_weights(self):
        return {"weight": ((self.params["size"],), "zero" if self.params.get("one_plus") else "norm")}

    def prepare(self, dtype, device) -> None:
        w = self.tensors["weight"].to(torch.float32)
        self.factor = ((1.0 + w) if self.params.get("one_plus") else w).contiguous()

    def forward(self, ctx, residual: torch.Tensor, delta, rows: int, row_index: Optional[torch.Tensor] = None,
                buffer: str = "normed", lazy: bool = False):
        from ..kernels import gated_sandwich as GS
        out = ctx.ws.get(buffer, (rows, self.params["size"]), ctx.dtype)
        GS.step(residual, delta, self.factor, out, float(self.params["eps"]), rows, row_index, ctx.stream)
        return out
