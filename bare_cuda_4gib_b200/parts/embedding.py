"""Token embedding and output head.

Embedding: x[t, :] = E[ids[t], :], no scale and no position term
(cuongvng/bare-cuda-4gib engine/kernels/embedding_lookup.cu:22-30), widened into the float32
residual stream.  Head: logits = normed lm_head^T in float32, only for the rows that were asked
for (the reference computes every row: engine/src/model.cpp:612-615).
"""

from __future__ import annotations

import torch

from ..kernels import lib as K
from .base import Part
from .linear import Linear
from .registry import register_embedding, register_head


@register_embedding("table")
class TokenEmbedding(Part):
    """params: `vocab`, `hidden`.  tensors: `weight` [vocab, hidden]."""

    def local_weights(self):
        return {"weight": ((int(self.params["vocab"]), int(self.params["hidden"])), "matrix")}

    def forward(self, ctx) -> torch.Tensor:
        x = ctx.ws.get("residual", (ctx.n_tokens, int(self.params["hidden"])), torch.float32)
        K.embed_gather(self.tensors["weight"], ctx.token_ids, x, ctx.n_tokens, ctx.stream)
        return x


@register_head("linear")
class OutputHead(Part):
    """params: `vocab`, `hidden`.  tensors: `weight` [vocab, hidden] (may be the embedding's)."""

    def local_weights(self):
        return {"weight": ((int(self.params["vocab"]), int(self.params["hidden"])), "matrix")}

    def prepare(self, dtype, device) -> None:
        self.linear = Linear(self.tensors["weight"], "lm_head")
        self.linear.prepare(dtype)

    takes_lazy_input = True

    def forward(self, ctx, normed, rows: int) -> torch.Tensor:
        return self.linear.forward(ctx, normed, rows, torch.float32, "logits").tensor


@register_embedding("table_positions")
class ScaledPositionEmbedding(Part):
    """x = E[id] * scale + P[position] (P a learned table, not scaled), in float32, written into
    every one of `streams` copies of the residual: the result is [tokens, streams * hidden].

    params: `vocab`, `hidden`, `scale`, `positions` (rows of the position table, or None for no
    position term), `streams`.  tensors: `weight` [vocab, hidden], `positions` [positions, hidden]."""

    def local_weights(self):
        p = self.params
        out = {"weight": ((int(p["vocab"]), int(p["hidden"])), "matrix")}
        if p.get("positions"):
            out["positions"] = ((int(p["positions"]), int(p["hidden"])), "matrix")
        return out

    def forward(self, ctx) -> torch.Tensor:
        from ..kernels import streams as SK
        p = self.params
        width, streams = int(p["hidden"]), int(p.get("streams") or 1)
        x = ctx.ws.get("streams", (ctx.n_tokens, streams * width), torch.float32)
        SK.embed_positions(self.tensors["weight"], self.tensors.get("positions"), ctx.token_ids, ctx.positions, x,
                           ctx.n_tokens, width, streams, float(p.get("scale", 1.0)), ctx.stream)
        return x


@register_embedding("table_norm")
class NormedEmbedding(Part):
    """x = rms_norm(E[id]) * w, in float32; with `one_plus` the weight is stored around zero and the
    factor is 1 + w, formed once in float32.

    params: `vocab`, `hidden`, `eps`, `one_plus` (optional).  tensors: `weight` [vocab, hidden], `norm` [hidden]."""

    def local_weights(self):
        p = self.params
        return {"weight": ((int(p["vocab"]), int(p["hidden"])), "matrix"),
                "norm": ((int(p["hidden"]),), "zero" if p.get("one_plus") else "norm")}

    def prepare(self, dtype, device) -> None:
        if self.params.get("one_plus"):
            self.norm = (1.0 + self.tensors["norm"].to(torch.float32)).contiguous()
        else:
            self.norm = self.tensors["norm"].to(self.tensors["weight"].dtype).contiguous()

    def forward(self, ctx) -> torch.Tensor:
        from ..kernels import sandwich as SW
        x = ctx.ws.get("residual", (ctx.n_tokens, int(self.params["hidden"])), torch.float32)
        SW.embed_rmsnorm(self.tensors["weight"], ctx.token_ids, self.norm, x, ctx.n_tokens, float(self.params["eps"]),
                         ctx.stream)
        return x
