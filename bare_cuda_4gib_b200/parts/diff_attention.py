"""Differential attention: every head has two softmax maps over the same values, and the second is
subtracted from the first.

    q = Wq h [heads][2][dim],  k = Wk h [kv_heads][2][dim],  v = Wv h [kv_heads][v_dim]  (no biases);
    every map of every head: rms_norm over dim with one weight for all of q (one for all of k), then
    the position encoding;  a_m = softmax((q_m . k_m) * scale) V over the keys the query sees;
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init  (one number for the layer);
    o = a_1 - lambda a_2;  o <- o / sqrt(mean(o^2) + eps) * out_scale  per head;
    heads concatenated, times sigmoid(Wg h) (with `gate`), then Wo.

Which keys a query at position p sees: j <= p, and with `window` the last `window` positions, with
`chunk` the positions of p's own block of `chunk` positions (blocks are counted from position 0 of
the sequence, not from where a prompt was cut).  A cached key head holds both maps side by side, so
the cache is asked for `kv_heads` heads of 2 * dim with values of `v_dim`; pages that no later
query can see are given back (a block is never longer than `chunk`).

One product makes [q | k | v | g]; one kernel norms, turns and caches; one kernel runs both maps
and finishes the heads (difference, unit norm, gate).

params: `hidden`, `heads`, `kv_heads`, `dim`, `v_dim`, `window`, `chunk`, `scale`, `eps`, `lambda_init`,
`out_scale`, `gate` (bool), `position` (a `PartSpec`: "rotary_halves", "rotary_pairs" or "none").
tensors: `q` [heads * 2 * dim, hidden], `k` [kv_heads * 2 * dim, hidden], `v` [kv_heads * v_dim, hidden],
`g` [heads * v_dim, hidden], `o` [hidden, heads * v_dim], `q_norm` [dim], `k_norm` [dim], `lq1`, `lk1`, `lq2`, `lk2` [dim].
"""

from __future__ import annotations

import math

import torch

from ..errors import ConfigError
from .base import KVCacheRequest, Part
from .linear import Linear
from .registry import build_part, register_mixer
from ..weights.loader import fused_rows

MAPS = 2


@register_mixer("differential_attention")
class DifferentialAttention(Part):
    takes_lazy_input = False

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.kv_heads, self.dim, self.v_dim = (
            int(p["hidden"]), int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["v_dim"]))
        if self.heads % self.kv_heads:
            raise ConfigError(f"differential_attention: {self.heads} heads cannot share {self.kv_heads} key/value heads")
        from ..kernels.diff_attention import MAX_V_DIM
        if self.v_dim > MAX_V_DIM:
            raise ConfigError(f"differential_attention: values of {self.v_dim} entries exceed the {MAX_V_DIM} the kernel takes")
        self.window, self.chunk = p.get("window"), p.get("chunk")
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.dim))
        self.eps, self.lambda_init = float(p["eps"]), float(p["lambda_init"])
        self.out_scale = float(p.get("out_scale", 1.0))
        self.has_gate = bool(p.get("gate", True))
        self.position = build_part("position", p["position"])

    def children(self):
        return [self.position]

    def _projections(self):
        return ("q", "k", "v", "g") if self.has_gate else ("q", "k", "v")

    def local_weights(self):
        qd, kd = self.heads * MAPS * self.dim, self.kv_heads * MAPS * self.dim
        out = {"q": ((qd, self.hidden), "matrix"), "k": ((kd, self.hidden), "matrix"),
               "v": ((self.kv_heads * self.v_dim, self.hidden), "matrix"),
               "o": ((self.hidden, self.heads * self.v_dim), "matrix"),
               "q_norm": ((self.dim,), "norm"), "k_norm": ((self.dim,), "norm")}
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[name] = ((self.dim,), "matrix")
        if self.has_gate:
            out["g"] = ((self.heads * self.v_dim, self.hidden), "matrix")
        return out

    def adjacent_weights(self):
        return [self._projections()]

    def cache_request(self):
        # a query never looks back further than its window, nor further than one block of `chunk` positions
        spans = [int(s) for s in (self.window, self.chunk) if s]
        return KVCacheRequest(self.kv_heads, MAPS * self.dim, min(spans) if spans else None, v_head_dim=self.v_dim)

    def state_request(self):
        return None

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.proj = Linear(fused_rows([t[n] for n in self._projections()]), "differential_attention.in")
        self.o = Linear(t["o"], "differential_attention.o")
        self.proj.prepare(dtype)
        self.o.prepare(dtype)
        self.q_norm, self.k_norm = t["q_norm"].to(dtype).contiguous(), t["k_norm"].to(dtype).contiguous()
        f = {n: t[n].to(torch.float32) for n in ("lq1", "lk1", "lq2", "lk2")}
        # one number for the layer, formed once in float32
        self.lam = float(torch.exp((f["lq1"] * f["lk1"]).sum()) - torch.exp((f["lq2"] * f["lk2"]).sum())) + self.lambda_init
        self.position.prepare(dtype, device)
        self.inv_freq = getattr(self.position, "inv_freq", None)
        self.rot_dims = int(getattr(self.position, "dims", 0)) if self.inv_freq is not None else 0
        if self.rot_dims > self.dim:
            raise ConfigError(f"differential_attention: {self.rot_dims} rotated entries in a map of {self.dim}")
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.halves = bool(getattr(self.position, "halves", False))

    def forward(self, ctx, call, h):
        from ..kernels import diff_attention as DA
        from ..kernels import head_prepare as HP
        n = ctx.n_tokens
        qd, kd, vd = self.heads * MAPS * self.dim, self.kv_heads * MAPS * self.dim, self.kv_heads * self.v_dim
        u = self.proj.forward(ctx, h, n, ctx.dtype, "mixer_in").tensor
        q = ctx.ws.get("q", (n, qd), ctx.dtype)
        HP.headnorm_rope_cache(ctx, u, 0, qd, qd + kd, self.q_norm, self.k_norm, self.eps, self.inv_freq, self.rot_dims,
                               self.magnitude, q, call.cache, self.heads, call.writes_cache, self.halves, MAPS)
        out = ctx.ws.get("attn_out", (n, self.heads * self.v_dim), ctx.dtype)
        DA.attention(ctx, q, out, u[:, qd + kd + vd:] if self.has_gate else None, call.cache, self.heads, self.scale,
                     int(self.window) if self.window else 0, int(self.chunk) if self.chunk else 0, self.lam, self.eps,
                     self.out_scale)
        return self.o.forward(ctx, out, n, torch.float32, "attn_proj", allow_partials=True)
