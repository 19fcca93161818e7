"""Attention whose keys and values are expanded from one cached latent vector per token.

    [c' | r'] = Wdkv h;  c = rms_norm(c') * w (the latent, `kv_rank` entries);  r = rotate(r') (`rot_dim`
    entries, one key part shared by all heads);  per head  k = [Uk c | r],  v = Uv c,
    q = [q_plain | rotate(q_rot)] from Wq h;  score = (q . k) * scale;  causal softmax, with `sink`
    also exp(sink_h) in the denominator;  heads concatenated, times sigmoid(Wg h), then Wo.

Options: with `q_rank` the queries go through a latent of their own, q = Wuq (rms_norm(Wdq h) * wq);
`gate` False leaves the sigmoid gate out; with `borrows` the run reads the [c | r] that an earlier run cached
(`LayerCall.cache_from`), has no Wdkv and writes nothing; `window` keeps the last positions, and
`cache_window` says how long the cache must keep a position where runs with wider windows read it too.

Only [c | r] is cached, as one key/value head of size kv_rank + rot_dim without values of its own.
The kernels never expand a cached token: Uk is applied to the queries (q_plain^T Uk, `kv_rank`
entries per head) and Uv to the weighted sum of latents, so every head reads the same cached
vectors (see csrc/latent_attention.cu).

params: `hidden`, `heads`, `dim`, `rot_dim`, `vdim`, `kv_rank`, `scale`, `eps`, `sink` (bool), `window`
(None = every key), `position` (a `PartSpec` for the rotated parts: "rotary_pairs", "rotary_halves" or "none"),
and optionally `q_rank`, `gate` (default True), `borrows`, `cache_window`.
tensors: `q` [heads * (dim + rot_dim), hidden] (or `dq` [q_rank, hidden], `dq_norm` [q_rank], `uq` [heads * (dim +
rot_dim), q_rank]), `dkv` [kv_rank + rot_dim, hidden], `dkv_norm` [kv_rank] (not with `borrows`), `uk` [heads * dim,
kv_rank], `uv` [heads * vdim, kv_rank], `sink` [heads], `g` [heads * vdim, hidden], `o` [hidden, heads * vdim].
"""

from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import latent as LT
from .base import KVCacheRequest, Part
from .linear import Linear
from .registry import build_part, register_mixer
from ..weights.loader import fused_rows


@register_mixer("latent_attention")
class LatentAttention(Part):
    takes_lazy_input = False

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.dim, self.rot, self.vdim, self.rank = (
            int(p["hidden"]), int(p["heads"]), int(p["dim"]), int(p["rot_dim"]), int(p["vdim"]), int(p["kv_rank"]))
        if self.rank > LT.MAX_RANK:
            raise ConfigError(f"latent_attention: a latent of {self.rank} entries exceeds the {LT.MAX_RANK} the kernel takes")
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.has_sink = bool(p.get("sink"))
        self.window = p.get("window")
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else 0
        self.has_gate = bool(p.get("gate", True))
        self.borrows = bool(p.get("borrows"))
        self.cache_window = p["cache_window"] if "cache_window" in p else self.window
        self.position = build_part("position", p["position"])

    def children(self):
        return [self.position]

    def local_weights(self):
        H, d, r, e, k, w = self.heads, self.dim, self.rot, self.vdim, self.rank, self.hidden
        out = {"uk": ((H * d, k), "matrix"), "uv": ((H * e, k), "matrix"), "o": ((w, H * e), "matrix")}
        if self.q_rank:
            out.update({"dq": ((self.q_rank, w), "matrix"), "dq_norm": ((self.q_rank,), "norm"),
                        "uq": ((H * (d + r), self.q_rank), "matrix")})
        else:
            out["q"] = ((H * (d + r), w), "matrix")
        if not self.borrows:
            out.update({"dkv": ((k + r, w), "matrix"), "dkv_norm": ((k,), "norm")})
        if self.has_gate:
            out["g"] = ((H * e, w), "matrix")
        if self.has_sink:
            out["sink"] = ((H,), "unit")
        return out

    def _inputs(self):
        """The tensors that multiply the mixer's input, in the order of the joint product's columns."""
        return ["dq" if self.q_rank else "q"] + ([] if self.borrows else ["dkv"]) + (["g"] if self.has_gate else [])

    def adjacent_weights(self):
        return [tuple(self._inputs())]

    def cache_request(self):
        return KVCacheRequest(1, self.rank + self.rot, self.cache_window, v_head_dim=0)

    def state_request(self):
        return None

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.proj = Linear(fused_rows([t[n] for n in self._inputs()]), "latent_attention.in")
        self.o = Linear(t["o"], "latent_attention.o")
        self.proj.prepare(dtype)
        self.o.prepare(dtype)
        self.uq = None
        if self.q_rank:
            self.uq = Linear(t["uq"], "latent_attention.uq")
            self.uq.prepare(dtype)
            self.q_norm_w = t["dq_norm"].to(dtype).contiguous()
        self.uk, self.uv = t["uk"].to(dtype).contiguous(), t["uv"].to(dtype).contiguous()
        self.norm_w = None if self.borrows else t["dkv_norm"].to(dtype).contiguous()
        self.sink = t["sink"].to(dtype).contiguous() if self.has_sink else None
        self.position.prepare(dtype, device)
        self.inv_freq = getattr(self.position, "inv_freq", None)
        self.rot_dims = int(getattr(self.position, "dims", 0)) if self.inv_freq is not None else 0
        if self.rot_dims > self.rot:
            raise ConfigError(f"latent_attention: {self.rot_dims} rotated entries in a part of {self.rot}")
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.halves = bool(getattr(self.position, "halves", False))

    def forward(self, ctx, call, h):
        n, H, D = ctx.n_tokens, self.heads, self.rank + self.rot
        q_cols = H * (self.dim + self.rot)
        first = self.q_rank if self.q_rank else q_cols
        u = self.proj.forward(ctx, h, n, ctx.dtype, "mixer_in").tensor
        if self.q_rank:
            cq = ctx.ws.get("latent_cq", (n, self.q_rank), ctx.dtype)
            LT.rows_rmsnorm(ctx, u[:, :first], self.q_norm_w, cq, n, self.eps)
            q = self.uq.forward(ctx, cq, n, ctx.dtype, "latent_q_in").tensor
        else:
            q = u
        c_rows = None if self.borrows else u[:, first: first + D]
        q_full = ctx.ws.get("latent_q", (n, H * D), ctx.dtype)
        LT.prepare(ctx, q, 0, c_rows, H, self.dim, self.rot, self.rank, self.norm_w, self.eps, self.inv_freq,
                   self.rot_dims, self.magnitude, q_full, call.cache, call.writes_cache and not self.borrows, self.halves)
        LT.per_head_linear(ctx, q[:, :q_cols].unflatten(1, (H, self.dim + self.rot)), self.uk, True,
                           q_full.unflatten(1, (H, D)), H, self.dim, self.rank, n)
        mixed = ctx.ws.get("latent_o", (n, H * self.rank), ctx.dtype)
        LT.attention(ctx, q_full, mixed, call.cache, self.rank, self.sink, H, self.scale,
                     int(self.window) if self.window else 0)
        out = ctx.ws.get("attn_out", (n, H * self.vdim), ctx.dtype)
        LT.per_head_linear(ctx, mixed.unflatten(1, (H, self.rank)), self.uv, False, out.unflatten(1, (H, self.vdim)), H,
                           self.rank, self.vdim, n, gate=u[:, u.shape[1] - H * self.vdim:] if self.has_gate else None)
        return self.o.forward(ctx, out, n, torch.float32, "attn_proj", allow_partials=True)
