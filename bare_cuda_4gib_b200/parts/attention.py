"""Causal grouped-query attention over the paged cache.

q = h Wq^T, k = h Wk^T, v = h Wv^T (no bias); q and k rotated by position; k and v appended to
the request's cache pages; scores (q . k) / sqrt(head_dim) over the keys at positions
<= the query's (and, with `window`, newer than position - window); softmax; weighted values;
output projection (cuongvng/bare-cuda-4gib engine/src/model.cpp:540-572,
engine/kernels/attention_qk.cu:49-68, softmax.cu:28-42, attention_av.cu:24-44).
The three projections are one matrix product against [Wq; Wk; Wv], fused at load.

params: `hidden`, `heads`, `kv_heads`, `head_dim`, `window` (None = every key), `position`
(a `PartSpec` of the position family).  tensors: `q`, `k`, `v`, `o`.
"""

from __future__ import annotations

import math

import torch

from ..errors import ConfigError
from ..kernels import lib as K
from .base import KVCacheRequest, Part
from .linear import Linear
from .registry import build_part, register_mixer
from ..weights.loader import fused_rows


@register_mixer("attention")
class Attention(Part):
    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.kv_heads, self.head_dim = (
            int(p["hidden"]), int(p["heads"]), int(p["kv_heads"]), int(p["head_dim"]))
        self.window = p.get("window")
        if self.heads % self.kv_heads:
            raise ConfigError(f"attention: {self.heads} heads cannot share {self.kv_heads} key/value heads")
        self.position = build_part("position", p["position"])
        self.scale = 1.0 / math.sqrt(self.head_dim)

    def children(self):
        return [self.position]

    def local_weights(self):
        qd, kvd = self.heads * self.head_dim, self.kv_heads * self.head_dim
        return {"q": ((qd, self.hidden), "matrix"), "k": ((kvd, self.hidden), "matrix"),
                "v": ((kvd, self.hidden), "matrix"), "o": ((self.hidden, qd), "matrix")}

    def adjacent_weights(self):
        return [("q", "k", "v")]

    def cache_request(self):
        return KVCacheRequest(self.kv_heads, self.head_dim, self.window)

    def state_request(self):
        return None

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.qkv = Linear(fused_rows([t.pop("q"), t.pop("k"), t.pop("v")]), "qkv")
        self.o = Linear(t.pop("o"), "o")
        self.qkv.prepare(dtype)
        self.o.prepare(dtype)
        self.position.prepare(dtype, device)
        if dtype == torch.bfloat16 and device.type == "cuda":
            from ..kernels import attention as fast
            self.fast = fast.plan_for(self.head_dim, self.heads, self.kv_heads)
        else:
            self.fast = None

    def plan_step(self, ctx) -> None:
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.step_tiles(ctx, self.fast)

    takes_lazy_input = True

    def forward(self, ctx, call, h):
        n = ctx.n_tokens
        qd = self.heads * self.head_dim
        # few rows: float32 partial results let the product split its inner dimension over more SMs
        qkv_dtype = torch.float32 if n <= 256 else ctx.dtype
        q = ctx.ws.get("q", (n, qd), ctx.dtype)
        inv_freq = self.position.fused_rotation()
        apply = getattr(self.position, "apply", None)
        if apply is not None:
            # a position encoding with kernels of its own: it changes q and k in place, as [tokens, heads,
            # head_dim] views of the finished projection, before k and v go into the cache
            qkv = self.qkv.forward(ctx, h, n, ctx.dtype, "qkv")
            kvd = self.kv_heads * self.head_dim
            apply(ctx, qkv.tensor[:, :qd].unflatten(1, (self.heads, self.head_dim)),
                  qkv.tensor[:, qd: qd + kvd].unflatten(1, (self.kv_heads, self.head_dim)))
        else:
            rotate = K.RotateAndCache(q, call.cache, ctx.positions, ctx.row_seq, inv_freq, self.heads, call.writes_cache)
            qkv = self.qkv.forward(ctx, h, n, qkv_dtype, "qkv", allow_partials=True, epilogue=rotate)
        if qkv is not None:
            K.rope_cache_write(qkv, q, call.cache, ctx.positions, ctx.row_seq, inv_freq, self.heads,
                               call.writes_cache, n, ctx.stream)
        out = ctx.ws.get("attn_out", (n, qd), ctx.dtype)
        window = int(self.window) if self.window else 0
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.run(ctx, self.fast, q, out, call.cache, self.scale, window)
        else:
            K.attention_plain(q, out, call.cache, ctx.positions, ctx.row_seq, self.heads, n,
                              self.scale, window, ctx.stream)
        residual = getattr(ctx, "residual", None)
        return self.o.forward(ctx, out, n, torch.float32, "attn_proj", allow_partials=True,
                              epilogue=K.AddTo(residual, getattr(ctx, "following_norm", None)) if residual is not None else None)


@register_mixer("gated_attention")
class GatedAttention(Part):
    """Grouped-query softmax attention whose queries and keys are RMS-normed per head (one weight
    per projection, shared by its heads) before the position encoding turns them, whose scores are
    (q . k) * `scale`, and whose concatenated heads are multiplied by sigmoid(Wg h) before the output
    projection.  With `values` = "keys" there is no value projection: a token's value is its key as
    projected, before norm and rotation.  `window` (None = every key) keeps the last positions.

    One product makes [q | k (| v) | g]; one kernel norms, turns and caches; then the engine's paged
    attention kernels run as they do for "attention".

    params: `hidden`, `heads`, `kv_heads`, `head_dim`, `window`, `scale`, `eps`, `values`
    ("keys" | "projection"), `position` (a `PartSpec`; "rotary_pairs" or "none").
    tensors: `q`, `k`, (`v`,) `g`, `o`, `q_norm` [head_dim], `k_norm` [head_dim]."""

    takes_lazy_input = False

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.kv_heads, self.head_dim = (
            int(p["hidden"]), int(p["heads"]), int(p["kv_heads"]), int(p["head_dim"]))
        self.window = p.get("window")
        self.own_values = p.get("values", "projection") != "keys"
        if self.heads % self.kv_heads:
            raise ConfigError(f"gated_attention: {self.heads} heads cannot share {self.kv_heads} key/value heads")
        self.position = build_part("position", p["position"])
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.head_dim))
        self.eps = float(p["eps"])

    def children(self):
        return [self.position]

    def _projections(self):
        return ("q", "k", "v", "g") if self.own_values else ("q", "k", "g")

    def local_weights(self):
        qd, kvd = self.heads * self.head_dim, self.kv_heads * self.head_dim
        out = {"q": ((qd, self.hidden), "matrix"), "k": ((kvd, self.hidden), "matrix"),
               "g": ((qd, self.hidden), "matrix"), "o": ((self.hidden, qd), "matrix"),
               "q_norm": ((self.head_dim,), "norm"), "k_norm": ((self.head_dim,), "norm")}
        if self.own_values:
            out["v"] = ((kvd, self.hidden), "matrix")
        return out

    def adjacent_weights(self):
        return [self._projections()]

    def cache_request(self):
        return KVCacheRequest(self.kv_heads, self.head_dim, self.window)

    def state_request(self):
        return None

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.proj = Linear(fused_rows([t[n] for n in self._projections()]), "gated_attention.in")
        self.o = Linear(t["o"], "gated_attention.o")
        self.proj.prepare(dtype)
        self.o.prepare(dtype)
        self.q_norm, self.k_norm = t["q_norm"].to(dtype).contiguous(), t["k_norm"].to(dtype).contiguous()
        self.position.prepare(dtype, device)
        self.inv_freq = getattr(self.position, "inv_freq", None)
        self.rot_dims = int(getattr(self.position, "dims", 0)) if self.inv_freq is not None else 0
        if self.rot_dims > self.head_dim:
            raise ConfigError(f"gated_attention: {self.rot_dims} rotated entries in a head of {self.head_dim}")
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.fast = None
        if dtype == torch.bfloat16 and device.type == "cuda":
            from ..kernels import attention as fast
            self.fast = fast.plan_for(self.head_dim, self.heads, self.kv_heads)

    def plan_step(self, ctx) -> None:
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.step_tiles(ctx, self.fast)

    def forward(self, ctx, call, h):
        from ..kernels import head_prepare as HP
        n = ctx.n_tokens
        qd, kvd = self.heads * self.head_dim, self.kv_heads * self.head_dim
        u = self.proj.forward(ctx, h, n, ctx.dtype, "mixer_in").tensor
        q = ctx.ws.get("q", (n, qd), ctx.dtype)
        HP.headnorm_rope_cache(ctx, u, 0, qd, qd + kvd if self.own_values else -1, self.q_norm, self.k_norm, self.eps,
                               self.inv_freq, self.rot_dims, self.magnitude, q, call.cache, self.heads, call.writes_cache)
        out = ctx.ws.get("attn_out", (n, qd), ctx.dtype)
        window = int(self.window) if self.window else 0
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.run(ctx, self.fast, q, out, call.cache, self.scale, window)
        else:
            K.attention_plain(q, out, call.cache, ctx.positions, ctx.row_seq, self.heads, n, self.scale, window, ctx.stream)
        HP.sigmoid_gate(ctx, out, u[:, u.shape[1] - qd:], n)
        return self.o.forward(ctx, out, n, torch.float32, "attn_proj", allow_partials=True)


@register_mixer("general_attention")
class GeneralAttention(Part):
    """Grouped-query causal softmax attention with the options several designs combine: biases on the
    q, k and v projections; an RMS norm per head on q and k (one weight per projection, used as stored)
    before the rotation; any position part that the norm-and-cache kernel turns (`rotary_halves`,
    `rotary_pairs`, `none`); a `scale` of its own; a cap on the scaled scores, cap * tanh(score / cap);
    value heads of their own size; a `window`; and value mixing: with `v_mix` = "source" the values this
    layer caches are also left for later layers of the step, with "mix" the cached value is (1 - l) v +
    l v_source of the same token, l the scalar tensor `v_lambda`.

    One product makes [q | k | v]; one kernel adds the biases, norms, turns, mixes and caches; then the
    engine's tensor-core attention kernels run in bfloat16 steps (all three for equal key and value sizes
    without a cap, the mma.sync kernel built for the value size and the cap otherwise), the plain kernel in
    float32 steps and for sizes that are no multiples of 16 up to 128.

    params: `hidden`, `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `eps`, `bias` (bool), `qk_norm` (bool),
    `softcap` (None: no cap), `window` (None: every key), `v_mix` (None | "source" | "mix"), `position`.
    tensors: `q`, `k`, `v`, `o`, (`q_bias`, `k_bias`, `v_bias`,) (`q_norm`, `k_norm` [dim],) (`v_lambda` [])."""

    takes_lazy_input = False

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p.get("vdim") or p["dim"])
        if self.heads % self.kv_heads:
            raise ConfigError(f"general_attention: {self.heads} heads cannot share {self.kv_heads} key/value heads")
        if self.vdim > 256:
            raise ConfigError(f"general_attention: value head size {self.vdim} exceeds the 256 the kernels take")
        self.window = p.get("window")
        self.has_bias, self.qk_norm = bool(p.get("bias")), bool(p.get("qk_norm"))
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.v_mix = p.get("v_mix")
        if self.v_mix not in (None, "source", "mix"):
            raise ConfigError(f"general_attention: v_mix must be None, 'source' or 'mix', got {self.v_mix!r}")
        self.position = build_part("position", p["position"])
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.dim))
        self.eps = float(p.get("eps", 1e-6))
        self.qd, self.kd, self.vd = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim

    def children(self):
        return [self.position]

    def local_weights(self):
        out = {"q": ((self.qd, self.hidden), "matrix"), "k": ((self.kd, self.hidden), "matrix"),
               "v": ((self.vd, self.hidden), "matrix"), "o": ((self.hidden, self.heads * self.vdim), "matrix")}
        if self.has_bias:
            out.update({"q_bias": ((self.qd,), "zero"), "k_bias": ((self.kd,), "zero"), "v_bias": ((self.vd,), "zero")})
        if self.qk_norm:
            out.update({"q_norm": ((self.dim,), "norm"), "k_norm": ((self.dim,), "norm")})
        if self.v_mix is not None:
            out["v_lambda"] = ((), "zero")      # the source layer has the tensor too and does not use it
        return out

    def adjacent_weights(self):
        return [("q", "k", "v")]

    def cache_request(self):
        return KVCacheRequest(self.kv_heads, self.dim, self.window, None if self.vdim == self.dim else self.vdim)

    def state_request(self):
        return None

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.proj = Linear(fused_rows([t["q"], t["k"], t["v"]]), "general_attention.in")
        self.o = Linear(t["o"], "general_attention.o")
        self.proj.prepare(dtype)
        self.o.prepare(dtype)
        self.bias = (torch.cat([t[n].to(torch.float32).reshape(-1) for n in ("q_bias", "k_bias", "v_bias")]).contiguous()
                     if self.has_bias else None)
        self.q_norm = t["q_norm"].to(dtype).contiguous() if self.qk_norm else None
        self.k_norm = t["k_norm"].to(dtype).contiguous() if self.qk_norm else None
        self.v_lambda = float(t["v_lambda"].to(torch.float32).reshape(-1)[0].item()) if self.v_mix == "mix" else 0.0
        self.position.prepare(dtype, device)
        self.inv_freq = getattr(self.position, "inv_freq", None)
        self.rot_dims = int(getattr(self.position, "dims", 0)) if self.inv_freq is not None else 0
        if self.rot_dims > self.dim:
            raise ConfigError(f"general_attention: {self.rot_dims} rotated entries in a head of {self.dim}")
        self.halves = bool(getattr(self.position, "halves", False))
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.fast = None
        if dtype == torch.bfloat16 and device.type == "cuda":
            # equal head sizes without a cap: the engine's tcgen05 prefill, cluster decode and mma.sync kernels;
            # otherwise the mma.sync kernel built for this value size and with the cap (sizes it takes)
            from ..kernels import attention as fast
            self.fast = fast.plan_for(self.dim, self.heads, self.kv_heads, False, self.vdim, self.softcap)

    def plan_step(self, ctx) -> None:
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.step_tiles(ctx, self.fast)

    def forward(self, ctx, call, h):
        from ..kernels import biased_attention as BA, head_prepare as HP
        n = ctx.n_tokens
        u = self.proj.forward(ctx, h, n, ctx.dtype, "mixer_in").tensor
        q = ctx.ws.get("q", (n, self.qd), ctx.dtype)
        shared = ctx.ws.get("mixed_values", (n, self.vd), torch.float32) if self.v_mix else None
        HP.headnorm_rope_cache(ctx, u, 0, self.qd, self.qd + self.kd, self.q_norm, self.k_norm, self.eps, self.inv_freq,
                               self.rot_dims, self.magnitude, q, call.cache, self.heads, call.writes_cache,
                               halves=self.halves, bias=self.bias, v_mix_in=shared if self.v_mix == "mix" else None,
                               v_mix=self.v_lambda, v_mix_out=shared if self.v_mix == "source" else None)
        out = ctx.ws.get("attn_out", (n, self.heads * self.vdim), ctx.dtype)
        window = int(self.window) if self.window else 0
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.run(ctx, self.fast, q, out, call.cache, self.scale, window)
        else:
            BA.attention(ctx, q, out, call.cache, None, self.heads, self.scale, window, 1.0, self.softcap)
        return self.o.forward(ctx, out, n, torch.float32, "attn_proj", allow_partials=True)
