"""Mamba-2 (state-space duality) as a mixer over state slots.

One input projection gives [z | x | B | C | dt] (z, x: heads * vdim; B, C: groups * state; dt: heads).
[x | B | C] pass a short causal convolution per channel (with bias) and silu; per head h of group
g = h / (heads / groups), with dt = softplus(dt + dt_bias) and a = exp(-exp(A_log) * dt):

    S_t = a S_(t-1) + dt B_t x_t^T  (state x vdim),    y_t = S_t^T C_t + D x_t

then y * silu(z), an RMS norm in `norm_groups` equal parts (each by its own root mean square), a
weight, and the output projection.  A request keeps S as a float32 state [heads, state, vdim] and the
convolution's last inputs as a second one (a ring of `taps` entries by position); the walk over a
step's tokens is the engine's state scan (`kernels.linear_attention.scan`) with one decay per token and
head, fed with float32 operands; the kernels of csrc/mamba2.cu come before and after it.  In a step of one
token per request one kernel with a block per (request, head) stands for operands, ring and scan.  In
bfloat16 steps with a portion of 32 tokens or more (state and value sizes that are multiples of 16) the
recurrence runs in chunks of 64 tokens on the tensor cores (csrc/mamba2_chunked.cu) instead of the scan.

params: `hidden`, `heads`, `vdim`, `state`, `groups`, `taps`, `norm_groups`, `eps`.
tensors: `in` [2 * heads * vdim + 2 * groups * state + heads, hidden], `conv` [channels, taps], `conv_bias`
[channels], `dt_bias`, `A_log`, `D` [heads], `norm` [heads * vdim], `o` [hidden, heads * vdim].
"""

from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import linear_attention as LA, mamba2 as MK
from .base import Part, StateRequest
from .linear import Linear
from .registry import register_mixer


@register_mixer("mamba2")
class Mamba2(Part):
    takes_lazy_input = False

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.vdim, self.state = int(p["hidden"]), int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.groups, self.taps, self.norm_groups = int(p["groups"]), int(p["taps"]), int(p["norm_groups"])
        self.eps = float(p["eps"])
        self.inner = self.heads * self.vdim
        self.conv_channels = self.inner + 2 * self.groups * self.state
        if self.heads % self.groups:
            raise ConfigError(f"mamba2: {self.heads} heads cannot share {self.groups} groups of B and C")
        if self.inner % self.norm_groups:
            raise ConfigError(f"mamba2: {self.inner} channels do not split into {self.norm_groups} equal parts for the norm")
        if self.state > LA.MAX_KEY_DIM:
            raise ConfigError(f"mamba2: state size {self.state} exceeds the {LA.MAX_KEY_DIM} the scan kernel takes")
        if self.taps < 1:
            raise ConfigError("mamba2: the convolution needs at least one tap")

    def local_weights(self):
        H, C = self.heads, self.conv_channels
        return {"in": ((self.inner + C + H, self.hidden), "matrix"), "conv": ((C, self.taps), "unit"),
                "conv_bias": ((C,), "zero"), "dt_bias": ((H,), "unit"), "A_log": ((H,), "zero"), "D": ((H,), "norm"),
                "norm": ((self.inner,), "norm"), "o": ((self.hidden, self.inner), "matrix")}

    def cache_request(self):
        return None

    def state_request(self):
        return StateRequest((self.heads, self.state, self.vdim), torch.float32)

    def cache_demands(self):
        """Two states per request: S, and the ring of the convolution's last inputs."""
        return [(None, self.state_request()),
                (None, StateRequest((self.taps, self.conv_channels), torch.float32))]

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.proj = Linear(t["in"], "mamba2.in")
        self.o = Linear(t["o"], "mamba2.o")
        self.proj.prepare(dtype)
        self.o.prepare(dtype)
        f = lambda x: x.to(torch.float32).contiguous()
        self.conv_w, self.conv_b = f(t["conv"]), f(t["conv_bias"])
        self.dt_bias, self.a_log, self.d_skip, self.norm_w = f(t["dt_bias"]), f(t["A_log"]), f(t["D"]), f(t["norm"])
        self.one_step = device.type == "cuda" and MK.step_takes(self.heads, self.vdim, self.state, self.groups)
        self.chunked = device.type == "cuda" and dtype == torch.bfloat16 and MK.chunked_takes(self.state, self.vdim)
        if self.chunked:
            self.chunk_columns = MK.chunked_columns(self.heads, self.vdim)
            MK.chunked_lib(self.state, self.vdim, self.chunk_columns)      # compiled with the model, not at its first long portion

    def forward(self, ctx, call, h):
        n, H, P, N = ctx.n_tokens, self.heads, self.vdim, self.state
        f32 = torch.float32
        u = self.proj.forward(ctx, h, n, ctx.dtype, "mixer_in").tensor
        state, ring = call.states[0], call.states[1]
        out = ctx.ws.get("mixer_act", (n, self.inner), ctx.dtype)
        xc = ctx.ws.get("mamba2_x", (n, self.inner), f32)
        scanned = ctx.ws.get("mamba2_scan", (n, self.inner), f32)
        if ctx.max_q_len == 1 and self.one_step:
            MK.step(ctx, u, self.conv_w, self.conv_b, ring, self.dt_bias, self.a_log, state, scanned, xc, H, P, N,
                    self.groups, call.writes_cache)
            MK.finish(ctx, scanned, xc, self.d_skip, u[:, : self.inner], self.norm_w, out, P, self.norm_groups, self.eps)
            return self.o.forward(ctx, out, n, torch.float32, "mixer_out", allow_partials=True)
        if ctx.dtype == torch.bfloat16 and self.chunked and ctx.max_q_len >= MK.CHUNKED_MIN_TOKENS and ctx.use_fast_attention:
            # long portions of a bfloat16 step: the recurrence in chunks on the tensor cores
            compact = ctx.ws.get("mamba2_compact", (n, self.conv_channels), torch.bfloat16)
            dt = ctx.ws.get("mamba2_dt", (n, H), f32)
            la = ctx.ws.get("mamba2_la", (n, H), f32)
            MK.operands(ctx, u, self.conv_w, self.conv_b, ring, self.dt_bias, self.a_log, None, None, None, xc, None, H, P, N,
                        self.groups, compact, dt, la)
            if call.writes_cache:
                MK.ring_write(ctx, u[:, self.inner: self.inner + self.conv_channels], ring, self.taps, self.conv_channels)
            MK.chunked(ctx, compact, dt, la, state, scanned, H, P, N, self.groups, self.chunk_columns)
            MK.finish(ctx, scanned, xc, self.d_skip, u[:, : self.inner], self.norm_w, out, P, self.norm_groups, self.eps)
            return self.o.forward(ctx, out, n, torch.float32, "mixer_out", allow_partials=True)
        qf = ctx.ws.get("mamba2_q", (n, H * N), f32)
        kf = ctx.ws.get("mamba2_k", (n, H * N), f32)
        vf = ctx.ws.get("mamba2_v", (n, self.inner), f32)
        decay = ctx.ws.get("mamba2_decay", (n, H), f32)
        MK.operands(ctx, u, self.conv_w, self.conv_b, ring, self.dt_bias, self.a_log, qf, kf, vf, xc, decay, H, P, N,
                    self.groups)
        if call.writes_cache:
            MK.ring_write(ctx, u[:, self.inner: self.inner + self.conv_channels], ring, self.taps, self.conv_channels)
        LA.scan(ctx, qf, kf, vf, decay, "token", state, scanned, H, N, P)
        MK.finish(ctx, scanned, xc, self.d_skip, u[:, : self.inner], self.norm_w, out, P, self.norm_groups, self.eps)
        return self.o.forward(ctx, out, n, torch.float32, "mixer_out", allow_partials=True)
