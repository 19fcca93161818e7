"""Launchers of `csrc/mamba2.cu`: the float32 operands of the state scan from a Mamba-2 input
projection (short convolution, silu, step sizes, decays), and the D term, gate and grouped norm after it."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build
from .lib import _check, _dev, dtype_code

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("mamba2.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_mamba2_operands.argtypes = [P, I, L, P, P, I, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P]
        l.llm_mamba2_finish.argtypes = [P, P, P, P, I, L, P, P, L, I, I, I, I, F, P]
        l.llm_mamba2_ring_write.argtypes = [P, I, L, P, I, I, P, P, P, P, I, P]
        l.llm_mamba2_step.argtypes = [P, I, L, P, P, I, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P]
        l.llm_mamba2_step_shared_bytes.argtypes = [I, I, I, I]
        l.llm_mamba2_step_shared_bytes.restype = c_longlong
        for name in ("llm_mamba2_operands", "llm_mamba2_finish", "llm_mamba2_ring_write", "llm_mamba2_step"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


def operands(ctx, u: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor, ring: torch.Tensor, dt_bias: torch.Tensor,
             a_log: torch.Tensor, qf, kf, vf, xc, decay, heads: int, vdim: int, state: int, groups: int) -> None:
    """u [rows, z | x | B | C | dt]: the convolution (history before the step from `ring`) and silu on
    [x | B | C]; qf, kf [rows, heads * state] = C, B of the head's group; vf [rows, heads * vdim] = dt * x;
    xc = x; decay [rows, heads] = exp(-exp(a_log) * dt) with dt = softplus(dt + dt_bias).  All float32."""
    _dev(u, conv_w, conv_b, ring, dt_bias, a_log, qf, kf, vf, xc, decay)
    for t in (conv_w, conv_b, ring, dt_bias, a_log, qf, kf, vf, xc, decay):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("mamba2 operands: constants, ring and operands must be contiguous float32")
    _check(lib().llm_mamba2_operands(
        u.data_ptr(), dtype_code(u.dtype), u.stride(0), conv_w.data_ptr(), conv_b.data_ptr(), conv_w.shape[1],
        ring.data_ptr(), dt_bias.data_ptr(), a_log.data_ptr(), qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), xc.data_ptr(),
        decay.data_ptr(), ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), ctx.seq_slot.data_ptr(),
        ctx.seq_q_start.data_ptr(), ctx.n_tokens, heads, vdim, state, groups, ctx.stream), "mamba2_operands")


def finish(ctx, scanned: torch.Tensor, xc: torch.Tensor, d_skip: torch.Tensor, z: torch.Tensor, norm_w: torch.Tensor,
           out: torch.Tensor, vdim: int, parts: int, eps: float) -> None:
    """out = rms_norm in `parts` equal parts of ((scanned + D x) * silu(z)) * norm_w; z may be a column view."""
    _dev(scanned, xc, d_skip, z, norm_w, out)
    if z.dtype != out.dtype or d_skip.dtype != torch.float32 or norm_w.dtype != torch.float32:
        raise TypeError("mamba2 finish: element types not as the kernel needs")
    _check(lib().llm_mamba2_finish(scanned.data_ptr(), xc.data_ptr(), d_skip.data_ptr(), z.data_ptr(), dtype_code(z.dtype),
                                   z.stride(0), norm_w.data_ptr(), out.data_ptr(), out.stride(0), ctx.n_tokens,
                                   scanned.shape[-1], vdim, parts, float(eps), ctx.stream), "mamba2_finish")


def ring_write(ctx, u: torch.Tensor, ring: torch.Tensor, taps: int, channels: int) -> None:
    """The rows [x | B | C] (u may be a column view) of each request's last taps - 1 positions into its ring
    [slots, taps, channels], entry position % taps."""
    _dev(u, ring)
    _check(lib().llm_mamba2_ring_write(u.data_ptr(), dtype_code(u.dtype), u.stride(0), ring.data_ptr(), taps, channels,
                                       ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), ctx.seq_slot.data_ptr(),
                                       ctx.seq_kv_len.data_ptr(), ctx.n_tokens, ctx.stream), "mamba2_ring_write")


STEP_MAX_SHARED = 160 * 1024


def step_takes(heads: int, vdim: int, state: int, groups: int) -> bool:
    """Whether the form for steps of one token per request takes these sizes (a head's channels fit in shared memory)."""
    if heads % groups:
        return False
    need = int(lib().llm_mamba2_step_shared_bytes(heads, vdim, state, groups))
    return 0 < need <= STEP_MAX_SHARED


def step(ctx, u: torch.Tensor, conv_w, conv_b, ring, dt_bias, a_log, state, scanned: torch.Tensor, xc: torch.Tensor,
         heads: int, vdim: int, state_size: int, groups: int, write_ring: bool) -> None:
    """A step of one token per request, a block per (request, head): convolution (and the ring's update), step
    size and decay, the state updated in place; scanned [rows, heads * vdim] = S^T C and xc = x, both float32,
    for `finish`."""
    _dev(u, conv_w, conv_b, ring, dt_bias, a_log, state, scanned, xc)
    if state.dtype != torch.float32 or ring.dtype != torch.float32 or scanned.dtype != torch.float32 or xc.dtype != torch.float32:
        raise TypeError("mamba2 step: states and results must be float32")
    _check(lib().llm_mamba2_step(
        u.data_ptr(), dtype_code(u.dtype), u.stride(0), conv_w.data_ptr(), conv_b.data_ptr(), conv_w.shape[1],
        ring.data_ptr(), dt_bias.data_ptr(), a_log.data_ptr(), state.data_ptr(), scanned.data_ptr(), xc.data_ptr(),
        ctx.positions.data_ptr(), ctx.seq_slot.data_ptr(), ctx.seq_q_start.data_ptr(), ctx.n_seqs, heads, vdim, state_size,
        groups, 1 if write_ring else 0, ctx.stream), "mamba2_step")
