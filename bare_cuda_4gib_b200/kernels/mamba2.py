"""Launchers of `csrc/mamba2.cu`: the float32 operands of the state scan from a Mamba-2 input
projection (short convolution, silu, step sizes, decays), and the D term, gate and grouped norm after it."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build
from .lib import _check, _dev, _ptr, dtype_code

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("mamba2.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_mamba2_operands.argtypes = [P, I, L, P, P, I, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P, P, P, P]
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
             a_log: torch.Tensor, qf, kf, vf, xc, decay, heads: int, vdim: int, state: int, groups: int,
             compact: Optional[torch.Tensor] = None, dt_out: Optional[torch.Tensor] = None,
             la_out: Optional[torch.Tensor] = None) -> None:
    """u [rows, z | x | B | C | dt]: the convolution (history before the step from `ring`) and silu on
    [x | B | C]; qf, kf [rows, heads * state] = C, B of the head's group; vf [rows, heads * vdim] = dt * x;
    xc = x; decay [rows, heads] = exp(-exp(a_log) * dt) with dt = softplus(dt + dt_bias).  All float32.
    With `compact` (bfloat16 [rows, channels]) the operands are left out: [x | B | C] goes there once per token,
    the step sizes to `dt_out` and the decays' logarithms to `la_out` (float32 [rows, heads]), and x to xc."""
    _dev(u, conv_w, conv_b, ring, dt_bias, a_log, qf, kf, vf, xc, decay, compact, dt_out, la_out)
    if compact is not None and (compact.dtype != torch.bfloat16 or not compact.is_contiguous() or dt_out is None or la_out is None):
        raise TypeError("mamba2 operands: the compact form is contiguous bfloat16 with float32 step sizes beside it")
    for t in (conv_w, conv_b, ring, dt_bias, a_log, qf, kf, vf, xc, decay, dt_out, la_out):
        if t is None:
            continue
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("mamba2 operands: constants, ring and operands must be contiguous float32")
    _check(lib().llm_mamba2_operands(
        u.data_ptr(), dtype_code(u.dtype), u.stride(0), conv_w.data_ptr(), conv_b.data_ptr(), conv_w.shape[1],
        ring.data_ptr(), dt_bias.data_ptr(), a_log.data_ptr(), _ptr(qf), _ptr(kf), _ptr(vf), xc.data_ptr(),
        _ptr(decay), ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), ctx.seq_slot.data_ptr(),
        ctx.seq_q_start.data_ptr(), ctx.n_tokens, heads, vdim, state, groups, _ptr(compact), _ptr(dt_out), _ptr(la_out),
        ctx.stream), "mamba2_operands")


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


CHUNKED_MIN_TOKENS = 32      # portions at least this long take the chunked walk
_chunked_libs = {}


def chunked_takes(state: int, vdim: int) -> bool:
    """Sizes the chunked walk on the tensor cores is built for (a library per pair)."""
    return state % 16 == 0 and 16 <= state <= 256 and vdim % 16 == 0 and 16 <= vdim <= 1024


def chunked_columns(heads: int, vdim: int) -> int:
    """Value columns of a block: 32, or 16 where one request's blocks (heads x vdim / 32) would not reach the
    number of SMs, so that a single long prompt still puts a block on every SM."""
    from .lib import sm_count
    return 32 if vdim % 32 == 0 and heads * (vdim // 32) >= sm_count() else 16


def chunked_lib(state: int, vdim: int, columns: int = 0):
    columns = columns or (32 if vdim % 32 == 0 else 16)
    l = _chunked_libs.get((state, vdim, columns))
    if l is None:
        l = build.load_library("mamba2_chunked.cu", (f"-DSSD_N={state}", f"-DSSD_P={vdim}", f"-DSSD_PC={columns}"))
        P, I, L = c_void_p, c_int, c_longlong
        l.llm_mamba2_chunked.argtypes = [P, P, P, L, P, P, P, P, P, P, P, I, I, I, I, I, P]
        l.llm_mamba2_chunked.restype = c_int
        _chunked_libs[(state, vdim, columns)] = l
    return l


def chunked(ctx, compact: torch.Tensor, dt: torch.Tensor, la: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
            heads: int, vdim: int, state_size: int, groups: int, columns: int = 0) -> None:
    """The recurrence of every request's portion in chunks of 64 tokens on the tensor cores: compact
    [rows, x | B | C] bfloat16, dt and la (the decays' logarithms) float32 [rows, heads]; the states
    [slots, heads, state, vdim] float32 are read and left as after the portions' last tokens; out [rows, heads *
    vdim] float32 = S_t^T C_t."""
    _dev(compact, dt, la, state, out)
    inner = heads * vdim
    if compact.dtype != torch.bfloat16 or state.dtype != torch.float32 or out.dtype != torch.float32 or not out.is_contiguous():
        raise TypeError("mamba2 chunked: element types or layout not as the kernel needs")
    base, esize = compact.data_ptr(), 2
    _check(chunked_lib(state_size, vdim, columns).llm_mamba2_chunked(
        base, base + inner * esize, base + (inner + groups * state_size) * esize, compact.stride(0), dt.data_ptr(),
        la.data_ptr(), state.data_ptr(), out.data_ptr(), ctx.seq_slot.data_ptr(), ctx.seq_q_start.data_ptr(),
        ctx.seq_q_len.data_ptr(), ctx.n_seqs, heads, groups, state_size, vdim, ctx.stream), "mamba2_chunked")
