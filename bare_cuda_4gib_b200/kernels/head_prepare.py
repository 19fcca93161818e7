"""Launchers of `csrc/head_prepare.cu`: per-head norms of queries and keys, the pairwise rotation
by position and the cache write in one kernel, and the sigmoid gate on a mixer's output."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build
from .lib import CacheView, _check, _dev, _ptr, dtype_code

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("head_prepare.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_headnorm_rope_cache.argtypes = [P, I, L, I, I, I, P, P, F, P, I, I, I, F, P, P, P, P, L, I, I, I, I, I, P, P,
                                              I, I, I, P, P, F, P, P]
        l.llm_sigmoid_gate.argtypes = [P, P, I, L, I, I, P]
        for name in ("llm_headnorm_rope_cache", "llm_sigmoid_gate"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


def headnorm_rope_cache(ctx, u: torch.Tensor, q_col: int, k_col: int, v_col: int, q_norm_w: Optional[torch.Tensor],
                        k_norm_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rot_dims: int,
                        mag: float, q_out: torch.Tensor, cache: CacheView, q_heads: int, write_cache: bool,
                        halves: bool = False, maps: int = 1, bias: Optional[torch.Tensor] = None,
                        v_mix_in: Optional[torch.Tensor] = None, v_mix: float = 0.0,
                        v_mix_out: Optional[torch.Tensor] = None) -> None:
    """u [rows, columns]: queries at column `q_col`, keys at `k_col`, values at `v_col` (-1: the
    keys as projected are the values).  Heads are RMS-normed with the shared weights (None: not
    normed), their first `rot_dims` entries turned pair by pair (2i with 2i + 1, or with `halves` i with
    i + rot_dims / 2); q to `q_out`, k and v to the cache.  With `maps` > 1 a query or key head (the
    cache's head size) is that many units side by side, each normed and turned by itself.  `bias` (float32,
    one entry per column of u) is added to q, k and v first.  With `v_mix_in` (float32 [rows, kv_heads *
    v_dim]) the cached value is (1 - v_mix) v + v_mix * v_mix_in; with `v_mix_out` it is also left there."""
    _dev(u, q_norm_w, k_norm_w, inv_freq, q_out, bias, v_mix_in, v_mix_out)
    for t in (bias, v_mix_in, v_mix_out):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise TypeError("headnorm_rope_cache: the bias and the mixed values must be contiguous float32")
    _check(lib().llm_headnorm_rope_cache(
        u.data_ptr(), dtype_code(u.dtype), u.stride(0), q_col, k_col, v_col, _ptr(q_norm_w), _ptr(k_norm_w), float(eps),
        _ptr(inv_freq), int(rot_dims), 1 if halves else 0, int(maps), float(mag), q_out.data_ptr(), cache.k_ptr, cache.v_ptr,
        cache.block_table.data_ptr(), cache.page_stride, cache.table_stride, cache.page_tokens, cache.kv_heads,
        cache.head_dim, cache.v_dim, ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), q_heads, 1 if write_cache else 0,
        ctx.n_tokens, _ptr(bias), _ptr(v_mix_in), float(v_mix), _ptr(v_mix_out), ctx.stream), "headnorm_rope_cache")


def sigmoid_gate(ctx, x: torch.Tensor, gate: torch.Tensor, rows: int) -> None:
    """x[:rows] *= sigmoid(gate[:rows]) in place; gate may be a column view."""
    _dev(x, gate)
    _check(lib().llm_sigmoid_gate(x.data_ptr(), gate.data_ptr(), dtype_code(x.dtype), gate.stride(0), rows,
                                  x.shape[-1], ctx.stream), "sigmoid_gate")
