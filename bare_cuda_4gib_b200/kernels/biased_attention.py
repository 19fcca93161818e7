"""Launchers of `csrc/biased_attention.cu`: the short convolution with whole-projection norms and
cache write, the ring of the convolution's last inputs, and softmax attention with a bias by
distance over the paged cache (key and value heads may differ in size)."""

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
        l = build.load_library("biased_attention.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_conv_norm_cache.argtypes = [P, I, L, P, I, P, P, P, P, P, P, P, L, I, I, I, I, I, P, P, P, P, I, I, F, F,
                                          I, I, P]
        l.llm_conv_ring_write.argtypes = [P, I, L, P, I, I, P, P, P, P, I, P]
        l.llm_biased_attention.argtypes = [P, P, I, L, P, P, P, L, I, I, I, I, I, P, I, P, P, I, I, F, I, F, F, P]
        for name in ("llm_conv_norm_cache", "llm_conv_ring_write", "llm_biased_attention"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


def conv_norm_cache(ctx, u: torch.Tensor, conv_w: torch.Tensor, ring: torch.Tensor, q_norm_w: torch.Tensor,
                    k_norm_w: torch.Tensor, q_out: torch.Tensor, cache: CacheView, q_heads: int, eps: float,
                    temp_coef: float, temp_every: int, write_cache: bool) -> None:
    """u [rows, q | k | v channels] (may be a column view) -> causal convolution over time with
    `conv_w` [channels, taps] (history before the step from `ring`), RMS norm of all q channels and
    of all k channels, the position factor on q; q to `q_out`, k and v into the cache."""
    _dev(u, conv_w, ring, q_norm_w, k_norm_w, q_out)
    _check(lib().llm_conv_norm_cache(
        u.data_ptr(), dtype_code(u.dtype), u.stride(0), conv_w.data_ptr(), conv_w.shape[1], ring.data_ptr(),
        q_norm_w.data_ptr(), k_norm_w.data_ptr(), q_out.data_ptr(), cache.k_ptr, cache.v_ptr,
        cache.block_table.data_ptr(), cache.page_stride, cache.table_stride, cache.page_tokens, cache.kv_heads,
        cache.head_dim, cache.v_dim, ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), ctx.seq_slot.data_ptr(),
        ctx.seq_q_start.data_ptr(), ctx.n_tokens, q_heads, float(eps), float(temp_coef), int(temp_every),
        1 if write_cache else 0, ctx.stream), "conv_norm_cache")


def conv_ring_write(ctx, u: torch.Tensor, ring: torch.Tensor, taps: int, channels: int) -> None:
    _dev(u, ring)
    _check(lib().llm_conv_ring_write(u.data_ptr(), dtype_code(u.dtype), u.stride(0), ring.data_ptr(), taps, channels,
                                     ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), ctx.seq_slot.data_ptr(),
                                     ctx.seq_kv_len.data_ptr(), ctx.n_tokens, ctx.stream), "conv_ring_write")


def attention(ctx, q: torch.Tensor, out: torch.Tensor, cache: CacheView, bias: Optional[torch.Tensor], q_heads: int,
              scale: float, window: int = 0, out_scale: float = 1.0, softcap: float = 0.0) -> None:
    """out[t, h] = out_scale * softmax_j((q[t, h] . k[j]) * scale + bias[h, distance]) v[j] over the
    keys at positions <= the query's (newer than position - window, if given).  `bias` is float32
    [heads, distances] or None; out may be a column view.  With `softcap` > 0 the scaled score (before the
    bias) becomes softcap * tanh(score / softcap)."""
    _dev(q, out, bias)
    _check(lib().llm_biased_attention(
        q.data_ptr(), out.data_ptr(), dtype_code(q.dtype), out.stride(0), cache.k_ptr, cache.v_ptr,
        cache.block_table.data_ptr(), cache.page_stride, cache.table_stride, cache.page_tokens, cache.kv_heads,
        cache.head_dim, cache.v_dim, _ptr(bias), bias.shape[1] if bias is not None else 0, ctx.positions.data_ptr(),
        ctx.row_seq.data_ptr(), q_heads, ctx.n_tokens, float(scale), int(window), float(out_scale), float(softcap), ctx.stream),
        "biased_attention")
