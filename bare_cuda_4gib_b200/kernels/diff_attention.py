"""Launchers of `csrc/diff_attention.cu`: differential attention (two softmax maps per head over the
same values, the second subtracted) with its finishing steps, over the paged cache."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build
from .lib import CacheView, _check, _dev, _ptr, dtype_code

MAX_V_DIM = 256      # value entries the plain kernel keeps per lane times 32
_lib = None
_mma_libs: dict = {}


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("diff_attention.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_diff_attention_plain.argtypes = [P, P, P, L, I, P, P, P, L, I, I, I, I, I, P, P, I, I, F, I, I, F, F, F, P]
        l.llm_diff_attention_plain.restype = c_int
        _lib = l
    return _lib


def mma_lib(dim: int, v_dim: int):
    """The tensor-core kernel built for maps of `dim` and values of `v_dim` entries."""
    key = (dim, v_dim)
    l = _mma_libs.get(key)
    if l is None:
        l = build.load_library("diff_attention.cu", mma_defines(dim, v_dim))
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_diff_attention_mma.argtypes = [P, P, P, L, P, P, P, L, I, I, I, I, I, P, P, P, I, I, I, I, F, I, I, F, F, F, P]
        l.llm_diff_attention_mma.restype = c_int
        _mma_libs[key] = l
    return l


def mma_defines(dim: int, v_dim: int):
    return [f"-DDA_DQ={dim}", f"-DDA_DV={v_dim}"]


def mma_takes(dtype, dim: int, v_dim: int) -> bool:
    """Whether the tensor-core kernel runs these sizes: bfloat16, a map a multiple of 16 up to 128, values a
    multiple of 16 up to 256."""
    return dtype == torch.bfloat16 and dim % 16 == 0 and 16 <= dim <= 128 and v_dim % 16 == 0 and 16 <= v_dim <= 256


def attention(ctx, q: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor], cache: CacheView, heads: int,
              scale: float, window: int, chunk: int, lam: float, eps: float, out_scale: float) -> None:
    """q [rows, heads, 2 * dim] (both maps of a head side by side, as the cache holds the keys); out [rows,
    heads * v_dim] = (a1 - lam * a2) / rms * out_scale * sigmoid(gate), a_m the m-th map's softmax attention
    over the keys that the query's position sees: `window` > 0 keeps the last positions, `chunk` > 0 the
    positions of the query's own block of that many; `gate` (or None) is a [rows, heads * v_dim] column view."""
    _dev(q, out, gate)
    if q.dtype != out.dtype or q.dtype != cache.dtype or (gate is not None and (gate.dtype != q.dtype or gate.stride(1) != 1)):
        raise TypeError("diff_attention: q, out, gate and the cache must share one element type")
    dim = cache.head_dim // 2
    if (mma_takes(q.dtype, dim, cache.v_dim) and q.data_ptr() % 16 == 0 and cache.k_ptr % 16 == 0 and cache.v_ptr % 16 == 0
            and cache.page_stride % 8 == 0 and q.is_contiguous()):
        single = 1 if ctx.max_q_len * (heads // cache.kv_heads) <= 16 else 0
        _check(mma_lib(dim, cache.v_dim).llm_diff_attention_mma(
            q.data_ptr(), out.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, cache.k_ptr, cache.v_ptr,
            cache.block_table.data_ptr(), cache.page_stride, cache.table_stride, cache.page_tokens, cache.kv_heads,
            cache.head_dim, cache.v_dim, ctx.seq_q_start.data_ptr(), ctx.seq_q_len.data_ptr(), ctx.seq_kv_len.data_ptr(),
            ctx.n_seqs, heads, ctx.n_tokens, single, float(scale), int(window), int(chunk), float(lam), float(eps),
            float(out_scale), ctx.stream), "diff_attention_mma")
        return
    _check(lib().llm_diff_attention_plain(
        q.data_ptr(), out.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, dtype_code(q.dtype),
        cache.k_ptr, cache.v_ptr, cache.block_table.data_ptr(), cache.page_stride, cache.table_stride, cache.page_tokens,
        cache.kv_heads, cache.head_dim, cache.v_dim, ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), heads,
        ctx.n_tokens, float(scale), int(window), int(chunk), float(lam), float(eps), float(out_scale), ctx.stream),
        "diff_attention_plain")
