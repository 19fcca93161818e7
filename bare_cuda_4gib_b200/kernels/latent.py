"""Launchers of `csrc/latent_attention.cu`: attention over a cached latent vector per token."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build
from .lib import CacheView, _check, _dev, _ptr, dtype_code

MAX_RANK = 512      # value entries the attention kernel keeps per lane times 32
ROWS_KERNEL_FROM = 8      # steps whose longest portion has at least this many tokens run the kernel for portions
_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("latent_attention.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_latent_prepare.argtypes = [P, I, L, I, P, L, I, I, I, I, P, F, P, I, I, F, P, P, P, L, I, I, P, P, I, I, P]
        l.llm_rows_rmsnorm.argtypes = [P, L, P, P, L, I, I, I, F, P]
        l.llm_per_head_linear.argtypes = [P, L, L, P, I, P, L, L, P, L, I, I, I, I, I, P]
        l.llm_latent_attention.argtypes = [P, P, I, P, P, L, I, I, I, I, P, P, P, I, I, F, I, P]
        l.llm_latent_attention_mma.argtypes = [P, P, P, P, P, L, I, I, I, I, P, P, P, I, I, F, I, I, P]
        l.llm_latent_attention_mma_scratch.argtypes = [I, I, I, I]
        l.llm_latent_attention_mma_scratch.restype = c_longlong
        l.llm_latent_attention_rows.argtypes = [P, P, P, P, L, I, I, I, I, P, P, P, P, P, I, I, I, F, I, P]
        for name in ("llm_latent_prepare", "llm_rows_rmsnorm", "llm_per_head_linear", "llm_latent_attention", "llm_latent_attention_mma",
                     "llm_latent_attention_rows"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


def prepare(ctx, u: torch.Tensor, q_col: int, c_rows: Optional[torch.Tensor], heads: int, dim: int, rot: int, rank: int,
            norm_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rot_dims: int, mag: float,
            q_full: torch.Tensor, cache: CacheView, write_cache: bool, halves: bool = False) -> None:
    """Norms the latent (`c_rows` [rows, rank + rot], a column view or a matrix of its own), rotates the
    shared key part and writes both to the cache; rotates the queries' rotated parts (u [rows, ...], the
    queries from column `q_col`) into the last `rot` entries of q_full [rows, heads, rank + rot].  A run that
    reads another run's cache gives no `c_rows` and writes nothing.  `halves`: entry i turns with entry
    i + rot_dims / 2 instead of 2i with 2i + 1."""
    _dev(u, c_rows, norm_w, inv_freq, q_full)
    write_cache = bool(write_cache and c_rows is not None)
    if c_rows is not None and (c_rows.dtype != u.dtype or c_rows.stride(1) != 1):
        raise TypeError("latent prepare: the compressed rows must have the queries' element type and unit column stride")
    _check(lib().llm_latent_prepare(
        u.data_ptr(), dtype_code(u.dtype), u.stride(0), q_col, _ptr(c_rows), c_rows.stride(0) if c_rows is not None else 0,
        heads, dim, rot, rank, _ptr(norm_w), float(eps), _ptr(inv_freq), int(rot_dims), 1 if halves else 0, float(mag),
        q_full.data_ptr(), cache.k_ptr, cache.block_table.data_ptr(), cache.page_stride, cache.table_stride,
        cache.page_tokens, ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), 1 if write_cache else 0, ctx.n_tokens,
        ctx.stream), "latent_prepare")


def rows_rmsnorm(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int, eps: float) -> None:
    """out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w; x may be a column view, sums are float32."""
    _dev(x, w, out)
    if not (x.dtype == w.dtype == out.dtype) or x.stride(1) != 1 or out.stride(1) != 1:
        raise TypeError("rows_rmsnorm: element types or layout not as the kernel needs")
    _check(lib().llm_rows_rmsnorm(x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0),
                                  dtype_code(x.dtype), rows, x.shape[1], float(eps), ctx.stream), "rows_rmsnorm")


def per_head_linear(ctx, x: torch.Tensor, w: torch.Tensor, w_in_rows: bool, out: torch.Tensor, heads: int, n_in: int,
                    n_out: int, rows: int, gate: Optional[torch.Tensor] = None) -> None:
    """out[t, h, :n_out] = x[t, h, :n_in] times head h's block of w: rows h * n_in .. of
    w [heads * n_in, n_out] (`w_in_rows`), or the transpose of rows h * n_out .. of w [heads * n_out,
    n_in].  x and out are [rows, heads, >= n] views (any row and head strides); with `gate`
    [rows, heads * n_out] the result is multiplied by its sigmoid."""
    _dev(x, w, out, gate)
    if not (x.dtype == w.dtype == out.dtype) or x.stride(2) != 1 or out.stride(2) != 1 or not w.is_contiguous():
        raise TypeError("per_head_linear: element types or layout not as the kernel needs")
    _check(lib().llm_per_head_linear(
        x.data_ptr(), x.stride(0), x.stride(1), w.data_ptr(), 1 if w_in_rows else 0, out.data_ptr(), out.stride(0),
        out.stride(1), _ptr(gate), gate.stride(0) if gate is not None else 0, dtype_code(x.dtype), rows, heads, n_in,
        n_out, ctx.stream), "per_head_linear")


def mma_takes(dtype: torch.dtype, D: int, rank: int) -> bool:
    """Whether the tensor-core kernel takes these sizes (else the float32 kernel runs)."""
    return dtype == torch.bfloat16 and D % 16 == 0 and rank % 32 == 0 and 32 <= rank <= MAX_RANK


_scratch = {}      # device -> float32 scratch of the split launches (outgrown ones are kept: graphs hold them)
_retired = []


def _split_scratch(device, floats: int) -> torch.Tensor:
    buf = _scratch.get(device)
    if buf is None or buf.numel() < floats:
        if buf is not None:
            _retired.append(buf)
        buf = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


def key_splits(n_tokens: int, heads: int) -> int:
    """Thread blocks that share a tile's keys: a step of few tokens (decoding) spreads every token's
    keys over about two blocks per SM in all.  It depends on the step's shape only, never on the
    requests' lengths, so a captured graph of the step stays valid while they grow."""
    from .lib import sm_count
    tiles = n_tokens * ((heads + 15) // 16)
    if tiles >= sm_count():
        return 1
    return max(1, min(32, (2 * sm_count()) // tiles))


def attention(ctx, q_full: torch.Tensor, out: torch.Tensor, cache: CacheView, rank: int, sink: Optional[torch.Tensor],
              heads: int, scale: float, window: int = 0) -> None:
    """out[t, h] = sum_j p_j c_j over the cached vectors [c_j | r_j] at positions <= the query's, p the
    softmax of (q_full[t, h] . [c_j | r_j]) * scale, with exp(sink[h]) in the denominator if given."""
    _dev(q_full, out, sink)
    if (ctx.use_fast_attention and q_full.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
            and ctx.max_q_len >= ROWS_KERNEL_FROM and cache.head_dim % 16 == 0 and rank % 16 == 0 and rank <= 256):
        # prompt portions: four tokens of a request share the cached blocks they read
        _check(lib().llm_latent_attention_rows(
            q_full.data_ptr(), out.data_ptr(), cache.k_ptr, cache.block_table.data_ptr(), cache.page_stride,
            cache.table_stride, cache.page_tokens, cache.head_dim, rank, _ptr(sink), ctx.positions.data_ptr(),
            ctx.seq_q_start.data_ptr(), ctx.seq_q_len.data_ptr(), ctx.row_seq.data_ptr(), heads, ctx.n_seqs,
            ctx.max_q_len, float(scale), int(window), ctx.stream), "latent_attention_rows")
        return
    if ctx.use_fast_attention and mma_takes(q_full.dtype, cache.head_dim, rank) and cache.dtype == torch.bfloat16:
        splits = key_splits(ctx.n_tokens, heads)
        floats = int(lib().llm_latent_attention_mma_scratch(ctx.n_tokens, heads, rank, splits))
        scratch = _split_scratch(q_full.device, floats).data_ptr() if floats else 0
        _check(lib().llm_latent_attention_mma(
            q_full.data_ptr(), out.data_ptr(), scratch, cache.k_ptr, cache.block_table.data_ptr(), cache.page_stride,
            cache.table_stride, cache.page_tokens, cache.head_dim, rank, _ptr(sink), ctx.positions.data_ptr(),
            ctx.row_seq.data_ptr(), heads, ctx.n_tokens, float(scale), int(window), splits, ctx.stream),
            "latent_attention_mma")
        if splits > 1:
            from .lib import LAUNCHES
            LAUNCHES[0] += 1      # the merge is a second kernel
        return
    _check(lib().llm_latent_attention(
        q_full.data_ptr(), out.data_ptr(), dtype_code(q_full.dtype), cache.k_ptr, cache.block_table.data_ptr(),
        cache.page_stride, cache.table_stride, cache.page_tokens, cache.head_dim, rank, _ptr(sink),
        ctx.positions.data_ptr(), ctx.row_seq.data_ptr(), heads, ctx.n_tokens, float(scale), int(window), ctx.stream),
        "latent_attention")
