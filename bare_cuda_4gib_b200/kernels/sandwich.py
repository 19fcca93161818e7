"""Launchers of `csrc/sandwich_norm.cu`: the embedding lookup with an RMS norm, and the kernel
between two sublayers of a stream that norms on both sides of every sublayer."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build
from .lib import Partials, _check, _dev, _ptr, dtype_code, stream_handle

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("sandwich_norm.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_embed_rmsnorm.argtypes = [P, P, P, I, I, P, I, I, F, P]
        l.llm_postnorm_add_rmsnorm.argtypes = [P, P, I, L, P, F, P, F, P, I, P, I, I, P]
        for name in ("llm_embed_rmsnorm", "llm_postnorm_add_rmsnorm"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


class NormedDelta:
    """A sublayer's result that still has to be normed (weight `weight`, `eps`) and added to the stream."""

    __slots__ = ("y", "weight", "eps")

    def __init__(self, y: Partials, weight: torch.Tensor, eps: float):
        self.y, self.weight, self.eps = y, weight, eps


def embed_rmsnorm(table: torch.Tensor, ids: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_tokens: int,
                  eps: float, stream=None) -> None:
    """out[t] = rms_norm(table[ids[t]]) * weight, float32; the weight has the table's type or is float32."""
    _dev(table, ids, weight, out)
    _check(lib().llm_embed_rmsnorm(table.data_ptr(), ids.data_ptr(), weight.data_ptr(), dtype_code(table.dtype),
                                   dtype_code(weight.dtype), out.data_ptr(), n_tokens, table.shape[1], float(eps),
                                   stream if stream is not None else stream_handle()), "embed_rmsnorm")


def postnorm_add_rmsnorm(residual: torch.Tensor, delta: Optional[NormedDelta], weight: Optional[torch.Tensor],
                         out: Optional[torch.Tensor], eps: float, rows: int, row_index: Optional[torch.Tensor] = None,
                         stream=None) -> None:
    """residual[r] += rms_norm(sum of delta's partial results)[r] * delta.weight, then
    out[i] = rms_norm(residual[r]) * weight with r = row_index[i] or i; either half may be left out."""
    _dev(residual, weight, out)
    y = delta.y if delta is not None else None
    if y is not None and y.tensor.dtype != torch.float32:
        raise TypeError("postnorm_add_rmsnorm: the sublayer's result must be float32")
    code = dtype_code(weight.dtype if weight is not None else delta.weight.dtype)
    _check(lib().llm_postnorm_add_rmsnorm(
        residual.data_ptr(), _ptr(y.tensor) if y is not None else 0, y.n if y is not None else 0,
        y.stride if y is not None else 0, _ptr(delta.weight) if delta is not None else 0,
        float(delta.eps) if delta is not None else 0.0, _ptr(weight), float(eps), _ptr(out), code, _ptr(row_index), rows,
        residual.shape[-1], stream if stream is not None else stream_handle()), "postnorm_add_rmsnorm")
