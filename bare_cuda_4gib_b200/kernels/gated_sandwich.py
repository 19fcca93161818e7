"""Launcher of `csrc/gated_sandwich.cu`: the kernel between two sublayers of a stream that norms on
both sides of every sublayer, multiplies a sublayer's result by a sigmoid gate first, and at a
layer's end replaces the stream by a weighted sum of every layer's result so far."""

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
        l = build.load_library("gated_sandwich.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_gated_sandwich_step.argtypes = [P, P, I, L, P, I, L, P, P, F, P, L, I, P, I, P, F, P, I, P, I, I, P]
        l.llm_gated_sandwich_step.restype = c_int
        _lib = l
    return _lib


class DepthMix:
    """Where a layer's result is kept and how the stream is formed from the results so far:
    `history` [entries, rows, width] float32, the row goes to entry `index`, and (with `weights`
    [index + 1] float32) the stream becomes sum_j weights[j] * entry j."""

    __slots__ = ("history", "index", "weights")

    def __init__(self, history: torch.Tensor, index: int, weights: Optional[torch.Tensor]):
        self.history, self.index, self.weights = history, index, weights


class GatedDelta:
    """A sublayer's result `y` that still has to be gated (`gate` pre-activations [rows, width] with
    `gate_bias`, or None), normed (`weight` float32, `eps`) and added to the stream, and what happens to
    the stream right after (`depth`, or None).  With `y` None only `depth` applies."""

    __slots__ = ("y", "gate", "gate_bias", "weight", "eps", "depth")

    def __init__(self, y: Optional[Partials], gate: Optional[torch.Tensor], gate_bias: Optional[torch.Tensor],
                 weight: Optional[torch.Tensor], eps: float, depth: Optional[DepthMix] = None):
        self.y, self.gate, self.gate_bias, self.weight, self.eps, self.depth = y, gate, gate_bias, weight, eps, depth


def step(residual: torch.Tensor, delta: Optional[GatedDelta], weight: Optional[torch.Tensor], out: Optional[torch.Tensor],
         eps: float, rows: int, row_index: Optional[torch.Tensor] = None, stream=None) -> None:
    """What `delta` describes, then out[i] = rms_norm(residual[r]) * weight with r = row_index[i] or i."""
    y = delta.y if delta is not None else None
    gate = delta.gate if delta is not None and y is not None else None
    depth = delta.depth if delta is not None else None
    _dev(residual, weight, out, gate)
    for t in (weight, delta.weight if delta is not None else None, delta.gate_bias if delta is not None else None,
              depth.weights if depth is not None else None, y.tensor if y is not None else None):
        if t is not None and t.dtype != torch.float32:
            raise TypeError("gated sandwich step: results, factors and biases must be float32")
    if gate is not None and gate.stride(1) != 1:
        raise TypeError("gated sandwich step: the gate's rows must be contiguous")
    hist = depth.history if depth is not None else None
    _check(lib().llm_gated_sandwich_step(
        residual.data_ptr(), _ptr(y.tensor) if y is not None else 0, y.n if y is not None else 0,
        y.stride if y is not None else 0, _ptr(gate), dtype_code(gate.dtype) if gate is not None else 0,
        gate.stride(0) if gate is not None else 0, _ptr(delta.gate_bias) if y is not None else 0,
        _ptr(delta.weight) if y is not None else 0, float(delta.eps) if y is not None else 0.0,
        _ptr(hist), hist.stride(0) if hist is not None else 0, depth.index if depth is not None else -1,
        _ptr(depth.weights) if depth is not None else 0, depth.index + 1 if depth is not None else 0,
        _ptr(weight), float(eps), _ptr(out), dtype_code(out.dtype) if out is not None else 0, _ptr(row_index), rows,
        residual.shape[-1], stream if stream is not None else stream_handle()), "gated_sandwich_step")
