"""Launchers of `csrc/moe.cu`: router, grouping of a step's (token, choice) slots by expert, the
experts' products over the grouped rows, and the sum of a token's slots."""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build
from .lib import Partials, _check, _dev, _ptr, dtype_code

MAX_EXPERTS = 512
_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load_library("moe.cu")
        P, I, L, F = c_void_p, c_int, c_longlong, c_float
        l.llm_moe_route.argtypes = [P, I, L, P, P, I, I, I, I, F, P, P, P, I, P]
        l.llm_moe_sort.argtypes = [P, I, I, I, P, P, P, P]
        l.llm_moe_grouped.argtypes = [P, L, P, P, I, I, P, P, P, P, I, I, I, I, P]
        l.llm_moe_combine.argtypes = [P, I, P, I, I, L, P, P, I, I, P]
        l.llm_moe_tile_rows.argtypes = []
        for name in ("llm_moe_route", "llm_moe_sort", "llm_moe_grouped", "llm_moe_combine", "llm_moe_tile_rows"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


def tile_rows() -> int:
    """Rows of one expert that a block of the grouped products takes."""
    return int(lib().llm_moe_tile_rows())


def max_tiles(n_slots: int, experts: int) -> int:
    """The most row tiles `n_slots` slots dealt to `experts` experts can make (a bound that depends
    on the step's shape only, so a captured graph of the step stays valid whatever the router picks)."""
    return -(-n_slots // tile_rows()) + min(experts, n_slots)


def route(ctx, h: torch.Tensor, w_router: torch.Tensor, w_shared_gate: Optional[torch.Tensor], top: int,
          router_scale: float, ids: torch.Tensor, weights: torch.Tensor, shared_gate: Optional[torch.Tensor], rows: int) -> None:
    """ids, weights [rows, top]: the `top` experts with the largest softmax(W_router h) (float32), and
    that score times `router_scale`; shared_gate [rows] = sigmoid(w_shared_gate . h)."""
    _dev(h, w_router, w_shared_gate, ids, weights, shared_gate)
    if w_shared_gate is not None and w_shared_gate.dtype != w_router.dtype:
        raise TypeError("moe route: the router and the shared gate must share one element type")
    _check(lib().llm_moe_route(h.data_ptr(), dtype_code(h.dtype), h.stride(0), w_router.data_ptr(), _ptr(w_shared_gate),
                               dtype_code(w_router.dtype), h.shape[1], w_router.shape[0], top, float(router_scale),
                               ids.data_ptr(), weights.data_ptr(), _ptr(shared_gate), rows, ctx.stream), "moe_route")


def sort(ctx, ids: torch.Tensor, n_slots: int, experts: int, sorted_slots: torch.Tensor, tiles: torch.Tensor,
         n_tiles: torch.Tensor) -> None:
    _dev(ids, sorted_slots, tiles, n_tiles)
    _check(lib().llm_moe_sort(ids.data_ptr(), n_slots, experts, tile_rows(), sorted_slots.data_ptr(), tiles.data_ptr(),
                              n_tiles.data_ptr(), ctx.stream), "moe_sort")


def grouped(ctx, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, down: bool, sorted_slots: torch.Tensor,
            tiles: torch.Tensor, n_tiles: torch.Tensor, weights: torch.Tensor, top: int, n: int, k: int, n_slots: int,
            experts: int) -> None:
    """up (`down` False): a [tokens, k], w [experts, 2n, k] (gate rows then up rows), out [slots, n] in the order
    of `sorted_slots` = silu(gate) * up.  down: a [slots, k] in that order, w [experts, n, k], out float32
    [slots, n] at the slot's own index, times the slot's weight."""
    _dev(a, w, out, sorted_slots, tiles, n_tiles, weights)
    if a.dtype != w.dtype or not w.is_contiguous() or a.stride(1) != 1:
        raise TypeError("moe grouped: element types or layout not as the kernel needs")
    _check(lib().llm_moe_grouped(a.data_ptr(), a.stride(0), w.data_ptr(), out.data_ptr(), dtype_code(a.dtype),
                                 1 if down else 0, sorted_slots.data_ptr(), tiles.data_ptr(), n_tiles.data_ptr(),
                                 weights.data_ptr(), top, n, k, max_tiles(n_slots, experts), ctx.stream), "moe_grouped")


def combine(ctx, y: torch.Tensor, top: int, shared: Optional[Partials], shared_gate: Optional[torch.Tensor],
            out: torch.Tensor, rows: int, hidden: int) -> None:
    """out[t] = sum_k y[t * top + k] (+ shared_gate[t] * shared[t]), float32."""
    st = shared.tensor if shared is not None else None
    _dev(y, st, shared_gate, out)
    _check(lib().llm_moe_combine(y.data_ptr(), top, _ptr(st), dtype_code(st.dtype) if st is not None else 0,
                                 shared.n if shared is not None else 0, shared.stride if shared is not None else 0,
                                 _ptr(shared_gate), out.data_ptr(), rows, hidden, ctx.stream), "moe_combine")
