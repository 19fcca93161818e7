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
        l.llm_moe_route.argtypes = [P, I, L, P, P, I, I, I, I, F, P, P, P, I, P, I, I, P]
        l.llm_moe_sort.argtypes = [P, I, I, I, P, P, P, P]
        l.llm_moe_grouped.argtypes = [P, L, P, P, I, I, P, P, P, P, I, I, I, I, I, P]
        l.llm_moe_combine.argtypes = [P, I, P, I, I, L, P, P, I, I, P, P, I, P, I, L, P]
        l.llm_moe_tile_rows.argtypes = []
        l.llm_moe_gather_rows.argtypes = [P, L, P, I, P, I, I, P]
        for name in ("llm_moe_route", "llm_moe_sort", "llm_moe_grouped", "llm_moe_combine", "llm_moe_tile_rows",
                     "llm_moe_gather_rows"):
            getattr(l, name).restype = c_int
        _lib = l
    return _lib


TENSOR_TILE_ROWS = 128      # rows of a tile of the tensor-core product (its MMA rows)


def tile_rows(tensor_cores: bool = False) -> int:
    """Rows of one expert that a block of the grouped products takes."""
    return TENSOR_TILE_ROWS if tensor_cores else int(lib().llm_moe_tile_rows())


def max_tiles(n_slots: int, experts: int, tensor_cores: bool = False) -> int:
    """The most row tiles `n_slots` slots dealt to `experts` experts can make (a bound that depends
    on the step's shape only, so a captured graph of the step stays valid whatever the router picks)."""
    return -(-n_slots // tile_rows(tensor_cores)) + min(experts, n_slots)


def route(ctx, h: torch.Tensor, w_router: torch.Tensor, w_shared_gate: Optional[torch.Tensor], top: int,
          router_scale: float, ids: torch.Tensor, weights: torch.Tensor, shared_gate: Optional[torch.Tensor], rows: int,
          correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1) -> None:
    """ids, weights [rows, top]: the `top` experts with the largest softmax(W_router h) (float32), and
    that score times `router_scale`; shared_gate [rows] = sigmoid(w_shared_gate . h).  With `correction`
    (float32, one per expert) the choice goes by score + correction while the weight stays the score; with
    `groups` > 1 the experts form that many equal groups of neighbours and only experts of the `keep`
    groups with the largest best choice value can be chosen."""
    _dev(h, w_router, w_shared_gate, ids, weights, shared_gate, correction)
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != w_router.shape[0]):
        raise TypeError("moe route: the correction must be float32, one number per router output")
    if w_shared_gate is not None and w_shared_gate.dtype != w_router.dtype:
        raise TypeError("moe route: the router and the shared gate must share one element type")
    _check(lib().llm_moe_route(h.data_ptr(), dtype_code(h.dtype), h.stride(0), w_router.data_ptr(), _ptr(w_shared_gate),
                               dtype_code(w_router.dtype), h.shape[1], w_router.shape[0], top, float(router_scale),
                               ids.data_ptr(), weights.data_ptr(), _ptr(shared_gate), rows, _ptr(correction), int(groups),
                               int(keep), ctx.stream), "moe_route")


def sort(ctx, ids: torch.Tensor, n_slots: int, experts: int, sorted_slots: torch.Tensor, tiles: torch.Tensor,
         n_tiles: torch.Tensor, tensor_cores: bool = False) -> None:
    _dev(ids, sorted_slots, tiles, n_tiles)
    _check(lib().llm_moe_sort(ids.data_ptr(), n_slots, experts, tile_rows(tensor_cores), sorted_slots.data_ptr(),
                              tiles.data_ptr(), n_tiles.data_ptr(), ctx.stream), "moe_sort")


def gather_rows(ctx, a: torch.Tensor, sorted_slots: torch.Tensor, top: int, out: torch.Tensor, n_slots: int) -> None:
    """out[i] = a[sorted_slots[i] // top]: the tokens' rows in the order of the list."""
    _dev(a, sorted_slots, out)
    if a.dtype != out.dtype or a.stride(1) != 1 or not out.is_contiguous() or out.shape[1] != a.shape[1]:
        raise TypeError("moe gather_rows: element types or layout not as the kernel needs")
    es = a.element_size()
    _check(lib().llm_moe_gather_rows(a.data_ptr(), a.stride(0) * es, sorted_slots.data_ptr(), top, out.data_ptr(),
                                     a.shape[1] * es, n_slots, ctx.stream), "moe_gather_rows")


class GroupedPlan:
    """Tensor maps of the experts' stacked matrices for the tensor-core grouped product: `w_up`
    [experts * 2 * ff, hidden] (an expert's gate rows, then its up rows; ungated experts: [experts * ff,
    hidden]) and `w_down` [experts * hidden, ff]."""

    UP_TILE, DOWN_TILE = 256, 128      # weight rows of a tile (the up tile is half gate rows, half up rows)

    def __init__(self, w_up: torch.Tensor, w_down: torch.Tensor, experts: int, gated: bool = True):
        from . import gemm
        self.experts, self.gated = experts, gated
        self.ff, self.hidden = w_down.shape[1], w_down.shape[0] // experts
        self.up = gemm.GemmPlan(w_up)
        self.down = gemm.GemmPlan(w_down)

    @staticmethod
    def takes(w_up: torch.Tensor, w_down: torch.Tensor) -> bool:
        from . import gemm
        return gemm.supports(w_up) and gemm.supports(w_down)


def grouped_tensor(ctx, plan: GroupedPlan, a: torch.Tensor, out: torch.Tensor, down: bool, sorted_slots: torch.Tensor,
                   tiles: torch.Tensor, n_tiles: torch.Tensor, weights: torch.Tensor, n_slots: int) -> None:
    """The grouped products on the tensor cores.  `a` [slots, k] bfloat16 in the order of the list.  up:
    out [slots, ff] = silu(gate) * up in that order.  down: out float32 [slots, hidden] at the slot's own
    index, times the slot's weight."""
    import ctypes
    from . import gemm
    _dev(a, out, sorted_slots, tiles, n_tiles, weights)
    p = plan.down if down else plan.up
    if a.dtype != torch.bfloat16 or a.stride(1) != 1 or a.shape[1] != p.k or a.data_ptr() % 16 or a.stride(0) % 8:
        raise TypeError("moe grouped (tensor cores): activations not as the kernel needs")
    bn = plan.DOWN_TILE if down else plan.UP_TILE
    n_out = plan.hidden if down else plan.ff
    err = gemm.error_word(a.device)
    if not down and not plan.gated:
        # ungated experts: a plain product of 128 weight rows a tile whose epilogue squares relu(x)
        from .lib import GROUPED_RELU2
        bn = plan.DOWN_TILE
        _check(gemm.lib(GROUPED_RELU2).llm_gemm_grouped_bf16(
            ctypes.addressof(p.weight_map(bn)), ctypes.addressof(p.act_map(a, gemm.BM)), out.data_ptr(), gemm.DT_BF16,
            max_tiles(n_slots, plan.experts, True), n_out, p.k, out.stride(0), bn, 0, 0, plan.ff, tiles.data_ptr(),
            n_tiles.data_ptr(), None, None, err.data_ptr(), ctx.stream), "gemm_tcgen05 (grouped, relu squared)")
        return
    _check(gemm.lib().llm_gemm_grouped_bf16(
        ctypes.addressof(p.weight_map(bn if down else bn // 2)), ctypes.addressof(p.act_map(a, gemm.BM)), out.data_ptr(),
        gemm.DT_F32 if down else gemm.DT_BF16, max_tiles(n_slots, plan.experts, True), n_out, p.k, out.stride(0), bn,
        0 if down else 1, 0 if down else plan.ff, plan.hidden if down else 2 * plan.ff, tiles.data_ptr(), n_tiles.data_ptr(),
        sorted_slots.data_ptr() if down else None, weights.data_ptr() if down else None, err.data_ptr(), ctx.stream),
        "gemm_tcgen05 (grouped)")


def grouped(ctx, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, down: bool, sorted_slots: torch.Tensor,
            tiles: torch.Tensor, n_tiles: torch.Tensor, weights: torch.Tensor, top: int, n: int, k: int, n_slots: int,
            experts: int, gated: bool = True) -> None:
    """up (`down` False): a [tokens, k], w [experts, 2n, k] (gate rows then up rows), out [slots, n] in the order
    of `sorted_slots` = silu(gate) * up; not `gated`: w [experts, n, k] and out = relu(up)^2.  down: a [slots, k] in that order, w [experts, n, k], out float32
    [slots, n] at the slot's own index, times the slot's weight."""
    _dev(a, w, out, sorted_slots, tiles, n_tiles, weights)
    if a.dtype != w.dtype or not w.is_contiguous() or a.stride(1) != 1:
        raise TypeError("moe grouped: element types or layout not as the kernel needs")
    _check(lib().llm_moe_grouped(a.data_ptr(), a.stride(0), w.data_ptr(), out.data_ptr(), dtype_code(a.dtype),
                                 1 if down else 0, sorted_slots.data_ptr(), tiles.data_ptr(), n_tiles.data_ptr(),
                                 weights.data_ptr(), top, n, k, max_tiles(n_slots, experts), 1 if gated else 0,
                                 ctx.stream), "moe_grouped")


def combine(ctx, y: torch.Tensor, top: int, shared: Optional[Partials], shared_gate: Optional[torch.Tensor],
            out: torch.Tensor, rows: int, hidden: int, ids: Optional[torch.Tensor] = None,
            weights: Optional[torch.Tensor] = None, experts: int = 0, h: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum_k y[t * top + k] (+ shared_gate[t] * shared[t]), float32.  With `ids`: a slot whose
    expert is `experts` or beyond is an identity expert and counts as weights[slot] * h[t]."""
    st = shared.tensor if shared is not None else None
    _dev(y, st, shared_gate, out, ids, weights, h)
    _check(lib().llm_moe_combine(y.data_ptr(), top, _ptr(st), dtype_code(st.dtype) if st is not None else 0,
                                 shared.n if shared is not None else 0, shared.stride if shared is not None else 0,
                                 _ptr(shared_gate), out.data_ptr(), rows, hidden, _ptr(ids), _ptr(weights), int(experts),
                                 _ptr(h), dtype_code(h.dtype) if h is not None else 0, h.stride(0) if h is not None else 0,
                                 ctx.stream), "moe_combine")
