"""Rotary position encoding with the rotate_half pairing (element p with p + head_dim / 2).

inv_freq[p] = 1 / theta^(2p / head_dim); the angle of position pos is the float32 product
float(pos) * inv_freq[p]; lo' = lo cos - hi sin, hi' = hi cos + lo sin
(cuongvng/bare-cuda-4gib engine/kernels/rope.cu:44-53; tools/references/reference_forward.py:89-104).
The frequencies are computed once on the host in float32 and kept on the device; the attention
kernels rotate q and k with them while they write the cache, so this part launches nothing.

params: `head_dim`, `theta`.  No tensors.
"""

from __future__ import annotations

import torch

from .base import Part
from .registry import register_position


@register_position("rope")
class RotaryPositions(Part):
    def prepare(self, dtype, device) -> None:
        d, theta = int(self.params["head_dim"]), float(self.params["theta"])
        exponent = torch.arange(d // 2, dtype=torch.float32) * 2.0 / d
        self.inv_freq = (1.0 / (theta ** exponent)).to(device)

    def fused_rotation(self):
        """Inverse frequencies for kernels that rotate q and k themselves."""
        return self.inv_freq


@register_position("none")
class NoPositions(Part):
    """No position information inside the mixer (keys and queries are used as projected)."""

    def fused_rotation(self):
        return None


@register_position("rotary_pairs")
class PairwiseRotaryPositions(Part):
    """Rotation of the first `dims` entries of a head in neighbouring pairs (entry 2i with 2i + 1;
    the rest pass) by the angle position * f_i, f_i = base^(-2i / dims).

    With `scaling` {factor, original, fast, slow} (YaRN): a frequency that turns more than `fast`
    times within `original` positions keeps f_i, one that turns fewer than `slow` times becomes
    f_i / factor, in between the two are blended linearly in i; cos and sin are multiplied by
    0.1 ln(factor) + 1.  With where(t) = dims ln(original / (2 pi t)) / (2 ln base), lo =
    max(floor(where(fast)), 0), hi = min(ceil(where(slow)), dims - 1), ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1): f_i <- f_i / factor * ramp_i + f_i (1 - ramp_i).

    The kernels that norm and cache q and k turn them with `inv_freq` and `magnitude` themselves.
    params: `dims`, `base`, `scaling` (or None).  No tensors."""

    def prepare(self, dtype, device) -> None:
        import math

        dims, base = int(self.params["dims"]), float(self.params["base"])
        self.dims = dims
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = base ** (-2.0 * i / dims)
        self.magnitude = 1.0
        sc = self.params.get("scaling")
        if sc:
            factor, original = float(sc["factor"]), float(sc["original"])

            def where(turns: float) -> float:
                return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

            lo = max(math.floor(where(float(sc["fast"]))), 0)
            hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.inv_freq = f.to(torch.float32).to(device)

    def fused_rotation(self):
        return None      # the pairing differs from the one the fused attention kernels apply


@register_position("rotary_halves")
class HalvesRotaryPositions(Part):
    """Rotation of the first `dims` entries of a head (or of a map of a head) with entry i paired with
    entry i + dims / 2 (the rest pass) by the angle position * f_i, f_i = base^(-2i / dims): the pair
    (u, v) becomes (u cos - v sin, v cos + u sin).

    With `scaling` {factor, low, high, original} (the rule of Llama 3.1, by wavelength l = 2 pi / f): a
    frequency with l < original / high stays, one with l > original / low becomes f / factor, and in
    between, with s = (original / l - low) / (high - low), it becomes (1 - s) f / factor + s f.

    The kernels that norm and cache q and k turn them with `inv_freq` themselves (`halves` tells them
    the pairing).  params: `dims`, `base`, `scaling` (or None).  No tensors."""

    halves = True
    magnitude = 1.0

    def prepare(self, dtype, device) -> None:
        import math

        dims, base = int(self.params["dims"]), float(self.params["base"])
        self.dims = dims
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = base ** (-2.0 * i / dims)
        sc = self.params.get("scaling")
        if sc:
            factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
            length = 2.0 * math.pi / f
            s = ((original / length - low) / (high - low)).clamp(0.0, 1.0) if high != low else torch.ones_like(f)
            blended = (1.0 - s) * f / factor + s * f
            f = torch.where(length < original / high, f, torch.where(length > original / low, f / factor, blended))
        self.inv_freq = f.to(torch.float32).to(device)

    def fused_rotation(self):
        return None      # the fused attention kernels turn whole heads; this one may turn a head's first entries only
