"""The Pudulorn decoder written out plainly in float64, one function per mechanism, whole sequences
at a time and with no cache: the oracle of the engine's tests.  It shares nothing with the engine.

Notation: x [n, width] is the residual stream of one sequence whose tokens sit at positions 0..n-1,
h a sublayer's input, t a dict of the model's tensors by name, m a layer's `mixer` entry.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    """The weight is used as stored."""
    return unit_rms(x, eps) * w


def rms_norm_around_zero(x, w, eps):
    """The weight is stored around zero: the factor is 1 + w."""
    return unit_rms(x, eps) * (1.0 + w)


def turn_halves(x, positions, dims, base):
    """x [n, ..., size]: entry i < dims/2 of the last axis is paired with entry i + dims/2 and the pair
    turned by the angle position * base^(-2i/dims); entries from `dims` on stay."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def sees_block(n, size):
    """[query, key]: the key is not later and lies in the query's block of `size` positions."""
    p = torch.arange(n)
    return (p[None, :] <= p[:, None]) & ((p[None, :] // size) == (p[:, None] // size))


def sees_window(n, size):
    """[query, key]: the key is the query's own or one of the size - 1 before it."""
    p = torch.arange(n)
    back = p[:, None] - p[None, :]
    return (back >= 0) & (back < size)


def softmax_attention(q, k, v, scale, sees):
    """q [n, dq], k [n, dq], v [n, dv] of one head: softmax over the keys a query sees."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~sees, -math.inf)
    return torch.softmax(s, -1) @ v


def difference_factor(t, p, diff):
    return (math.exp(float((t[p + "lq1"] * t[p + "lk1"]).sum())) - math.exp(float((t[p + "lq2"] * t[p + "lk2"]).sum()))
            + diff)


def differential_attention(t: Dict[str, torch.Tensor], p: str, m, h, eps):
    n = h.shape[0]
    heads, groups, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(n)
    q = (h @ t[p + "q"].T).view(n, heads, 2, d)
    k = (h @ t[p + "k"].T).view(n, groups, 2, d)
    v = (h @ t[p + "v"].T).view(n, groups, dv)
    q = turn_halves(rms_norm(q, t[p + "q.norm"], eps), pos, m["rot"]["dims"], m["rot"]["base"])
    k = turn_halves(rms_norm(k, t[p + "k.norm"], eps), pos, m["rot"]["dims"], m["rot"]["base"])
    sees = sees_block(n, m["mask"]["size"])
    lam = difference_factor(t, p, m["diff"])
    out = []
    for head in range(heads):
        g = head // (heads // groups)
        first = softmax_attention(q[:, head, 0], k[:, g, 0], v[:, g], m["scale"], sees)
        second = softmax_attention(q[:, head, 1], k[:, g, 1], v[:, g], m["scale"], sees)
        out.append(unit_rms(first - lam * second, eps) * (1.0 - m["diff"]))
    o = torch.cat(out, -1) * torch.sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def compressed_keys(t, p, m, h, eps):
    """What a latent layer caches per token: the normed latent and the turned key part all heads share."""
    rank = m["kv_rank"]
    both = h @ t[p + "dkv"].T
    latent = rms_norm(both[:, :rank], t[p + "dkv.norm"], eps)
    shared = turn_halves(both[:, rank:], torch.arange(h.shape[0]), m["rot"]["dims"], m["rot"]["base"])
    return latent, shared


def latent_attention(t, p, m, h, eps, cached=None):
    """`cached`: (latent, shared key part) of the layer this one reads from; None: its own."""
    n = h.shape[0]
    heads, d, r, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    latent, shared = compressed_keys(t, p, m, h, eps) if cached is None else cached
    q = (rms_norm(h @ t[p + "dq"].T, t[p + "dq.norm"], eps) @ t[p + "uq"].T).view(n, heads, d + r)
    q_turned = turn_halves(q[..., d:], torch.arange(n), m["rot"]["dims"], m["rot"]["base"])
    keys = (latent @ t[p + "uk"].T).view(n, heads, d)
    values = (latent @ t[p + "uv"].T).view(n, heads, dv)
    sees = sees_window(n, m["mask"]["size"])
    out = []
    for head in range(heads):
        q_full = torch.cat([q[:, head, :d], q_turned[:, head]], -1)
        k_full = torch.cat([keys[:, head], shared], -1)
        out.append(softmax_attention(q_full, k_full, values[:, head], m["scale"], sees))
    return torch.cat(out, -1) @ t[p + "o"].T, (latent, shared)


def clamped_feed_forward(t, p, mlp, h):
    limit = mlp["limit"]
    g = torch.clamp(h @ t[p + "gate"].T, max=limit)
    u = torch.clamp(h @ t[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t[p + "down"].T


def expert(t, p, h):
    z = h @ t[p + "gate"].T
    return (z * torch.sigmoid(z) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def router(t, p, mlp, h, margins=None):
    """[n, experts]: score times router scale for a token's chosen experts, zero for the others.
    `margins` (a list) receives, per token, how far the last chosen score lies above the first one
    left out, relative to itself (1 where every expert is chosen)."""
    r = mlp["router"]
    s = torch.softmax(h @ t[p + "router"].T, -1)
    chosen = torch.topk(s, r["top"], -1).indices
    keep = torch.zeros_like(s).scatter_(1, chosen, 1.0)
    if margins is not None:
        v = torch.sort(s, -1, descending=True).values
        top = r["top"]
        margins.append((v[:, top - 1] - v[:, top]) / v[:, top - 1] if top < s.shape[1] else torch.ones_like(v[:, 0]))
    return s * keep * r["scale"]


def mixture_of_experts(t, p, mlp, h, margins=None):
    w = router(t, p, mlp, h, margins)
    out = torch.zeros_like(h)
    for e in range(mlp["router"]["experts"]):
        rows = torch.nonzero(w[:, e] != 0).flatten()
        if len(rows):
            out[rows] += w[rows, e, None] * expert(t, f"{p}e{e}.", h[rows])
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ t[p + "shared.sg"].T) * expert(t, p + "shared.", h)
    return out


def feed_forward(t, p, mlp, h, margins=None):
    return clamped_feed_forward(t, p, mlp, h) if mlp["kind"] == "dense" else mixture_of_experts(t, p, mlp, h, margins)


def forward(cfg, tensors: Dict[str, torch.Tensor], ids: List[int], streams: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence; with `streams` a list, the residual stream after every layer is appended;
    with `margins` a list, every router's per-token margin between the chosen and the other experts."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = t["embed"][torch.tensor(ids)]
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = rms_norm_around_zero(x, t[p + "norm1"], eps)
        if layer["type"] == "attention":
            x = x + differential_attention(t, p + "mix.", m, h, eps)
        else:
            src = m.get("kv_from")
            y, cached[i] = latent_attention(t, p + "mix.", m, h, eps, None if src is None else cached[src])
            x = x + y
        if layer.get("mlp") is not None:
            x = x + feed_forward(t, p + "mlp.", layer["mlp"], rms_norm_around_zero(x, t[p + "norm2"], eps), margins)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm_around_zero(x, t["final.norm"], eps) @ t["head"].T
