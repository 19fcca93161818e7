"""The Gurolix decoder written out plainly in float64, one function per mechanism, whole sequences
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


def norm_around_zero(x, w, eps):
    """The weight is stored around zero: the factor is 1 + w."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain_weight(x, w, eps):
    return unit_rms(x, eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def frequencies(rot) -> torch.Tensor:
    """f_i = base^(-2i/dims); with `scaling`, a frequency whose wavelength is longer than
    original/low is divided by factor, one shorter than original/high stays, and between the two
    the divided and the kept value are blended by how many turns fit into `original` positions."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, original = sc["factor"], sc["low"], sc["high"], sc["original"]
        out = []
        for fi in f:
            length = 2.0 * math.pi / fi
            if length < original / high:
                out.append(fi)
            elif length > original / low:
                out.append(fi / factor)
            else:
                s = (original / length - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def turn_halves(x, positions, freq, dims):
    """x [n, heads, size]: entry i < dims/2 is paired with entry i + dims/2, the pair turned by
    position * freq[i]; entries from `dims` on stay."""
    half = dims // 2
    angle = positions.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def causal_softmax_attention(q, k, v, scale, softcap=None):
    """One head: q [n, d], k [n, d], v [n, dv]; key j is seen by query i when j <= i."""
    n = q.shape[0]
    s = (q @ k.T) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    p = torch.arange(n)
    s = s.masked_fill(p[None, :] > p[:, None], -math.inf)
    return torch.softmax(s, -1) @ v


def attention(t: Dict[str, torch.Tensor], p: str, m, h, eps, kind: str, v_first: Optional[torch.Tensor]):
    """Returns (the mixer's output, the values it used [n, G, dv]).  `v_first` is what the first
    value-mixing layer used (None in that layer itself and in layers that do not mix)."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).view(n, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).view(n, G, d)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).view(n, G, dv)
    if kind == "attention":
        q = norm_plain_weight(q, t[p + "q.norm"], eps)
        k = norm_plain_weight(k, t[p + "k.norm"], eps)
    pos = torch.arange(n)
    freq = frequencies(m["rot"])
    q = turn_halves(q, pos, freq, m["rot"]["dims"])
    k = turn_halves(k, pos, freq, m["rot"]["dims"])
    if v_first is not None:
        lam = t[p + "vmix"].to(F64).reshape(())
        v = (1.0 - lam) * v + lam * v_first
    cap = m.get("softcap")
    outs = []
    for head in range(H):
        g = head // (H // G)
        outs.append(causal_softmax_attention(q[:, head], k[:, g], v[:, g], m["scale"], cap))
    return torch.cat(outs, -1) @ t[p + "o"].T, v


def short_convolution(u, w, b):
    """u [n, channels]; w [channels, taps] whose last column meets the current token; zeros before
    the start."""
    n, taps = u.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    out = b[None, :].expand(n, -1).clone()
    for j in range(taps):
        out = out + padded[j: j + n] * w[:, j][None, :]
    return out


def mamba2(t: Dict[str, torch.Tensor], p: str, m, h, eps):
    n = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ t[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner: 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, t[p + "conv"], t[p + "conv.b"]))
    x = xbc[:, :inner].view(n, H, P)
    B = xbc[:, inner: inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = softplus(dt + t[p + "dt_bias"])
    decay = torch.exp(-torch.exp(t[p + "A_log"])[None, :] * dt)
    y = torch.zeros(n, H, P, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for i in range(n):
            S = decay[i, head] * S + dt[i, head] * torch.outer(B[i, g], x[i, head])
            y[i, head] = S.T @ C[i, g] + t[p + "D"][head] * x[i, head]
    y = y.reshape(n, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * t[p + "norm"]
    return y @ t[p + "o"].T


def route(t: Dict[str, torch.Tensor], p: str, r, h, margins: Optional[list] = None):
    """Returns (ids [n, top], weights [n, top]); ids from `experts` on are identity experts.  `margins`
    receives, per token, how far the last group kept lies above the first one barred, and the last expert
    chosen above the first one left out (infinite where there is no such pair)."""
    z = h @ t[p + "router"].T
    s = torch.softmax(z, -1)
    choice = s + t[p + "correction"]
    total = r["experts"] + (r.get("identity") or 0)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    best = choice.view(-1, count, total // count).max(-1).values
    ranked = best.sort(-1, descending=True).values
    kept = torch.zeros_like(best, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, -1).indices, True)
    allowed = kept[:, :, None].expand(-1, -1, total // count).reshape(-1, total)
    choice = choice.masked_fill(~allowed, -math.inf)
    ids = choice.topk(r["top"], -1).indices
    if margins is not None:
        inf = torch.full((h.shape[0],), math.inf, dtype=F64)
        order = choice.sort(-1, descending=True).values
        margins.append(ranked[:, keep - 1] - ranked[:, keep] if keep < count else inf)
        margins.append(torch.nan_to_num(order[:, r["top"] - 1] - order[:, r["top"]], nan=math.inf, posinf=math.inf)
                       if r["top"] < total else inf)
    return ids, s.gather(1, ids)


def expert(t, p: str, e: int, h):
    return torch.relu(h @ t[f"{p}e{e}.up"].T) ** 2 @ t[f"{p}e{e}.down"].T


def mixture(t: Dict[str, torch.Tensor], p: str, mlp, h, margins: Optional[list] = None):
    r = mlp["router"]
    ids, weights = route(t, p, r, h, margins)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e, w in zip(ids[i].tolist(), weights[i]):
            out[i] += w * (h[i] if e >= r["experts"] else expert(t, p, e, h[i][None, :])[0])
    return out


def residual_gate(t, name: str, h):
    return torch.sigmoid(h @ t[name].T + t[name + ".b"])


def forward(config, tensors: Dict[str, torch.Tensor], tokens: List[int], collect: Optional[list] = None,
            margins: Optional[list] = None):
    """Logits [n, vocab] of one sequence; `collect` receives the stream after every layer, `margins` the
    routers' margins (see `route`)."""
    t = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = norm_around_zero(t["embed"][torch.tensor(tokens)], t["embed.norm"], eps)
    history = [x]
    v_first = None
    seen_first = False
    for i, layer in enumerate(config["layers"]):
        name = f"l{i}."
        m = layer["mixer"]
        h = norm_around_zero(x, t[name + "norm1"], eps)
        if layer["type"] == "mamba2":
            y = mamba2(t, name + "mix.", m, h, eps)
        else:
            mixes = bool(m.get("v_mix"))
            y, v = attention(t, name + "mix.", m, h, eps, layer["type"], v_first if (mixes and seen_first) else None)
            if mixes and not seen_first:
                v_first, seen_first = v, True
        x = x + norm_around_zero(y * residual_gate(t, name + "rg1", h), t[name + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = norm_around_zero(x, t[name + "norm2"], eps)
            y = mixture(t, name + "mlp.", layer["mlp"], h, margins)
            x = x + norm_around_zero(y * residual_gate(t, name + "rg2", h), t[name + "norm2b"], eps)
        history.append(x)
        w = t[name + "dwa"]
        x = sum(w[j] * history[j] for j in range(len(history)))
        if collect is not None:
            collect.append(x)
    return norm_around_zero(x, t["final.norm"], eps) @ t["head"].T
