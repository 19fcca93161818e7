"""The Pudulorn decoder laid out as parts.

Every layer is a pre-norm block, x += mixer(norm(x)) and then, where it has one, x += ff(norm(x)),
with RMS norms whose weight is stored around zero (the factor is 1 + w).  Mixers, by the layer's
`type`: "attention" (differential attention: two softmax maps per head over the same values, the
second subtracted times lambda; per-map norms of queries and keys; rotation of the first entries of
a map in halves; keys seen in blocks of `mask.size` positions counted from the sequence's first; a
unit norm per head and a sigmoid gate on the output) and "latent_attention" (queries through a
normed latent; keys and values of all heads expanded from one cached latent vector, a rotated key
part shared by the heads; a window of the last `mask.size` positions; with `kv_from` the layer
reads the latent an earlier layer cached and has no compression of its own).  Feed-forwards:
"dense" (a gated one with clamped gate and up, g sigmoid(1.702 g) (u + 1)) and "moe" (routed
experts with a softmax router, plus a gated shared expert).

Tensor names: `embed`, `final.norm`, `head`, and per layer i `l<i>.norm1|norm2`, `l<i>.mix.*`,
`l<i>.mlp.gate|up|down` or `l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`, `l<i>.mlp.shared.gate|up|down|sg`.
"""

from __future__ import annotations

from ..config.pudulorn import PudulornConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

SWISH_ALPHA = 1.702      # the dense feed-forward's gate is g * sigmoid(1.702 g)


def _rotation(rot) -> PartSpec:
    return PartSpec("rotary_halves", {"dims": rot["dims"], "base": rot["base"]})


def _mask_size(m):
    return m["mask"]["size"] if m.get("mask") is not None else None


def _attention(cfg: PudulornConfig, m, p: str, extra) -> PartSpec:
    return PartSpec("differential_attention",
                    {"hidden": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                     "v_dim": m["vdim"], "chunk": _mask_size(m), "window": None, "scale": m["scale"],
                     "eps": cfg.norm_eps, "lambda_init": m["diff"], "out_scale": 1.0 - m["diff"], "gate": True,
                     "position": _rotation(m["rot"])},
                    {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "o": p + "o", "q_norm": p + "q.norm",
                     "k_norm": p + "k.norm", "lq1": p + "lq1", "lk1": p + "lk1", "lq2": p + "lq2", "lk2": p + "lk2"})


def _latent(cfg: PudulornConfig, m, p: str, extra) -> PartSpec:
    borrows = m.get("kv_from") is not None
    names = {"dq": p + "dq", "dq_norm": p + "dq.norm", "uq": p + "uq", "uk": p + "uk", "uv": p + "uv", "o": p + "o"}
    if not borrows:
        names.update({"dkv": p + "dkv", "dkv_norm": p + "dkv.norm"})
    return PartSpec("latent_attention",
                    {"hidden": cfg.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                     "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"], "eps": cfg.norm_eps,
                     "sink": False, "gate": False, "borrows": borrows, "window": _mask_size(m),
                     "cache_window": extra["cache_window"], "position": _rotation(m["rot"])}, names)


_MIXERS = {"attention": _attention, "latent_attention": _latent}


def _feed_forward(cfg: PudulornConfig, mlp, p: str) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("glu", {"hidden": cfg.width, "intermediate": mlp["ff"], "activation": "clamped_swish",
                                "limit": mlp["limit"], "alpha": SWISH_ALPHA},
                        {"gate": p + "gate", "up": p + "up", "down": p + "down"})
    r, shared = mlp["router"], mlp.get("shared")
    names = {"router": p + "router"}
    for e in range(r["experts"]):
        names.update({f"e{e}.{t}": f"{p}e{e}.{t}" for t in ("gate", "up", "down")})
    if shared is not None:
        names.update({f"shared.{t}": f"{p}shared.{t}" for t in ("gate", "up", "down", "sg")})
    return PartSpec("moe", {"hidden": cfg.width, "experts": r["experts"], "top": r["top"], "router_scale": r["scale"],
                            "intermediate": mlp["expert"]["ff"],
                            "shared_intermediate": shared["ff"] if shared is not None else None,
                            "shared_gate": shared is not None}, names)


def pudulorn_spec(cfg: PudulornConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "one_plus": True}, {"weight": name})

    # a cached latent must outlive the widest window among the layers that read it
    reach = {}
    for i, layer in enumerate(cfg.layers):
        if layer["type"] == "latent_attention":
            src = layer["mixer"].get("kv_from")
            src = i if src is None else src
            size = _mask_size(layer["mixer"])
            reach[src] = None if (size is None or reach.get(src, 0) is None) else max(reach.get(src, 0), size)
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        name = f"l{i}"
        mlp = layer.get("mlp")
        m = layer["mixer"]
        extra = {"cache_window": reach.get(m.get("kv_from") if m.get("kv_from") is not None else i)}
        layers.append(LayerSpec(
            mixer_norm=norm(name + ".norm1"),
            mixer=_MIXERS[layer["type"]](cfg, m, name + ".mix.", extra),
            ffn_norm=norm(name + ".norm2") if mlp is not None else None,
            ffn=_feed_forward(cfg, mlp, name + ".mlp.") if mlp is not None else None,
            block="prenorm"))
        order.append(LayerCall(i, cache_from=m.get("kv_from") if layer["type"] == "latent_attention" else None))
    sizes = {"vocab": cfg.vocab, "hidden": cfg.width}
    return ModelSpec(
        architecture=PudulornConfig.ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=None,
        embed=PartSpec("table", sizes, {"weight": "embed"}),
        layers=layers, order=order, final_norm=norm("final.norm"), head=PartSpec("linear", sizes, {"weight": "head"}))


register_architecture(PudulornConfig.ARCHITECTURE, PudulornConfig, pudulorn_spec)
