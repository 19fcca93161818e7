"""The Gurolix decoder laid out as parts.

The embedding is RMS-normed.  Every layer norms on both sides of each sublayer, multiplies a sublayer's
result by sigmoid(W_g h + b_g) of the sublayer's own input first, and hands a weighted sum of all layers'
results so far (the embedding's output included) on to the next layer (block "gated_sandwich"); all norm
weights are stored around zero (the factor is 1 + w).  Mixers, by the layer's `type`: "attention"
(grouped-query softmax attention with biased projections, per-head norms of queries and keys, rotation
of a head's first entries in halves), "attention_2" (the same without the norms, with the rotation's
frequencies rescaled by wavelength and a tanh cap on the scores) and "mamba2"; attention layers that
say `v_mix` blend their values with those of the first such layer.  The feed-forward is a mixture of
ungated experts W_down relu(W_up h)^2 with identity experts, a correction for the choice and a limit
to the best groups of experts.

Tensor names: `embed`, `embed.norm`, `final.norm`, `head`, and per layer i `l<i>.norm1|norm2|norm1b|norm2b`,
`l<i>.rg1|rg2` (+ `.b`), `l<i>.dwa`, `l<i>.mix.*`, `l<i>.mlp.router|correction`, `l<i>.mlp.e<j>.up|down`.
"""

from __future__ import annotations

from ..config.gurolix import GurolixConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _attention(cfg: GurolixConfig, m, p: str, second: bool, v_mix) -> PartSpec:
    rot = m["rot"]
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_bias": p + "q.b", "k_bias": p + "k.b",
             "v_bias": p + "v.b"}
    if not second:
        names.update({"q_norm": p + "q.norm", "k_norm": p + "k.norm"})
    if v_mix is not None:
        names["v_lambda"] = p + "vmix"
    return PartSpec("general_attention",
                    {"hidden": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                     "scale": m["scale"], "eps": cfg.norm_eps, "bias": True, "qk_norm": not second,
                     "softcap": m.get("softcap"), "window": None, "v_mix": v_mix,
                     "position": PartSpec("rotary_halves", {"dims": rot["dims"], "base": rot["base"],
                                                            "scaling": rot.get("scaling")})}, names)


def _mamba2(cfg: GurolixConfig, m, p: str) -> PartSpec:
    return PartSpec("mamba2", {"hidden": cfg.width, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"],
                               "groups": m["groups"], "taps": m["conv"], "norm_groups": m["norm_groups"], "eps": cfg.norm_eps},
                    {"in": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
                     "A_log": p + "A_log", "D": p + "D", "norm": p + "norm", "o": p + "o"})


def _feed_forward(cfg: GurolixConfig, mlp, p: str) -> PartSpec:
    r = mlp["router"]
    names = {"router": p + "router", "correction": p + "correction"}
    for e in range(r["experts"]):
        names.update({f"e{e}.{t}": f"{p}e{e}.{t}" for t in ("up", "down")})
    g = r.get("groups") or {}
    return PartSpec("moe", {"hidden": cfg.width, "experts": r["experts"], "top": r["top"], "router_scale": 1.0,
                            "intermediate": mlp["expert"]["ff"], "shared_intermediate": None, "shared_gate": False,
                            "expert_form": "relu2", "identity": r.get("identity") or 0, "correction": True,
                            "groups": g.get("count"), "keep": g.get("keep")}, names)


def gurolix_spec(cfg: GurolixConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("gated_sandwich_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "one_plus": True}, {"weight": name})

    def gate(name):
        return PartSpec("residual_gate", {"size": cfg.width}, {"weight": name, "bias": name + ".b"})

    layers, order = [], []
    source_seen = False
    for i, layer in enumerate(cfg.layers):
        name = f"l{i}"
        m, mlp = layer["mixer"], layer.get("mlp")
        if layer["type"] == "mamba2":
            mixer = _mamba2(cfg, m, name + ".mix.")
        else:
            v_mix = None
            if m.get("v_mix"):
                v_mix, source_seen = ("mix" if source_seen else "source"), True
            mixer = _attention(cfg, m, name + ".mix.", layer["type"] == "attention_2", v_mix)
        extras = {"post1": norm(name + ".norm1b"), "gate1": gate(name + ".rg1"),
                  "depth": PartSpec("depth_average", {"index": i, "entries": len(cfg.layers) + 1, "size": cfg.width},
                                    {"weights": name + ".dwa"})}
        if mlp is not None:
            extras.update({"post2": norm(name + ".norm2b"), "gate2": gate(name + ".rg2")})
        layers.append(LayerSpec(
            mixer_norm=norm(name + ".norm1"), mixer=mixer,
            ffn_norm=norm(name + ".norm2") if mlp is not None else None,
            ffn=_feed_forward(cfg, mlp, name + ".mlp.") if mlp is not None else None,
            block="gated_sandwich", extras=extras))
        order.append(LayerCall(i))
    sizes = {"vocab": cfg.vocab, "hidden": cfg.width}
    return ModelSpec(
        architecture=GurolixConfig.ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=None,
        embed=PartSpec("table_norm", dict(sizes, eps=cfg.norm_eps, one_plus=True), {"weight": "embed", "norm": "embed.norm"}),
        layers=layers, order=order, final_norm=norm("final.norm"), head=PartSpec("linear", sizes, {"weight": "head"}))


register_architecture(GurolixConfig.ARCHITECTURE, GurolixConfig, gurolix_spec)
