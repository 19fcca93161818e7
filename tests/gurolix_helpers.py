"""Small Gurolix configurations with random weights made here (names and shapes written out from
the configuration, independent of the engine's own list), their model folders, and the comparison
of replayed logits with the plain implementation."""

from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import torch

import helpers as H
import plain_gurolix as P


def moe(experts, top, ff, identity=0, groups=None):
    r = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def attention(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, scale=None, v_mix=False, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix,
                      "rot": {"base": base, "dims": rot_dims}, "scale": dim ** -0.5 if scale is None else scale}}


def attention_2(heads, kv_heads, dim, vdim, rot_dims, softcap, scaling, base=10000.0, scale=None, v_mix=False, mlp=None):
    """`scaling` = (factor, low, high, original)."""
    rot = {"base": base, "dims": rot_dims,
           "scaling": dict(zip(("factor", "low", "high", "original"), scaling))}
    return {"type": "attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix, "softcap": softcap,
                      "rot": rot, "scale": dim ** -0.5 if scale is None else scale}}


def mamba2(heads, vdim, state, groups, conv, norm_groups, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def _cfg_a():
    layers = [mamba2(4, 8, 16, 2, 4, 4, mlp=moe(5, 2, 24, identity=1, groups=(3, 2))),
              attention_2(4, 2, 16, 24, 8, 5.0, (8.0, 1.0, 4.0, 64), scale=0.3, v_mix=True, mlp=moe(6, 3, 16, identity=3, groups=(3, 2))),
              attention(4, 2, 32, 24, 32, base=500.0, scale=0.2, v_mix=True),                       # no feed-forward
              attention_2(2, 1, 24, 8, 24, 2.0, (2.0, 2.0, 8.0, 32), base=100.0, mlp=moe(4, 1, 40)),   # mixes no values; plain router
              mamba2(2, 16, 8, 1, 2, 1),
              attention(2, 2, 8, 24, 4, scale=0.5, v_mix=True, mlp=moe(3, 3, 8, identity=5, groups=(4, 3)))]
    return {"architecture": "Gurolix", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "layers": layers}


def _cfg_b():
    # what another model makes equal or 1: key and value heads of one size, every head its own keys, one key
    # head for all, a group of B and C per head, one part for the norm, a convolution of one tap, one choice
    layers = [attention(3, 3, 32, 32, 16, base=50.0, v_mix=True, mlp=moe(2, 1, 48, identity=2, groups=(2, 1))),
              mamba2(3, 32, 24, 3, 1, 1, mlp=moe(7, 2, 16, identity=1, groups=(1, 1))),
              attention_2(6, 1, 16, 16, 16, 50.0, (4.0, 1.0, 2.0, 16), base=20.0, scale=0.4, mlp=moe(5, 5, 8)),   # all experts
              mamba2(6, 16, 40, 2, 5, 3, mlp=moe(9, 4, 24, identity=3, groups=(6, 3))),
              attention_2(3, 3, 64, 32, 2, 10.0, (16.0, 0.5, 3.0, 100), scale=0.1, v_mix=True)]
    return {"architecture": "Gurolix", "vocab": 131, "width": 96, "norm": {"eps": 1e-6}, "layers": layers}


CFG_A, CFG_B = _cfg_a(), _cfg_b()
CONFIGS = {"A": (CFG_A, 16), "B": (CFG_B, 32)}


def every_expert_chosen(cfg):
    """The same model with routers that choose every expert (identity experts included) and bar no group.
    A router's choice is a discontinuity: where two choice values nearly tie, the rounding of a bfloat16
    run picks the other expert and the row moves by a whole expert's result, which says nothing about the
    kernels.  bfloat16 runs are therefore compared on this variant, whose logits are continuous in every
    rounding error, with the same tensors; the choice itself is compared in float32, where a tie within
    rounding is rare enough to be drawn around (`clear_ids`)."""
    import copy
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer.get("mlp") is not None:
            r = layer["mlp"]["router"]
            r["top"] = r["experts"] + (r.get("identity") or 0)
            r.pop("groups", None)
    return out


def config_for(name: str, dtype: str):
    cfg, page = CONFIGS[name]
    return (every_expert_chosen(cfg) if dtype == "bfloat16" else cfg), page


def tensor_shapes(cfg) -> Dict[str, Tuple[int, ...]]:
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "embed.norm": (W,), "final.norm": (W,), "head": (cfg["vocab"], W)}
    mixes = False
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out.update({p + "norm1": (W,), p + "norm1b": (W,), p + "rg1": (W, W), p + "rg1.b": (W,), p + "dwa": (i + 2,)})
        if layer["type"] == "mamba2":
            H_, P_, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            ch = H_ * P_ + 2 * G * N
            out.update({p + "mix.in": (H_ * P_ + ch + H_, W), p + "mix.conv": (ch, m["conv"]), p + "mix.conv.b": (ch,),
                        p + "mix.dt_bias": (H_,), p + "mix.A_log": (H_,), p + "mix.D": (H_,), p + "mix.norm": (H_ * P_,),
                        p + "mix.o": (W, H_ * P_)})
        else:
            n, g, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (n * d, W), p + "mix.q.b": (n * d,), p + "mix.k": (g * d, W), p + "mix.k.b": (g * d,),
                        p + "mix.v": (g * e, W), p + "mix.v.b": (g * e,), p + "mix.o": (W, n * e)})
            if layer["type"] == "attention":
                out.update({p + "mix.q.norm": (d,), p + "mix.k.norm": (d,)})
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
        mlp = layer["mlp"]
        if mlp is None:
            continue
        r = mlp["router"]
        total = r["experts"] + (r.get("identity") or 0)
        out.update({p + "norm2": (W,), p + "norm2b": (W,), p + "rg2": (W, W), p + "rg2.b": (W,),
                    p + "mlp.router": (total, W), p + "mlp.correction": (total,)})
        for e in range(r["experts"]):
            out.update({f"{p}mlp.e{e}.up": (mlp["expert"]["ff"], W), f"{p}mlp.e{e}.down": (W, mlp["expert"]["ff"])})
    return out


def random_tensors(cfg, seed: int) -> Dict[str, torch.Tensor]:
    """Values of a size that keeps every activation of order one; bfloat16, as files store them."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        x = torch.randn(shape, generator=g)
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b") or name in ("final.norm", "embed.norm"):
            x = 0.2 * x                                   # stored around zero
        elif last == "norm":
            x = 1.0 + 0.2 * x
        elif last == "b":
            x = 0.3 * x
        elif last == "dwa":
            x = 0.3 * x
            x[-1] += 1.0                                  # mostly the layer's own result, some of every earlier one
        elif last == "vmix":
            x = 0.4 + 0.1 * x
        elif last == "router":
            x = 3.0 * x / shape[1] ** 0.5
        elif last == "correction":
            x = 0.1 * x
        elif last == "conv":
            x = x / shape[1] ** 0.5
        elif last == "A_log":
            x = 0.5 * x - 1.0
        elif last == "D":
            x = 1.0 + 0.3 * x
        elif len(shape) == 2 and name != "embed":
            x = x / shape[1] ** 0.5
        out[name] = x.to(torch.bfloat16)
    return out


def write_folder(folder, cfg, tensors) -> None:
    from bare_cuda_4gib_b200.weights.safetensors_io import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    write_safetensors(folder / "model.safetensors", tensors)
    (folder / "config.json").write_text(json.dumps(cfg))


_tensors: Dict[str, Dict[str, torch.Tensor]] = {}


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 3, dtype: str = "float32"):
    """The folder of configuration `name`; for bfloat16 runs the variant whose routers choose every expert."""
    cfg, _page = config_for(name, dtype)
    folder = H.tmp_root() / f"gurolix{name}-{seed}-{dtype}"
    register(folder, cfg, random_tensors(CONFIGS[name][0], seed))
    return folder


def register(folder, cfg, tensors) -> None:
    write_folder(folder, cfg, tensors)
    _tensors[str(folder)] = tensors


# Per logits row: max |got - want| / max |want| against the float64 plain implementation.  A logic
# fault (a key, a state, a tap of the convolution, an expert, a mixed value or a layer's share of the
# depth sum lost or shifted) shows at 1e-2 and more in float32, where every row has to be within the
# tolerance.  In bfloat16 single rows are ill-conditioned (the router reads a rounded input, so a close
# second choice can go to another expert): a bfloat16 run has to have `BF16_SHARE` of its rows within the
# tolerance and none beyond `BF16_WORST`.
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}
BF16_SHARE, BF16_WORST = 0.95, 0.6

_plain: Dict[Tuple, torch.Tensor] = {}


def plain_logits(folder, ids: Sequence[int]) -> torch.Tensor:
    key = (str(folder), tuple(ids))
    if key not in _plain:
        cfg = json.loads((folder / "config.json").read_text())
        _plain[key] = P.forward(cfg, _tensors[str(folder)], list(ids))
    return _plain[key]


CLEAR_MARGIN = 2e-4


def clear_ids(folder, rng, n: int, vocab: int) -> List[int]:
    """`n` random ids on which no router of the model in `folder` makes a close call: where the last group
    kept or the last expert chosen lies within `CLEAR_MARGIN` of the first one left out, float32 rounding may
    choose the other, which is no fault; such a draw is thrown away and the next one taken."""
    cfg = json.loads((folder / "config.json").read_text())
    for _ in range(200):
        ids = H.random_ids(rng, n, vocab)
        margins: list = []
        logits = P.forward(cfg, _tensors[str(folder)], ids, None, margins)
        if all(float(m.min()) > CLEAR_MARGIN for m in margins):
            _plain[(str(folder), tuple(ids))] = logits
            return ids
    raise AssertionError("no draw without a close call of a router")


def check(folder, requests: Dict[str, List[int]], got, dtype: str, expect_all: bool = True) -> None:
    errors = []
    for rid, ids in requests.items():
        want = plain_logits(folder, ids)
        places = sorted(p for (r, p) in got if r == rid)
        if expect_all:
            assert places == list(range(len(ids))), f"request {rid}: places {places}"
        for p in places:
            err = H.row_error(got[(rid, p)], want[p])
            errors.append(err)
            if dtype == "float32":
                assert err <= TOLERANCE[dtype], f"request {rid} position {p} of {len(ids)}: error {err:.3e}"
    if dtype != "float32":
        errors.sort()
        over = sum(e > TOLERANCE[dtype] for e in errors)
        assert errors[-1] <= BF16_WORST, f"worst row: error {errors[-1]:.3e}"
        assert over <= (1.0 - BF16_SHARE) * len(errors) or over <= 1, \
            f"{over} of {len(errors)} rows beyond {TOLERANCE[dtype]:.0e}: {errors[-5:]}"
