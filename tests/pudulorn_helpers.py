"""Small Pudulorn configurations with random weights made here (names and shapes written out from
the configuration, independent of the engine's own list), their model folders, and the comparison
of replayed logits with the plain implementation."""

from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import torch

import helpers as H
import plain_pudulorn as P


def dense(ff, limit=1.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, scale=1.0, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def attention(heads, kv_heads, dim, vdim, chunk, rot_dims, diff=0.5, base=10000.0, scale=None, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "mask": {"size": chunk},
                      "rot": {"base": base, "dims": rot_dims}, "scale": dim ** -0.5 if scale is None else scale}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, scale=None, base=10000.0, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim},
         "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mlp": mlp, "mixer": m}


def _cfg_p():
    layers = [attention(4, 2, 16, 24, 24, 8, diff=0.3, mlp=dense(80, 2.0)),
              latent(3, 12, 8, 20, 24, 40, 17, scale=0.2, base=5000.0, mlp=moe(5, 2, 24, 1.5, shared=40)),
              latent(2, 8, 8, 12, 24, 16, 30, base=5000.0, kv_from=1),            # a wider window than the layer it reads from
              attention(2, 2, 8, 8, 7, 8, diff=0.8, base=300.0, scale=0.3, mlp=moe(3, 1, 32)),   # one expert a token, no shared one
              latent(5, 4, 8, 4, 24, 8, 9, scale=0.4, base=5000.0, kv_from=1, mlp=dense(48, 0.5))]
    return {"architecture": "Pudulorn", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "layers": layers}


def _cfg_q():
    layers = [latent(2, 24, 16, 8, 64, 32, 40, scale=0.15, base=100.0, mlp=dense(64, 3.0)),
              attention(6, 1, 32, 64, 1000, 2, diff=0.1, mlp=moe(4, 4, 16, 0.5, shared=16)),   # a block wider than any request; all experts
              latent(5, 16, 4, 16, 32, 16, 1, base=20.0),                                       # a window of the token itself
              latent(1, 40, 16, 32, 64, 48, 64, base=100.0, kv_from=0, mlp=moe(9, 3, 8, 2.0, shared=24)),
              attention(3, 3, 64, 32, 33, 64, diff=0.6, base=500.0, scale=0.1, mlp=dense(72, 1.0))]
    return {"architecture": "Pudulorn", "vocab": 77, "width": 96, "norm": {"eps": 1e-6}, "layers": layers}


CFG_P, CFG_Q = _cfg_p(), _cfg_q()
CONFIGS = {"P": (CFG_P, 16), "Q": (CFG_Q, 32)}


def tensor_shapes(cfg) -> Dict[str, Tuple[int, ...]]:
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (W,)
        if layer["type"] == "attention":
            n, g, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (n * 2 * d, W), p + "mix.k": (g * 2 * d, W), p + "mix.v": (g * e, W),
                        p + "mix.q.norm": (d,), p + "mix.k.norm": (d,), p + "mix.lq1": (d,), p + "mix.lk1": (d,),
                        p + "mix.lq2": (d,), p + "mix.lk2": (d,), p + "mix.g": (n * e, W), p + "mix.o": (W, n * e)})
        else:
            n, d, r, e, k, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (n * (d + r), qr),
                        p + "mix.uk": (n * d, k), p + "mix.uv": (n * e, k), p + "mix.o": (W, n * e)})
            if m.get("kv_from") is None:
                out.update({p + "mix.dkv": (k + r, W), p + "mix.dkv.norm": (k,)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)

        def gated(q, ff):
            out.update({q + "gate": (ff, W), q + "up": (ff, W), q + "down": (W, ff)})

        if mlp["kind"] == "dense":
            gated(p + "mlp.", mlp["ff"])
        else:
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                gated(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            if mlp.get("shared") is not None:
                gated(p + "mlp.shared.", mlp["shared"]["ff"])
                out[p + "mlp.shared.sg"] = (1, W)
    return out


def random_tensors(cfg, seed: int) -> Dict[str, torch.Tensor]:
    """Values of a size that keeps every activation of order one; bfloat16, as files store them."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        x = torch.randn(shape, generator=g)
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            x = 0.2 * x                                   # stored around zero
        elif last == "norm":
            x = 1.0 + 0.2 * x
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            x = 0.4 * x
        elif last == "router":
            x = 3.0 * x / shape[1] ** 0.5
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
def model_folder(name: str, seed: int = 3):
    cfg, _page = CONFIGS[name]
    folder = H.tmp_root() / f"pudulorn{name}-{seed}"
    register(folder, cfg, random_tensors(cfg, seed))
    return folder


def register(folder, cfg, tensors) -> None:
    write_folder(folder, cfg, tensors)
    _tensors[str(folder)] = tensors


# Per logits row: max |got - want| / max |want| against the float64 plain implementation.  A logic
# fault (a key, a block's or a window's edge, an expert or a cached latent lost or shifted) shows at 1e-2
# and more in float32, where every row has to be within the tolerance.  In bfloat16 single rows are
# ill-conditioned: the router reads a rounded input, so a close second choice can go to another expert,
# and the unit norm behind the difference of the two maps enlarges rounding where the maps nearly
# cancel.  So a bfloat16 run has to have `BF16_SHARE` of its rows within the tolerance and none beyond
# `BF16_WORST`.
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}
BF16_SHARE, BF16_WORST = 0.95, 0.6

_plain: Dict[Tuple, torch.Tensor] = {}


def plain_logits(folder, ids: Sequence[int]) -> torch.Tensor:
    key = (str(folder), tuple(ids))
    if key not in _plain:
        cfg = json.loads((folder / "config.json").read_text())
        _plain[key] = P.forward(cfg, _tensors[str(folder)], list(ids))
    return _plain[key]


CLEAR_MARGIN = 1e-3


def clear_ids(folder, rng, n: int, vocab: int) -> List[int]:
    """`n` random ids on which no router of the model in `folder` makes a close call: where the last chosen
    expert's score lies within `CLEAR_MARGIN` (relative) of the first one left out, float32 rounding may
    choose the other, which is no fault; such a draw is thrown away and the next one taken."""
    cfg = json.loads((folder / "config.json").read_text())
    for _ in range(50):
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
