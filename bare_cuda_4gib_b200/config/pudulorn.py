"""Typed configuration of the Pudulorn decoder, read from its own `config.json` layout:

    architecture, vocab, width, norm.eps,
    layers: [{type: "attention" | "latent_attention", mixer: {...}, mlp: {...} | null}, ...]

    attention mixer:         heads, kv_heads, dim, vdim, diff, scale, mask.size, rot.{dims, base}
    latent_attention mixer:  heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask.size, rot.{dims, base},
                             kv_from (optional: the earlier layer whose cached latent this one reads)
    mlp, dense:              kind "dense", ff, limit
    mlp, mixture of experts: kind "moe", expert.ff, router.{experts, top, scale}, shared.ff (optional)

Every size and every constant that may differ between models of the design is read here and
nowhere else; a key that is wrong or missing is named in the error.  The design states no largest
position: a request is as long as the cache pool lets it be.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from ..errors import ConfigError
from .dopudra import _get

MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _rotation(rot, where: str, most: int) -> None:
    dims = _get(rot, "dims", where)
    _get(rot, "base", where, float)
    if dims % 2:
        raise ConfigError(f"config.json: '{where}dims' must be even (entries are turned in pairs), got {dims}")
    if dims > most:
        raise ConfigError(f"config.json: '{where}dims' {dims} exceeds the {most} entries it is applied to")


def _mask(m, where: str) -> None:
    if m.get("mask") is not None:
        _get(m.get("mask"), "size", where + "mask.")


def _attention(m, where: str, layers, i) -> None:
    heads, kv = _get(m, "heads", where), _get(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: '{where}heads' {heads} is not a multiple of '{where}kv_heads' {kv}")
    dim = _get(m, "dim", where)
    _get(m, "vdim", where)
    _get(m, "scale", where, float)
    _get(m, "diff", where, float, positive=False)
    _mask(m, where)
    _rotation(m.get("rot"), where + "rot.", dim)


def _latent(m, where: str, layers, i) -> None:
    for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
        _get(m, key, where)
    _get(m, "scale", where, float)
    _mask(m, where)
    _rotation(m.get("rot"), where + "rot.", m["rot_dim"])
    src = m.get("kv_from")
    if src is not None:
        if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < i):
            raise ConfigError(f"config.json: '{where}kv_from' must name an earlier layer, got {src!r}")
        other = layers[src]
        om = other.get("mixer") if isinstance(other, dict) else None
        if not isinstance(other, dict) or other.get("type") != "latent_attention" or not isinstance(om, dict) \
                or om.get("kv_from") is not None:
            raise ConfigError(f"config.json: '{where}kv_from' names layer {src}, which caches no latent of its own")
        for key in ("kv_rank", "rot_dim"):
            if om.get(key) != m[key]:
                raise ConfigError(f"config.json: '{where}{key}' {m[key]} differs from layer {src}'s, whose cache it reads")
        if om.get("rot") != m["rot"]:
            raise ConfigError(f"config.json: '{where}rot' differs from layer {src}'s, whose cache it reads")


def _mlp(mlp, where: str) -> None:
    if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"config.json: '{where}kind' must be one of {list(MLP_KINDS)} (or 'mlp' null)")
    if mlp["kind"] == "dense":
        _get(mlp, "ff", where)
        _get(mlp, "limit", where, float)
        return
    _get(mlp.get("expert"), "ff", where + "expert.")
    r = mlp.get("router")
    experts, top = _get(r, "experts", where + "router."), _get(r, "top", where + "router.")
    _get(r, "scale", where + "router.", float)
    if top > experts:
        raise ConfigError(f"config.json: '{where}router.top' {top} exceeds '{where}router.experts' {experts}")
    if mlp.get("shared") is not None:
        _get(mlp["shared"], "ff", where + "shared.")


_CHECKS = {"attention": _attention, "latent_attention": _latent}


@dataclass
class PudulornConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]] = field(default_factory=list)
    norm_eps: float = 1e-6

    ARCHITECTURE = "Pudulorn"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PudulornConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=_get(d, "vocab", ""), width=_get(d, "width", ""), layers=copy.deepcopy(layers),
                  norm_eps=_get(d.get("norm"), "eps", "norm.", float))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}type' must be one of {list(MIXER_TYPES)}, "
                                  f"got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            if not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"config.json: required key '{where}mixer' is missing")
            _CHECKS[layer["type"]](layer["mixer"], where + "mixer.", self.layers, i)
            if layer.get("mlp") is not None:
                _mlp(layer["mlp"], where + "mlp.")

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        return {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}

    # the names the command line tools read from any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def stop_ids(self) -> List[int]:
        return []
