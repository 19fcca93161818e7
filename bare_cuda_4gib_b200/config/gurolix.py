"""Typed configuration of the Gurolix decoder, read from its own `config.json` layout:

    architecture, vocab, width, norm.eps,
    layers: [{type: "attention" | "attention_2" | "mamba2", mixer: {...}, mlp: {...} | null}, ...]

    attention mixer:    heads, kv_heads, dim, vdim, scale, v_mix, rot.{dims, base}
                        (queries and keys are normed per head)
    attention_2 mixer:  heads, kv_heads, dim, vdim, scale, softcap, v_mix, rot.{dims, base,
                        scaling.{factor, low, high, original}}  (no norms)
                        (`softcap` and `rot.scaling` are applied wherever an attention mixer states them)
    mamba2 mixer:       heads, vdim, state, groups, conv, norm_groups
    mlp:                kind "moe", expert.ff, router.{experts, top, identity, groups.{count, keep}}

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

MIXER_TYPES = ("attention", "attention_2", "mamba2")


def _rotation(rot, where: str, most: int) -> None:
    dims = _get(rot, "dims", where)
    _get(rot, "base", where, float)
    if dims % 2:
        raise ConfigError(f"config.json: '{where}dims' must be even (entries are turned in pairs), got {dims}")
    if dims > most:
        raise ConfigError(f"config.json: '{where}dims' {dims} exceeds the {most} entries it is applied to")
    sc = rot.get("scaling")
    if sc is not None:
        for key in ("factor", "low", "high", "original"):
            _get(sc, key, where + "scaling.", float)
        if not sc["high"] > sc["low"]:
            raise ConfigError(f"config.json: '{where}scaling.high' must exceed '{where}scaling.low'")


def _attention(m, where: str, second: bool) -> None:
    heads, kv = _get(m, "heads", where), _get(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: '{where}heads' {heads} is not a multiple of '{where}kv_heads' {kv}")
    dim = _get(m, "dim", where)
    _get(m, "vdim", where)
    _get(m, "scale", where, float)
    if m.get("softcap") is not None:
        _get(m, "softcap", where, float)
    if not isinstance(m.get("v_mix", False), bool):
        raise ConfigError(f"config.json: '{where}v_mix' must be true or false, got {m.get('v_mix')!r}")
    _rotation(m.get("rot"), where + "rot.", dim)


def _mamba2(m, where: str) -> None:
    heads, groups = _get(m, "heads", where), _get(m, "groups", where)
    if heads % groups:
        raise ConfigError(f"config.json: '{where}heads' {heads} is not a multiple of '{where}groups' {groups}")
    vdim = _get(m, "vdim", where)
    _get(m, "state", where)
    _get(m, "conv", where)
    parts = _get(m, "norm_groups", where)
    if (heads * vdim) % parts:
        raise ConfigError(f"config.json: '{where}norm_groups' {parts} does not divide heads * vdim = {heads * vdim}")


def _mlp(mlp, where: str) -> None:
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: '{where}kind' must be 'moe' (or 'mlp' null)")
    _get(mlp.get("expert"), "ff", where + "expert.")
    r = mlp.get("router")
    experts, top = _get(r, "experts", where + "router."), _get(r, "top", where + "router.")
    identity = r.get("identity") or 0
    if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
        raise ConfigError(f"config.json: '{where}router.identity' must be a count, got {identity!r}")
    outputs = experts + identity
    g = r.get("groups")
    allowed = outputs
    if g is not None:
        count, keep = _get(g, "count", where + "router.groups."), _get(g, "keep", where + "router.groups.")
        if outputs % count:
            raise ConfigError(f"config.json: '{where}router.groups.count' {count} does not divide the {outputs} router outputs")
        if keep > count:
            raise ConfigError(f"config.json: '{where}router.groups.keep' {keep} exceeds '{where}router.groups.count' {count}")
        allowed = keep * (outputs // count)
    if top > allowed:
        raise ConfigError(f"config.json: '{where}router.top' {top} exceeds the {allowed} experts that can be chosen")


@dataclass
class GurolixConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]] = field(default_factory=list)
    norm_eps: float = 1e-5

    ARCHITECTURE = "Gurolix"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GurolixConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=_get(d, "vocab", ""), width=_get(d, "width", ""), layers=copy.deepcopy(layers),
                  norm_eps=_get(d.get("norm"), "eps", "norm.", float))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        mixed = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}type' must be one of {list(MIXER_TYPES)}, "
                                  f"got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: required key '{where}mixer' is missing")
            if layer["type"] == "mamba2":
                _mamba2(m, where + "mixer.")
            else:
                _attention(m, where + "mixer.", layer["type"] == "attention_2")
                if m.get("v_mix"):
                    # mixed values are another layer's values of the same token: the layers' value sizes agree
                    size = (m["kv_heads"], m["vdim"])
                    if mixed is not None and size != mixed[1]:
                        raise ConfigError(f"config.json: '{where}mixer' mixes values with layer {mixed[0]}, whose "
                                          f"kv_heads and vdim {mixed[1]} differ from {size}")
                    mixed = mixed or (i, size)
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
