"""Typed configuration of the Ropelix decoder, read from its config.json.

The file names its architecture with one string, ``"architecture": "Ropelix"``, and gives the model's sizes
(``vocab``, ``width``), the token embedding's factor (``embedding.scale``), the norm's eps (``norm.eps``), the
constant on every sublayer's result (``residual_mult``) and a list ``layers`` whose entries say which mixer the layer
has (``type``: parallel | attention | delta), the mixer's sizes and constants (``mixer``) and the feed-forward
(``mlp``: ``kind`` dense, or null for none).  Every size and constant is taken from there; nothing is assumed equal
between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .errors import ConfigError

MIXER_TYPES = ("parallel", "attention", "delta")
MLP_KINDS = ("dense",)


def _int(where: str, d: dict, key: str, low: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < low:
        raise ConfigError(f"{where}: key {key!r} must be an integer >= {low}, got {v!r}")
    return int(v)


def _num(where: str, d: dict, key: str, positive: bool = False) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"{where}: key {key!r} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


def _obj(where: str, d: dict, key: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object, got {v!r}")
    return v


def _check_heads(where: str, m: dict) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _int(where, m, k)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")


def _check_mask(where: str, m: dict) -> None:
    if m.get("mask") is not None:
        _int(where + ".mask", _obj(where, m, "mask"), "size")


def _check_left(where: str, m: dict) -> None:
    _check_heads(where, m)
    _num(where, m, "scale")
    if m.get("softcap") is not None:
        _num(where, m, "softcap")
    _check_mask(where, m)
    if m.get("rot") is not None:
        rot = _obj(where, m, "rot")
        dims = _int(where + ".rot", rot, "dims", 0)
        if dims % 2 or dims > m["dim"]:
            raise ConfigError(f"{where}.rot: 'dims' must be even and at most 'dim' ({m['dim']}), got {dims}")
        if dims:
            _num(where + ".rot", rot, "base", positive=True)


def _check_right(where: str, m: dict) -> None:
    for k in ("width", "blocks", "conv"):
        _int(where, m, k)
    if m["width"] % m["blocks"]:
        raise ConfigError(f"{where}: {m['width']} channels do not split into {m['blocks']} blocks")


def _check_parallel(where: str, m: dict) -> None:
    _check_left(where + ".left", _obj(where, m, "left"))
    _check_right(where + ".right", _obj(where, m, "right"))
    _num(where, m, "left_scale")
    _num(where, m, "right_scale")


def _check_attention(where: str, m: dict) -> None:
    _check_heads(where, m)
    if m["vdim"] > m["dim"]:
        raise ConfigError(f"{where}: the values are the keys, so 'vdim' ({m['vdim']}) cannot exceed 'dim' ({m['dim']})")
    _int(where, m, "conv")
    _num(where, m, "scale")
    _check_mask(where, m)


def _check_delta(where: str, m: dict) -> None:
    _check_heads(where, m)
    _int(where, m, "conv")


def _check_mlp(where: str, mlp: dict) -> None:
    if mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"{where}: 'kind' must be one of {', '.join(MLP_KINDS)}, got {mlp.get('kind')!r}")
    _int(where, mlp, "ff")
    _num(where, mlp, "limit", positive=True)


_CHECKS = {"parallel": _check_parallel, "attention": _check_attention, "delta": _check_delta}


@dataclass
class RopelixLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class RopelixConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    residual_mult: float
    layers: List[RopelixLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "RopelixConfig":
        vocab, width = _int("config", d, "vocab"), _int("config", d, "width")
        scale = _num("config key 'embedding'", _obj("config", d, "embedding"), "scale")
        eps = _num("config key 'norm'", _obj("config", d, "norm"), "eps")
        mult = _num("config", d, "residual_mult") if d.get("residual_mult") is not None else 1.0
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config key 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(raw):
            where = f"config layers[{i}]"
            if not isinstance(e, dict) or e.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}: 'type' must be one of {', '.join(MIXER_TYPES)}, got "
                                  f"{e.get('type') if isinstance(e, dict) else e!r}")
            m = dict(_obj(where, e, "mixer"))
            _CHECKS[e["type"]](where + ".mixer", m)
            mlp = e.get("mlp")
            if mlp is not None:
                mlp = dict(_obj(where, e, "mlp"))
                _check_mlp(where + ".mlp", mlp)
            layers.append(RopelixLayer(e["type"], m, mlp))
        eos = d.get("eos_token_id")
        return cls(vocab, width, scale, eps, mult, layers, None if eos is None else int(eos))

    def to_dict(self) -> dict:
        return {"vocab": self.vocab, "width": self.width, "embedding_scale": self.embedding_scale,
                "norm_eps": self.norm_eps, "residual_mult": self.residual_mult,
                "layers": [f"{l.type} {l.mixer}" + (f" + mlp {l.mlp}" if l.mlp else "") for l in self.layers]}
