"""Typed configuration of the Puzorax decoder, read from its config.json.

The file names its architecture with one string, ``"architecture": "Puzorax"``, and gives the model's sizes
(``vocab``, ``width``), the norm's eps (``norm.eps``), the hashed bigram table of the embedding
(``embedding.bigram``: ``buckets``, ``mul_prev``, ``mul_cur``), a list ``layers`` whose entries say which mixer the
layer has (``type``: latent_attention | channel_delta), the mixer's sizes and constants (``mixer``) and the
feed-forward (``mlp``: ``kind`` moe, or null for none), and ``loop`` (``start``, ``stop``, ``times``; absent: no run
of layers is repeated): the layers start .. stop - 1 run ``times`` times in a row with the same weights.  Every size
and constant is taken from there; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .errors import ConfigError

MIXER_TYPES = ("latent_attention", "channel_delta")
MLP_KINDS = ("moe",)


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


def _check_latent(where: str, m: dict) -> None:
    for k in ("heads", "dim", "vdim", "kv_rank"):
        _int(where, m, k)
    rd = _int(where, m, "rot_dim", 0)
    _num(where, m, "scale")
    if m.get("mask") is not None:
        _int(where + ".mask", _obj(where, m, "mask"), "size")
    if m.get("rot") is not None:
        rot = _obj(where, m, "rot")
        dims = _int(where + ".rot", rot, "dims", 0)
        if dims % 2 or dims > rd:
            raise ConfigError(f"{where}.rot: 'dims' must be even and at most 'rot_dim' ({rd}), got {dims}")
        if dims:
            _num(where + ".rot", rot, "base", positive=True)


def _check_delta(where: str, m: dict) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
        _int(where, m, k)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")


def _check_mlp(where: str, mlp: dict) -> None:
    if mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"{where}: 'kind' must be one of {', '.join(MLP_KINDS)}, got {mlp.get('kind')!r}")
    _int(where + ".expert", _obj(where, mlp, "expert"), "ff")
    r = _obj(where, mlp, "router")
    E, top = _int(where + ".router", r, "experts"), _int(where + ".router", r, "top")
    ident = 0 if r.get("identity") is None else _int(where + ".router", r, "identity", 0)
    if r.get("scale") is not None:
        _num(where + ".router", r, "scale")
    if top > E + ident:
        raise ConfigError(f"{where}.router: {top} of {E} + {ident} experts cannot be chosen")


@dataclass
class PuzoraxLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class PuzoraxLoop:
    start: int
    stop: int
    times: int


@dataclass
class PuzoraxConfig:
    vocab: int
    width: int
    norm_eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: List[PuzoraxLayer] = field(default_factory=list)
    loop: Optional[PuzoraxLoop] = None
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "PuzoraxConfig":
        vocab, width = _int("config", d, "vocab"), _int("config", d, "width")
        eps = _num("config key 'norm'", _obj("config", d, "norm"), "eps")
        bg = _obj("config key 'embedding'", _obj("config", d, "embedding"), "bigram")
        buckets = _int("config embedding.bigram", bg, "buckets")
        mul_prev, mul_cur = _int("config embedding.bigram", bg, "mul_prev", 0), _int("config embedding.bigram", bg, "mul_cur", 0)
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
            (_check_latent if e["type"] == "latent_attention" else _check_delta)(where + ".mixer", m)
            mlp = e.get("mlp")
            if mlp is not None:
                mlp = dict(_obj(where, e, "mlp"))
                _check_mlp(where + ".mlp", mlp)
            layers.append(PuzoraxLayer(e["type"], m, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = _obj("config", d, "loop")
            loop = PuzoraxLoop(_int("config loop", lp, "start", 0), _int("config loop", lp, "stop", 0),
                               _int("config loop", lp, "times"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"config loop: layers {loop.start} .. {loop.stop} - 1 of {len(layers)}")
            if loop.start == loop.stop:
                loop = None                       # an empty run: nothing is repeated and nothing is added
        eos = d.get("eos_token_id")
        return cls(vocab, width, eps, buckets, mul_prev, mul_cur, layers, loop, None if eos is None else int(eos))

    def to_dict(self) -> dict:
        return {"vocab": self.vocab, "width": self.width, "norm_eps": self.norm_eps,
                "bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur},
                "loop": None if self.loop is None else vars(self.loop),
                "layers": [f"{l.type} {l.mixer}" + (f" + mlp {l.mlp}" if l.mlp else "") for l in self.layers]}
