"""Typed configuration of the Tevirax decoder, read from its config.json.

The file names its architecture with one string, ``"architecture": "Tevirax"``, and gives the model's sizes
(``vocab``, ``width``, ``max_positions``: the position table's rows, taken from the checkpoint where absent), the token embedding's factor (``embedding.scale``), the norm's eps
(``norm.eps``), the cap on the logits (``logit_softcap``) and a list ``layers`` whose entries say which mixer the
layer has (``type``: mamba2 | parallel), the mixer's sizes and constants (``mixer``) and the feed-forward
(``mlp``: ``kind`` dense | moe, or null for none).  Every size and constant is taken from there; nothing is
assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .errors import ConfigError

MIXER_TYPES = ("mamba2", "parallel")
MLP_KINDS = ("dense", "moe")


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


def _check_rotation(where: str, rot: dict, dim: int) -> None:
    dims = _int(where, rot, "dims", 0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"{where}: 'dims' must be even and at most 'dim' ({dim}), got {dims}")
    if dims:
        _num(where, rot, "base", positive=True)
    sc = rot.get("scaling")
    if sc is not None:
        sc = _obj(where, rot, "scaling")
        if _num(where + ".scaling", sc, "factor", positive=True) < 1.0:
            raise ConfigError(f"{where}.scaling: 'factor' must be at least 1")
        for k in ("original", "fast", "slow"):
            _num(where + ".scaling", sc, k, positive=True)


def _check_softmax_side(where: str, m: dict) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _int(where, m, k)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
    _num(where, m, "scale")
    if m.get("mask") is not None:
        _int(where + ".mask", _obj(where, m, "mask"), "size")
    if m.get("rot") is not None:
        _check_rotation(where + ".rot", _obj(where, m, "rot"), m["dim"])


def _check_memory_side(where: str, m: dict) -> None:
    for k in ("heads", "dim", "vdim"):
        _int(where, m, k)
    _num(where, m, "gate_cap", positive=True)


def _check_mamba2(where: str, m: dict) -> None:
    for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
        _int(where, m, k)
    if m["heads"] % m["groups"]:
        raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['groups']} groups")
    if (m["heads"] * m["vdim"]) % m["norm_groups"]:
        raise ConfigError(f"{where}: {m['heads'] * m['vdim']} channels do not split into {m['norm_groups']} norm_groups")


def _check_mlp(where: str, mlp: dict) -> None:
    if mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"{where}: 'kind' must be one of {', '.join(MLP_KINDS)}, got {mlp.get('kind')!r}")
    if mlp["kind"] == "dense":
        _int(where, mlp, "ff")
        return
    _int(where + ".expert", _obj(where, mlp, "expert"), "ff")
    r = _obj(where, mlp, "router")
    E, top = _int(where + ".router", r, "experts"), _int(where + ".router", r, "top")
    count, keep = 1, 1
    if r.get("groups") is not None:
        g = _obj(where + ".router", r, "groups")
        count, keep = _int(where + ".router.groups", g, "count"), _int(where + ".router.groups", g, "keep")
    if E % count or keep > count or top > keep * (E // count):
        raise ConfigError(f"{where}.router: {top} of {E} experts cannot be chosen from {keep} of {count} equal groups")
    if mlp.get("shared") is not None:
        _int(where + ".shared", _obj(where, mlp, "shared"), "ff")


@dataclass
class TeviraxLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class TeviraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    max_positions: Optional[int]
    logit_softcap: float
    layers: List[TeviraxLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "TeviraxConfig":
        vocab, width = _int("config", d, "vocab"), _int("config", d, "width")
        eps = _num("config key 'norm'", _obj("config", d, "norm"), "eps")
        emb = d.get("embedding")
        scale = _num("config key 'embedding'", emb, "scale") if isinstance(emb, dict) and emb.get("scale") is not None else 1.0
        # absent: the position table's length is the checkpoint's to say
        max_positions = None if d.get("max_positions") is None else _int("config", d, "max_positions")
        cap = d.get("logit_softcap")
        cap = 0.0 if cap is None else _num("config", d, "logit_softcap", positive=True)
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
            if e["type"] == "mamba2":
                _check_mamba2(where + ".mixer", m)
            else:
                _check_softmax_side(where + ".mixer.left", _obj(where + ".mixer", m, "left"))
                _check_memory_side(where + ".mixer.right", _obj(where + ".mixer", m, "right"))
                for k in ("left_scale", "right_scale"):
                    _num(where + ".mixer", m, k)
            mlp = e.get("mlp")
            if mlp is not None:
                mlp = dict(_obj(where, e, "mlp"))
                _check_mlp(where + ".mlp", mlp)
            layers.append(TeviraxLayer(e["type"], m, mlp))
        eos = d.get("eos_token_id")
        return cls(vocab, width, eps, scale, max_positions, cap, layers, None if eos is None else int(eos))

    def to_dict(self) -> dict:
        return {"vocab": self.vocab, "width": self.width, "norm_eps": self.norm_eps, "embedding_scale": self.embedding_scale,
                "max_positions": self.max_positions, "logit_softcap": self.logit_softcap,
                "layers": [f"{l.type} {l.mixer}" + (f" + mlp {l.mlp}" if l.mlp else "") for l in self.layers]}
