"""Typed configuration of the Votavik decoder, read from its config.json.

The file names its architecture with one string, ``"architecture": "Votavik"``, gives the model's
sizes (``vocab``, ``width``), the norm's eps (``norm.eps``), the size of the per-layer token input
(``token_side.dim``; the key absent or null: none) and a list ``layers`` whose entries say which mixer
the layer has (``type``: gla | attention | lightning), the mixer's sizes and constants (``mixer``) and
the feed-forward (``mlp``, null for none).  Every size and constant is taken from there; nothing is
assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .errors import ConfigError

MIXER_TYPES = ("gla", "attention", "lightning")
MLP_KINDS = ("dense",)


def _int(where: str, d: dict, key: str, low: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < low:
        raise ConfigError(f"{where}: key {key!r} must be an integer >= {low}, got {v!r}")
    return int(v)


def _num(where: str, d: dict, key: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: key {key!r} must be a number, got {v!r}")
    return float(v)


def _obj(where: str, d: dict, key: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object, got {v!r}")
    return v


@dataclass
class VotavikLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class VotavikConfig:
    vocab: int
    width: int
    norm_eps: float
    side_dim: int
    layers: List[VotavikLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None
    max_positions: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "VotavikConfig":
        vocab, width = _int("config", d, "vocab"), _int("config", d, "width")
        eps = _num("config key 'norm'", _obj("config", d, "norm"), "eps")
        side = d.get("token_side")
        side_dim = _int("config key 'token_side'", side, "dim") if isinstance(side, dict) else 0
        if side is not None and not isinstance(side, dict):
            raise ConfigError(f"config key 'token_side' must be an object or null, got {side!r}")
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
            mw = where + ".mixer"
            for k in ("heads", "dim", "vdim"):
                _int(mw, m, k)
            if e["type"] == "gla":
                if _num(mw, m, "tau") <= 0:
                    raise ConfigError(f"{mw}: 'tau' must be positive")
                if m.get("rank") is not None:
                    _int(mw, m, "rank")
            elif e["type"] == "lightning":
                dec = m.get("decay")
                if not isinstance(dec, list) or len(dec) != m["heads"] or \
                        any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in dec):
                    raise ConfigError(f"{mw}: 'decay' must list one number for each of the {m['heads']} heads")
            else:
                if m["heads"] % _int(mw, m, "kv_heads"):
                    raise ConfigError(f"{mw}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
                _num(mw, m, "scale")
                if m.get("softcap") is not None and _num(mw, m, "softcap") < 0:
                    raise ConfigError(f"{mw}: 'softcap' must not be negative")
                if m.get("mask") is not None:
                    mask = _obj(mw, m, "mask")
                    _int(mw + ".mask", mask, "size")
                    if mask.get("keep_first") is not None:
                        _int(mw + ".mask", mask, "keep_first", 0)
                if m.get("rot") is not None:
                    rot = _obj(mw, m, "rot")
                    dims = _int(mw + ".rot", rot, "dims", 0)
                    if dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"{mw}.rot: 'dims' must be even and at most 'dim' ({m['dim']}), got {dims}")
                    if dims and _num(mw + ".rot", rot, "base") <= 0:
                        raise ConfigError(f"{mw}.rot: 'base' must be positive")
            mlp = e.get("mlp")
            if mlp is not None:
                mlp = dict(_obj(where, e, "mlp"))
                if mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"{where}.mlp: 'kind' must be one of {', '.join(MLP_KINDS)}, got {mlp.get('kind')!r}")
                _int(where + ".mlp", mlp, "ff")
                _num(where + ".mlp", mlp, "limit")
            layers.append(VotavikLayer(e["type"], m, mlp))
        eos = d.get("eos_token_id")
        mp = d.get("max_positions")
        return cls(vocab, width, eps, side_dim, layers, None if eos is None else int(eos), None if mp is None else int(mp))

    def to_dict(self) -> dict:
        return {"vocab": self.vocab, "width": self.width, "norm_eps": self.norm_eps, "side_dim": self.side_dim,
                "layers": [f"{l.type} {l.mixer}" + (f" + mlp {l.mlp}" if l.mlp else "") for l in self.layers]}
