"""Typed configuration of the Rirulix decoder, read from its own ``config.json``.

The file lists the layers one by one; each names its mixer (``type``: ``attention`` or ``rglru``)
with the mixer's sizes, and its feed-forward (``mlp``, or null for none).  Every size and every
constant that may differ between models of the design is read from the file; nothing is filled in.

    {"architecture": "Rirulix", "vocab": V, "width": H, "max_positions": P,
     "norm": {"eps": e, "groups": g},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "v_mix", "mask": {"size", "keep_first"}},
                 "mlp": {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff", "limit"},
                         "shared": {"ff", "limit"} | null} | null},
                {"type": "rglru", "mixer": {"width", "blocks", "conv"}, "mlp": ...}, ...]}
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .text_config import ConfigError


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no {key!r}")
    return d[key]


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    keep_first: int
    v_mix: bool


@dataclass(frozen=True)
class RecurrentMixerConfig:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class RoutedMlpConfig:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: Optional[int]
    shared_limit: Optional[float]


@dataclass(frozen=True)
class RirulixLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[RoutedMlpConfig]


@dataclass(frozen=True)
class RirulixConfig:
    vocab_size: int
    hidden_size: int
    max_positions: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[RirulixLayerConfig, ...]
    eos_token_id: Optional[int] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "RirulixConfig":
        norm = _need(raw, "norm", "the model")
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the model")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            m = _need(entry, "mixer", where)
            if kind == "attention":
                mask = m.get("mask") or {}
                window = mask.get("size")
                mixer = AttentionMixerConfig(
                    heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)), dim=int(_need(m, "dim", where)),
                    vdim=int(m["vdim"]) if m.get("vdim") is not None else int(m["dim"]), scale=float(_need(m, "scale", where)),
                    window=int(window) if window else None, keep_first=int(mask.get("keep_first") or 0),
                    v_mix=bool(m.get("v_mix", False)))
            elif kind == "rglru":
                mixer = RecurrentMixerConfig(width=int(_need(m, "width", where)), blocks=int(_need(m, "blocks", where)),
                                             conv=int(_need(m, "conv", where)))
            else:
                raise ConfigError(f"config.json: {where} has the unknown type {kind!r}; known: attention, rglru")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp has the unknown kind {mlp.get('kind')!r}; known: moe")
                router, expert, shared = _need(mlp, "router", where + ".mlp"), _need(mlp, "expert", where + ".mlp"), mlp.get("shared")
                mlp = RoutedMlpConfig(
                    experts=int(_need(router, "experts", where)), top=int(_need(router, "top", where)),
                    ff=int(_need(expert, "ff", where)), limit=float(_need(expert, "limit", where)),
                    shared_ff=int(_need(shared, "ff", where)) if shared else None,
                    shared_limit=float(_need(shared, "limit", where)) if shared else None)
            layers.append(RirulixLayerConfig(kind, mixer, mlp))
        eos = raw.get("eos_token_id")
        return cls(vocab_size=int(_need(raw, "vocab", "the model")), hidden_size=int(_need(raw, "width", "the model")),
                   max_positions=int(_need(raw, "max_positions", "the model")), norm_eps=float(_need(norm, "eps", "norm")),
                   norm_groups=int(norm.get("groups") or 1), layers=tuple(layers), eos_token_id=None if eos is None else int(eos))
