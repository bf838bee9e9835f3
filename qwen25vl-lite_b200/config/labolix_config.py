"""Typed configuration of the Labolix decoder, read from its own ``config.json``.

The file lists the layers one by one; each names its mixer (``type``: ``attention``,
``latent_attention`` or ``retention``) with the mixer's sizes, and its feed-forward (``mlp``, or null
for none).  A layer with ``weights_of: j`` has no tensors of its own and runs with layer j's.  Every
size and every constant that may differ between models of the design is read from the file; nothing
is filled in.

    {"architecture": "Labolix", "vocab": V, "width": W, "norm": {"eps": e}, "logit_softcap": c,
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                           "rot": {"dims", "base", "scaling": {"factor", "low", "high", "original"} | absent}},
                 "mlp": {"kind": "dense", "ff", "limit"} | null},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "mask": {"size"},
                           "rot": {"dims", "base", "scaling": {"factor", "original", "fast", "slow"} | absent}}, ...},
                {"type": "retention", "mixer": {"heads", "dim", "vdim", "decay": [...], "rot": {"dims", "base"}}, ...},
                {..., "weights_of": j}, ...]}
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
class RotaryConfig:
    dims: int
    base: float
    # None, or ("wavelength", factor, low, high, original) / ("ramp", factor, original, fast, slow) as a dict with "kind"
    scaling: Optional[Tuple[Tuple[str, Any], ...]] = None

    def scaling_dict(self) -> Optional[Dict[str, Any]]:
        return dict(self.scaling) if self.scaling else None


@dataclass(frozen=True)
class SoftmaxMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot: Optional[RotaryConfig]


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot: Optional[RotaryConfig]


@dataclass(frozen=True)
class RetentionMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[RotaryConfig]


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class LabolixLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[DenseMlpConfig]
    weights_of: Optional[int] = None


SCALING_KEYS = {"wavelength": ("factor", "low", "high", "original"), "ramp": ("factor", "original", "fast", "slow")}


def _rotary(m: Dict[str, Any], where: str, scaling_kind: Optional[str]) -> Optional[RotaryConfig]:
    rot = m.get("rot")
    if rot is None:
        return None
    dims = int(_need(rot, "dims", where + ".rot"))
    scaling = rot.get("scaling")
    if scaling:
        if scaling_kind is None:
            raise ConfigError(f"config.json: {where}.rot has a 'scaling', which this mixer does not take")
        scaling = (("kind", scaling_kind),) + tuple((k, float(_need(scaling, k, where + ".rot.scaling"))) for k in SCALING_KEYS[scaling_kind])
    if dims < 0 or dims % 2:
        raise ConfigError(f"config.json: {where}.rot.dims must be even, got {dims}")
    return RotaryConfig(dims, float(_need(rot, "base", where + ".rot")), scaling or None)


def _window(m: Dict[str, Any]) -> Optional[int]:
    size = (m.get("mask") or {}).get("size")
    return int(size) if size else None


@dataclass(frozen=True)
class LabolixConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_softcap: float
    layers: Tuple[LabolixLayerConfig, ...]
    eos_token_id: Optional[int] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "LabolixConfig":
        norm = _need(raw, "norm", "the model")
        entries = _need(raw, "layers", "the model")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            m = _need(entry, "mixer", where)
            need = lambda key: _need(m, key, where + ".mixer")
            if kind == "attention":
                heads = int(need("heads"))
                mixer = SoftmaxMixerConfig(heads=heads, kv_heads=int(m["kv_heads"]) if m.get("kv_heads") else heads, dim=int(need("dim")),
                                           vdim=int(m["vdim"]) if m.get("vdim") else int(m["dim"]), scale=float(need("scale")),
                                           window=_window(m), rot=_rotary(m, where + ".mixer", "wavelength"))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: {where}: {mixer.heads} heads cannot share {mixer.kv_heads} kv_heads")
            elif kind == "latent_attention":
                mixer = LatentMixerConfig(heads=int(need("heads")), dim=int(need("dim")), rot_dim=int(need("rot_dim")), vdim=int(need("vdim")),
                                          kv_rank=int(need("kv_rank")), scale=float(need("scale")), window=_window(m),
                                          rot=_rotary(m, where + ".mixer", "ramp"))
                if mixer.rot is not None and mixer.rot.dims > mixer.rot_dim:
                    raise ConfigError(f"config.json: {where}: rot.dims {mixer.rot.dims} exceeds rot_dim {mixer.rot_dim}")
            elif kind == "retention":
                heads = int(need("heads"))
                decay = tuple(float(d) for d in need("decay"))
                if len(decay) != heads:
                    raise ConfigError(f"config.json: {where}: {heads} heads but {len(decay)} decays")
                mixer = RetentionMixerConfig(heads=heads, dim=int(need("dim")), vdim=int(m["vdim"]) if m.get("vdim") else int(m["dim"]),
                                             decay=decay, rot=_rotary(m, where + ".mixer", None))
            else:
                raise ConfigError(f"config.json: {where} has the unknown type {kind!r}; known: attention, latent_attention, retention")
            if getattr(mixer, "rot", None) is not None and mixer.rot.dims > mixer.dim and kind != "latent_attention":
                raise ConfigError(f"config.json: {where}: rot.dims {mixer.rot.dims} exceeds the head size {mixer.dim}")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp has the unknown kind {mlp.get('kind')!r}; known: dense")
                mlp = DenseMlpConfig(ff=int(_need(mlp, "ff", where + ".mlp")), limit=float(_need(mlp, "limit", where + ".mlp")))
            owner = entry.get("weights_of")
            if owner is not None:
                owner = int(owner)
                if not 0 <= owner < len(entries) or owner == i:
                    raise ConfigError(f"config.json: {where}.weights_of names layer {owner}, which is not another layer of the model")
            layers.append(LabolixLayerConfig(kind, mixer, mlp, owner))
        for i, layer in enumerate(layers):
            if layer.weights_of is None:
                continue
            owner = layers[layer.weights_of]
            if owner.weights_of is not None:
                raise ConfigError(f"config.json: layers[{i}].weights_of names layer {layer.weights_of}, which has no tensors of its own")
            if (owner.type, owner.mixer, owner.mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}] runs with the tensors of layer {layer.weights_of} but describes another layer")
        eos = raw.get("eos_token_id")
        cap = raw.get("logit_softcap")
        return cls(vocab_size=int(_need(raw, "vocab", "the model")), hidden_size=int(_need(raw, "width", "the model")),
                   norm_eps=float(_need(norm, "eps", "norm")), logit_softcap=float(cap) if cap else 0.0, layers=tuple(layers),
                   eos_token_id=None if eos is None else int(eos))
