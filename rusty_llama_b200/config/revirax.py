"""Typed configuration of the Revirax architecture, read from config.json.

The file lists its layers one by one; every layer names which mixer it has (`type`), the mixer's sizes and constants and
its feed-forward, so two models of the architecture may differ in everything, the order of layer kinds included.  Keys:

    architecture: "Revirax", vocab, width, norm: {eps},
    layers: [ {type: "lightning", mixer: {heads, dim, vdim, decay: [one per head]}, mlp}
            | {type: "attention", mixer: <softmax attention>, mlp}
            | {type: "parallel",  mixer: {left: <softmax attention>, right: {width}, left_scale, right_scale}, mlp} ... ]
    <softmax attention>: {heads, kv_heads, dim, vdim, scale, rot: {base, dims, scaling: {...} or null}, mask: {size} (optional)}
    mlp: null | {kind: "dense", ff}

A rotation's scaling is told by its keys: {factor, low, high, original} rescales by wavelength bands, {factor, original, fast,
slow} by a ramp over the pair index with a magnitude on cosines and sines.  What else a mixer has (a sink per head, mixed
scores, biases, an output gate) belongs to its layer type and is fixed by the design, not by the file.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..errors import ConfigError
from .rope_scaling import RopeScaling
from .vezatar import _get, _int, _num

ARCHITECTURE = "Revirax"
MAX_POSITIONS = 1 << 20  # the design names no limit; the library's bookkeeping wants one


@dataclass(frozen=True)
class SoftmaxMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: RopeScaling
    window: int = 0  # 0: every earlier position is seen


@dataclass(frozen=True)
class LightningMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SoftmaxMixerConfig
    right_width: int
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class ReviraxLayerConfig:
    type: str
    mixer: Union[SoftmaxMixerConfig, LightningMixerConfig, ParallelMixerConfig]
    mlp: Optional[DenseMlpConfig]


@dataclass(frozen=True)
class ReviraxConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[ReviraxLayerConfig, ...]
    architecture: str = ARCHITECTURE

    @classmethod
    def from_json(cls, d: Mapping[str, Any]) -> "ReviraxConfig":
        layers = _get(d, "layers", "config.json")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        return cls(
            vocab=_int(d, "vocab", "config.json"),
            width=_int(d, "width", "config.json"),
            eps=_num(_get(d, "norm", "config.json"), "eps", "norm"),
            layers=tuple(_layer(i, layer) for i, layer in enumerate(layers)),
        )


def _scaling(sc, where: str) -> RopeScaling:
    if sc is None:
        return RopeScaling()
    if not isinstance(sc, Mapping):
        raise ConfigError(f"{where} must be an object or null")
    if "fast" in sc or "slow" in sc:
        out = RopeScaling(
            kind="yarn", factor=_num(sc, "factor", where), original_max_position_embeddings=_int(sc, "original", where),
            beta_fast=_num(sc, "fast", where), beta_slow=_num(sc, "slow", where),
        )
    elif "low" in sc or "high" in sc:
        out = RopeScaling(
            kind="llama3", factor=_num(sc, "factor", where), low_freq_factor=_num(sc, "low", where),
            high_freq_factor=_num(sc, "high", where), original_max_position_embeddings=_int(sc, "original", where),
        )
    else:
        raise ConfigError(f"{where} names neither (low, high) nor (fast, slow): the kind of scaling cannot be told")
    out.validate()
    return out


def _softmax_mixer(m, where: str) -> SoftmaxMixerConfig:
    rot = m.get("rot") if isinstance(m, Mapping) else None
    if rot is None:
        base, dims, scaling = 10000.0, 0, RopeScaling()
    else:
        dims = _int(rot, "dims", where + ".rot", 0)
        base = _num(rot, "base", where + ".rot")
        scaling = _scaling(rot.get("scaling"), where + ".rot.scaling")
    dim = _int(m, "dim", where)
    if dims > dim or dims % 2:
        raise ConfigError(f"{where}.rot.dims = {dims} must be even and at most dim = {dim}")
    mask = m.get("mask")
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
    return SoftmaxMixerConfig(
        heads=heads, kv_heads=kv_heads, dim=dim, vdim=_int(m, "vdim", where), scale=_num(m, "scale", where),
        rot_base=base, rot_dims=dims, rot_scaling=scaling, window=_int(mask, "size", where + ".mask") if mask is not None else 0,
    )


def _layer(i: int, d: Mapping[str, Any]) -> ReviraxLayerConfig:
    where = f"layers[{i}]"
    kind = _get(d, "type", where)
    m = _get(d, "mixer", where)
    w = where + ".mixer"
    if kind == "lightning":
        heads = _int(m, "heads", w)
        decay = _get(m, "decay", w)
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"{w}.decay must list one number per head ({heads})")
        mixer = LightningMixerConfig(
            heads=heads, dim=_int(m, "dim", w), vdim=_int(m, "vdim", w),
            decay=tuple(_num({"decay": x}, "decay", w, positive=False) for x in decay),
        )
    elif kind == "attention":
        mixer = _softmax_mixer(m, w)
    elif kind == "parallel":
        mixer = ParallelMixerConfig(
            left=_softmax_mixer(_get(m, "left", w), w + ".left"), right_width=_int(_get(m, "right", w), "width", w + ".right"),
            left_scale=_num(m, "left_scale", w, positive=False), right_scale=_num(m, "right_scale", w, positive=False),
        )
    else:
        raise ConfigError(f"{where}.type '{kind}' is not a mixer of this architecture (known: lightning, attention, parallel)")
    mlp = d.get("mlp")
    if mlp is None:
        parsed = None
    else:
        mk = _get(mlp, "kind", where + ".mlp")
        if mk != "dense":
            raise ConfigError(f"{where}.mlp.kind '{mk}' is not a feed-forward of this architecture (known: dense)")
        parsed = DenseMlpConfig(ff=_int(mlp, "ff", where + ".mlp"))
    return ReviraxLayerConfig(kind, mixer, parsed)
