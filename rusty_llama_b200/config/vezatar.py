"""Typed configuration of the Vezatar architecture, read from config.json.

The file lists its layers one by one: every layer names its mixer (with the mixer's sizes and
constants) and its feed-forward (dense, routed, or none), so two models of the architecture may
differ in everything, the order of layer kinds included.  Keys:

    architecture: "Vezatar", vocab, width, norm: {eps},
    layers: [ {type: "latent_attention",
               mixer: {heads, dim, rot_dim, vdim, kv_rank, scale, kv_from (optional: the layer whose cache is read),
                       rot: {base, dims, scaling: {factor, original, fast, slow} or null}},
               mlp: null
                  | {kind: "dense", ff, limit}
                  | {kind: "moe", router: {experts, top}, expert: {ff}, shared: {ff} or null}} ... ]
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..errors import ConfigError
from .rope_scaling import RopeScaling

ARCHITECTURE = "Vezatar"

# Constants the design fixes
DENSE_GATE_ALPHA = 1.702  # the dense feed-forward's gate is g * logistic(1.702 g)
MAX_POSITIONS = 1 << 20  # the design names no limit; the library's bookkeeping wants one


def _get(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping):
        raise ConfigError(f"{where} must be an object")
    if key not in d:
        raise ConfigError(f"{where} lacks '{key}'")
    return d[key]


def _int(d, key, where, minimum=1) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"{where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d, key, where, positive=True) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)) or (positive and float(v) <= 0):
        raise ConfigError(f"{where}.{key} must be a finite{' positive' if positive else ''} number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: RopeScaling
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeMlpConfig:
    experts: int
    top: int
    expert_ff: int
    shared_ff: int = 0  # 0: no shared expert


@dataclass(frozen=True)
class VezatarLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: Union[DenseMlpConfig, MoeMlpConfig, None]


@dataclass(frozen=True)
class VezatarConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[VezatarLayerConfig, ...]
    architecture: str = ARCHITECTURE

    @classmethod
    def from_json(cls, d: Mapping[str, Any]) -> "VezatarConfig":
        layers = _get(d, "layers", "config.json")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = tuple(_layer(i, layer) for i, layer in enumerate(layers))
        for i, layer in enumerate(parsed):
            src = layer.mixer.kv_from
            if src is None:
                continue
            if not 0 <= src < i:
                raise ConfigError(f"layers[{i}].mixer.kv_from names layer {src}, which does not run before it")
            other = parsed[src].mixer
            if other.kv_from is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from names layer {src}, which has no cache of its own")
            mine = layer.mixer
            if (mine.kv_rank, mine.rot_dim, mine.rot_base, mine.rot_dims, mine.rot_scaling) != (
                other.kv_rank, other.rot_dim, other.rot_base, other.rot_dims, other.rot_scaling):
                raise ConfigError(f"layers[{i}] reads the cache of layer {src}, but their kv_rank, rot_dim or rotation differ")
        return cls(
            vocab=_int(d, "vocab", "config.json"),
            width=_int(d, "width", "config.json"),
            eps=_num(_get(d, "norm", "config.json"), "eps", "norm"),
            layers=parsed,
        )


def _layer(i: int, d: Mapping[str, Any]) -> VezatarLayerConfig:
    where = f"layers[{i}]"
    kind = _get(d, "type", where)
    if kind != "latent_attention":
        raise ConfigError(f"{where}.type '{kind}' is not a mixer of this architecture (known: latent_attention)")
    m = _get(d, "mixer", where)
    rot = _get(m, "rot", where + ".mixer")
    sc = rot.get("scaling") if isinstance(rot, Mapping) else None
    if sc is None:
        scaling = RopeScaling()
    else:
        w = where + ".mixer.rot.scaling"
        scaling = RopeScaling(
            kind="yarn", factor=_num(sc, "factor", w), original_max_position_embeddings=_int(sc, "original", w),
            beta_fast=_num(sc, "fast", w), beta_slow=_num(sc, "slow", w),
        )
        scaling.validate()
    rot_dim = _int(m, "rot_dim", where + ".mixer", 0)
    rot_dims = _int(rot, "dims", where + ".mixer.rot", 0)
    if rot_dims > rot_dim or rot_dims % 2:
        raise ConfigError(f"{where}.mixer.rot.dims = {rot_dims} must be even and at most rot_dim = {rot_dim}")
    kv_from = m.get("kv_from")
    if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
        raise ConfigError(f"{where}.mixer.kv_from must be a layer index, got {kv_from!r}")
    mixer = LatentMixerConfig(
        heads=_int(m, "heads", where + ".mixer"), dim=_int(m, "dim", where + ".mixer", 0), rot_dim=rot_dim,
        vdim=_int(m, "vdim", where + ".mixer"), kv_rank=_int(m, "kv_rank", where + ".mixer"),
        scale=_num(m, "scale", where + ".mixer"), rot_base=_num(rot, "base", where + ".mixer.rot"), rot_dims=rot_dims,
        rot_scaling=scaling, kv_from=kv_from,
    )
    mlp = d.get("mlp")
    if mlp is None:
        parsed = None
    else:
        w = where + ".mlp"
        mk = _get(mlp, "kind", w)
        if mk == "dense":
            parsed = DenseMlpConfig(ff=_int(mlp, "ff", w), limit=_num(mlp, "limit", w))
        elif mk == "moe":
            router = _get(mlp, "router", w)
            shared = mlp.get("shared")
            parsed = MoeMlpConfig(
                experts=_int(router, "experts", w + ".router"), top=_int(router, "top", w + ".router"),
                expert_ff=_int(_get(mlp, "expert", w), "ff", w + ".expert"),
                shared_ff=_int(shared, "ff", w + ".shared") if shared is not None else 0,
            )
            if parsed.top > parsed.experts:
                raise ConfigError(f"{w}.router: {parsed.top} of {parsed.experts} experts")
        else:
            raise ConfigError(f"{w}.kind '{mk}' is neither 'dense' nor 'moe'")
    return VezatarLayerConfig(kind, mixer, parsed)
