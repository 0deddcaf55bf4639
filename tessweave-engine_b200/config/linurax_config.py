"""Typed view of a Linurax ``config.json``.

The file names the design under ``architecture``, the residual width, the vocabulary, the embedding's
scale, the norms' eps, and a list of layers; a layer names its mixer (``attention`` or ``mingru``) with
the mixer's own sizes and constants, and its feed-forward (``dense`` or none).  Layers may differ from one
another in everything.  Every size and constant comes from here; anything this engine does not implement
(another mixer, another feed-forward kind, a value size that differs from the key size although the values
are the keys) is refused before a weight is read.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

from .model_config import ConfigError


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _positive_int(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {value!r}")
    return value


def _finite(value, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ConfigError(f"config.json: {what} must be a finite number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "AttentionConfig":
        rot = _need(d, "rot", where)
        cfg = cls(heads=_positive_int(_need(d, "heads", where), f"{where}.heads"),
                  kv_heads=_positive_int(_need(d, "kv_heads", where), f"{where}.kv_heads"),
                  dim=_positive_int(_need(d, "dim", where), f"{where}.dim"),
                  vdim=_positive_int(_need(d, "vdim", where), f"{where}.vdim"),
                  scale=_finite(_need(d, "scale", where), f"{where}.scale"),
                  rot_dims=int(_need(rot, "dims", f"{where}.rot")),
                  rot_base=_finite(_need(rot, "base", f"{where}.rot"), f"{where}.rot.base"))
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}: heads must be a multiple of kv_heads")
        if cfg.vdim != cfg.dim:
            raise ConfigError(f"config.json: {where}: the values are the keys, so vdim must equal dim")
        if cfg.rot_dims < 0 or cfg.rot_dims % 2 or cfg.rot_dims > cfg.dim or not cfg.rot_base > 0:
            raise ConfigError(f"config.json: {where}.rot: dims must be even and at most dim, base positive")
        if cfg.dim > 256:
            raise ConfigError(f"config.json: {where}: head sizes above 256 are not supported")
        return cfg


@dataclass(frozen=True)
class MinGRUConfig:
    width: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MinGRUConfig":
        return cls(width=_positive_int(_need(d, "width", where), f"{where}.width"))


@dataclass(frozen=True)
class DenseFeedForwardConfig:
    ff: int


MIXERS = {"attention": AttentionConfig, "mingru": MinGRUConfig}


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: AttentionConfig | MinGRUConfig
    mlp: DenseFeedForwardConfig | None


@dataclass(frozen=True)
class LinuraxConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple[LayerConfig, ...]
    eos_token_ids: tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict) -> "LinuraxConfig":
        layers = []
        raw_layers = _need(d, "layers", "the top level")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, layer in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r} is not implemented (known: {', '.join(sorted(MIXERS))})")
            mixer = MIXERS[kind].from_dict(_need(layer, "mixer", where), f"{where}.mixer")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", f"{where}.mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp: feed-forward kind {mlp['kind']!r} is not implemented (known: dense)")
                mlp = DenseFeedForwardConfig(ff=_positive_int(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff"))
            layers.append(LayerConfig(kind, mixer, mlp))
        cfg = cls(architecture=str(d.get("architecture", "Linurax")),
                  vocab=_positive_int(_need(d, "vocab", "the top level"), "vocab"),
                  width=_positive_int(_need(d, "width", "the top level"), "width"),
                  embedding_scale=_finite(_need(_need(d, "embedding", "the top level"), "scale", "embedding"), "embedding.scale"),
                  norm_eps=_finite(_need(_need(d, "norm", "the top level"), "eps", "norm"), "norm.eps"),
                  layers=tuple(layers))
        if not cfg.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg

    @classmethod
    def read(cls, folder) -> "LinuraxConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))
