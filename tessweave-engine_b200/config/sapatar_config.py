"""Typed view of a Sapatar ``config.json``.

The file names the design under ``architecture``, the residual width, the vocabulary, the norms' eps, optionally
the number of parallel copies of the residual stream (``streams``: hyper-connections), and a list of layers.  A
layer names its mixer by ``type`` -- ``wkv`` (time mixing with token-dependent decays), ``retention`` (linear
attention with a constant decay per head) or ``parallel`` (softmax attention over a sliding window beside an mLSTM
matrix memory, summed with two scales) -- with the mixer's sizes and constants under ``mixer``, and its
feed-forward under ``mlp`` (``moe`` or null).  A layer with ``weights_of: j`` has no tensors of its own: it runs
with layer j's, on a cache and state of its own.  Every size and constant comes from here; the one size the file
does not give, the inner size of a wkv layer's decay projection, is read from the checkpoint's tensor shapes
(or from the key ``decay_rank`` where a configuration is written before its weights exist).  Anything this engine
does not implement is refused before a weight is read.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, replace
from pathlib import Path

from .linurax_config import _finite, _need, _positive_int
from .model_config import ConfigError


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float

    @classmethod
    def from_dict(cls, d: dict, where: str, head_dim: int) -> "RotationConfig":
        dims = _need(d, "dims", where)
        base = _finite(_need(d, "base", where), f"{where}.base")
        if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > head_dim or not base > 0:
            raise ConfigError(f"config.json: {where}: dims must be even and at most the head size {head_dim}, base positive")
        return cls(dims, base)


@dataclass(frozen=True)
class WkvConfig:
    heads: int
    dim: int
    decay_rank: int | None      # None until the checkpoint's shapes have been seen

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "WkvConfig":
        rank = d.get("decay_rank")
        return cls(heads=_positive_int(_need(d, "heads", where), f"{where}.heads"),
                   dim=_positive_int(_need(d, "dim", where), f"{where}.dim"),
                   decay_rank=None if rank is None else _positive_int(rank, f"{where}.decay_rank"))


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: RotationConfig

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "RetentionConfig":
        heads = _positive_int(_need(d, "heads", where), f"{where}.heads")
        dim = _positive_int(_need(d, "dim", where), f"{where}.dim")
        decay = _need(d, "decay", where)
        if not isinstance(decay, list) or len(decay) != heads:
            raise ConfigError(f"config.json: {where}.decay must list one decay per head")
        return cls(heads=heads, dim=dim, vdim=_positive_int(_need(d, "vdim", where), f"{where}.vdim"),
                   decay=tuple(_finite(x, f"{where}.decay") for x in decay),
                   rot=RotationConfig.from_dict(_need(d, "rot", where), f"{where}.rot", dim))


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
    rot: RotationConfig

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "WindowAttentionConfig":
        heads = _positive_int(_need(d, "heads", where), f"{where}.heads")
        kv_heads = _positive_int(_need(d, "kv_heads", where), f"{where}.kv_heads")
        dim = _positive_int(_need(d, "dim", where), f"{where}.dim")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: heads must be a multiple of kv_heads")
        mask = d.get("mask")
        window = None if mask is None else _positive_int(_need(mask, "size", f"{where}.mask"), f"{where}.mask.size")
        cfg = cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_positive_int(_need(d, "vdim", where), f"{where}.vdim"),
                  scale=_finite(_need(d, "scale", where), f"{where}.scale"), window=window,
                  rot=RotationConfig.from_dict(_need(d, "rot", where), f"{where}.rot", dim))
        if max(cfg.dim, cfg.vdim) > 256:
            raise ConfigError(f"config.json: {where}: head sizes above 256 are not supported")
        return cfg


@dataclass(frozen=True)
class MlstmConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MlstmConfig":
        cfg = cls(heads=_positive_int(_need(d, "heads", where), f"{where}.heads"),
                  dim=_positive_int(_need(d, "dim", where), f"{where}.dim"),
                  vdim=_positive_int(_need(d, "vdim", where), f"{where}.vdim"),
                  gate_cap=_finite(_need(d, "gate_cap", where), f"{where}.gate_cap"))
        if not cfg.gate_cap > 0:
            raise ConfigError(f"config.json: {where}.gate_cap must be positive")
        return cfg


@dataclass(frozen=True)
class ParallelConfig:
    left: WindowAttentionConfig
    right: MlstmConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ParallelConfig":
        return cls(left=WindowAttentionConfig.from_dict(_need(d, "left", where), f"{where}.left"),
                   right=MlstmConfig.from_dict(_need(d, "right", where), f"{where}.right"),
                   left_scale=_finite(_need(d, "left_scale", where), f"{where}.left_scale"),
                   right_scale=_finite(_need(d, "right_scale", where), f"{where}.right_scale"))


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    ff: int
    shared_ff: int | None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MoeConfig":
        router = _need(d, "router", where)
        shared = d.get("shared")
        cfg = cls(experts=_positive_int(_need(router, "experts", f"{where}.router"), f"{where}.router.experts"),
                  top=_positive_int(_need(router, "top", f"{where}.router"), f"{where}.router.top"),
                  ff=_positive_int(_need(_need(d, "expert", where), "ff", f"{where}.expert"), f"{where}.expert.ff"),
                  shared_ff=None if shared is None else _positive_int(_need(shared, "ff", f"{where}.shared"), f"{where}.shared.ff"))
        if cfg.top > cfg.experts:
            raise ConfigError(f"config.json: {where}.router: top exceeds the number of experts")
        return cfg


MIXERS = {"wkv": WkvConfig, "retention": RetentionConfig, "parallel": ParallelConfig}


@dataclass(frozen=True)
class SapatarLayer:
    type: str
    mixer: WkvConfig | RetentionConfig | ParallelConfig
    mlp: MoeConfig | None
    weights_of: int | None = None


@dataclass(frozen=True)
class SapatarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    streams: int | None
    layers: tuple[SapatarLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict) -> "SapatarConfig":
        raw_layers = _need(d, "layers", "the top level")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: list[SapatarLayer] = []
        for i, layer in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r} is not implemented (known: {', '.join(sorted(MIXERS))})")
            mixer = MIXERS[kind].from_dict(_need(layer, "mixer", where), f"{where}.mixer")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", f"{where}.mlp") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp: feed-forward kind {mlp['kind']!r} is not implemented (known: moe)")
                mlp = MoeConfig.from_dict(mlp, f"{where}.mlp")
            owner = layer.get("weights_of")
            if owner is not None:
                if isinstance(owner, bool) or not isinstance(owner, int) or not 0 <= owner < i:
                    raise ConfigError(f"config.json: {where}.weights_of must name an earlier layer")
                while layers[owner].weights_of is not None:
                    owner = layers[owner].weights_of
                mine = SapatarLayer(kind, mixer, mlp)
                if replace(mine, mixer=_without_rank(mixer)) != replace(layers[owner], mixer=_without_rank(layers[owner].mixer)):
                    raise ConfigError(f"config.json: {where} uses the weights of layer {owner} but describes another layer")
                mixer = layers[owner].mixer
            layers.append(SapatarLayer(kind, mixer, mlp, owner))
        streams = d.get("streams")
        cfg = cls(architecture=str(d.get("architecture", "Sapatar")),
                  vocab=_positive_int(_need(d, "vocab", "the top level"), "vocab"),
                  width=_positive_int(_need(d, "width", "the top level"), "width"),
                  norm_eps=_finite(_need(_need(d, "norm", "the top level"), "eps", "norm"), "norm.eps"),
                  streams=None if streams is None else _positive_int(streams, "streams"),
                  layers=tuple(layers))
        if not cfg.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg

    def with_tensor_shapes(self, shapes: dict[str, tuple]) -> "SapatarConfig":
        """Fill the sizes only the checkpoint gives (the inner size of a wkv layer's decay projection, from
        ``l<i>.mix.w1``) and refuse a configured one that the checkpoint contradicts."""
        layers = list(self.layers)
        for i, layer in enumerate(layers):
            if not isinstance(layer.mixer, WkvConfig):
                continue
            owner = i if layer.weights_of is None else layer.weights_of
            shape = shapes.get(f"l{owner}.mix.w1")
            rank = layer.mixer.decay_rank
            if shape is not None:
                if len(shape) != 2 or (rank is not None and rank != shape[0]):
                    raise ConfigError(f"config.json: layers[{i}].mixer.decay_rank {rank} contradicts l{owner}.mix.w1 {list(shape)}")
                rank = int(shape[0])
            layers[i] = replace(layer, mixer=replace(layer.mixer, decay_rank=rank))
        return replace(self, layers=tuple(layers))

    @classmethod
    def read(cls, folder) -> "SapatarConfig":
        folder = Path(folder)
        cfg = cls.from_dict(json.loads((folder / "config.json").read_text()))
        return cfg.with_tensor_shapes(safetensors_shapes(folder))


def _without_rank(mixer):
    return replace(mixer, decay_rank=None) if isinstance(mixer, WkvConfig) else mixer


def safetensors_shapes(folder: Path) -> dict[str, tuple]:
    """name -> shape of every tensor in the folder's ``*.safetensors`` files, from their headers alone
    (8 bytes of little-endian length, then that many bytes of JSON)."""
    shapes: dict[str, tuple] = {}
    for path in sorted(Path(folder).glob("*.safetensors")):
        with open(path, "rb") as f:
            (length,) = struct.unpack("<Q", f.read(8))
            if length > 1 << 28:
                raise ConfigError(f"{path.name}: the header claims {length} bytes")
            header = json.loads(f.read(length))
        for name, entry in header.items():
            if name != "__metadata__":
                shapes[name] = tuple(entry["shape"])
    return shapes
