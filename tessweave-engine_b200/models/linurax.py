"""The Linurax decoder as a ``ModelSpec``.

A stack of layers that differ from one another: each has one mixer -- sigmoid attention with mixed heads
over a paged cache (``attention``) or a minGRU recurrence with a fixed-size state (``mingru``) -- and
optionally a dense gated feed-forward.  The norm of a sub-layer sits on its output (block kind
``output_norm``).  The embedding rows are scaled; the output matrix is the embedding matrix itself.
Tensor names: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.gate|up|down``.
"""
from __future__ import annotations

from ..config.linurax_config import AttentionConfig, LayerConfig, LinuraxConfig, MinGRUConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry

LINURAX_LAYER_NAMES = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp"}
NO_POSITION_LIMIT = 2 ** 31 - 1        # the design has no table of positions; int32 positions bound a request


def mixer_spec(cfg: LinuraxConfig, layer: LayerConfig) -> PartSpec:
    m = layer.mixer
    if isinstance(m, AttentionConfig):
        return PartSpec("sigmoid_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale,
            "eps": cfg.norm_eps, "mix_heads": True, "score_bias": True, "output_gate": True, "window": None,
            "position": PartSpec("rope_interleaved", {"theta": m.rot_base, "dims": m.rot_dims})})
    if isinstance(m, MinGRUConfig):
        return PartSpec("mingru", {"hidden": cfg.width, "width": m.width})
    raise TypeError(f"no part for mixer configuration {m!r}")


def linurax_spec(cfg: LinuraxConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        params = {"hidden": cfg.width, "norm1": norm, "mixer": mixer_spec(cfg, layer), "names": LINURAX_LAYER_NAMES}
        if layer.mlp is not None:
            params["norm2"] = norm
            params["feed_forward"] = PartSpec("swiglu", {"hidden": cfg.width, "intermediate": layer.mlp.ff,
                                                         "names": ("gate", "up", "down")})
        layers.append(LayerSpec(PartSpec("output_norm", params), f"l{i}"))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "scale": cfg.embedding_scale,
                                               "weight_name": ""}),
        embedding_prefix="embed", final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.width}), head_prefix="head",
        tie_word_embeddings=True, max_position_embeddings=NO_POSITION_LIMIT, eos_token_ids=cfg.eos_token_ids)


register_architecture("Linurax", LinuraxConfig, linurax_spec)
