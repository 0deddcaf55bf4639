"""The Sapatar decoder as a ``ModelSpec``.

Pre-norm layers that differ from one another, each with one mixer -- ``wkv`` (time mixing with token-dependent
decays), ``retention`` (linear attention with a constant decay per head), or softmax attention over a sliding
window beside an mLSTM matrix memory, summed with two scales (``weighted_sum`` of ``gqa_attention`` and ``mlstm``)
-- and optionally a mixture-of-experts feed-forward with a shared expert (``routed_experts``).  With ``streams``
the residual is kept as that many parallel copies (block kind ``hyper_pre_norm``), else the block is ``pre_norm``.
A layer may run with an earlier layer's tensors on a cache and state of its own: the schedule then names that layer
again.  Tensor names: ``embed``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1|norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``l<i>.hc1|hc2.in|out|mix``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sapatar_config import (MlstmConfig, ParallelConfig, RetentionConfig, SapatarConfig, SapatarLayer,
                                     WindowAttentionConfig, WkvConfig)
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry

SAPATAR_LAYER_NAMES = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp"}
ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}
NO_POSITION_LIMIT = 2 ** 31 - 1        # the design has no table of positions; int32 positions bound a request


def window_attention_spec(cfg: SapatarConfig, m: WindowAttentionConfig) -> PartSpec:
    return PartSpec("gqa_attention", {
        "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
        "qkv_bias": True, "scale": m.scale, "window": m.window, "names": ATTENTION_NAMES,
        "position": PartSpec("rope", {"theta": m.rot.base, "dims": m.rot.dims})})


def mlstm_spec(cfg: SapatarConfig, m: MlstmConfig) -> PartSpec:
    return PartSpec("mlstm", {"hidden": cfg.width, "n_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
                              "gate_cap": m.gate_cap, "eps": cfg.norm_eps})


def mixer_spec(cfg: SapatarConfig, layer: SapatarLayer, where: str) -> PartSpec:
    m = layer.mixer
    if isinstance(m, WkvConfig):
        if m.decay_rank is None:
            raise ValueError(f"{where}: the inner size of the decay projection is known neither from 'decay_rank' nor from a checkpoint")
        return PartSpec("wkv", {"hidden": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "decay_rank": m.decay_rank,
                                "eps": cfg.norm_eps})
    if isinstance(m, RetentionConfig):
        return PartSpec("retention", {"hidden": cfg.width, "n_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
                                      "decay": m.decay, "eps": cfg.norm_eps,
                                      "position": PartSpec("rope", {"theta": m.rot.base, "dims": m.rot.dims})})
    if isinstance(m, ParallelConfig):
        return PartSpec("weighted_sum", {"hidden": cfg.width, "members": (
            ("left", window_attention_spec(cfg, m.left), m.left_scale),
            ("right", mlstm_spec(cfg, m.right), m.right_scale))})
    raise TypeError(f"no part for mixer configuration {m!r}")


def sapatar_spec(cfg: SapatarConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""})
    layers, spec_index, schedule = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            schedule.append(ScheduleEntry(spec_index[layer.weights_of]))
            continue
        params = {"hidden": cfg.width, "norm1": norm, "mixer": mixer_spec(cfg, layer, f"layers[{i}]"),
                  "names": SAPATAR_LAYER_NAMES}
        if layer.mlp is not None:
            mlp = layer.mlp
            shared = None
            if mlp.shared_ff is not None:
                shared = PartSpec("swiglu", {"hidden": cfg.width, "intermediate": mlp.shared_ff, "names": ("gate", "up", "down")})
            params["norm2"] = norm
            params["feed_forward"] = PartSpec("routed_experts", {
                "hidden": cfg.width, "experts": mlp.experts, "top": mlp.top, "intermediate": mlp.ff, "shared": shared,
                "shared_gate": shared is not None})
        if cfg.streams is not None:
            block = PartSpec("hyper_pre_norm", {**params, "copies": cfg.streams})
        else:
            block = PartSpec("pre_norm", params)
        spec_index[i] = len(layers)
        layers.append(LayerSpec(block, f"l{i}"))
        schedule.append(ScheduleEntry(spec_index[i]))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
        schedule=tuple(schedule),
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "weight_name": ""}),
        embedding_prefix="embed", final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": cfg.width, "weight_name": ""}), head_prefix="head",
        tie_word_embeddings=False, max_position_embeddings=NO_POSITION_LIMIT, eos_token_ids=cfg.eos_token_ids)


register_architecture("Sapatar", SapatarConfig, sapatar_spec)
