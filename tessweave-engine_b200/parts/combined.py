"""Mixers made of other mixers."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import (Mixer, PartSpec, Runtime, SeveralNeeds, SeveralViews, StepContext, WeightDecl, build_part, dense_delta,
                   join_name, register_part)


@register_part("mixer", "weighted_sum")
class WeightedSumMixer(Mixer):
    """Several mixers side by side on the same input: delta = sum_m scale_m * mixer_m(h).

    ``members``: (checkpoint prefix, mixer spec, scale) per member, in order.  Each member keeps the cache or
    state it needs itself (``SeveralNeeds`` / ``SeveralViews``, in the members' order); the sum is formed in fp32
    and rounded once.
    """

    def __init__(self, runtime: Runtime, hidden: int, members: tuple):
        super().__init__(runtime)
        if not members:
            raise ValueError("weighted_sum: at least one member")
        self.hidden = hidden
        self.prefixes = [str(p) for p, _, _ in members]
        self.scales = [float(s) for _, _, s in members]
        self.members = [build_part("mixer", spec, runtime) for _, spec, _ in members]
        self.graph_safe = all(m.graph_safe for m in self.members)

    def weights(self) -> list[WeightDecl]:
        return [WeightDecl(join_name(prefix, w.name), w.shape, w.role, w.init, w.dest)
                for prefix, member in zip(self.prefixes, self.members) for w in member.weights()]

    def redundant_names(self) -> list[str]:
        return [join_name(prefix, n) for prefix, member in zip(self.prefixes, self.members) for n in member.redundant_names()]

    def finalize(self) -> None:
        for member in self.members:
            member.finalize()

    def cache_need(self) -> SeveralNeeds:
        return SeveralNeeds(tuple(member.cache_need() for member in self.members))

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        if not isinstance(cache, SeveralViews) or len(cache.views) != len(self.members):
            raise TypeError("weighted_sum needs one cache view per member")
        n, dt = ctx.n_tokens, self.runtime.dtype
        acc = ctx.workspace.get("weighted_sum.acc", (n, self.hidden), torch.float32)
        out = ctx.workspace.get("weighted_sum.delta", (n, self.hidden), dt)
        last = len(self.members) - 1
        for i, (member, scale, view) in enumerate(zip(self.members, self.scales, cache.views)):
            delta = dense_delta(ctx, member.forward(ctx, h, view, write_cache), dt)[:n]
            ops.scaled_accumulate(acc, out if i == last else None, delta, scale, first=(i == 0))
        return out
