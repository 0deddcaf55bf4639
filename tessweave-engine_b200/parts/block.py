"""Arrangements of parts around the residual stream."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import (Block, PartSpec, ResidualStream, Runtime, StepContext, WeightDecl, build_part, join_name,
                   register_part)


class ArrangedBlock(Block):
    """What every arrangement shares: sub-parts under their checkpoint prefixes (``names``), their
    weight declarations, and the mixer's cache need.  A sub-part may be absent (``None``)."""

    ROLES = ("norm1", "mixer", "norm2", "feed_forward")

    def __init__(self, runtime: Runtime, hidden: int, names: dict[str, str] | None = None):
        super().__init__(runtime)
        self.hidden = hidden
        self.names = {role: role for role in self.ROLES}
        self.names.update(names or {})

    def parts(self):
        return {role: getattr(self, role) for role in self.ROLES if getattr(self, role) is not None}

    def weights(self) -> list[WeightDecl]:
        return [WeightDecl(join_name(self.names[role], w.name), w.shape, w.role, w.init, w.dest)
                for role, part in self.parts().items() for w in part.weights()]

    def redundant_names(self) -> list[str]:
        return [join_name(self.names[role], name) for role, part in self.parts().items() for name in part.redundant_names()]

    def finalize(self) -> None:
        for part in self.parts().values():
            part.finalize()

    def cache_need(self):
        return self.mixer.cache_need()


@register_part("block", "pre_norm")
class PreNormBlock(ArrangedBlock):
    """x = x + mixer(norm1(x));  x = x + feed_forward(norm2(x)).

    Reference: flow_engine/model.py:179-202.  The residual stream is fp32; each
    sub-layer's output is handed to the next norm as a pending delta, so the add
    and the norm are one kernel.  ``names`` gives the checkpoint's prefix of each
    sub-part inside the layer.
    """

    def __init__(self, runtime: Runtime, hidden: int, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec,
                 feed_forward: PartSpec, names: dict[str, str] | None = None):
        super().__init__(runtime, hidden, names)
        self.norm1 = build_part("norm", norm1, runtime)
        self.mixer = build_part("mixer", mixer, runtime)
        self.norm2 = build_part("norm", norm2, runtime)
        self.feed_forward = build_part("feed_forward", feed_forward, runtime)
        self.graph_safe = all(p.graph_safe for p in self.parts().values())

    def forward(self, ctx: StepContext, stream: ResidualStream, cache, write_cache: bool) -> None:
        n = ctx.n_tokens
        stream.rounded = None
        h = ctx.workspace.get("block.h", (n, self.hidden), self.runtime.dtype)
        self.norm1.apply(ctx, h, stream.resid, stream.pending, n)
        ctx.upcoming_weights = self.feed_forward.streamed_first()
        delta = self.mixer.forward(ctx, h, cache, write_cache)
        ctx.upcoming_weights = None
        self.norm2.apply(ctx, h, stream.resid, delta, n)
        stream.pending = self.feed_forward.forward(ctx, h)      # whoever normalises next adds it


@register_part("block", "output_norm")
class OutputNormBlock(ArrangedBlock):
    """x = x + norm1(mixer(x));  x = x + norm2(feed_forward(x)): the norm sits on what a sub-layer returns,
    and the sub-layers read the residual rows themselves.  ``feed_forward`` (with ``norm2``) may be None: the
    layer then has its first half only.

    The residual stream stays fp32; the matrix products read a copy of its rows in the run's type, which the
    norm kernel writes while it adds (in float32 runs the stream itself is read).  Nothing is left pending.
    """

    def __init__(self, runtime: Runtime, hidden: int, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec | None = None,
                 feed_forward: PartSpec | None = None, names: dict[str, str] | None = None):
        super().__init__(runtime, hidden, names)
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("output_norm block: norm2 and feed_forward come together or not at all")
        self.norm1 = build_part("norm", norm1, runtime)
        self.mixer = build_part("mixer", mixer, runtime)
        self.norm2 = build_part("norm", norm2, runtime) if norm2 is not None else None
        self.feed_forward = build_part("feed_forward", feed_forward, runtime) if feed_forward is not None else None
        self.graph_safe = all(p.graph_safe for p in self.parts().values())

    def _rows(self, ctx: StepContext, stream: ResidualStream) -> tuple[torch.Tensor, torch.Tensor | None]:
        """(the rows a sub-layer reads, the buffer the next norm writes their successor into)."""
        n = ctx.n_tokens
        if self.runtime.dtype == torch.float32:
            return stream.resid[:n], None
        copy = ctx.workspace.get("block.rows", (n, self.hidden), self.runtime.dtype)
        if stream.rounded is None or stream.rounded.data_ptr() != copy.data_ptr():
            ops.round_rows(copy, stream.resid, n)
        return copy, copy

    def forward(self, ctx: StepContext, stream: ResidualStream, cache, write_cache: bool) -> None:
        n = ctx.n_tokens
        if stream.pending is not None:
            raise RuntimeError("output_norm block: the block before left a delta that only a norm of its own kind can add")
        h, copy = self._rows(ctx, stream)
        ctx.upcoming_weights = self.feed_forward.streamed_first() if self.feed_forward is not None else None
        delta = self.mixer.forward(ctx, h, cache, write_cache)
        ctx.upcoming_weights = None
        self.norm1.add_normed(ctx, stream.resid, delta, n, copy)
        stream.rounded = copy
        if self.feed_forward is not None:
            delta = self.feed_forward.forward(ctx, h)
            self.norm2.add_normed(ctx, stream.resid, delta, n, copy)
