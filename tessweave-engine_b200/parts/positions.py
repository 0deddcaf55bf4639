"""Position encodings."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import PositionEncoding, RotaryPlan, Runtime, StepContext, register_part


@register_part("position", "rope")
class RotaryEmbedding(PositionEncoding):
    """Rotate-half rotary encoding over the whole head.

    inv_freq[i] = theta ** (-(2 i) / D), angle = float(position) * inv_freq[i], pairs
    (i, i + D/2); all in fp32 (reference: flow_engine/model.py:26-33).  The table of
    inverse frequencies is made on the host with the reference's own expression and
    uploaded once per head size, so the device only multiplies by the position.
    """

    def __init__(self, runtime: Runtime, theta: float):
        super().__init__(runtime)
        if not theta > 0:
            raise ValueError("rope theta must be positive")
        self.theta = float(theta)
        self._tables: dict[int, torch.Tensor] = {}

    def fused_rotary_table(self, head_dim: int) -> torch.Tensor:
        table = self._tables.get(head_dim)
        if table is None:
            if head_dim % 2:
                raise ValueError(f"rope needs an even head_dim, got {head_dim}")
            inv = self.theta ** (-torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)
            table = inv.to(self.runtime.device)
            self._tables[head_dim] = table
        return table

    def rotary_plan(self, head_dim: int) -> RotaryPlan:
        return RotaryPlan(self.fused_rotary_table(head_dim), head_dim, interleaved=False)

    def apply(self, ctx: StepContext, qk: torch.Tensor, n_heads: int, head_dim: int) -> None:
        """Rotate ``n_heads`` heads at the start of each packed row in place (nothing else is touched).
        A mixer with a kernel that rotates on the way (``fused_rotary_table``) gets the same numbers."""
        ops.rotate_heads(qk, None, ctx.positions, ctx.seq_of_token, self.fused_rotary_table(head_dim), ctx.n_tokens,
                         n_heads, head_dim)


@register_part("position", "rope_interleaved")
class InterleavedRotaryEmbedding(PositionEncoding):
    """Rotary encoding on neighbouring pairs, over the first ``dims`` values of a head (all of it when
    ``dims`` is None); the rest of the head passes unchanged.

        f_i = theta ** (-(2 i) / dims),  a = float(position) * f_i,  i < dims / 2
        (x[2i], x[2i+1]) -> (x[2i] cos a - x[2i+1] sin a,  x[2i+1] cos a + x[2i] sin a)

    all in fp32.  The table of f_i is made once per head size on the host.
    """

    def __init__(self, runtime: Runtime, theta: float, dims: int | None = None):
        super().__init__(runtime)
        if not theta > 0:
            raise ValueError("rope theta must be positive")
        if dims is not None and (dims < 0 or dims % 2):
            raise ValueError(f"rope needs an even number of rotated dims, got {dims}")
        self.theta, self.dims = float(theta), dims
        self._plans: dict[int, RotaryPlan] = {}

    def rotary_plan(self, head_dim: int) -> RotaryPlan:
        plan = self._plans.get(head_dim)
        if plan is None:
            dims = head_dim if self.dims is None else self.dims
            if dims > head_dim or dims % 2:
                raise ValueError(f"rope over {dims} dims does not fit a head of {head_dim}")
            inv = self.theta ** (-torch.arange(0, dims, 2, dtype=torch.float32) / max(dims, 1))
            plan = RotaryPlan(inv.to(self.runtime.device), dims, interleaved=True)
            self._plans[head_dim] = plan
        return plan

    def apply(self, ctx: StepContext, qk: torch.Tensor, n_heads: int, head_dim: int) -> None:
        plan = self.rotary_plan(head_dim)
        ops.rotate_pairs(qk, ctx.positions, ctx.seq_of_token, plan.inv_freq, ctx.n_tokens, n_heads, head_dim,
                         plan.rot_dims, plan.interleaved)


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries and keys as they are."""

    def apply(self, ctx: StepContext, qk, n_heads, head_dim) -> None:
        return None
