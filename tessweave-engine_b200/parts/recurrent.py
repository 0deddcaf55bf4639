"""Recurrent mixers: a state of fixed size per request instead of a cache that grows."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FixedState, Mixer, Runtime, StateView, StepContext, WeightDecl, register_part
from .linear import linear


@register_part("mixer", "mingru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token.

        z = sigmoid(h Wz^T + bz),  u = h Wx^T + bx,  c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
        S_t = (1 - z_t) S_{t-1} + z_t c_t            element by element, fp32, zero before the first token
        delta = (S_t * silu(h Wg^T)) Wo^T

    The state (``width`` fp32 values per request) lives in a slot of the cache manager, which zeroes it
    when a request is admitted; a step reads it at a request's first row and writes it back after its
    last, so prompts may be cut anywhere.  z, u and the gate are one packed product [Wz; Wx; Wg].

    ``names`` gives the checkpoint's tensor names: z, z_bias, x, x_bias, gate, out.
    """

    NAMES = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "gate": "g", "out": "o"}

    def __init__(self, runtime: Runtime, hidden: int, width: int, names: dict[str, str] | None = None):
        super().__init__(runtime)
        if min(hidden, width) <= 0:
            raise ValueError("mingru needs positive sizes")
        self.hidden, self.width = hidden, width
        self.names = {**self.NAMES, **(names or {})}
        self.w_in = runtime.empty(3 * width, hidden)                  # rows [Wz; Wx; Wg]
        self.b_z = runtime.empty(width, dtype=torch.float32)
        self.b_x = runtime.empty(width, dtype=torch.float32)
        self.w_o = runtime.empty(hidden, width)

    def weights(self) -> list[WeightDecl]:
        w, nm = self.width, self.names
        return [WeightDecl(nm["z"], (w, self.hidden), dest=self.w_in[:w]),
                WeightDecl(nm["z_bias"], (w,), role="vector", dest=self.b_z),
                WeightDecl(nm["x"], (w, self.hidden), dest=self.w_in[w:2 * w]),
                WeightDecl(nm["x_bias"], (w,), role="vector", dest=self.b_x),
                WeightDecl(nm["gate"], (w, self.hidden), dest=self.w_in[2 * w:]),
                WeightDecl(nm["out"], (self.hidden, w), dest=self.w_o)]

    def cache_need(self) -> FixedState:
        return FixedState(self.width, torch.float32)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        if not isinstance(cache, StateView):
            raise TypeError("mingru needs a fixed-size state per request")
        return self.project_out(ctx, self.recur(ctx, self.project_in(ctx, h), cache, write_cache))

    def project_in(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        """h @ [Wz; Wx; Wg].T, rows [z | x | gate] before their biases and activations."""
        return linear(ctx, "mingru.in", h, self.w_in)

    def recur(self, ctx: StepContext, proj: torch.Tensor, cache: StateView, write_state: bool = True) -> torch.Tensor:
        """[rows, width]: S_t * silu(gate) for the step's rows; the requests' states move on."""
        out = ctx.workspace.get("mingru.out", (ctx.n_tokens, self.width), self.runtime.dtype)
        ops.mingru_scan(out, proj, self.b_z, self.b_x, cache.state, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len,
                        ctx.n_seqs, ctx.max_q_len, self.width, write_state)
        return out

    def project_out(self, ctx: StepContext, out: torch.Tensor):
        return linear(ctx, "mixer.delta", out, self.w_o, allow_split=True)
