"""Sigmoid attention with mixed heads over a paged cache."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PagedKV, PagedView, PartSpec, Runtime, StepContext, WeightDecl, build_part, register_part
from .linear import linear


@register_part("mixer", "sigmoid_attention")
class SigmoidAttention(Mixer):
    """Grouped-query attention whose weights are sigmoids, not a softmax, and whose values are its keys.

        q = rms(h Wq^T) * nq,  k = rms(h Wk^T) * nk        each norm over the whole projection, all heads at once
        v = h Wk^T                                          the key as projected: no norm, no rotation, no Wv
        q, k = position(q), position(k)
        s_g(i, j)  = scale * q_g(i) . k_{g // group}(j)     j <= i [, j > i - window]
        s'_h(i, j) = sum_g M[h, g] s_g(i, j)                M [H, H] mixes the heads' scores   (``mix_heads``)
        w_h(i, j)  = sigmoid(s'_h(i, j) + b_h)              b [H]                               (``score_bias``)
        o_h(i)     = sum_j w_h(i, j) v_{h // group}(j)      not normalised over j
        delta      = (o * sigmoid(h Wg^T)) Wo^T             the gate reads the mixer's input   (``output_gate``)

    The cache holds two things per position and key/value head: the normalised, rotated key and the raw key
    (as the value).  q, k and the gate are one packed product [Wq; Wk; Wg].  The mixing of heads is linear in
    the queries and is folded into them once per token (csrc/sigmoid_attention.cu), so the kernels that meet
    the keys see ordinary heads with a query of ``n_kv_heads * head_dim`` values.

    ``names`` gives the checkpoint's tensor names: q, k, q_norm, k_norm, mix, bias, gate, out.
    """

    NAMES = {"q": "q", "k": "k", "q_norm": "q.norm", "k_norm": "k.norm", "mix": "talk", "bias": "pb", "gate": "g",
             "out": "o"}

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 eps: float, position: PartSpec, mix_heads: bool = True, score_bias: bool = True,
                 output_gate: bool = True, window: int | None = None, names: dict[str, str] | None = None):
        super().__init__(runtime)
        if min(hidden, n_heads, n_kv_heads, head_dim) <= 0 or n_heads % n_kv_heads:
            raise ValueError("sigmoid attention: heads must be positive and n_heads a multiple of n_kv_heads")
        if head_dim > 256:
            raise ValueError(f"sigmoid attention: head_dim {head_dim} above 256 is not supported")
        if window is not None and window <= 0:
            raise ValueError("sigmoid attention: window must be positive or None")
        if not eps > 0:
            raise ValueError("sigmoid attention: eps must be positive")
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.scale, self.eps, self.window = float(scale), float(eps), window
        self.names = {**self.NAMES, **(names or {})}
        self.q_size, self.kv_size = n_heads * head_dim, n_kv_heads * head_dim
        self.gate_size = self.q_size if output_gate else 0
        self.position = build_part("position", position, runtime)
        self.w_in = runtime.empty(self.q_size + self.kv_size + self.gate_size, hidden)      # rows [Wq; Wk; Wg]
        self.q_norm = runtime.empty(self.q_size, dtype=torch.float32)
        self.k_norm = runtime.empty(self.kv_size, dtype=torch.float32)
        self.mix = runtime.empty(n_heads, n_heads, dtype=torch.float32) if mix_heads else None
        self.bias = runtime.empty(n_heads, dtype=torch.float32) if score_bias else None
        self.w_o = runtime.empty(hidden, self.q_size)

    def weights(self) -> list[WeightDecl]:
        q, kv, nm = self.q_size, self.kv_size, self.names
        decls = [WeightDecl(nm["q"], (q, self.hidden), dest=self.w_in[:q]),
                 WeightDecl(nm["k"], (kv, self.hidden), dest=self.w_in[q:q + kv]),
                 WeightDecl(nm["q_norm"], (q,), role="vector", init="one_plus_normal", dest=self.q_norm),
                 WeightDecl(nm["k_norm"], (kv,), role="vector", init="one_plus_normal", dest=self.k_norm)]
        if self.mix is not None:
            decls.append(WeightDecl(nm["mix"], (self.n_heads, self.n_heads), role="vector", init="eye_plus_normal", dest=self.mix))
        if self.bias is not None:
            decls.append(WeightDecl(nm["bias"], (self.n_heads,), role="vector", dest=self.bias))
        if self.gate_size:
            decls.append(WeightDecl(nm["gate"], (q, self.hidden), dest=self.w_in[q + kv:]))
        decls.append(WeightDecl(nm["out"], (self.hidden, q), dest=self.w_o))
        return decls

    def cache_need(self) -> PagedKV:
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        if not isinstance(cache, PagedView):
            raise TypeError("sigmoid_attention needs a paged key/value cache")
        return self.project_out(ctx, self.attend(ctx, self.project_in(ctx, h), cache, write_cache))

    def project_in(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        """h @ [Wq; Wk; Wg].T, rows [q | k | gate]."""
        return linear(ctx, "sigattn.in", h, self.w_in)

    def prepare(self, ctx: StepContext, proj: torch.Tensor, cache: PagedView, write_cache: bool) -> torch.Tensor:
        """Norms, rotation, cache write and the folded queries [rows, Hq, Hkv * D] of the step's rows."""
        n = ctx.n_tokens
        qf = ctx.workspace.get("sigattn.qf", (n, self.n_heads, self.kv_size), self.runtime.dtype)
        plan = self.position.rotary_plan(self.head_dim)
        if plan is None:
            raise NotImplementedError("sigmoid_attention needs a position encoding that is a rotation of pairs "
                                      "(its norm runs before the rotation, inside one kernel)")
        ops.sigmoid_attention_prepare(qf, proj, self.q_norm, self.k_norm, self.eps, self.mix, self.scale,
                                      plan.inv_freq if plan.rot_dims else None, plan.rot_dims, plan.interleaved,
                                      ctx.positions, ctx.seq_of_token, ctx.seq_slot, cache.block_table, cache.k_pages,
                                      cache.v_pages, n, self.n_heads, self.n_kv_heads, self.head_dim, write_cache,
                                      ctx.status)
        return qf

    def attend(self, ctx: StepContext, proj: torch.Tensor, cache: PagedView, write_cache: bool) -> torch.Tensor:
        """[rows, Hq * D]: the gated heads of the step's rows."""
        return self.attend_prepared(ctx, self.prepare(ctx, proj, cache, write_cache), proj, cache)

    def attend_prepared(self, ctx: StepContext, qf: torch.Tensor, proj: torch.Tensor, cache: PagedView) -> torch.Tensor:
        """The attention itself, over the cache as ``prepare`` left it; the gate is read from ``proj``."""
        n = ctx.n_tokens
        out = ctx.workspace.get("sigattn.out", (n, self.q_size), self.runtime.dtype)
        gate = proj[:, self.q_size + self.kv_size:] if self.gate_size else None
        window = self.window or 0
        if not ops.sigmoid_attention_tensor_cores(self.runtime.dtype, self.head_dim, self.n_kv_heads):
            # float32, and shapes the tensor-core kernels do not take: one block per (token, head)
            ops.sigmoid_attention_generic(out, qf, self.bias, gate, ctx.positions, ctx.seq_of_token, ctx.seq_slot,
                                          cache.block_table, cache.k_pages, cache.v_pages, n, self.n_heads, self.n_kv_heads,
                                          self.head_dim, window, ctx.status)
            return out
        # bfloat16: portions on the tile kernel, single tokens on the kernel that cuts their keys into slices; both
        # read the same flat batch and skip the other's requests
        singles = ctx.decode_only or ctx.fixed_shape or any(count == 1 for count in ctx.host_q_len)
        if not ctx.decode_only:
            # long portions: tcgen05 kernel (TMA, S and O in tensor memory); short ones, and the shapes it does not
            # take, stay on the mma.sync kernel, which starts faster
            prefill = ops.sigmoid_attention_prefill
            if ops.sigmoid_attention_tcgen05(self.runtime.dtype, self.head_dim, self.n_kv_heads, cache.k_pages.shape[2],
                                             ctx.max_q_len):
                prefill = ops.sigmoid_attention_prefill_tcgen05
            prefill(out, qf, self.bias, gate, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len,
                                          ctx.seq_slot, cache.block_table, cache.k_pages, cache.v_pages, ctx.n_seqs,
                                          ctx.max_q_len, self.n_heads, self.n_kv_heads, self.head_dim, window, singles,
                                          ctx.status)
        if singles:
            nsplit = ops.sigmoid_decode_splits(ctx.n_seqs, self.n_heads, ctx.max_kv_len)
            partial = ctx.workspace.get("sigattn.partial", (ctx.n_seqs, nsplit, self.n_heads, self.head_dim), torch.float32)
            ops.sigmoid_attention_decode(out, partial, qf, self.bias, gate, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len,
                                         ctx.seq_slot, cache.block_table, cache.k_pages, cache.v_pages, ctx.n_seqs,
                                         self.n_heads, self.n_kv_heads, self.head_dim, window, nsplit, ctx.status)
        return out

    def project_out(self, ctx: StepContext, out: torch.Tensor):
        return linear(ctx, "mixer.delta", out, self.w_o, allow_split=True)
