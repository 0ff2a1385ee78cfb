"""Gated linear attention: a matrix of state per head, decayed channel by channel.

Per head, with q and k of ``dim`` numbers and v of ``vdim``: ``S_t = diag(a_t) S_(t-1) + k_t
v_t^T`` (S is dim x vdim, zero before a request's first token; the decay multiplies the rows that
belong to key channels) and ``o_t = S_t^T q_t``.  The decay is ``a = sigmoid(z) ** (1 / tau)``
with ``z = W_a2 (W_a1 h) + b`` (a projection through ``decay_rank`` numbers), q is scaled by ``dim
** -0.5``.  Each head's o is divided by its root mean square over vdim (times a weight shared by
the heads), the heads are joined, multiplied by ``silu(W_g h)`` and projected by W_o.

The state is float32 and lives in a state slot of the request; the projections may run in the
activation type, everything that enters the recurrence after them (the decay from z on, the
scaled q, k, v, the state, the outputs and their norm) is float32 in both precisions.  The
recurrence is walked token by token in one order whatever the step's cut, so a position's result
does not depend on how the prompt was portioned.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import KEEP32, MATRIX, ParamSpec
from .base import Mixer, SlotStateNeed, SlotStateView, StepContext, register_mixer
from .scored_attention import SEQUENCE_TILE


class GatedLinearAttention(Mixer):
    graph_safe = True  # kernels only; launches depend on the step's sizes

    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "decay_down": "a1",
             "decay_up": "a2", "decay_bias": "a2.b"}

    def __init__(self, width: int, heads: int, dim: int, vdim: int, tau: float, decay_rank: int, eps: float = 1e-6,
                 names: Optional[Dict[str, str]] = None):
        for what, v in (("heads", heads), ("dim", dim), ("vdim", vdim), ("decay_rank", decay_rank)):
            if v <= 0:
                raise ValueError(f"gated linear attention: {what} must be positive, got {v}")
        if not tau > 0:
            raise ValueError("gated linear attention: tau must be positive")
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.tau, self.decay_rank, self.eps = float(tau), decay_rank, float(eps)
        self.names = dict(self.NAMES, **(names or {}))
        self.qk_cols, self.v_cols = heads * dim, heads * vdim
        self.w_in = self.w_decay_down = self.w_decay_up = self.decay_bias = self.norm = self.w_o = None

    def cache_need(self):
        return SlotStateNeed((self.heads, self.dim, self.vdim), torch.float32)

    def query_tile_rows(self, ops=None):
        return [SEQUENCE_TILE]

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        n = self.names
        return [ParamSpec(f"{prefix}.{n['q']}", (self.qk_cols, self.width), MATRIX),
                ParamSpec(f"{prefix}.{n['k']}", (self.qk_cols, self.width), MATRIX),
                ParamSpec(f"{prefix}.{n['v']}", (self.v_cols, self.width), MATRIX),
                ParamSpec(f"{prefix}.{n['gate']}", (self.v_cols, self.width), MATRIX),
                ParamSpec(f"{prefix}.{n['out']}", (self.width, self.v_cols), MATRIX),
                ParamSpec(f"{prefix}.{n['norm']}", (self.vdim,), KEEP32, init="ones"),
                ParamSpec(f"{prefix}.{n['decay_down']}", (self.decay_rank, self.width), MATRIX),
                ParamSpec(f"{prefix}.{n['decay_up']}", (self.qk_cols, self.decay_rank), MATRIX),
                ParamSpec(f"{prefix}.{n['decay_bias']}", (self.qk_cols,), KEEP32)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        n = self.names
        # one product yields rows laid out [q | k | v | gate]
        self.w_in = torch.cat([state[f"{prefix}.{n[k]}"] for k in ("q", "k", "v", "gate")], 0).contiguous()
        self.w_decay_down = state[f"{prefix}.{n['decay_down']}"]
        self.w_decay_up = state[f"{prefix}.{n['decay_up']}"]
        self.decay_bias = state[f"{prefix}.{n['decay_bias']}"]
        self.norm = state[f"{prefix}.{n['norm']}"]
        self.w_o = state[f"{prefix}.{n['out']}"]

    def param_bytes(self) -> int:
        ts = (self.w_in, self.w_decay_down, self.w_decay_up, self.decay_bias, self.norm, self.w_o)
        return sum(t.numel() * t.element_size() for t in ts)

    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor, cache: SlotStateView,
                accumulate: bool = True) -> None:
        """``accumulate`` False: the output is written to ``x`` instead of added to it."""
        ops, ws, n = ctx.ops, ctx.workspace, ctx.n
        u = ws.rows("gla_in32", n, 2 * self.qk_cols + 2 * self.v_cols, torch.float32)
        ops.linear(xn, self.w_in, u)
        low = ws.rows("gla_decay_low", n, self.decay_rank, ctx.act_dtype)
        ops.linear(xn, self.w_decay_down, low)
        z = ws.rows("gla_decay32", n, self.qk_cols, torch.float32)
        ops.linear(low, self.w_decay_up, z)
        gated = ws.rows("gla_out", n, self.v_cols, ctx.act_dtype)
        o32 = ws.rows("gla_out32", n, self.v_cols, torch.float32)
        ops.gla_scan(u, z, self.decay_bias, self.tau, cache.state, self.norm, self.eps, gated, self.heads, self.dim,
                     self.vdim, self.dim ** -0.5, ctx, ctx.query_tiles(SEQUENCE_TILE), scratch=o32)
        ops.linear(gated, self.w_o, x, residual=x if accumulate else None)


register_mixer("gated_linear_attention", GatedLinearAttention)
