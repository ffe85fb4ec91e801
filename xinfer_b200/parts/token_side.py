"""A layer's own input from the token ids: a small table over the vocabulary, shared by all layers, of which every
layer owns a range of columns.  With e the token's row of the layer's columns,

    y = W_proj ( gelu_tanh(W_gate x) * e )

x being the residual stream as it stands.  The result leaves in the type the residual stream takes its branches
in; a norm on it is the block's business.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import TokenSideSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext, register_feed_forward
from .linear import linear


class TokenSide(FeedForward):
    kind = "token_side"
    graph_safe = True

    def __init__(self, spec: TokenSideSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if not (0 <= spec.column and spec.column + spec.dim <= spec.columns):
            raise ValueError(f"columns {spec.column}..{spec.column + spec.dim} lie outside a table of {spec.columns}")
        self.table = self.w_gate = self.w_proj = None

    @classmethod
    def weight_specs(cls, spec: TokenSideSpec, prefix: str) -> List[WeightSpec]:
        return [WeightSpec(spec.table, (spec.vocab, spec.columns), "unit"),
                WeightSpec(prefix + spec.names[0], (spec.dim, spec.hidden)),
                WeightSpec(prefix + spec.names[1], (spec.hidden, spec.dim))]

    def load(self, store) -> None:
        s = self.spec
        # the layer's own columns of the shared table, as a matrix of its own
        self.table = store.get(s.table, self.device, self.dtype, operand=True, columns=(s.column, s.column + s.dim))
        self.w_gate = store.get(self.prefix + s.names[0], self.device, self.dtype, operand=True)
        self.w_proj = store.get(self.prefix + s.names[1], self.device, self.dtype, operand=True)

    def forward(self, x, ctx: StepContext):
        s = self.spec
        T = x.shape[0]
        ws = ctx.workspace
        u = ws.get("tside.u", (T, s.dim), self.dtype)
        linear(u, x, self.w_gate, ctx.err)
        g = ws.get("tside.g", (T, s.dim), self.dtype)
        kernels.token_gate(g, u, self.table, 0, ctx.token_ids, ctx.sampled, ctx.req_of_token, ctx.err)
        out = ws.get("tside.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        linear(out, g, self.w_proj, ctx.err)
        return out


register_feed_forward("token_side", TokenSide)
