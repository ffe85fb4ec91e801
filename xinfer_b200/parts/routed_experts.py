"""Mixture of small gated experts chosen by a learned router, with an optional expert that every token runs.

    scores   s = sigmoid(W_router h)                     float32
    choice   on s + correction, among the experts of the ``keep`` best of ``groups`` groups of neighbours
             (a group's score: the sum of its ``group_best`` largest choice scores); the ``top`` largest win
    weights  the chosen experts' plain scores s (optionally divided by their sum)
    expert   W_down_e ( act(W_gate_e h) * f(W_up_e h) ),  no biases; ``act`` by the spec (``kernels.ACTIVATIONS``)
    out      = sum over the token's experts of weight * expert  (+ shared(h))

The router kernel leaves the step's choices and weights on the device, a row per token; from there the forms of
the table-driven experts (``parts/table_experts.py``) are reused with that table in place of one over token ids:

* few tokens in bfloat16 (a decode step): ONE dense product with the gate/up matrices stacked, a kernel that keeps a
  token's own experts (times their weights) and zeroes the others, ONE product with the down matrices side by side;
* otherwise: the (token, choice) pairs are grouped by expert on the device, two grouped products run (gate/up with
  the activation applied in the same kernel, then down), and a last kernel sums a token's experts in the order of
  its choices, each times its weight, onto the shared expert's result;
* large prompt steps in bfloat16: the grouping's offsets (one number per expert) are read back, and each expert's
  contiguous rows go through the library's matrix product (gate/up, the gate kernel, down).  The read waits for the
  device once per layer; where every product is large that costs far less than the grouped kernels lose to the
  library's (about 200 against 1,400 TFLOP/s).

Steps that are (or will be) replayed from a CUDA graph take the first two forms only: nothing comes back to the host.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import RoutedExpertsSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext, build_part, part_class, register_feed_forward
from .linear import linear

# up to this many tokens a bfloat16 step takes the dense form (all experts' matrices are read once, as they would be
# anyway once most experts are in use)
DENSE_MAX_TOKENS = 32
# bfloat16 steps whose products are large enough go through per-expert library products (tests switch it off to reach
# the grouped kernels); rows per expert are rounded up to ROW_STEP so that the library meets few distinct shapes
PER_EXPERT_LIBRARY_PRODUCTS = True
ROW_STEP = 128
LIBRARY_FROM_FLOP_PER_CALL = 8e9


class RoutedExperts(FeedForward):
    kind = "routed_experts"
    graph_safe = True

    def __init__(self, spec: RoutedExpertsSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if not (0 < spec.top <= spec.experts):
            raise ValueError(f"a token cannot use {spec.top} of {spec.experts} experts")
        if spec.groups <= 0 or spec.experts % spec.groups or not (0 < spec.keep <= spec.groups):
            raise ValueError(f"{spec.experts} experts do not form {spec.groups} equal groups of which {spec.keep} are kept")
        if spec.top > spec.keep * (spec.experts // spec.groups):
            raise ValueError(f"{spec.keep} groups of {spec.experts // spec.groups} experts cannot give a token {spec.top}")
        kernels.activation_args(spec.activation, spec.act_params)
        self.shared = None
        if spec.shared is not None:
            self.shared = build_part("feed_forward", spec.shared, prefix + "shared.", dtype, device)
            self.shared.scratch = "experts.shared"
        self.w_gate_up = self.w_down = self.w_router = self.correction = None

    @classmethod
    def weight_specs(cls, spec: RoutedExpertsSpec, prefix: str) -> List[WeightSpec]:
        out = []
        for e in range(spec.experts):
            p = f"{prefix}e{e}."
            out += [WeightSpec(p + "gate", (spec.intermediate, spec.hidden)),
                    WeightSpec(p + "up", (spec.intermediate, spec.hidden)),
                    WeightSpec(p + "down", (spec.hidden, spec.intermediate))]
        out.append(WeightSpec(prefix + "router", (spec.experts, spec.hidden), "unit"))
        if spec.correction:
            out.append(WeightSpec(prefix + "correction", (spec.experts,), "around_zero"))
        if spec.shared is not None:
            out += part_class("feed_forward", spec.shared.kind).weight_specs(spec.shared, prefix + "shared.")
        return out

    def load(self, store) -> None:
        s, p = self.spec, self.prefix
        gu, dn = [], []
        for e in range(s.experts):
            q = f"{p}e{e}."
            gu.append(torch.cat([store.get(q + "gate", self.device, self.dtype, operand=True),
                                 store.get(q + "up", self.device, self.dtype, operand=True)], dim=0))
            dn.append(store.get(q + "down", self.device, self.dtype, operand=True))
        self.w_gate_up = torch.stack(gu).contiguous()      # [experts, 2 ff, hidden]
        self.w_down = torch.cat(dn, dim=1).contiguous()    # [hidden, experts * ff]: side by side along K
        # the router works in float32 whatever the engine's type
        self.w_router = store.get(p + "router", self.device, torch.float32).float().contiguous()
        if s.correction:
            self.correction = store.get(p + "correction", self.device, torch.float32).float().contiguous()
        if self.shared is not None:
            self.shared.load(store)

    def forward(self, x, ctx: StepContext):
        s = self.spec
        T = x.shape[0]
        ws = ctx.workspace
        choice = ws.get("experts.choice", (T, s.top), torch.int32)
        weight = ws.get("experts.weight", (T, s.top), torch.float32)
        kernels.expert_router(choice, weight, x, self.w_router, self.correction, ctx.req_of_token, s.top, s.groups, s.keep,
                              s.group_best, s.renormalize)
        base = self.shared.forward(x, ctx) if self.shared is not None else None
        out = ws.get("experts.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        if self.dtype == torch.bfloat16 and T <= DENSE_MAX_TOKENS:
            gu = ws.get("experts.gu_all", (T, s.experts * 2 * s.intermediate), self.dtype)
            linear(gu, x, self.w_gate_up.view(s.experts * 2 * s.intermediate, s.hidden), ctx.err)
            act = ws.get("experts.act_all", (T, s.experts * s.intermediate), self.dtype)
            kernels.expert_select_gate(act, gu, choice, None, None, ctx.req_of_token, s.top, s.experts, ctx.err,
                                       weights=weight, activation=s.activation, params=s.act_params)
            linear(out, act, self.w_down, ctx.err)
            if base is not None:
                kernels.add(out, out, base)
            return out
        n = T * s.top
        offsets = ws.get("experts.offsets", (s.experts + 1,), torch.int32)
        perm = ws.get("experts.perm", (n,), torch.int32)
        inv = ws.get("experts.inv", (n,), torch.int32)
        kernels.expert_route(offsets, perm, inv, choice, None, None, ctx.req_of_token, T, s.top, s.experts, ctx.err)
        by_library = (PER_EXPERT_LIBRARY_PRODUCTS and self.dtype == torch.bfloat16 and not ctx.fixed_shapes
                      and 6.0 * n * s.hidden * s.intermediate > LIBRARY_FROM_FLOP_PER_CALL * 3 * s.experts)
        if by_library:
            # Each expert's rows are rounded up to a multiple of ROW_STEP.  The extra rows are the next expert's: what
            # is computed for them here is overwritten when that expert's turn comes, and past the last expert lies
            # spare room that nobody reads.
            bounds = offsets.cpu().tolist()         # (the one wait of this form)
            room = n + ROW_STEP
            act = ws.get("experts.act", (room, s.intermediate), self.dtype)
            y = ws.get("experts.y", (room, s.hidden), torch.float32)
            xp = ws.get("experts.x_grouped", (room, s.hidden), self.dtype)
            kernels.expert_gather(xp[:n], x, perm, offsets, s.top)
            gu = ws.get("experts.gate_up", (room, 2 * s.intermediate), self.dtype)
            for e in range(s.experts):
                at, c = bounds[e], bounds[e + 1] - bounds[e]
                if c == 0:
                    continue
                m = min((c + ROW_STEP - 1) // ROW_STEP * ROW_STEP, room - at)
                torch.mm(xp[at:at + m], self.w_gate_up[e].t(), out=gu[at:at + m])
                kernels.swiglu(act[at:at + m], gu[at:at + m], s.activation, s.act_params)
                torch.mm(act[at:at + m], self.w_down[:, e * s.intermediate:(e + 1) * s.intermediate].t(),
                         out_dtype=torch.float32, out=y[at:at + m])
            y = y[:n]
        else:
            act = ws.get("experts.act", (n, s.intermediate), self.dtype)
            y = ws.get("experts.y", (n, s.hidden), torch.float32)
            kernels.expert_gemm(act, x, self.w_gate_up, offsets, perm, True, s.top, True, activation=s.activation,
                                params=s.act_params)
            kernels.expert_gemm(y, act, self.w_down, offsets, perm, False, s.top, False, side_by_side=True)
        kernels.expert_combine(out, y, inv, s.top, weights=weight, base=base)
        return out


register_feed_forward("routed_experts", RoutedExperts)
