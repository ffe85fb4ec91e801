"""Gated feed-forward: ``down( act(gate(x)) * up(x) )`` with gate and up concatenated into
one projection at load (src/models/layers/mlp.rs:447-466, forward :613-697), no biases.  ``act`` is SiLU
(the reference's), the tanh form of GELU, ReLU, or a clamped swish that also clamps and shifts the up half
(``kernels.ACTIVATIONS``; its parameters come in ``act_params``); the three tensors' names may be given by the spec."""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import FeedForwardSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext, register_feed_forward
from . import gemm_backend
from .linear import linear


_DEFAULT_NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


class SwiGLU(FeedForward):
    kind = "swiglu"
    graph_safe = True

    def __init__(self, spec: FeedForwardSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"the gated feed-forward supports {', '.join(sorted(kernels.ACTIVATIONS))}, not '{spec.activation}'")
        kernels.activation_args(spec.activation, spec.act_params)      # (raises on parameters that do not fit)
        self.names = tuple(spec.names) if spec.names else _DEFAULT_NAMES
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None
        # the workspace buffers' name: a part that holds a feed-forward of this kind inside gives it another
        self.scratch = "ffn"

    @classmethod
    def weight_specs(cls, spec: FeedForwardSpec, prefix: str) -> List[WeightSpec]:
        p = prefix
        n = tuple(spec.names) if spec.names else _DEFAULT_NAMES
        out = [
            WeightSpec(p + n[0], (spec.intermediate, spec.hidden)),
            WeightSpec(p + n[1], (spec.intermediate, spec.hidden)),
            WeightSpec(p + n[2], (spec.hidden, spec.intermediate)),
        ]
        if spec.bias_suffix:
            out += [WeightSpec(p + n[0] + spec.bias_suffix, (spec.intermediate,), "around_zero"),
                    WeightSpec(p + n[1] + spec.bias_suffix, (spec.intermediate,), "around_zero"),
                    WeightSpec(p + n[2] + spec.bias_suffix, (spec.hidden,), "around_zero")]
        return out

    def load(self, store) -> None:
        p = self.prefix
        g = store.get(p + self.names[0], self.device, self.dtype, operand=True)
        u = store.get(p + self.names[1], self.device, self.dtype, operand=True)
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        del g, u
        self.w_down = store.get(p + self.names[2], self.device, self.dtype, operand=True)
        sfx = self.spec.bias_suffix
        if sfx:
            self.b_gate_up = torch.cat([store.get(p + self.names[i] + sfx, self.device, torch.float32).float()
                                        for i in range(2)]).contiguous()
            self.b_down = store.get(p + self.names[2] + sfx, self.device, torch.float32).float().contiguous()

    def forward(self, x, ctx: StepContext):
        s = self.spec
        T = x.shape[0]
        ws = ctx.workspace
        act = ws.get(self.scratch + ".act", (T, s.intermediate), self.dtype)
        if self.b_gate_up is not None:
            # biases: the packed product leaves float32, the gate kernel adds them before the activation
            gu = ws.get(self.scratch + ".gate_up32", (T, 2 * s.intermediate), torch.float32)
            linear(gu, x, self.w_gate_up, ctx.err)
            kernels.swiglu_bias(act, gu, self.b_gate_up, s.activation)
        elif s.activation != "silu" or not gemm_backend.try_fused_gate(act, x, self.w_gate_up, ctx.err):
            gu = ws.get(self.scratch + ".gate_up", (T, 2 * s.intermediate), self.dtype)
            linear(gu, x, self.w_gate_up, ctx.err)
            kernels.swiglu(act, gu, s.activation, s.act_params)
        # the result leaves in the type the residual stream takes its branches in (float32 accumulators unrounded
        # where the stream is float32)
        out = ws.get(self.scratch + ".out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        linear(out, act, self.w_down, ctx.err)
        if self.b_down is not None:
            kernels.add_bias(out, self.b_down)
        return out


register_feed_forward("swiglu", SwiGLU)
