"""A state-space mixer in the form of Mamba-2 (state-space duality).

    [z | x | B | C | dt] = W_in h                 z, x: heads * head_dim;  B, C: groups * state;  dt: heads
    [x | B | C] <- silu(conv([x | B | C]))        a causal convolution per channel, with a bias
    dt <- softplus(dt + dt_bias)
    S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T       per head, S of state x head_dim, zero at a sequence's start
    y_t = S_t^T C_t + D x_t
    out = W_o ( rms_norm_in_parts(y * silu(z)) * w )       gated first, normed second

The projection leaves float32; the convolution, the step sizes, the decays, the state and the gated norm are
float32 in both engine types.  A request keeps the state matrices and the convolution's last inputs in its row of
the engine's per-request state tables.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import SelectiveStateSpec
from ..weights.loader import WeightSpec
from .base import Mixer, StepContext, register_mixer
from .linear import linear


class SelectiveState(Mixer):
    kind = "selective_state"
    graph_safe = True

    def __init__(self, spec: SelectiveStateSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.heads % spec.groups:
            raise ValueError(f"{spec.heads} heads do not divide into {spec.groups} groups")
        if (spec.heads * spec.head_dim) % spec.norm_groups:
            raise ValueError(f"{spec.heads * spec.head_dim} channels do not divide into {spec.norm_groups} norm parts")
        if not (1 <= spec.conv <= kernels.CONV_MAX_TAPS):
            raise ValueError(f"a short convolution has 1 to {kernels.CONV_MAX_TAPS} taps, got {spec.conv}")
        self.inner = spec.heads * spec.head_dim
        self.conv_channels = self.inner + 2 * spec.groups * spec.state
        self.w_in = self.w_o = self.taps = self.conv_bias = self.dt_bias = self.a_log = self.d_skip = self.norm_w = None

    @classmethod
    def weight_specs(cls, spec: SelectiveStateSpec, prefix: str) -> List[WeightSpec]:
        n = spec.names
        inner, H = spec.heads * spec.head_dim, spec.heads
        C = inner + 2 * spec.groups * spec.state
        return [WeightSpec(prefix + n[0], (inner + C + H, spec.hidden)),
                WeightSpec(prefix + n[1], (C, spec.conv), "unit"), WeightSpec(prefix + n[1] + ".b", (C,), "around_zero"),
                WeightSpec(prefix + n[2], (H,), "unit"), WeightSpec(prefix + n[3], (H,), "around_zero"),
                WeightSpec(prefix + n[4], (H,), "norm"), WeightSpec(prefix + n[5], (inner,), "norm"),
                WeightSpec(prefix + n[6], (spec.hidden, inner))]

    def load(self, store) -> None:
        p, n = self.prefix, self.spec.names

        def f32(name):
            return store.get(p + name, self.device, torch.float32).float().contiguous()
        self.w_in = store.get(p + n[0], self.device, self.dtype, operand=True)
        self.w_o = store.get(p + n[6], self.device, self.dtype, operand=True)
        self.taps, self.conv_bias = f32(n[1]), f32(n[1] + ".b")
        self.dt_bias, self.a_log, self.d_skip, self.norm_w = f32(n[2]), f32(n[3]), f32(n[4]), f32(n[5])

    def state_need(self):
        s = self.spec
        need = {"S": ((s.heads, s.state, s.head_dim), torch.float32)}
        if s.conv > 1:
            need["conv"] = ((s.conv - 1, self.conv_channels), torch.float32)
        return need

    def forward(self, x, ctx: StepContext, cache=None, state=None, writes_cache: bool = True):
        s = self.spec
        T, inner, C = x.shape[0], self.inner, self.conv_channels
        ws = ctx.workspace
        proj = ws.get("sstate.proj", (T, inner + C + s.heads), torch.float32)
        linear(proj, x, self.w_in, ctx.err)
        xbc = ws.get("sstate.xbc", (T, C), torch.float32)
        kernels.conv_silu(xbc, proj, inner, self.taps, self.conv_bias, state.get("conv"), ctx.req_of_token, ctx.q_start,
                          ctx.slots, ctx.num_entries)
        y = ws.get("sstate.y", (T, inner), torch.float32)
        kernels.selective_scan(y, xbc, proj, inner + C, self.dt_bias, self.a_log, self.d_skip, state["S"], ctx.q_start,
                               ctx.slots, ctx.num_entries, s.heads, s.head_dim, s.state, s.groups)
        gated = ws.get("sstate.gated", (T, inner), self.dtype)
        kernels.gated_head_norm(gated, y, proj, 0, self.norm_w, inner // s.norm_groups, s.eps, gate_after=False)
        out = ws.get("sstate.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        linear(out, gated, self.w_o, ctx.err)
        return out


register_mixer("selective_state", SelectiveState)
