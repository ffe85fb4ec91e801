"""The gated delta rule: a matrix state per head that forgets per key channel, corrects what it holds under the
current key towards the current value, and is read by the query after the token's own write.

    q = W_q h, k = W_k h (kv_heads x head_dim), v = W_v h (heads x v_head_dim); each through a causal convolution
    per channel and SiLU; q, k -> unit vectors per head, q also times head_dim^-1/2
    beta = sigmoid(W_b h)                                   per head
    g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) + dt_bias))    per head and key channel
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out = W_o ( o / rms(o) * w * sigmoid(W_g2 (W_g1 h)) )   norm per head, w shared by the heads

Three products feed it: [q | k | v | beta] (float32 out), the two low-rank maps' first halves side by side, and
their second halves as one block-diagonal product (float32 out).  The convolutions, unit norms, decays, beta,
the state and the output norm and gate are float32 in both engine types.  A request keeps the state matrices and
the convolutions' last inputs in its row of the engine's per-request state tables.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import GatedDeltaSpec
from ..weights.loader import WeightSpec
from .base import Mixer, StepContext, register_mixer
from .linear import linear


class GatedDelta(Mixer):
    kind = "gated_delta"
    graph_safe = True

    def __init__(self, spec: GatedDeltaSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.heads % spec.kv_heads:
            raise ValueError(f"{spec.heads} heads do not divide into {spec.kv_heads} query/key heads")
        if not (1 <= spec.conv <= kernels.CONV_MAX_TAPS):
            raise ValueError(f"a short convolution has 1 to {kernels.CONV_MAX_TAPS} taps, got {spec.conv}")
        self.qk = spec.kv_heads * spec.head_dim
        self.vw = spec.heads * spec.v_head_dim
        self.conv_channels = 2 * self.qk + self.vw
        self.w_main = self.w_low = self.w_second = self.w_o = None
        self.taps = self.dt_bias = self.a_log = self.norm_w = None

    @classmethod
    def weight_specs(cls, spec: GatedDeltaSpec, prefix: str) -> List[WeightSpec]:
        G, H, d, dv, K = spec.kv_heads, spec.heads, spec.head_dim, spec.v_head_dim, spec.conv
        ra = -1 if spec.decay_rank is None else spec.decay_rank
        rg = -1 if spec.gate_rank is None else spec.gate_rank
        R = spec.DEFAULT_RANK
        return [WeightSpec(prefix + "q", (G * d, spec.hidden)), WeightSpec(prefix + "q.conv", (G * d, K), "unit"),
                WeightSpec(prefix + "k", (G * d, spec.hidden)), WeightSpec(prefix + "k.conv", (G * d, K), "unit"),
                WeightSpec(prefix + "v", (H * dv, spec.hidden)), WeightSpec(prefix + "v.conv", (H * dv, K), "unit"),
                WeightSpec(prefix + "b", (H, spec.hidden)), WeightSpec(prefix + "A_log", (H,), "around_zero"),
                WeightSpec(prefix + "norm", (dv,), "norm"),
                WeightSpec(prefix + "a1", (ra, spec.hidden), "linear", R), WeightSpec(prefix + "a2", (H * d, ra), "linear", R),
                WeightSpec(prefix + "dt_bias", (H * d,), "unit"),
                WeightSpec(prefix + "g1", (rg, spec.hidden), "linear", R), WeightSpec(prefix + "g2", (H * dv, rg), "linear", R),
                WeightSpec(prefix + "o", (spec.hidden, H * dv))]

    def load(self, store) -> None:
        p, s = self.prefix, self.spec

        def operand(name):
            return store.get(p + name, self.device, self.dtype, operand=True)

        def f32(name):
            return store.get(p + name, self.device, torch.float32).float().contiguous()
        self.w_main = torch.cat([operand("q"), operand("k"), operand("v"), operand("b")], dim=0).contiguous()
        a1, g1, a2, g2 = operand("a1"), operand("g1"), operand("a2"), operand("g2")
        ra, rg = a1.shape[0], g1.shape[0]
        if a2.shape[1] != ra or g2.shape[1] != rg:
            raise ValueError(f"'{p}': the two halves of a low-rank map disagree about its inner size")
        self.w_low = torch.cat([a1, g1], dim=0).contiguous()
        # the second halves as one block-diagonal matrix over [a1 h | g1 h] (the zero blocks add exact zeros)
        second = torch.zeros((a2.shape[0] + g2.shape[0], ra + rg), dtype=self.dtype, device=self.device)
        second[: a2.shape[0], :ra] = a2
        second[a2.shape[0]:, ra:] = g2
        self.w_second = second
        self.w_o = operand("o")
        self.taps = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).contiguous()
        self.dt_bias, self.a_log, self.norm_w = f32("dt_bias"), f32("A_log"), f32("norm")

    def state_need(self):
        s = self.spec
        need = {"S": ((s.heads, s.head_dim, s.v_head_dim), torch.float32)}
        if s.conv > 1:
            need["conv"] = ((s.conv - 1, self.conv_channels), torch.float32)
        return need

    def forward(self, x, ctx: StepContext, cache=None, state=None, writes_cache: bool = True):
        s = self.spec
        T, C, H = x.shape[0], self.conv_channels, s.heads
        ws = ctx.workspace
        proj = ws.get("gdelta.proj", (T, C + H), torch.float32)
        linear(proj, x, self.w_main, ctx.err)
        low = ws.get("gdelta.low", (T, self.w_low.shape[0]), self.dtype)
        linear(low, x, self.w_low, ctx.err)
        ag = ws.get("gdelta.ag", (T, self.w_second.shape[0]), torch.float32)
        linear(ag, low, self.w_second, ctx.err)
        qkv = ws.get("gdelta.qkv", (T, C), torch.float32)
        kernels.conv_silu(qkv, proj, 0, self.taps, None, state.get("conv"), ctx.req_of_token, ctx.q_start, ctx.slots,
                          ctx.num_entries)
        o = ws.get("gdelta.o", (T, self.vw), torch.float32)
        kernels.delta_rule(o, qkv, proj, C, ag, self.dt_bias, self.a_log, state["S"], ctx.q_start, ctx.slots, ctx.num_entries,
                           H, s.kv_heads, s.head_dim, s.v_head_dim, s.unit_eps)
        gated = ws.get("gdelta.gated", (T, self.vw), self.dtype)
        kernels.gated_head_norm(gated, o, ag, H * s.head_dim, self.norm_w, s.v_head_dim, s.eps, gate_after=True)
        out = ws.get("gdelta.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        linear(out, gated, self.w_o, ctx.err)
        return out


register_mixer("gated_delta", GatedDelta)
