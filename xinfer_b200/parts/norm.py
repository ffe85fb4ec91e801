"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * (offset + w)``, statistics and weight product in
float32 (src/models/layers/others.rs:22-46, 65-85), with the fused form that first adds a branch
to the residual stream and returns both the sum and its norm (others.rs:48-62, 87-125)."""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import DynamicTanhSpec, NormSpec
from ..weights.loader import WeightSpec
from .base import Norm, register_norm


class RMSNorm(Norm):
    """Over a float32 residual stream it can take the whole residual step around it into its kernel: a branch that is
    scaled (``branch_scale``), multiplied by a learned vector (``branch_gain``) and first passed through an RMS norm of
    its own (``branch_norm``) before it is added."""

    kind = "rmsnorm"
    graph_safe = True
    takes_branch_scale = True
    takes_branch_norm = True
    takes_branch_gain = True

    def __init__(self, spec: NormSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.weight = None

    @staticmethod
    def accepts_branch_norm(norm) -> bool:
        return isinstance(norm, RMSNorm) and not isinstance(norm, IdentityNorm)

    @classmethod
    def weight_specs(cls, spec: NormSpec, prefix: str) -> List[WeightSpec]:
        return [WeightSpec(prefix + spec.weight_name, (spec.dim,), spec.init)]

    def load(self, store) -> None:
        # norm weights are held in float32 whatever the activations are (src/models/qwen3.rs:83)
        self.weight = store.get(self.prefix + self.spec.weight_name, self.device, torch.float32).float().contiguous()

    def forward(self, out, x, ctx, branch=None, sum_out=None, rows=None, branch_scale: float = 1.0, branch_norm=None,
                branch_gain=None):
        if branch_scale == 1.0 and branch_norm is None and branch_gain is None and self.weight is not None:
            kernels.rmsnorm(out, x, self.weight, self.spec.eps, ctx.err, branch=branch, sum_out=sum_out,
                            rows=rows, weight_offset=self.spec.weight_offset)
            return out
        chain(out, x, ctx, self, branch, branch_scale, branch_norm, branch_gain, sum_out, rows)
        return out


def chain(out, x, ctx, norm, branch, branch_scale, branch_norm, branch_gain, sum_out, rows):
    """``kernels.rms_chain`` from norm parts: ``norm`` (an RMSNorm, an IdentityNorm or None) acts on the sum,
    ``branch_norm`` (an RMSNorm or None) on the branch."""
    if x.dtype != torch.float32:
        raise kernels.KernelError("a branch with a norm, a gain or a scale of its own is added into a float32 residual stream")
    ident = norm is None or isinstance(norm, IdentityNorm)
    kernels.rms_chain(out, x, None if ident else norm.weight, 0.0 if ident else norm.spec.eps, ctx.err, branch=branch,
                      branch_weight=branch_norm.weight if branch_norm is not None else None,
                      branch_eps=branch_norm.spec.eps if branch_norm is not None else 0.0,
                      branch_offset=branch_norm.spec.weight_offset if branch_norm is not None else 0.0, gain=branch_gain,
                      branch_scale=branch_scale, sum_out=sum_out, rows=rows,
                      weight_offset=0.0 if ident else norm.spec.weight_offset)


class IdentityNorm(RMSNorm):
    """No norm at all: ``out`` receives the sum itself in the engine's type.  It stands where a part reads the
    residual stream directly, and takes the additions that wait for the stream into its one pass like any norm."""

    kind = "identity"

    @classmethod
    def weight_specs(cls, spec: NormSpec, prefix: str) -> List[WeightSpec]:
        return []

    def load(self, store) -> None:
        self.weight = None


class DynamicTanh(Norm):
    """``y = tanh(alpha * x) * w + b``: no mean, no variance, every element alone.  Being elementwise, it can
    take the whole residual step around it into its kernel: a branch that is scaled (``branch_scale``) and first
    passed through a Dynamic Tanh of its own (``branch_norm``) before it is added."""

    kind = "dynamic_tanh"
    graph_safe = True
    takes_branch_scale = True
    takes_branch_norm = True

    def __init__(self, spec: DynamicTanhSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.weight = self.bias = self.alpha = None

    @classmethod
    def weight_specs(cls, spec: DynamicTanhSpec, prefix: str) -> List[WeightSpec]:
        return [WeightSpec(prefix + spec.weight_name, (spec.dim,), "norm"),
                WeightSpec(prefix + spec.bias_name, (spec.dim,), "around_zero"),
                WeightSpec(prefix + spec.alpha_name, (), "norm")]

    def load(self, store) -> None:
        def f32(name):
            return store.get(self.prefix + name, self.device, torch.float32).float().contiguous()
        self.weight, self.bias, self.alpha = f32(self.spec.weight_name), f32(self.spec.bias_name), f32(self.spec.alpha_name)

    def params(self):
        return (self.alpha, self.weight, self.bias)

    def forward(self, out, x, ctx, branch=None, sum_out=None, rows=None, branch_scale: float = 1.0, branch_norm=None):
        kernels.dyt_norm(out, x, self.alpha, self.weight, self.bias, ctx.err, branch=branch, branch_scale=branch_scale,
                         branch_norm=branch_norm.params() if branch_norm is not None else None, sum_out=sum_out, rows=rows)
        return out


register_norm("rmsnorm", RMSNorm)
register_norm("identity", IdentityNorm)
register_norm("dynamic_tanh", DynamicTanh)
