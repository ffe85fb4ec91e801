"""Two mixers side by side on the same input: ``left_scale * left(h) + right_scale * right(h)``.

Both mixers must end in an output projection and offer their halves (``Mixer.inner_width``): their inner
activations, each times its scale, are written side by side into one buffer and ONE product with the
concatenated output matrices ``[W_o left | W_o right]`` forms the scaled sum in its float32 accumulators.
Tensor names: the left mixer's under ``left.``, the right one's under ``right.``.  At most one of the two
may keep pages; both may keep per-request state.

With ``out_norms`` every mixer's finished result is RMS-normed over the model width with a weight of its own
before the scaled sum: the two mixers then run whole, each with its own output projection, and one kernel norms
both and adds them.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..config.plan import ParallelMixerSpec
from ..weights.loader import WeightSpec
from .base import LayerCache, Mixer, StepContext, build_part, part_class, register_mixer
from .linear import linear


class ParallelMixer(Mixer):
    kind = "parallel"

    def __init__(self, spec: ParallelMixerSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.left: Mixer = build_part("mixer", spec.left, prefix + "left.", dtype, device)
        self.right: Mixer = build_part("mixer", spec.right, prefix + "right.", dtype, device)
        self.norm_l = self.norm_r = None
        for name, m in (("left", self.left), ("right", self.right)):
            if spec.out_norms is None and m.inner_width() is None:
                raise ValueError(f"the {name} mixer ('{m.kind}') does not offer its output projection separately")
        if self.left.cache_need() is not None and self.right.cache_need() is not None:
            raise ValueError("only one of two parallel mixers may keep pages")
        self.graph_safe = bool(self.left.graph_safe and self.right.graph_safe)
        self.w_o = None

    @classmethod
    def weight_specs(cls, spec: ParallelMixerSpec, prefix: str) -> List[WeightSpec]:
        out = (part_class("mixer", spec.left.kind).weight_specs(spec.left, prefix + "left.")
               + part_class("mixer", spec.right.kind).weight_specs(spec.right, prefix + "right."))
        if spec.out_norms is not None:
            out += [WeightSpec(prefix + n, (spec.hidden,), "norm") for n in spec.out_norms]
        return out

    def load(self, store) -> None:
        self.left.load(store)
        self.right.load(store)
        if self.spec.out_norms is not None:
            self.norm_l, self.norm_r = (store.get(self.prefix + n, self.device, torch.float32).float().contiguous()
                                        for n in self.spec.out_norms)
            return
        self.w_o = torch.cat([self.left.output_weight(), self.right.output_weight()], dim=1).contiguous()

    def cache_need(self):
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self) -> Optional[Dict]:
        out = {}
        for tag, m in (("left.", self.left), ("right.", self.right)):
            for name, v in (m.state_need() or {}).items():
                out[tag + name] = v
        return out or None

    def prepare_step(self, ctx: StepContext, cache: Optional[LayerCache]) -> None:
        self.left.prepare_step(ctx, cache if self.left.cache_need() is not None else None)
        self.right.prepare_step(ctx, cache if self.right.cache_need() is not None else None)

    @staticmethod
    def _own(state, tag: str):
        if not state:
            return None
        return {k[len(tag):]: v for k, v in state.items() if k.startswith(tag)} or None

    def forward(self, x, ctx: StepContext, cache, state=None, writes_cache: bool = True):
        s = self.spec
        T = x.shape[0]
        if s.out_norms is not None:
            lo = self.left.forward(x, ctx, cache if self.left.cache_need() is not None else None, self._own(state, "left."),
                                   writes_cache)
            ro = self.right.forward(x, ctx, cache if self.right.cache_need() is not None else None, self._own(state, "right."),
                                    writes_cache)
            out = ctx.workspace.get("parallel.out", (T, s.hidden), lo.dtype)
            kernels.dual_rms_sum(out, lo, ro, self.norm_l, self.norm_r, s.out_norm_eps, s.left_scale, s.right_scale,
                                 s.out_norm_offset)
            return out
        wl, wr = self.left.inner_width(), self.right.inner_width()
        inner = ctx.workspace.get("parallel.inner", (T, wl + wr), self.dtype)
        self.left.forward_inner(x, ctx, cache if self.left.cache_need() is not None else None, self._own(state, "left."),
                                writes_cache, inner[:, :wl], s.left_scale)
        self.right.forward_inner(x, ctx, cache if self.right.cache_need() is not None else None, self._own(state, "right."),
                                 writes_cache, inner[:, wl:], s.right_scale)
        out = ctx.workspace.get("parallel.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        linear(out, inner, self.w_o, ctx.err)
        return out


register_mixer("parallel", ParallelMixer)
