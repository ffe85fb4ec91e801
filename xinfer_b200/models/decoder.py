"""The generic decoder: builds any ``ModelPlan`` from registered parts and runs one step of it.

embedding (times the plan's ``embed_scale``, if it has one) -> the plan's layer runs in order (a run may add the
embedding's output to the stream again: layers that are run several times in a row start every pass but the first so) ->
final norm on the wanted rows -> output head -> the plan's logit scale and soft cap, if any.
(The reference's forward for this architecture: src/models/qwen3.rs:311-374.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import kernels, tracing
from ..config.plan import ModelPlan
from ..parts import Block, LayerCache, StepContext, build_part, part_class
from ..parts.block import Addend, Stream, fused_norm
from ..parts.linear import linear
from ..weights.loader import WeightSpec, WeightStore


def model_weight_specs(plan: ModelPlan) -> List[WeightSpec]:
    """Every tensor the model needs, in file order."""
    specs = [WeightSpec(plan.embed_name, (plan.vocab_size, plan.hidden), "embedding")]
    if plan.pair_embedding is not None:
        specs.append(WeightSpec(plan.pair_embedding.name, (plan.pair_embedding.buckets + 1, plan.hidden), "embedding"))
    if plan.position_table is not None:
        specs.append(WeightSpec(plan.position_table, (plan.max_positions, plan.hidden), "embedding"))
    for b in plan.blocks:
        specs += Block.weight_specs(b)
    specs += part_class("norm", plan.final_norm.kind).weight_specs(plan.final_norm, plan.final_norm_name)
    if plan.head_name is not None:
        specs.append(WeightSpec(plan.head_name, (plan.vocab_size, plan.hidden), "linear"))
    # a tensor that several parts read (a table shared by all layers) is declared by each of them, alike
    seen: Dict[str, WeightSpec] = {}
    out: List[WeightSpec] = []
    for s in specs:
        if s.name not in seen:
            seen[s.name] = s
            out.append(s)
        elif seen[s.name] != s:
            raise ValueError(f"the plan declares the tensor '{s.name}' twice, with different shapes or kinds")
    return out


class DecoderModel:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device):
        plan.validate()
        self.plan = plan
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks = [Block(b, dtype, self.device) for b in plan.blocks]
        self.final_norm = build_part("norm", plan.final_norm, plan.final_norm_name, dtype, self.device)
        # the residual stream's dtype: the engine's, or float32 where the plan says so
        self.stream_dtype = torch.float32 if plan.residual_dtype == "float32" else dtype
        self.embed = None
        self.head = None
        self.pair_table = self.pos_table = None
        # the model's own per-request state (``state_need_of_model``), bound by the runner
        self.model_state: Dict[str, torch.Tensor] = {}

    # ---- weights -------------------------------------------------------------------------------
    def load(self, store: WeightStore) -> None:
        store.check(model_weight_specs(self.plan))
        self.embed = store.get(self.plan.embed_name, self.device, self.dtype, operand=True)
        if self.plan.pair_embedding is not None:
            self.pair_table = store.get(self.plan.pair_embedding.name, self.device, self.dtype, operand=True)
        if self.plan.position_table is not None:
            self.pos_table = store.get(self.plan.position_table, self.device, self.dtype, operand=True)
        for b in self.blocks:
            b.load(store)
        self.final_norm.load(store)
        self.head = self.embed if self.plan.head_name is None else store.get(
            self.plan.head_name, self.device, self.dtype, operand=True)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        visit(self)
        visit(self.final_norm)
        for b in self.blocks:
            for t in b.gains.values():
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
            for part in b.all_parts():
                visit(part)
                inner = getattr(part, "shared", None)
                if inner is not None and hasattr(inner, "spec"):
                    visit(inner)            # a feed-forward inside a mixture of experts holds its own weights
                if getattr(getattr(part, "spec", None), "out_norms", None) is not None:
                    # two mixers side by side that keep their output projections apart hold their own weights
                    visit(part.left)
                    visit(part.right)
        return total

    def graph_safe(self) -> bool:
        """Every part takes what it needs of a step from device tensors: decode steps can be replayed from CUDA graphs."""
        return self.final_norm.graph_safe and all(p.graph_safe for b in self.blocks for p in b.all_parts())

    # ---- what the runs need from the cache ---------------------------------------------------------
    def cache_needs(self):
        """Per layer run: the mixer's paged-cache need (None if it has none or reads another run's)."""
        out = []
        for run in self.plan.runs:
            mixer = self.blocks[run.block].mixer
            out.append(mixer.cache_need() if mixer is not None else None)
        return out

    def state_need_of_model(self):
        """Per-request state that belongs to no layer: the token before, for the pair embedding."""
        if self.plan.pair_embedding is not None:
            return {"prev_token": ((), torch.int32)}
        return None

    def bind_state(self, tables: Dict[str, torch.Tensor]) -> None:
        self.model_state = dict(tables)

    def state_needs(self):
        mixers = [self.blocks[run.block].mixer for run in self.plan.runs]
        return [m.state_need() if m is not None else None for m in mixers]

    # ---- one step ------------------------------------------------------------------------------------
    def forward(self, ctx: StepContext, caches: List[Optional[LayerCache]],
                states: List[Optional[Dict[str, torch.Tensor]]]) -> torch.Tensor:
        """Runs the step's tokens through the layer runs and returns float32 logits
        ``[num_logit_rows, vocab]`` for ``ctx.logit_rows``."""
        T, H, V = ctx.num_tokens, self.plan.hidden, self.plan.vocab_size
        ws = ctx.workspace
        x = ws.get("model.x", (T, H), self.stream_dtype)
        ctx.branch_dtype = self.stream_dtype
        # what mixers decide once per step from its metadata, before the step's first kernel
        for pos, run in enumerate(self.plan.runs):
            mixer = self.blocks[run.block].mixer
            if mixer is not None:
                mixer.prepare_step(ctx, caches[pos if run.cache_from is None else run.cache_from])
        trace = tracing.ENABLED
        if trace:
            tracing.push("embedding")
        if self.pair_table is not None or self.pos_table is not None:
            pair = self.plan.pair_embedding
            prev = self.model_state.get("prev_token")
            if pair is not None and prev is None:
                raise RuntimeError("the pair embedding needs the model's per-request state (bind_state)")
            kernels.embed_sum(x, self.embed, ctx.token_ids, ctx.err, sampled=ctx.sampled, scale=self.plan.embed_scale,
                              pair=self.pair_table, pair_rule=(pair.buckets, pair.mul_prev, pair.mul_cur) if pair else None,
                              pos_table=self.pos_table, positions=ctx.positions, req_of_token=ctx.req_of_token,
                              q_start=ctx.q_start, slots=ctx.slots, prev_state=prev)
            if pair is not None:
                kernels.prev_store(prev, ctx.token_ids, ctx.sampled, ctx.q_start, ctx.slots, ctx.num_entries)
        else:
            kernels.embedding(x, self.embed, ctx.token_ids, ctx.err, ctx.sampled, scale=self.plan.embed_scale)
        if trace:
            tracing.pop()
        stream = Stream(x)
        x0 = None
        if any(run.add_input for run in self.plan.runs):
            # runs that add the embedding's output again: it is kept apart from the stream that the blocks change
            x0 = ws.get("model.x0", (T, H), self.stream_dtype)
            x0.copy_(x)
        for pos, run in enumerate(self.plan.runs):
            if run.add_input:
                stream.pending.append(Addend(x0))      # summed by whoever reads the stream next
            src = pos if run.cache_from is None else run.cache_from
            stream = self.blocks[run.block].forward(stream, ctx, caches[src], states[pos],
                                                    writes_cache=run.cache_from is None)
        R = ctx.num_logit_rows
        logits = ws.get("model.logits", (max(R, 1), V), torch.float32)[:R]
        if R == 0:
            return logits      # nothing reads the stream again: its waiting additions are void
        if trace:
            tracing.push("head")
        y = ws.get("model.final", (R, H), self.dtype)
        fused_norm(self.final_norm, y, stream.x, ctx, stream.settle(ctx, keep_last=True), rows=ctx.logit_rows)
        linear(logits, y, self.head, ctx.err)
        if self.plan.logit_scale is not None or self.plan.logit_softcap is not None:
            kernels.logits_post(logits, self.plan.logit_scale, self.plan.logit_softcap)
        if trace:
            tracing.pop()
        return logits
