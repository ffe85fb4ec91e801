"""One layer: the parts of a ``BlockSpec`` and the executor of its program.

A block's arrangement is data (``BlockSpec.program``): operations ``norm``, ``mixer``,
``feed_forward`` and ``add`` over named activations, ``"x"`` being the residual stream.  The
reference wires its one arrangement by hand, ``x + mixer(norm(x))`` then ``x + mlp(norm(x))``
(src/models/qwen3.rs:108-134), and fuses each residual sum with the norm after it
(src/models/layers/others.rs:48-62).

Here an addition is carried out when its sum is next read.  Where a norm reads it, the norm
kernel forms the sum in float32, stores it and norms it in one pass - also across the block
boundary: the last addition of a block waits in the ``Stream`` that the next block (or the
decoder's final norm) receives.  Where a mixer or a feed-forward runs next, an addition kernel
runs first (for every waiting addition: the part may reuse the buffer an addend lives in).
The pre-norm block therefore launches exactly the kernels a hand-written one would.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels, tracing
from ..config.plan import BlockSpec
from ..weights.loader import WeightSpec
from .base import LayerCache, Part, StepContext, build_part, part_class
from .norm import RMSNorm, chain as norm_chain

_FAMILY = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}


def _width_of(spec: BlockSpec) -> int:
    """The width of the residual stream, from the block's first norm or part that names it."""
    for o in spec.program:
        if o.spec is not None:
            w = getattr(o.spec, "dim", 0) if o.op == "norm" else getattr(o.spec, "hidden", 0)
            if w:
                return int(w)
    raise ValueError(f"block '{spec.prefix}': no part names the width of the residual stream")


class Addend:
    """A value that waits to be added into another: ``scale * gain * norm(t)``, where ``norm`` (a norm part, or None)
    has not been carried out yet - the kernel that forms the sum may do it, if its kind offers that - and ``gain`` is
    a learned vector over the channels (or None)."""

    __slots__ = ("t", "scale", "norm", "gain")

    def __init__(self, t: torch.Tensor, scale: float = 1.0, norm=None, gain=None):
        self.t = t
        self.scale = scale
        self.norm = norm
        self.gain = gain

    def plain(self, ctx) -> torch.Tensor:
        """The tensor with its norm carried out (in place: the unnormed value is read by nobody else)."""
        if self.norm is not None:
            self.norm.forward(self.t, self.t, ctx)
            self.norm = None
        return self.t


def _add_into(dst: torch.Tensor, a: Addend, ctx) -> None:
    if a.gain is not None or (a.norm is not None and isinstance(a.norm, RMSNorm) and dst.dtype == torch.float32):
        # one pass: the branch's own RMS norm, the gain, the scale and the sum
        norm, a.norm = a.norm, None
        if norm is not None and not RMSNorm.accepts_branch_norm(norm):
            norm.forward(a.t, a.t, ctx)
            norm = None
        norm_chain(None, dst, ctx, None, a.t, a.scale, norm, a.gain, dst, None)
        return
    kernels.add(dst, dst, a.plain(ctx), a.scale)


def fused_norm(part, out, src, ctx, last: Optional[Addend], rows=None):
    """``out = part(src + last)`` in one kernel where the norm's kind takes what the addend needs (a scale, a norm of
    its own of the same kind); the sum is stored back into ``src`` unless rows are gathered."""
    if last is None:
        return part.forward(out, src, ctx, rows=rows) if rows is not None else part.forward(out, src, ctx)
    kw = {}
    if last.norm is not None:
        accepts = getattr(part, "accepts_branch_norm", None)
        if getattr(part, "takes_branch_norm", False) and (accepts(last.norm) if accepts else type(last.norm) is type(part)):
            kw["branch_norm"] = last.norm
        else:
            last.plain(ctx)
    if last.gain is not None:
        if getattr(part, "takes_branch_gain", False):
            kw["branch_gain"] = last.gain
        else:
            _add_into(src, last, ctx)
            return part.forward(out, src, ctx, rows=rows) if rows is not None else part.forward(out, src, ctx)
    if last.scale != 1.0:
        if getattr(part, "takes_branch_scale", False):
            kw["branch_scale"] = last.scale
        else:
            # the norm cannot scale its branch: the sum is formed by an addition kernel first
            _add_into(src, last, ctx)
            return part.forward(out, src, ctx, rows=rows) if rows is not None else part.forward(out, src, ctx)
    if rows is not None:
        return part.forward(out, src, ctx, branch=last.t, rows=rows, **kw)
    return part.forward(out, src, ctx, branch=last.t, sum_out=src, **kw)


class Stream:
    """The residual stream between blocks: its tensor and the branches still to be added to it."""

    __slots__ = ("x", "pending")

    def __init__(self, x: torch.Tensor, pending: Optional[List[Addend]] = None):
        self.x = x
        self.pending: List[Addend] = pending or []

    def settle(self, ctx, keep_last: bool = False) -> Optional[Addend]:
        """Carry out the waiting additions; with ``keep_last`` the last one is handed back for a
        norm kernel to fuse."""
        last = self.pending.pop() if (keep_last and self.pending) else None
        for b in self.pending:
            _add_into(self.x, b, ctx)
        self.pending = []
        return last


class Block:
    def __init__(self, spec: BlockSpec, dtype, device):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.parts: Dict[Tuple[str, str], Part] = {}
        for o in spec.program:
            if o.op == "add":
                continue
            key = (o.op, o.name)
            if key not in self.parts:
                self.parts[key] = build_part(_FAMILY[o.op], o.spec, spec.prefix + o.name, dtype, device)
        mixers = [p for (op, _), p in self.parts.items() if op == "mixer"]
        self.mixer = mixers[0] if mixers else None
        self.device = device
        self.gains: Dict[str, torch.Tensor] = {}      # learned vectors of the additions, by tensor name after the prefix

    @staticmethod
    def weight_specs(spec: BlockSpec) -> List[WeightSpec]:
        out: List[WeightSpec] = []
        seen = set()
        for o in spec.program:
            if o.op == "add" or (o.op, o.name) in seen:
                continue
            seen.add((o.op, o.name))
            out += part_class(_FAMILY[o.op], o.spec.kind).weight_specs(o.spec, spec.prefix + o.name)
        for name in sorted({o.gain for o in spec.program if o.op == "add" and o.gain is not None}):
            out.append(WeightSpec(spec.prefix + name, (_width_of(spec),), "norm"))
        return out

    def all_parts(self) -> List[Part]:
        return list(self.parts.values())

    def load(self, store) -> None:
        for part in self.parts.values():
            part.load(store)
        for o in self.spec.program:
            if o.op == "add" and o.gain is not None and o.gain not in self.gains:
                self.gains[o.gain] = store.get(self.spec.prefix + o.gain, self.device, torch.float32).float().contiguous()

    def forward(self, stream: Stream, ctx: StepContext, cache: Optional[LayerCache], state, writes_cache: bool) -> Stream:
        """Runs the program on the residual stream; returns the stream with the additions that
        still wait."""
        ws = ctx.workspace
        vals: Dict[str, torch.Tensor] = {"x": stream.x}
        waiting: Dict[str, List[Addend]] = {"x": stream.pending}
        lazy: Dict[str, Part] = {}      # block-local values whose norm waits for the addition that follows it

        def read(name: str) -> torch.Tensor:
            """The value with every addition into it carried out."""
            t = vals[name]
            if name in lazy:
                part = lazy.pop(name)
                part.forward(t, t, ctx)
            for b in waiting.pop(name, ()):
                _add_into(t, b, ctx)
            return t

        def settle_all() -> None:
            # a part is about to run and may reuse the buffer that a waiting addend lives in
            for name in list(waiting):
                read(name)

        program = self.spec.program
        for idx, o in enumerate(program):
            if o.op == "add":
                gain = self.gains[o.gain] if o.gain is not None else None
                if o.src in lazy and not waiting.get(o.src):
                    waiting.setdefault(o.dst, []).append(Addend(vals[o.src], o.scale, lazy.pop(o.src), gain))
                else:
                    waiting.setdefault(o.dst, []).append(Addend(read(o.src), o.scale, None, gain))
                continue
            part = self.parts[(o.op, o.name)]
            if o.op == "norm":
                nxt = program[idx + 1] if idx + 1 < len(program) else None
                if (o.src == o.dst and o.src != "x" and o.src not in lazy and not waiting.get(o.src)
                        and getattr(part, "takes_branch_norm", False)
                        and nxt is not None and nxt.op == "add" and nxt.src == o.dst):
                    # a norm in place of a block-local value that is only added into another value next: it
                    # waits, and the kernel that forms that sum carries it out
                    lazy[o.dst] = part
                    continue
                src = vals[o.src]
                if o.src in lazy:
                    read(o.src)
                adds = waiting.pop(o.src, [])
                for b in adds[:-1]:
                    _add_into(src, b, ctx)
                last = adds[-1] if adds else None
                out = ws.get("block." + o.dst, tuple(src.shape), self.dtype)
                if any(out.data_ptr() == t.data_ptr() for t in (src, *([last.t] if last else []))):
                    # a norm back into its own input (or over its addend) gets a buffer of its own
                    out = ws.get("block." + o.dst + "'", tuple(src.shape), self.dtype)
                if tracing.ENABLED:
                    tracing.push("norm")
                fused_norm(part, out, src, ctx, last)
                if tracing.ENABLED:
                    tracing.pop()
            else:
                settle_all()
                if tracing.ENABLED:
                    tracing.push(o.op + ":" + part.kind)
                if o.op == "mixer":
                    out = part.forward(vals[o.src], ctx, cache, state, writes_cache)
                else:
                    out = part.forward(vals[o.src], ctx)
                if tracing.ENABLED:
                    tracing.pop()
            waiting.pop(o.dst, None)      # additions that waited for the value this one replaces are void
            lazy.pop(o.dst, None)
            vals[o.dst] = out
        # additions into block-local values that nothing read are void; the stream's wait for its next reader
        return Stream(vals["x"], waiting.get("x", []))
