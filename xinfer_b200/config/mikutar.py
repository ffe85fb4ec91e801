"""Typed configuration of the Mikutar decoder, read from the keys of its own config.json, and its arrangement
of parts.

A Mikutar model lists its layers one by one (``layers``), each with its own type and sizes.  A layer has ONE norm
whose output both sublayers read, and adds their results together:

    h = norm1(x);   x <- x + (mixer(h) + ff(h))                       (the feed-forward is optional)

``loop`` = {start, stop, times}: layers start .. stop-1 run ``times`` times in a row with the same weights (each
pass with a cache of its own), and before every pass but the first the embedding's output is added to the stream.
The mixer is one of two kinds of grouped-query softmax attention with a sigmoid gate of one number per head:

* ``attention``: biases on q, k and the output; the keys as projected double as values; one RMS norm over the whole
  q (and k) projection; rotation of neighbouring channels; a sliding window;
* ``attention_2``: no biases, no rotation; capped scores, a bias on the distance (slope ``2^(-8 (h + 1) / heads)``
  for head h), a chunked mask.

The feed-forward is ReLU-gated, or a mixture of experts with a sigmoid router, a correction on the choice scores,
a choice among groups and an expert that every token runs.  The logits come from the embedding table and pass a
soft cap.  The residual stream is float32 whatever the engine's dtype is.

Every size and every constant that config.json gives is read here and handed to the parts through their specs;
the design fixes the tensor names, the arrangement and the constants below.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .plan import (AttentionSpec, BlockOp, BlockSpec, FeedForwardSpec, LayerRun, ModelPlan, NormSpec, RopeSpec,
                   RoutedExpertsSpec)

ARCHITECTURE = "Mikutar"
# the engine's own bound on a sequence (the model has no position table)
MAX_POSITIONS = 1 << 20
# constants of the design
SWISH_ALPHA = 1.702            # an expert's gate: a * sigmoid(1.702 a)
GROUP_BEST = 2                 # a group's score: the sum of its two largest choice scores
SLOPE_EXPONENT = 8.0           # the distance bias of head h: 2^(-8 (h + 1) / heads) per position


def _get(raw, key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks '{where}{key}'")
    return raw[key]


def _int(raw, key: str, where: str, least: int = 1) -> int:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"config key '{where}{key}' must be an integer >= {least}, got {v!r}")
    return v


def _num(raw, key: str, where: str, positive: bool = False) -> float:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"config key '{where}{key}' must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class MikutarAttention:
    """Either kind of mixer: ``rot`` = (dims, base) or None; ``softcap`` None where scores are not capped."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask: int
    rot: Optional[Tuple[int, float]]
    softcap: Optional[float]


@dataclass(frozen=True)
class MikutarExpert:
    ff: int
    limit: float


@dataclass(frozen=True)
class MikutarMlp:
    """``kind`` "dense": ``ff``.  "moe": ``expert``, the router's ``experts``, ``top``, ``groups``, ``keep`` and
    an optional ``shared`` expert."""
    kind: str
    ff: int = 0
    expert: Optional[MikutarExpert] = None
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    shared: Optional[MikutarExpert] = None


@dataclass(frozen=True)
class MikutarLayer:
    type: str
    mixer: MikutarAttention
    mlp: Optional[MikutarMlp]


@dataclass(frozen=True)
class MikutarConfig:
    vocab: int
    width: int
    eps: float
    logit_softcap: Optional[float]
    loop: Optional[Tuple[int, int, int]]        # start, stop, times
    layers: Tuple[MikutarLayer, ...]

    ARCHITECTURE = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MikutarConfig":
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        eps = _num(_get(raw, "norm", ""), "eps", "norm.", positive=True)
        softcap = _num(raw, "logit_softcap", "", positive=True) if raw.get("logit_softcap") is not None else None
        layers = _get(raw, "layers", "")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            w = f"layers[{i}]."
            kind = _get(layer, "type", w)
            if kind not in ("attention", "attention_2"):
                raise ConfigError(f"config key '{w}type' is '{kind}'; known: attention, attention_2")
            m, wm = _get(layer, "mixer", w), w + "mixer."
            heads, kv = _int(m, "heads", wm), _int(m, "kv_heads", wm)
            if heads % kv:
                raise ConfigError(f"'{wm}heads' {heads} is not a multiple of '{wm}kv_heads' {kv}")
            dim, vdim = _int(m, "dim", wm), _int(m, "vdim", wm)
            rot = None
            cap = None
            if kind == "attention":
                if vdim != dim:
                    raise ConfigError(f"'{wm}vdim' {vdim} differs from '{wm}dim' {dim}, but this layer's keys are its values")
                if m.get("rot") is not None:
                    r, wr = m["rot"], wm + "rot."
                    dims = _int(r, "dims", wr, least=0)
                    if dims % 2 or dims > dim:
                        raise ConfigError(f"'{wr}dims' {dims} must be even and at most '{wm}dim' {dim}")
                    if dims:
                        rot = (dims, _num(r, "base", wr, positive=True))
            elif m.get("softcap") is not None:
                cap = _num(m, "softcap", wm, positive=True)
            mixer = MikutarAttention(heads, kv, dim, vdim, _num(m, "scale", wm), _int(_get(m, "mask", wm), "size", wm + "mask."),
                                     rot, cap)
            mlp = None
            if layer.get("mlp") is not None:
                f, wf = layer["mlp"], w + "mlp."
                mk = _get(f, "kind", wf)
                if mk == "dense":
                    mlp = MikutarMlp("dense", ff=_int(f, "ff", wf))
                elif mk == "moe":
                    def expert(key):
                        e, we = _get(f, key, wf), f"{wf}{key}."
                        return MikutarExpert(_int(e, "ff", we), _num(e, "limit", we, positive=True))
                    r, wr = _get(f, "router", wf), wf + "router."
                    experts, top = _int(r, "experts", wr), _int(r, "top", wr)
                    groups, keep = 1, 1
                    if r.get("groups") is not None:
                        groups = _int(r["groups"], "count", wr + "groups.")
                        keep = _int(r["groups"], "keep", wr + "groups.")
                    if experts % groups or keep > groups:
                        raise ConfigError(f"'{wr}experts' {experts} do not form {groups} equal groups of which {keep} are kept")
                    if top > keep * (experts // groups):
                        raise ConfigError(f"'{wr}top' {top} is more than the {keep} kept groups of {experts // groups} experts hold")
                    mlp = MikutarMlp("moe", expert=expert("expert"), experts=experts, top=top, groups=groups, keep=keep,
                                     shared=expert("shared") if f.get("shared") is not None else None)
                else:
                    raise ConfigError(f"config key '{wf}kind' is '{mk}'; known: dense, moe")
            out.append(MikutarLayer(kind, mixer, mlp))
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            start, stop, times = _int(lp, "start", "loop.", least=0), _int(lp, "stop", "loop."), _int(lp, "times", "loop.")
            if not (start < stop <= len(out)):
                raise ConfigError(f"'loop' {start}..{stop} does not lie within the {len(out)} layers")
            loop = (start, stop, times)
        return cls(vocab=vocab, width=width, eps=eps, logit_softcap=softcap, loop=loop, layers=tuple(out))

    # ---- the order of layer runs --------------------------------------------------------------------
    def runs(self) -> Tuple[LayerRun, ...]:
        n = len(self.layers)
        if self.loop is None:
            return tuple(LayerRun(block=i) for i in range(n))
        start, stop, times = self.loop
        runs = [LayerRun(block=i) for i in range(start)]
        for t in range(times):
            runs += [LayerRun(block=i, add_input=(t > 0 and i == start)) for i in range(start, stop)]
        return tuple(runs + [LayerRun(block=i) for i in range(stop, n)])

    # ---- the arrangement of parts ---------------------------------------------------------
    def plan(self) -> ModelPlan:
        def norm():
            return NormSpec(kind="rmsnorm", dim=self.width, eps=self.eps, weight_offset=0.0, weight_name="")

        def gated(ff: int, activation: str, params=()):
            return FeedForwardSpec(kind="swiglu", hidden=self.width, intermediate=ff, activation=activation,
                                   names=("gate", "up", "down"), act_params=tuple(params))

        blocks = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            common = dict(kind="talking_attention", hidden=self.width, num_heads=m.heads, num_kv_heads=m.kv_heads,
                          head_dim=m.dim, v_head_dim=m.vdim, scale=m.scale, talking_heads=False, sink=False,
                          names=("q", "k", "v", "o", "talk"), gate_name="g", gate_per_head=True)
            if layer.type == "attention":
                rope = None
                if m.rot is not None:
                    rope = RopeSpec(kind="rope", head_dim=m.dim, rotary_dim=m.rot[0], theta=m.rot[1],
                                    max_positions=MAX_POSITIONS, layout="interleaved", tables=False)
                mixer = AttentionSpec(**common, qk_norm=True, qk_norm_eps=self.eps, qk_norm_weight=True, qk_norm_whole=True,
                                      qk_norm_names=("q.norm", "k.norm"), rope=rope, window=m.mask, bias_suffix=".b",
                                      out_bias=True, value_from_key=True)
            else:
                mixer = AttentionSpec(**common, qk_norm=False, rope=None, window=None, chunk=m.mask,
                                      score_softcap=m.softcap, distance_slope_exponent=SLOPE_EXPONENT)
            prog = [BlockOp("norm", "x", "h", norm(), "norm1"),
                    BlockOp("mixer", "h", "a", mixer, "mix.")]
            if layer.mlp is not None:
                f = layer.mlp
                if f.kind == "dense":
                    ff = gated(f.ff, "relu")
                else:
                    ff = RoutedExpertsSpec(kind="routed_experts", hidden=self.width, intermediate=f.expert.ff,
                                           experts=f.experts, top=f.top, groups=f.groups, keep=f.keep, group_best=GROUP_BEST,
                                           correction=True, renormalize=False, activation="swish_clamp",
                                           act_params=(f.expert.limit, SWISH_ALPHA),
                                           shared=gated(f.shared.ff, "swish_clamp", (f.shared.limit, SWISH_ALPHA))
                                           if f.shared is not None else None)
                prog.append(BlockOp("feed_forward", "h", "f", ff, "mlp."))
            # both sublayers read the one normed input; their results are summed into the stream
            prog.append(BlockOp("add", "a", "x"))
            if layer.mlp is not None:
                prog.append(BlockOp("add", "f", "x"))
            blocks.append(BlockSpec(f"l{i}.", tuple(prog)))
        plan = ModelPlan(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden=self.width, embed_name="embed",
            blocks=tuple(blocks), runs=self.runs(), final_norm=norm(), final_norm_name="final.norm", head_name=None,
            max_positions=MAX_POSITIONS, logit_softcap=self.logit_softcap, residual_dtype="float32")
        plan.validate()
        return plan
