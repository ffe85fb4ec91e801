"""Typed configuration of the Gulipel decoder, read from the keys of its own config.json, and its arrangement
of parts.

A Gulipel model lists its layers one by one (``layers``), each with its own type and sizes.  A layer norms a
sublayer's input *and* its output, multiplies the normed output by a learned vector and adds it:

    x <- x + ls1 * norm1b(mixer(norm1(x)));   x <- x + ls2 * norm2b(ff(norm2(x)))        (the second half is optional)
    x <- x + side_norm(W_proj(gelu_tanh(W_gate x) * e))      e: the layer's columns of a table over token ids

Every norm is an RMS norm with a plain weight.  The mixer is a state-space mixer (types ``mamba2`` and ``mamba2_2``,
one mechanism under two names) or two mixers side by side (``parallel``): causal grouped-query softmax attention
without rotation - biases on q, k, v, a weighted RMS norm per head on q and k, a query temperature that grows with
the logarithm of the position, a sigmoid gate on the heads - beside a gated delta rule; each side's result is
RMS-normed over the width and the two are averaged.  The feed-forward is SiLU-gated with biases on all three
projections.  The embedding row is scaled and joined by a row of a table over hashed (previous token, token) pairs
and a learned vector per position; the logits pass a soft cap.  The residual stream is float32 whatever the
engine's dtype is.

Every size and every constant that config.json gives is read here and handed to the parts through their specs;
nothing is fixed in code but the tensor names, the arrangement, the average of the two sides (1/2 each) and the
1e-6 under the root of the delta rule's unit vectors.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .plan import (AttentionSpec, BlockOp, BlockSpec, FeedForwardSpec, GatedDeltaSpec, LayerRun, ModelPlan, NormSpec,
                   PairEmbeddingSpec, ParallelMixerSpec, SelectiveStateSpec, TokenSideSpec)

ARCHITECTURE = "Gulipel"
# the engine's own bound on a sequence where the model has no position table
MAX_POSITIONS = 1 << 20
STATE_SPACE_TYPES = ("mamba2", "mamba2_2")


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


def _opt_int(raw, key: str, where: str) -> Optional[int]:
    return _int(raw, key, where) if isinstance(raw, Mapping) and raw.get(key) is not None else None


@dataclass(frozen=True)
class GulipelStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class GulipelLeft:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[Tuple[float, int]]


@dataclass(frozen=True)
class GulipelRight:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int]
    gate_rank: Optional[int]


@dataclass(frozen=True)
class GulipelLayer:
    type: str
    mixer: Any               # GulipelStateSpace, or (GulipelLeft, GulipelRight)
    ff: Optional[int]        # width of the dense feed-forward; None: the layer has none


@dataclass(frozen=True)
class GulipelConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    bigram: Optional[Tuple[int, int, int]]      # buckets, mul_prev, mul_cur
    max_positions: Optional[int]                # rows of the position table; None: the model has none
    side_dim: Optional[int]
    logit_softcap: Optional[float]
    layers: Tuple[GulipelLayer, ...]

    ARCHITECTURE = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "GulipelConfig":
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        eps = _num(_get(raw, "norm", ""), "eps", "norm.", positive=True)
        emb = _get(raw, "embedding", "")
        embed_scale = _num(emb, "scale", "embedding.")
        bigram = None
        if emb.get("bigram") is not None:
            b, wb = emb["bigram"], "embedding.bigram."
            bigram = (_int(b, "buckets", wb), _int(b, "mul_prev", wb, least=0), _int(b, "mul_cur", wb, least=0))
        max_positions = _opt_int(raw, "max_positions", "")
        side_dim = _opt_int(raw.get("token_side"), "dim", "token_side.")
        softcap = _num(raw, "logit_softcap", "", positive=True) if raw.get("logit_softcap") is not None else None
        layers = _get(raw, "layers", "")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            w = f"layers[{i}]."
            kind = _get(layer, "type", w)
            m, wm = _get(layer, "mixer", w), w + "mixer."
            if kind in STATE_SPACE_TYPES:
                heads, groups = _int(m, "heads", wm), _int(m, "groups", wm)
                if heads % groups:
                    raise ConfigError(f"'{wm}heads' {heads} is not a multiple of '{wm}groups' {groups}")
                vdim, parts = _int(m, "vdim", wm), _int(m, "norm_groups", wm)
                if (heads * vdim) % parts:
                    raise ConfigError(f"'{wm}norm_groups' {parts} does not divide the {heads * vdim} inner channels")
                mixer = GulipelStateSpace(heads, vdim, _int(m, "state", wm), groups, _int(m, "conv", wm), parts)
            elif kind == "parallel":
                left, wl = _get(m, "left", wm), wm + "left."
                heads, kv = _int(left, "heads", wl), _int(left, "kv_heads", wl)
                if heads % kv:
                    raise ConfigError(f"'{wl}heads' {heads} is not a multiple of '{wl}kv_heads' {kv}")
                q_temp = None
                if left.get("q_temp") is not None:
                    q_temp = (_num(left["q_temp"], "coef", wl + "q_temp."), _int(left["q_temp"], "every", wl + "q_temp."))
                lf = GulipelLeft(heads, kv, _int(left, "dim", wl), _int(left, "vdim", wl), _num(left, "scale", wl), q_temp)
                right, wr = _get(m, "right", wm), wm + "right."
                heads, kv = _int(right, "heads", wr), _int(right, "kv_heads", wr)
                if heads % kv:
                    raise ConfigError(f"'{wr}heads' {heads} is not a multiple of '{wr}kv_heads' {kv}")
                rt = GulipelRight(heads, kv, _int(right, "dim", wr), _int(right, "vdim", wr), _int(right, "conv", wr),
                                  _opt_int(right, "decay_rank", wr), _opt_int(right, "gate_rank", wr))
                mixer = (lf, rt)
            else:
                raise ConfigError(f"config key '{w}type' is '{kind}'; known: parallel, {', '.join(STATE_SPACE_TYPES)}")
            ff = None
            if layer.get("mlp") is not None:
                mlp, wf = layer["mlp"], w + "mlp."
                mk = _get(mlp, "kind", wf)
                if mk != "dense":
                    raise ConfigError(f"config key '{wf}kind' is '{mk}'; known: dense")
                ff = _int(mlp, "ff", wf)
            out.append(GulipelLayer(kind, mixer, ff))
        return cls(vocab=vocab, width=width, eps=eps, embed_scale=embed_scale, bigram=bigram, max_positions=max_positions,
                   side_dim=side_dim, logit_softcap=softcap, layers=tuple(out))

    # ---- the arrangement of parts ---------------------------------------------------------
    def plan(self) -> ModelPlan:
        def norm(kind: str = "rmsnorm"):
            return NormSpec(kind=kind, dim=self.width, eps=self.eps, weight_offset=0.0, weight_name="")

        blocks = []
        for i, layer in enumerate(self.layers):
            if layer.type in STATE_SPACE_TYPES:
                m = layer.mixer
                mixer = SelectiveStateSpec(kind="selective_state", hidden=self.width, heads=m.heads, head_dim=m.vdim,
                                           state=m.state, groups=m.groups, conv=m.conv, norm_groups=m.norm_groups, eps=self.eps)
            else:
                lf, rt = layer.mixer
                left = AttentionSpec(kind="talking_attention", hidden=self.width, num_heads=lf.heads, num_kv_heads=lf.kv_heads,
                                     head_dim=lf.dim, v_head_dim=lf.vdim, scale=lf.scale, qk_norm=True, qk_norm_eps=self.eps,
                                     qk_norm_weight=True, qk_norm_after_rope=False, rope=None, talking_heads=False, sink=False,
                                     names=("q", "k", "v", "o", "talk"), bias_suffix=".b", qk_norm_names=("q.norm", "k.norm"),
                                     q_temp=lf.q_temp, gate_name="g")
                right = GatedDeltaSpec(kind="gated_delta", hidden=self.width, heads=rt.heads, kv_heads=rt.kv_heads,
                                       head_dim=rt.dim, v_head_dim=rt.vdim, conv=rt.conv, eps=self.eps, unit_eps=1e-6,
                                       decay_rank=rt.decay_rank, gate_rank=rt.gate_rank)
                mixer = ParallelMixerSpec(kind="parallel", hidden=self.width, left=left, right=right, left_scale=0.5,
                                          right_scale=0.5, out_norms=("left.out", "right.out"), out_norm_eps=self.eps)
            prog = [BlockOp("norm", "x", "h", norm(), "norm1"),
                    BlockOp("mixer", "h", "a", mixer, "mix."),
                    BlockOp("norm", "a", "a", norm(), "norm1b"),
                    BlockOp("add", "a", "x", gain="ls1")]
            if layer.ff is not None:
                ff = FeedForwardSpec(kind="swiglu", hidden=self.width, intermediate=layer.ff, activation="silu",
                                     names=("gate", "up", "down"), bias_suffix=".b")
                prog += [BlockOp("norm", "x", "h", norm(), "norm2"),
                         BlockOp("feed_forward", "h", "f", ff, "mlp."),
                         BlockOp("norm", "f", "f", norm(), "norm2b"),
                         BlockOp("add", "f", "x", gain="ls2")]
            if self.side_dim is not None:
                side = TokenSideSpec(kind="token_side", hidden=self.width, dim=self.side_dim, vocab=self.vocab,
                                     table="side.embed", column=i * self.side_dim, columns=len(self.layers) * self.side_dim)
                # the part reads the stream as it stands: a norm that is none hands it over in the engine's type
                prog += [BlockOp("norm", "x", "h", norm("identity"), "side.in"),
                         BlockOp("feed_forward", "h", "s", side, "side."),
                         BlockOp("norm", "s", "s", norm(), "side.norm"),
                         BlockOp("add", "s", "x")]
            blocks.append(BlockSpec(f"l{i}.", tuple(prog)))
        pair = None
        if self.bigram is not None:
            pair = PairEmbeddingSpec("bigram", self.bigram[0], self.bigram[1], self.bigram[2])
        plan = ModelPlan(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden=self.width, embed_name="embed",
            blocks=tuple(blocks), runs=tuple(LayerRun(block=i) for i in range(len(blocks))),
            final_norm=norm(), final_norm_name="final.norm", head_name="head",
            max_positions=self.max_positions if self.max_positions is not None else MAX_POSITIONS,
            embed_scale=self.embed_scale, logit_softcap=self.logit_softcap, residual_dtype="float32",
            pair_embedding=pair, position_table="pos" if self.max_positions is not None else None)
        plan.validate()
        return plan
