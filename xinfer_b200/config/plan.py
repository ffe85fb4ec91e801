"""Typed descriptions of a decoder: what each layer is made of and in which order layers run.

A model is described as data before anything is built:

* a *part spec* per part (mixer, feed-forward, norm, position encoding) carrying every size and
  constant the part needs, so no part ever looks at a model configuration;
* a ``BlockSpec`` per set of weights: its parts and their arrangement as a short program of
  operations (norm, mixer, feed-forward, add) over named activations, so that pre-norm, post-norm,
  sandwich-norm and parallel arrangements, and blocks without a feed-forward, are all data;
* a ``LayerRun`` list: the order in which blocks execute.  A block may be named twice (its
  weights are reused, each run keeps a cache of its own), and a run may read the cache that an
  earlier run wrote instead of writing one (``cache_from``).

The reference wires one struct per architecture by hand (src/models/qwen3.rs:20-135 for the
layer, :137-290 for the stack); here the same information is a ``ModelPlan`` that a generic
decoder builds from.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple, Union


@dataclass(frozen=True)
class PartSpec:
    """Base of every part spec. ``kind`` selects the implementation in the part registry."""

    kind: str

    def params(self) -> Dict[str, Any]:
        d = dict(self.__dict__)
        d.pop("kind")
        return d


@dataclass(frozen=True)
class RopeScaling:
    """Slower turning for long wavelengths (the rule of Llama 3.1): a pair whose wavelength
    ``2 pi / f`` is shorter than ``original / high`` keeps its frequency f, one longer than
    ``original / low`` turns at ``f / factor``, and between the two the frequency is
    ``(1 - s) f / factor + s f`` with ``s = (original / wavelength - low) / (high - low)``."""

    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class YarnScaling:
    """Slower turning for the pairs that turn slowly (the rule of YaRN), decided by how many turns a pair
    makes within the ``original`` length: with ``pair(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)``
    the pair index at which ``t`` turns are made, ``lo = max(floor(pair(fast)), 0)``,
    ``hi = min(ceil(pair(slow)), rotary_dim - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``,
    pair i turns at ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RopeSpec(PartSpec):
    """Rotary position encoding over the first ``rotary_dim`` channels of each head.

    ``layout`` is "neox" (channel j pairs with j + rotary_dim/2) or "interleaved" (2j with 2j+1).
    ``scaling`` changes the frequencies (None: ``theta^(-2j / rotary_dim)`` as they are).
    ``tables`` False: no cos/sin table is built; kernels take the frequencies and form
    ``position * frequency`` in float32 themselves, so no longest position has to be known.
    ``magnitude``: cos and sin are both multiplied by it (1: a pure rotation).
    """

    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    layout: str = "neox"
    scaling: Optional[Union[RopeScaling, YarnScaling]] = None
    tables: bool = True
    magnitude: float = 1.0


@dataclass(frozen=True)
class NormSpec(PartSpec):
    dim: int = 0
    eps: float = 1e-6
    # weight enters as (offset + w): 0 for plain RMSNorm, 1 for the "(1 + w)" family
    weight_offset: float = 0.0
    # the tensor's name after the part's prefix ("" where the prefix is the whole name)
    weight_name: str = "weight"
    # how the random-weights mode draws the weight: "norm" (around one) or "around_zero"
    init: str = "norm"


@dataclass(frozen=True)
class DynamicTanhSpec(PartSpec):
    """A norm without statistics: ``y = tanh(alpha * x) * w + b`` with a learned scalar ``alpha`` and learned
    vectors ``w`` and ``b``.  The three names follow the part's prefix."""

    dim: int = 0
    weight_name: str = "weight"
    bias_name: str = "bias"
    alpha_name: str = "alpha"


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    hidden: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    rope: Optional[RopeSpec] = None
    # a query at position p sees keys j with p - window < j <= p; None = all earlier keys
    window: Optional[int] = None
    # size of a value head (None: head_dim)
    v_head_dim: Optional[int] = None
    # q/k norm: with a learned weight per channel or without; before the rotation or after it
    qk_norm_weight: bool = True
    qk_norm_after_rope: bool = False
    # the scores of all heads for one (query, key) pair are mixed by a learned [heads, heads] matrix
    # before the softmax: score_h <- sum_g talk[h, g] score_g
    talking_heads: bool = False
    # the softmax has one more entry of score 0 that carries no value: p_j = e^s_j / (1 + sum e^s)
    sink: bool = False
    # tensor names of the q, k, v, output (and talk) matrices after the part's prefix; None: the
    # "q_proj.weight" family
    names: Optional[Tuple[str, ...]] = None
    # q, k and v have biases: the matrix's name with this suffix (None: no biases)
    bias_suffix: Optional[str] = None
    # names of the q and k norm weights after the prefix (None: "q_norm.weight", "k_norm.weight")
    qk_norm_names: Optional[Tuple[str, str]] = None
    # query temperature (coef, every): the query at position p is multiplied by
    # 1 + coef * ln(floor((p + 1) / every) + 1), after its norm and rotation
    q_temp: Optional[Tuple[float, int]] = None
    # the concatenated heads are multiplied by sigmoid(W_g h) before the output projection; the name of W_g
    gate_name: Optional[str] = None
    # the gate is one number per head (W_g has ``num_heads`` rows) instead of one per channel
    gate_per_head: bool = False
    # the keys as projected (with their bias, before norm and rotation) double as values: there is no W_v
    value_from_key: bool = False
    # q/k norm with ONE root mean square over the whole q projection (and one over the whole k projection) and
    # weights of that size, instead of one per head
    qk_norm_whole: bool = False
    # the output projection has a bias too (its matrix's name with ``bias_suffix``)
    out_bias: bool = False
    # scores pass cap * tanh(score / cap) before the softmax
    score_softcap: Optional[float] = None
    # a distance bias after the cap: head h's score of a key ``dist`` positions back loses
    # 2^(-x (h + 1) / num_heads) * dist, x this exponent
    distance_slope_exponent: Optional[float] = None
    # a query sees the earlier keys of its own chunk of this many positions (chunks counted from position 0 of the
    # sequence) instead of a window
    chunk: Optional[int] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """Attention whose keys and values are linear maps of one cached latent vector per token.

    A token's ``kv_rank`` latent channels (RMS-normed with a learned weight, ``norm_eps``) and one rotated key part
    of ``rope_dim`` channels shared by all heads are all that is cached.  Head h has ``head_dim`` plain and
    ``rope_dim`` rotated query channels; its plain key is ``W_uk,h c`` and its value ``W_uv,h c`` (``v_head_dim``
    channels).  ``window`` as for attention.  ``sink``: every head's softmax has one more entry with a learned score
    and no value.  ``gate``: the concatenated heads are multiplied by ``sigmoid(W_g h)`` before the output projection.
    ``shares_cache``: the layer has no latent projection of its own and reads the rows another layer cached.
    ``cache_window``: how long cached rows must be kept (None: for ever): the largest window among the layers that
    read them.  ``names``: the tensors q, latent projection, its norm, uk, uv, sink, gate, output after the prefix."""

    hidden: int = 0
    num_heads: int = 0
    head_dim: int = 0
    rope_dim: int = 0
    v_head_dim: int = 0
    kv_rank: int = 0
    scale: float = 1.0
    rope: Optional[RopeSpec] = None
    window: Optional[int] = None
    cache_window: Optional[int] = None
    norm_eps: float = 1e-6
    sink: bool = False
    gate: bool = False
    shares_cache: bool = False
    names: Tuple[str, ...] = ("q", "dkv", "dkv.norm", "uk", "uv", "sink", "g", "o")


@dataclass(frozen=True)
class GatedRecurrenceSpec(PartSpec):
    """A recurrence over ``width`` channels whose gates read only the current token (minGRU):
    z = sigmoid(W_z h + b_z), u = W_x h + b_x, candidate c = u + 1/2 where u >= 0 and sigmoid(u)
    elsewhere, state S <- (1 - z) S + z c per channel (float32, zero at a sequence's start),
    output W_o (S * silu(W_g h))."""

    hidden: int = 0
    width: int = 0


@dataclass(frozen=True)
class SelectiveStateSpec(PartSpec):
    """A state-space mixer in the form of Mamba-2: ``heads`` heads of ``head_dim`` channels, a state of ``state``
    rows per head, input and output maps B and C shared by the heads of one of ``groups`` groups.  One input
    projection gives ``[z | x | B | C | dt]``; x, B and C pass a causal convolution of ``conv`` taps per channel
    (with a bias) and SiLU; dt = softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T and
    y = S^T C + D x; y * silu(z) is RMS-normed in ``norm_groups`` equal parts (``eps``) with one weight over all
    channels, then projected out.  ``names``: the input projection, the convolution (its bias: that name plus
    ``.b``), dt_bias, A_log, D, the norm and the output projection after the prefix."""

    hidden: int = 0
    heads: int = 0
    head_dim: int = 0
    state: int = 0
    groups: int = 1
    conv: int = 4
    norm_groups: int = 1
    eps: float = 1e-6
    names: Tuple[str, ...] = ("in", "conv", "dt_bias", "A_log", "D", "norm", "o")


@dataclass(frozen=True)
class GatedDeltaSpec(PartSpec):
    """The gated delta rule: ``heads`` value heads of ``v_head_dim`` channels over ``kv_heads`` query/key heads of
    ``head_dim``.  q, k, v pass a causal convolution of ``conv`` taps per channel (no bias) and SiLU; q and k become
    unit vectors per head (``unit_eps`` under the root), q also times head_dim^-1/2; beta = sigmoid(W_b h) per head;
    a decay per head and key channel, g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) + dt_bias)); per head
    S <- diag(g) S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q; o is RMS-normed per head (``eps``) with one
    weight shared by the heads, times sigmoid(W_g2 (W_g1 h)), then projected out.  ``decay_rank`` / ``gate_rank``:
    the inner sizes of the two low-rank maps; None: whatever the tensors' shapes say (the random-weights mode then
    draws ``DEFAULT_RANK``)."""

    hidden: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    conv: int = 4
    eps: float = 1e-6
    unit_eps: float = 1e-6
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None

    DEFAULT_RANK = 16


@dataclass(frozen=True)
class ParallelMixerSpec(PartSpec):
    """Two mixers that read the same input; the result is left_scale * left + right_scale * right.
    ``out_norms`` = (left name, right name): each mixer's result (after its own output projection) is first
    RMS-normed over the model width with a learned weight of that name after the prefix (``out_norm_eps``; the
    weight enters as ``out_norm_offset + w``)."""

    hidden: int = 0
    left: Optional[PartSpec] = None
    right: Optional[PartSpec] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    out_norms: Optional[Tuple[str, str]] = None
    out_norm_eps: float = 1e-6
    out_norm_offset: float = 0.0


@dataclass(frozen=True)
class FeedForwardSpec(PartSpec):
    hidden: int = 0
    intermediate: int = 0
    activation: str = "silu"
    eps: float = 1e-6      # of activations that norm (polynorm)
    # tensor names of the gate, up and down matrices after the part's prefix; None: the "gate_proj.weight" family
    names: Optional[Tuple[str, ...]] = None
    # the three projections have biases: the matrix's name with this suffix (None: no biases)
    bias_suffix: Optional[str] = None
    # parameters of activations that take some ("swish_clamp": limit, alpha)
    act_params: Tuple[float, ...] = ()


@dataclass(frozen=True)
class RoutedExpertsSpec(PartSpec):
    """``experts`` small gated feed-forwards (``e0.``, ``e1.``, ... after the prefix, without biases) of which a
    learned router gives every token ``top``.  Scores are ``sigmoid(W_router h)`` in float32; the choice is made
    on ``score + correction`` (a learned vector; ``correction`` False: on the scores), the weights are the chosen
    experts' plain scores (``renormalize``: divided by their sum).  Experts form ``groups`` equal groups of
    neighbours; a group's score is the sum of its ``group_best`` largest choice scores and only experts of the
    ``keep`` best groups can be chosen.  ``activation`` / ``act_params`` as in ``FeedForwardSpec``.  ``shared``:
    a gated feed-forward of its own sizes (``shared.`` after the prefix) that every token runs and that is added."""

    hidden: int = 0
    intermediate: int = 0
    experts: int = 0
    top: int = 1
    groups: int = 1
    keep: int = 1
    group_best: int = 2
    correction: bool = True
    renormalize: bool = False
    activation: str = "silu"
    act_params: Tuple[float, ...] = ()
    shared: Optional[FeedForwardSpec] = None


@dataclass(frozen=True)
class TokenSideSpec(PartSpec):
    """A layer's own input from the token ids: with e the ``dim`` columns from ``column`` of the row of a table
    over token ids (``table``: the tensor's full name, shared by all layers, ``columns`` wide),
    y = W_proj (gelu_tanh(W_gate x) * e).  ``names``: W_gate and W_proj after the prefix."""

    hidden: int = 0
    dim: int = 0
    vocab: int = 0
    table: str = ""
    column: int = 0
    columns: int = 0
    names: Tuple[str, str] = ("gate", "proj")


@dataclass(frozen=True)
class ExpertTableSpec(PartSpec):
    """``experts`` small SiLU-gated feed-forwards of which every token uses ``top``, named by a
    table over token ids (no router); each chosen expert has weight 1 / top."""

    hidden: int = 0
    intermediate: int = 0
    experts: int = 0
    top: int = 1
    vocab: int = 0


@dataclass(frozen=True)
class BlockOp:
    """One operation of a block's program.  A program works on named activations of shape
    ``[tokens, hidden]``; ``"x"`` is the residual stream that enters and leaves the block, every
    other name is local to the block.

    * ``op="norm"``: ``dst = norm(src)`` with the norm ``spec``;
    * ``op="mixer"`` / ``op="feed_forward"``: ``dst = part(src)`` with the part ``spec``;
    * ``op="add"``: ``dst = dst + scale * gain * src`` (no spec); ``gain`` names a learned vector over the
      channels (its tensor name after the block's prefix; None: ones).

    ``name`` is the tensor-name piece between the block's prefix and the part's own tensor names;
    two operations with the same ``op`` and ``name`` are the same part (one set of weights).
    An addition into a value is carried out when that value is next read: by the norm kernel
    that reads it where a norm follows (sum and norm in one pass, the sum in float32), by an
    addition kernel otherwise.  A norm of a block-local value that is only added into another value afterwards
    may likewise be carried out by the kernel that forms that sum, where its kind offers that."""

    op: str
    src: str
    dst: str
    spec: Optional[PartSpec] = None
    name: str = ""
    scale: float = 1.0
    gain: Optional[str] = None


BLOCK_OPS = ("norm", "mixer", "feed_forward", "add")


@dataclass(frozen=True)
class BlockSpec:
    """One set of layer weights and the arrangement of its parts: ``program`` lists the block's
    operations in order.  ``prefix`` is the tensor-name prefix of the block's weights.  A block
    holds at most one mixer (a layer with two is written as two blocks, the first without a
    feed-forward); it may hold none."""

    prefix: str
    program: Tuple[BlockOp, ...]

    def ops_of(self, op: str) -> Tuple[BlockOp, ...]:
        return tuple(o for o in self.program if o.op == op)

    @property
    def mixer(self) -> Optional[PartSpec]:
        ops = self.ops_of("mixer")
        return ops[0].spec if ops else None

    @property
    def feed_forward(self) -> Optional[PartSpec]:
        ops = self.ops_of("feed_forward")
        return ops[0].spec if ops else None

    def norms(self) -> Tuple[PartSpec, ...]:
        return tuple(o.spec for o in self.ops_of("norm"))

    def validate(self) -> None:
        defined = {"x"}
        mixers = set()
        for i, o in enumerate(self.program):
            where = f"block '{self.prefix}' operation {i} ({o.op})"
            if o.op not in BLOCK_OPS:
                raise ValueError(f"{where}: unknown operation; known: {', '.join(BLOCK_OPS)}")
            if o.src not in defined:
                raise ValueError(f"{where}: reads '{o.src}', which no earlier operation has produced")
            if o.op == "add":
                if o.dst not in defined:
                    raise ValueError(f"{where}: adds into '{o.dst}', which no earlier operation has produced")
                if o.spec is not None:
                    raise ValueError(f"{where}: an addition has no part")
                if o.src == o.dst:
                    raise ValueError(f"{where}: adds '{o.src}' to itself")
            elif o.scale != 1.0 or o.gain is not None:
                raise ValueError(f"{where}: only an addition has a scale or a gain")
            else:
                if o.spec is None:
                    raise ValueError(f"{where}: needs a part spec")
                if o.dst == o.src and o.op != "norm":
                    raise ValueError(f"{where}: a part may not write the value it reads")
                defined.add(o.dst)
            if o.op == "mixer":
                mixers.add(o.name)
        if len(mixers) > 1:
            raise ValueError(f"block '{self.prefix}' holds {len(mixers)} mixers; a block holds at most one "
                             f"(write the layer as several blocks)")


def pre_norm_block(prefix: str, norm_in: NormSpec, mixer: PartSpec, norm_post: NormSpec, feed_forward: PartSpec, *,
                   norm_in_name: str = "input_layernorm.", mixer_name: str = "self_attn.",
                   norm_post_name: str = "post_attention_layernorm.", feed_forward_name: str = "mlp.") -> BlockSpec:
    """The pre-norm residual block ``x += mixer(norm_in(x)); x += feed_forward(norm_post(x))``
    (src/models/qwen3.rs:108-134)."""
    return BlockSpec(prefix, (
        BlockOp("norm", "x", "h", norm_in, norm_in_name),
        BlockOp("mixer", "h", "a", mixer, mixer_name),
        BlockOp("add", "a", "x"),
        BlockOp("norm", "x", "h", norm_post, norm_post_name),
        BlockOp("feed_forward", "h", "f", feed_forward, feed_forward_name),
        BlockOp("add", "f", "x"),
    ))


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """A table of ``buckets + 1`` rows added to the embedding: a token after ``prev`` takes row
    ``(prev * mul_prev + token * mul_cur) mod buckets``, a sequence's first token the last row."""

    name: str
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class LayerRun:
    """One execution of a block.  ``cache_from`` names an earlier position in the run list whose
    cache this run reads instead of writing its own (None = own cache).  ``add_input``: the embedding's
    output (the residual stream as it was before the first run) is added to the stream before this run."""

    block: int
    cache_from: Optional[int] = None
    add_input: bool = False


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden: int
    embed_name: str
    blocks: Tuple[BlockSpec, ...]
    runs: Tuple[LayerRun, ...]
    final_norm: PartSpec
    final_norm_name: str  # tensor-name prefix of the final norm
    # None = the head reuses the embedding table
    head_name: Optional[str]
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    # the embedding rows are multiplied by this (rounded to the activation dtype) before the first block
    embed_scale: Optional[float] = None
    # what happens to the float32 logits after the head: logits *= logit_scale, then
    # logits = logit_softcap * tanh(logits / logit_softcap); None = off
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    # the residual stream's dtype ("float32"); None = the engine's dtype
    residual_dtype: Optional[str] = None
    # added to every token's embedding row: a row of a table over hashed (previous token, token) pairs, and a
    # learned vector per position (the tensor's name; it has max_positions rows)
    pair_embedding: Optional["PairEmbeddingSpec"] = None
    position_table: Optional[str] = None
    # standard deviations used by the random-weights mode
    init_std: float = 0.02
    norm_init_std: float = 0.1

    def validate(self) -> None:
        if not self.blocks:
            raise ValueError("a model plan needs at least one block")
        for b in self.blocks:
            b.validate()
        if self.residual_dtype not in (None, "float32"):
            raise ValueError(f"residual_dtype must be None or 'float32', got {self.residual_dtype!r}")
        if (self.pair_embedding is not None or self.position_table is not None) and self.residual_dtype != "float32":
            raise ValueError("a pair embedding or a position table is summed into a float32 residual stream")
        if self.logit_softcap is not None and not (self.logit_softcap > 0):
            raise ValueError(f"logit_softcap must be positive, got {self.logit_softcap}")
        for pos, run in enumerate(self.runs):
            if not (0 <= run.block < len(self.blocks)):
                raise ValueError(f"run {pos} names block {run.block}, but there are {len(self.blocks)}")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < pos):
                    raise ValueError(f"run {pos} reads the cache of run {run.cache_from}, which is not earlier")
                if self.runs[run.cache_from].cache_from is not None:
                    raise ValueError(f"run {pos} reads the cache of run {run.cache_from}, which owns none")
