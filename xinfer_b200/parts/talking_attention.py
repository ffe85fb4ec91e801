"""Grouped-query attention whose heads talk to each other before the softmax.

    q = W_q h, k = W_k h, v = W_v h         heads of size head_dim (q, k) and v_head_dim (v)
    q, k: per-head norm (with or without a learned weight) before or after the rotary encoding
    raw_g[i, j] = scale * q_g[i] . k_kv(g)[j]
    s_h[i, j]   = sum_g talk[h, g] raw_g[i, j]                          (``talking_heads``)
    p_h[i, j]   = exp(s_h[i, j]) / (sink + sum_j' exp(s_h[i, j']))      sink = 1 (``sink``) or 0
    out         = W_o concat_h( sum_j p_h[i, j] v_kv(h)[j] )

Options of the spec beyond that: biases on q, k, v (and the output projection); keys that double as values
(``value_from_key``: v is the k projection with its bias, before norm and rotation, and there is no W_v); ONE norm
over the whole q (k) projection instead of one per head; a cap on the scores, ``cap * tanh(s / cap)``; a bias on
the distance after the cap, ``- 2^(-x (h + 1) / heads) * (i - j)``; a chunked mask (a query sees the earlier keys
of its own chunk of positions, counted from the sequence's start); a sigmoid gate on the heads' outputs, one number
per channel or per head.

Causal, optionally within a window; query head h reads key/value head h // (heads / kv_heads).  With a
sink the weights of a row sum to less than one: a query may attend to nothing.  Keys after rotation and
norm, and values, live in the paged cache; scores, mix, softmax and value sums are float32.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import AttentionSpec
from ..weights.loader import WeightSpec
from .base import CacheTensor, LayerCache, Mixer, PagedCacheNeed, StepContext, build_part, register_mixer
from .linear import linear

_DEFAULT_NAMES = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "talk.weight")
_DEFAULT_NORM_NAMES = ("q_norm.weight", "k_norm.weight")
# a single-token step cuts every token's keys into ranges so that about this many blocks run: one per SM (the
# kernel's shared memory allows one block per SM; 8 requests at context 4,096 take 71.7 us in one wave of 144
# blocks and 80.2 us in 256 blocks)
_DECODE_BLOCKS = 148
_DECODE_MIN_KEYS = 128
# bfloat16: both products on tensor cores where the sizes allow; tests switch it off to compare the two forms
USE_TENSOR_CORES = True
# without a mix and a sink the attention is the ordinary one: use the kernels of the engine's attention backend
USE_ATTENTION_BACKEND = True


class TalkingAttention(Mixer):
    kind = "talking_attention"
    graph_safe = True

    def __init__(self, spec: AttentionSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads do not divide into {spec.num_kv_heads} key/value heads")
        self.position = build_part("position", spec.rope, prefix, dtype, device) if spec.rope is not None else None
        if self.position is not None and not hasattr(self.position, "frequencies"):
            raise ValueError("this attention needs a rotary position encoding that offers its frequencies")
        self.names = tuple(spec.names) if spec.names else _DEFAULT_NAMES
        self.w_qkv = self.w_o = self.talk = self.q_norm = self.k_norm = self.bias = self.b_o = None
        if spec.value_from_key and spec.value_dim != spec.head_dim:
            raise ValueError(f"keys of {spec.head_dim} channels cannot double as values of {spec.value_dim}")
        if spec.chunk is not None and spec.window is not None:
            raise ValueError("an attention takes a window or a chunked mask, not both")
        if (spec.score_softcap is not None or spec.distance_slope_exponent is not None or spec.chunk is not None) and (
                spec.talking_heads or spec.sink):
            raise ValueError("a score cap, a distance bias and a chunked mask are not built for talking heads or a sink")

    @classmethod
    def weight_specs(cls, spec: AttentionSpec, prefix: str) -> List[WeightSpec]:
        n = tuple(spec.names) if spec.names else _DEFAULT_NAMES
        d, dv = spec.head_dim, spec.value_dim
        out = [
            WeightSpec(prefix + n[0], (spec.num_heads * d, spec.hidden)),
            WeightSpec(prefix + n[1], (spec.num_kv_heads * d, spec.hidden)),
        ]
        if not spec.value_from_key:
            out.append(WeightSpec(prefix + n[2], (spec.num_kv_heads * dv, spec.hidden)))
        out.append(WeightSpec(prefix + n[3], (spec.hidden, spec.num_heads * dv)))
        if spec.talking_heads:
            out.append(WeightSpec(prefix + n[4], (spec.num_heads, spec.num_heads), "unit"))
        if spec.qk_norm and spec.qk_norm_weight:
            qn, kn = spec.qk_norm_names or _DEFAULT_NORM_NAMES
            nq, nk = (spec.num_heads * d, spec.num_kv_heads * d) if spec.qk_norm_whole else (d, d)
            out += [WeightSpec(prefix + qn, (nq,), "norm"), WeightSpec(prefix + kn, (nk,), "norm")]
        if spec.bias_suffix:
            out += [WeightSpec(prefix + n[0] + spec.bias_suffix, (spec.num_heads * d,), "around_zero"),
                    WeightSpec(prefix + n[1] + spec.bias_suffix, (spec.num_kv_heads * d,), "around_zero")]
            if not spec.value_from_key:
                out.append(WeightSpec(prefix + n[2] + spec.bias_suffix, (spec.num_kv_heads * dv,), "around_zero"))
            if spec.out_bias:
                out.append(WeightSpec(prefix + n[3] + spec.bias_suffix, (spec.hidden,), "around_zero"))
        if spec.gate_name:
            out.append(WeightSpec(prefix + spec.gate_name, (spec.num_heads * (1 if spec.gate_per_head else dv), spec.hidden)))
        return out

    def load(self, store) -> None:
        p, n, s = self.prefix, self.names, self.spec
        own = (0, 1) if s.value_from_key else (0, 1, 2)      # keys that double as values: the row is [q | k (| gate)]
        parts = [store.get(p + n[i], self.device, self.dtype, operand=True) for i in own]
        if s.gate_name:     # the gate reads the same input: one product gives [q | k | v | gate]
            parts.append(store.get(p + s.gate_name, self.device, self.dtype, operand=True))
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        del parts
        if s.bias_suffix:
            self.bias = torch.cat([store.get(p + n[i] + s.bias_suffix, self.device, torch.float32).float()
                                   for i in own]).contiguous()
            if s.out_bias:
                self.b_o = store.get(p + n[3] + s.bias_suffix, self.device, torch.float32).float().contiguous()
        self.w_o = store.get(p + n[3], self.device, self.dtype, operand=True)
        if s.talking_heads:
            self.talk = store.get(p + n[4], self.device, torch.float32).float().contiguous()
        if s.qk_norm and s.qk_norm_weight:
            qn, kn = s.qk_norm_names or _DEFAULT_NORM_NAMES
            self.q_norm = store.get(p + qn, self.device, torch.float32).float().contiguous()
            self.k_norm = store.get(p + kn, self.device, torch.float32).float().contiguous()

    def cache_need(self) -> PagedCacheNeed:
        s = self.spec
        return PagedCacheNeed((("k", CacheTensor((s.num_kv_heads, s.head_dim), None, 1)),
                               ("v", CacheTensor((s.num_kv_heads, s.value_dim), None, 1))), s.window)

    def _plain_softmax(self) -> bool:
        """No mix across heads, no sink, key and value heads of one size in bfloat16: the attention itself is the
        ordinary grouped-query one, and the engine's tcgen05 kernels (work lists, decode plans) take it."""
        s = self.spec
        return (USE_ATTENTION_BACKEND and not s.talking_heads and not s.sink and s.value_dim == s.head_dim
                and self.dtype == torch.bfloat16 and kernels.attn_tiled_supported(self.dtype, s.head_dim))

    def _changed_scores(self) -> bool:
        """A cap, a distance bias or a chunked mask: what the ordinary attention kernels do not know."""
        s = self.spec
        return s.score_softcap is not None or s.distance_slope_exponent is not None or s.chunk is not None

    def prepare_step(self, ctx: StepContext, cache: LayerCache) -> None:
        if self._plain_softmax():
            from . import attention_backend
            s = self.spec
            attention_backend.prepare_step(ctx, self.dtype, s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size,
                                           kernels.mask_code(s.window, s.chunk), ctx.strides[cache.group])

    # ---- the two halves ---------------------------------------------------------------------------
    def inner_width(self) -> int:
        return self.spec.num_heads * self.spec.value_dim

    def output_weight(self) -> torch.Tensor:
        return self.w_o

    def forward_inner(self, x, ctx: StepContext, cache: LayerCache, state, writes_cache, out, out_scale) -> None:
        s = self.spec
        T = x.shape[0]
        nh, nkv, d, dv = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        ws = ctx.workspace
        nqkv = (nh + nkv) * d + (0 if s.value_from_key else nkv * dv)
        if s.gate_name:
            proj = ws.get("tattn.qkvg", (T, nqkv + nh * (1 if s.gate_per_head else dv)), self.dtype)
            linear(proj, x, self.w_qkv, ctx.err)
            qkv = proj
        else:
            qkv = ws.get("tattn.qkv", (T, nqkv), self.dtype)
            linear(qkv, x, self.w_qkv, ctx.err)
        q = ws.get("tattn.q", (T, nh, d), self.dtype)
        table, stride = ctx.tables[cache.group], ctx.strides[cache.group]
        rope = self.position.spec if self.position is not None else None
        norm_mode = 0 if not s.qk_norm else (2 if s.qk_norm_after_rope else (3 if s.qk_norm_whole else 1))
        kernels.qkv_prepare(q, cache["k"], cache["v"], qkv, self.q_norm, self.k_norm,
                            self.position.frequencies() if rope is not None else None, ctx.positions, ctx.req_of_token,
                            table, stride, nh, nkv, d, dv, rope.rotary_dim if rope is not None else 0,
                            rope is not None and rope.layout == "interleaved", norm_mode, s.qk_norm_eps, writes_cache,
                            ctx.err, rot_magnitude=rope.magnitude if rope is not None else 1.0, bias=self.bias,
                            q_temp=s.q_temp, row_len=qkv.shape[1], value_offset=nh * d if s.value_from_key else None)
        self._attend(q, ctx, cache, table, stride, out, out_scale)
        if s.gate_name:
            kernels.gate_sigmoid(out, out.view(T, nh, dv).transpose(0, 1), qkv[:, nqkv:])

    def _attend(self, q, ctx: StepContext, cache: LayerCache, table, stride, out, out_scale) -> None:
        s = self.spec
        T = q.shape[0]
        nh, nkv, d, dv = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        ws = ctx.workspace
        if self._plain_softmax() and out_scale == 1.0 and out.is_contiguous():
            from . import attention_backend
            attention_backend.attend(out.view(T, nh, dv), q, cache, ctx, table, stride, s.window, s.scale,
                                     softcap=s.score_softcap, slope_exponent=s.distance_slope_exponent, chunk=s.chunk)
            return
        # queries per block: the longest portion decides (a step of single tokens takes one query per block
        # and cuts the keys instead); a replayed step must not look at its actual lengths
        single = ctx.all_single or ctx.fixed_shapes
        longest = 1 if single else int((ctx.h_q_start[1:] - ctx.h_q_start[:-1]).max())
        mma = (USE_TENSOR_CORES and self.dtype == torch.bfloat16 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0
               and kernels.attn_talking_mma_tile(nh, nkv, d, dv, longest) > 0)
        bq = kernels.attn_talking_mma_tile(nh, nkv, d, dv, longest) if mma else kernels.attn_talking_tile(nh, d, dv, longest)
        if self._changed_scores():
            if out_scale != 1.0 or not out.is_contiguous():
                raise kernels.KernelError("attention with changed scores writes a contiguous, unscaled result")
            kernels.attention_plain(out.view(T, nh, dv), q, cache["k"], cache["v"], ctx.positions, ctx.req_of_token, table,
                                    stride, s.window, s.scale, ctx.err, softcap=s.score_softcap,
                                    slope_exponent=s.distance_slope_exponent, chunk=s.chunk)
            return
        if bq <= 0 and not s.talking_heads and out_scale == 1.0 and out.is_contiguous():
            # no mix across heads: a head needs no other head in its block, and the kernel with one warp per
            # (token, head) takes any number of heads of any size (a silent entry of score 0 is a sink of zeros)
            if s.sink and getattr(self, "_zero_sink", None) is None:
                self._zero_sink = torch.zeros(nh, dtype=torch.float32, device=self.device)
            kernels.attention_plain(out.view(T, nh, dv), q, cache["k"], cache["v"], ctx.positions, ctx.req_of_token, table,
                                    stride, s.window, s.scale, ctx.err, sink=self._zero_sink if s.sink else None)
            return
        if bq <= 0:
            raise kernels.KernelError(f"attention with {nh} heads of {d}/{dv} channels does not fit the kernel's tile")
        parts, part_o, part_ml = 1, None, None
        if single and bq == 1:      # (a single-token step always gets a tile of one query)
            bound = stride * cache.page_size if ctx.fixed_shapes else ctx.max_context
            if s.window:
                bound = min(bound, s.window + 32)
            parts = max(1, min(_DECODE_BLOCKS // max(T, 1), bound // _DECODE_MIN_KEYS, 64))
            if parts > 1:
                part_o = ws.get("tattn.part_o", (T * parts * nh * dv,), torch.float32)
                part_ml = ws.get("tattn.part_ml", (T * parts * nh * 2,), torch.float32)
        (kernels.attn_talking_mma if mma else kernels.attn_talking)(out, q, cache["k"], cache["v"], self.talk, ctx.q_start, ctx.start_pos, ctx.num_entries, table,
                             stride, s.window, s.scale, s.sink, out_scale, bq, ctx.err, parts, part_o, part_ml)

    def forward(self, x, ctx: StepContext, cache: LayerCache, state=None, writes_cache: bool = True):
        T = x.shape[0]
        inner = ctx.workspace.get("tattn.inner", (T, self.inner_width()), self.dtype)
        self.forward_inner(x, ctx, cache, state, writes_cache, inner, 1.0)
        out = ctx.workspace.get("tattn.out", (T, self.spec.hidden), ctx.branch_dtype or self.dtype)
        linear(out, inner, self.w_o, ctx.err)
        if self.b_o is not None:
            kernels.add_bias(out, self.b_o)
        return out


register_mixer("talking_attention", TalkingAttention)
