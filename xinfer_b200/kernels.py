"""Python faces of the CUDA kernels.  Each wrapper checks devices, dtypes, shapes and contiguity,
launches on the current torch stream and raises on a launch error.  Nothing here computes on the
CPU or through a library: a missing extension or a CPU tensor is an error.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np
import torch

from .native import kernels_lib

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    """The checks every wrapper makes on its tensors; the message is only put together on failure
    (these run a few thousand times in a step of a small model)."""
    try:
        ok = t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype)
    except AttributeError:
        ok = False
    if ok and shape is not None:
        ts = t.shape
        if len(ts) != len(shape):
            ok = False
        else:
            for want, have in zip(shape, ts):
                if want is not None and want != have:
                    ok = False
                    break
    if not ok:
        _need_failed(t, name, dtype, shape)


def _need_failed(t, name, dtype, shape) -> None:
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous (shape {tuple(t.shape)}, strides {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    raise KernelError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")


try:    # the raw handle of the current stream without building a Stream object for every launch
    _raw_stream, _device_index = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:  # pragma: no cover - other torch builds
    _raw_stream = None


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(_device_index())
    return torch.cuda.current_stream().cuda_stream


_launches = 0
_by_name: dict = {}

# Use the 16-byte-access bfloat16 kernels for norm / gate / q-k preparation where sizes allow;
# tests switch this off to compare them with the plain kernels.
vectorized = True
# From this many rows (tokens) on, the SiLU gate runs in its many-row form (blocks that stay on
# their SM and walk over rows with the next row's loads in flight); below, in the form shaped for a
# decode step's few rows.  The two forms give the same bits; tests move this bound to compare them.
many_rows = int(os.environ.get("XINFER_B200_MANY_ROWS", "256"))


def launch_count() -> int:
    """Kernels of this engine launched so far by this process (captured launches included)."""
    return _launches


def launch_counts() -> dict:
    """Launches so far by wrapper name (a copy): which kernels a step really ran."""
    return dict(_by_name)


def _ok(status: int, what: str, n: int = 1) -> None:
    global _launches
    if status != 0:
        raise KernelError(f"{what}: CUDA error {status} at launch")
    _launches += n
    _by_name[what] = _by_name.get(what, 0) + n


# device-side error word -------------------------------------------------------------------------
ERR_BAD_TOKEN, ERR_BAD_PAGE, ERR_WAIT, ERR_BAD_ROW, ERR_SCRATCH, ERR_BAD_POSITION = 1, 2, 4, 8, 16, 32


def describe_error(word: int) -> str:
    parts = []
    if word & ERR_BAD_TOKEN:
        parts.append("a token id outside the vocabulary")
    if word & ERR_BAD_PAGE:
        parts.append("a block-table entry outside the page pool")
    if word & ERR_WAIT:
        parts.append("a bounded wait inside a kernel gave up")
    if word & ERR_BAD_ROW:
        parts.append("a requested row outside the step's tokens")
    if word & ERR_BAD_POSITION:
        parts.append("a token position outside the position table")
    if word & ERR_SCRATCH:
        parts.append("scratch memory that a kernel must find zeroed was not")
    return "; ".join(parts) or "no error"


# ---- wrappers --------------------------------------------------------------------------------------
def embedding(out, table, ids, err, sampled=None, scale=None):
    """out[t] = table[ids[t]] (times ``scale``, if given, rounded to the table's dtype); an id -1 - i
    is replaced on the device by ``sampled[i]`` (int32 ids a sampler left there)."""
    T, H = out.shape
    wide = out.dtype == torch.float32 and table.dtype != torch.float32     # a float32 stream over a bfloat16 table
    _need(out, "out", torch.float32 if wide else table.dtype, (T, H))
    _need(table, "table", None, (None, H))
    _need(ids, "ids", torch.int32)
    if ids.numel() < T:
        raise KernelError(f"ids holds {ids.numel()} entries for {T} tokens")
    _need(err, "err", torch.int32)
    if sampled is not None:
        _need(sampled, "sampled", torch.int32)
    if wide:
        _ok(kernels_lib().xb_embedding_f32(dtype_code(table.dtype), out.data_ptr(), table.data_ptr(), ids.data_ptr(),
                                           _ptr(sampled), sampled.numel() if sampled is not None else 0, T, H, table.shape[0],
                                           1.0 if scale is None else float(scale), err.data_ptr(), _stream()), "embedding_f32")
        return
    _ok(kernels_lib().xb_embedding(dtype_code(table.dtype), out.data_ptr(), table.data_ptr(), ids.data_ptr(),
                                   _ptr(sampled), sampled.numel() if sampled is not None else 0,
                                   T, H, table.shape[0], 1.0 if scale is None else float(scale), err.data_ptr(),
                                   _stream()), "embedding")


def logits_post(logits, scale=None, softcap=None):
    """In place on float32 logits: ``logits *= scale``, then ``logits = softcap * tanh(logits / softcap)``."""
    _need(logits, "logits", torch.float32)
    _ok(kernels_lib().xb_logits_post(logits.data_ptr(), logits.numel(), 1.0 if scale is None else float(scale),
                                     0.0 if softcap is None else float(softcap), _stream()), "logits_post")


def rmsnorm(out, x, weight, eps, err, *, branch=None, sum_out=None, rows=None, weight_offset=0.0):
    """out = norm(s) * (offset + w) with s = x (+ branch), optionally gathered at ``rows``;
    ``sum_out`` receives s (it may be x itself when no rows are given)."""
    dim = x.shape[-1]
    n = out.shape[0]
    _need(x, "x", None, (None, dim))
    _need(weight, "weight", torch.float32, (dim,))
    if x.dtype == torch.float32 and (out.dtype != torch.float32 or (branch is not None and branch.dtype != torch.float32)):
        # a float32 stream beside activations in the engine's type
        _need(out, "out", None, (n, dim))
        if branch is not None:
            _need(branch, "branch", None, tuple(x.shape))
        if sum_out is not None:
            _need(sum_out, "sum_out", torch.float32, (n, dim))
        if rows is not None:
            _need(rows, "rows", torch.int32)
            if rows.numel() < n:
                raise KernelError(f"rows holds {rows.numel()} entries for {n} output rows")
        elif n != x.shape[0]:
            raise KernelError(f"out has {n} rows, x has {x.shape[0]} and no row list was given")
        _ok(kernels_lib().xb_rmsnorm_f32(dtype_code(branch.dtype) if branch is not None else F32, dtype_code(out.dtype),
                                         out.data_ptr(), _ptr(sum_out), x.data_ptr(), _ptr(branch), _ptr(rows),
                                         weight.data_ptr(), n, dim, x.shape[0], float(eps), float(weight_offset),
                                         err.data_ptr(), _stream()), "rmsnorm_f32")
        return
    _need(out, "out", x.dtype, (n, dim))
    if branch is not None:
        _need(branch, "branch", x.dtype, tuple(x.shape))
    if sum_out is not None:
        _need(sum_out, "sum_out", x.dtype, (n, dim))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n:
            raise KernelError(f"rows holds {rows.numel()} entries for {n} output rows")
    elif n != x.shape[0]:
        raise KernelError(f"out has {n} rows, x has {x.shape[0]} and no row list was given")
    if vectorized and x.dtype == torch.bfloat16 and dim % 8 == 0 and dim <= 32768:
        _ok(kernels_lib().xb_rmsnorm_bf16(out.data_ptr(), _ptr(sum_out), x.data_ptr(), _ptr(branch), _ptr(rows),
                                          weight.data_ptr(), n, dim, x.shape[0], float(eps), float(weight_offset),
                                          err.data_ptr(), _stream()), "rmsnorm_bf16")
        return
    _ok(kernels_lib().xb_rmsnorm(dtype_code(x.dtype), out.data_ptr(), _ptr(sum_out), x.data_ptr(), _ptr(branch),
                                 _ptr(rows), weight.data_ptr(), n, dim, x.shape[0], float(eps),
                                 float(weight_offset), err.data_ptr(), _stream()), "rmsnorm")


def add(out, x, branch, scale: float = 1.0):
    """out = x + scale * branch (the sum in float32)."""
    _need(x, "x")
    if x.dtype == torch.float32 and branch.dtype != torch.float32:
        _need(branch, "branch", None, tuple(x.shape))
        _need(out, "out", torch.float32, tuple(x.shape))
        _ok(kernels_lib().xb_add_f32(dtype_code(branch.dtype), out.data_ptr(), x.data_ptr(), branch.data_ptr(), x.numel(),
                                     float(scale), _stream()), "add_f32")
        return
    _need(branch, "branch", x.dtype, tuple(x.shape))
    _need(out, "out", x.dtype, tuple(x.shape))
    _ok(kernels_lib().xb_add(dtype_code(x.dtype), out.data_ptr(), x.data_ptr(), branch.data_ptr(), x.numel(), float(scale),
                             _stream()), "add")


def dyt_norm(out, x, alpha, weight, bias, err, *, branch=None, branch_scale: float = 1.0, branch_norm=None, sum_out=None,
             rows=None):
    """Dynamic Tanh: out = tanh(alpha * s) * weight + bias with s = x + branch_scale * br, optionally gathered at
    ``rows``; ``br`` is the branch, or with ``branch_norm`` = (alpha, weight, bias) its own Dynamic Tanh first.
    ``sum_out`` receives s (it may be x itself when no rows are given); ``out`` None: only the sum is formed.
    x and sum_out share a type, the branch and out may have another; the arithmetic is float32."""
    dim = x.shape[-1]
    n = out.shape[0] if out is not None else x.shape[0]
    _need(x, "x", None, (None, dim))
    for name, t, shape in (("alpha", alpha, ()), ("weight", weight, (dim,)), ("bias", bias, (dim,))):
        _need(t, name, torch.float32, shape)
    if out is not None:
        _need(out, "out", None, (n, dim))
    if branch is not None:
        _need(branch, "branch", None, tuple(x.shape))
    if branch_norm is not None:
        if branch is None:
            raise KernelError("a branch norm needs a branch")
        for name, t, shape in (("branch alpha", branch_norm[0], ()), ("branch weight", branch_norm[1], (dim,)),
                               ("branch bias", branch_norm[2], (dim,))):
            _need(t, name, torch.float32, shape)
    if sum_out is not None:
        _need(sum_out, "sum_out", x.dtype, (n, dim))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n:
            raise KernelError(f"rows holds {rows.numel()} entries for {n} output rows")
    elif n != x.shape[0]:
        raise KernelError(f"out has {n} rows, x has {x.shape[0]} and no row list was given")
    bn = branch_norm or (None, None, None)
    _ok(kernels_lib().xb_dyt_norm(dtype_code(x.dtype), dtype_code(branch.dtype) if branch is not None else F32,
                                  dtype_code(out.dtype) if out is not None else F32, _ptr(out), _ptr(sum_out), x.data_ptr(),
                                  _ptr(branch), _ptr(rows), alpha.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                  float(branch_scale), _ptr(bn[0]), _ptr(bn[1]), _ptr(bn[2]), n, dim, x.shape[0],
                                  err.data_ptr(), _stream()), "dyt_norm")


def gemm_plain(out, a, w):
    """out[M, N] = a[M, K] . w[N, K]^T with float32 FMA accumulation (no tensor cores)."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", None, (M, K))
    _need(w, "w", None, (N, K))
    _need(out, "out", None, (M, N))
    _ok(kernels_lib().xb_gemm_plain(dtype_code(a.dtype), dtype_code(w.dtype), dtype_code(out.dtype), out.data_ptr(),
                                    a.data_ptr(), w.data_ptr(), M, N, K, _stream()), "gemm_plain")


def rope_table(cos_t, sin_t, inv_freq):
    max_pos, half = cos_t.shape
    _need(cos_t, "cos", torch.float32, (max_pos, half))
    _need(sin_t, "sin", torch.float32, (max_pos, half))
    _need(inv_freq, "inv_freq", torch.float32, (half,))
    _ok(kernels_lib().xb_rope_table(cos_t.data_ptr(), sin_t.data_ptr(), inv_freq.data_ptr(), max_pos, half, _stream()), "rope_table")


def qk_norm_rope_write(q_out, k_cache, v_cache, qkv, q_w, k_w, cos_t, sin_t, positions, req_of_token,
                       block_table, table_stride, nh, nkv, d, rot, interleaved, eps, write_kv, err):
    T = qkv.shape[0]
    _need(qkv, "qkv", None, (T, (nh + 2 * nkv) * d))
    _need(q_out, "q_out", qkv.dtype, (T, nh, d))
    if write_kv:
        _need(k_cache, "k_cache", qkv.dtype, (None, nkv, None, d))
        _need(v_cache, "v_cache", qkv.dtype, tuple(k_cache.shape))
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    page_size = k_cache.shape[2] if k_cache is not None else 1
    for name, w_ in (("q_norm", q_w), ("k_norm", k_w)):
        if w_ is not None:
            _need(w_, name, torch.float32, (d,))
    max_pos = 0
    if cos_t is not None:
        _need(cos_t, "cos", torch.float32, (None, rot // 2))
        _need(sin_t, "sin", torch.float32, tuple(cos_t.shape))
        max_pos = cos_t.shape[0]
    if (vectorized and qkv.dtype == torch.bfloat16 and d % 16 == 0 and d <= 512
            and (cos_t is None or interleaved or rot == d)):
        _ok(kernels_lib().xb_qk_norm_rope_write_bf16(
            q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache), qkv.data_ptr(), _ptr(q_w), _ptr(k_w), _ptr(cos_t), _ptr(sin_t),
            positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(), int(table_stride), T, nh, nkv, d, rot,
            int(bool(interleaved)), page_size, num_pages, max_pos, float(eps), int(bool(write_kv)), err.data_ptr(),
            _stream()), "qk_norm_rope_write_bf16")
        return
    _ok(kernels_lib().xb_qk_norm_rope_write(
        dtype_code(qkv.dtype), q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache), qkv.data_ptr(), _ptr(q_w), _ptr(k_w),
        _ptr(cos_t), _ptr(sin_t), positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(),
        int(table_stride), T, nh, nkv, d, rot, int(bool(interleaved)), page_size, num_pages, max_pos, float(eps),
        int(bool(write_kv)), err.data_ptr(), _stream()), "qk_norm_rope_write")


def attention_plain(out, q, k_cache, v_cache, positions, req_of_token, block_table, table_stride, window, scale, err, *,
                    sink=None, value_dim=None, softcap=None, slope_exponent=None, chunk=None):
    """Attention of every token over its request's cached positions, one warp per (token, head), float32 scores,
    softmax and value sums.  ``q`` is ``[T, heads, d]``, ``out`` ``[T, heads, dv]``.  The caches are
    ``[page, kv_head, slot, d]`` and ``[page, kv_head, slot, dv]``; with ``value_dim`` the values are the first
    ``value_dim`` channels of the key rows themselves (``v_cache`` is then ignored).  ``sink`` (float32 per head):
    one more softmax entry of that score without a value.  ``softcap``: scores pass ``cap * tanh(s / cap)``;
    ``slope_exponent`` x: head h's score of a key ``dist`` positions back loses ``2^(-x (h + 1) / heads) * dist``
    (after the cap); ``chunk``: a query sees the keys of its own chunk of that many positions, counted from the
    sequence's start, instead of a window."""
    T, nh, d = q.shape
    _need(q, "q", None, (T, nh, d))
    _need(k_cache, "k_cache", q.dtype, (None, None, None, d))
    num_pages, nkv, page_size, _ = k_cache.shape
    if value_dim is not None:
        dv = int(value_dim)
        if not (0 < dv <= d):
            raise KernelError(f"values of {dv} channels cannot be the first channels of {d}-channel keys")
        v_cache, v_stride = k_cache, d
    else:
        dv = v_cache.shape[-1]
        _need(v_cache, "v_cache", q.dtype, (num_pages, nkv, page_size, dv))
        v_stride = dv
    _need(out, "out", q.dtype, (T, nh, dv))
    if sink is not None:
        _need(sink, "sink", torch.float32, (nh,))
    if nh % nkv:
        raise KernelError(f"{nh} query heads do not divide into {nkv} key/value heads")
    if max(d, dv) > 1024:
        raise KernelError(f"head size {max(d, dv)} is larger than the plain attention kernel's limit of 1024")
    _ok(kernels_lib().xb_attention_plain(
        dtype_code(q.dtype), out.data_ptr(), q.data_ptr(), nh * d, d, k_cache.data_ptr(), v_cache.data_ptr(), d, v_stride,
        _ptr(sink), positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(), int(table_stride), T, nh, nkv, d,
        dv, page_size, num_pages, int(window or 0), float(scale), float(softcap or 0.0), float(slope_exponent or 0.0),
        int(chunk or 0), err.data_ptr(), _stream()), "attention_plain")


# activations of a gated feed-forward by code.  "swish_clamp" takes two parameters (limit, alpha): with
# a = min(gate, limit) and b = clamp(up, -limit, limit) the product is a * sigmoid(alpha * a) * (b + 1).
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu": 2, "swish_clamp": 3}


def activation_args(activation: str, params=()) -> tuple:
    """(code, p0, p1) of an activation and its parameters for the kernels."""
    code = ACTIVATIONS[activation]
    params = tuple(float(p) for p in (params or ()))
    if activation == "swish_clamp":
        if len(params) != 2 or not params[0] > 0:
            raise KernelError(f"'swish_clamp' takes (limit > 0, alpha), got {params}")
        return code, params[0], params[1]
    if params:
        raise KernelError(f"the activation '{activation}' takes no parameters")
    return code, 0.0, 0.0


def swiglu(out, gate_up, activation: str = "silu", params=()):
    """out[t, i] = act(gate_up[t, i]) * f(gate_up[t, I + i]); ``activation``: a key of ``ACTIVATIONS``."""
    act, p0, p1 = activation_args(activation, params)
    T, two_i = gate_up.shape
    _need(gate_up, "gate_up", None, (T, two_i))
    _need(out, "out", gate_up.dtype, (T, two_i // 2))
    if vectorized and gate_up.dtype == torch.bfloat16 and two_i % 16 == 0:
        if T >= many_rows:
            _ok(kernels_lib().xb_swiglu_rows_bf16(out.data_ptr(), gate_up.data_ptr(), T, two_i // 2, act, p0, p1, _stream()), "swiglu_rows_bf16")
            return
        _ok(kernels_lib().xb_swiglu_bf16(out.data_ptr(), gate_up.data_ptr(), T, two_i // 2, act, p0, p1, _stream()), "swiglu_bf16")
        return
    _ok(kernels_lib().xb_swiglu(dtype_code(gate_up.dtype), out.data_ptr(), gate_up.data_ptr(), T, two_i // 2, act, p0, p1, _stream()), "swiglu")


def widen_bf16(out, x):
    _need(x, "x", torch.bfloat16)
    _need(out, "out", torch.float32, tuple(x.shape))
    _ok(kernels_lib().xb_widen_bf16(out.data_ptr(), x.data_ptr(), x.numel(), _stream()), "widen_bf16")


SAMPLE_PARAMS = np.dtype([
    ("temperature", np.float32), ("top_k", np.int32), ("top_p", np.float32),
    ("seed_lo", np.uint32), ("seed_hi", np.uint32), ("draw", np.uint32),
    ("frequency_penalty", np.float32), ("presence_penalty", np.float32),
    ("history_offset", np.int32), ("history_len", np.int32),
])


def sample_scratch_bytes(capacity: int) -> int:
    """Bytes of scratch for a sampler that sees at most ``capacity`` rows in one call."""
    return int(kernels_lib().xb_sample_scratch_bytes(int(capacity)))


def sample(out_tokens, logits, params_dev, history_dev, apply_penalties: bool, scratch, err_word=None, *,
           capacity: Optional[int] = None):
    """One token per logits row into ``out_tokens``; with ``err_word`` (a device int32) its value is
    written to ``out_tokens[R]``, so that one copy brings tokens and error word to the host.
    ``scratch``: uint8 device buffer of ``sample_scratch_bytes(capacity)``, zero before its first use
    and laid out by ``capacity`` (default: the rows of this call): calls that share a buffer must
    give the same capacity, whatever their rows."""
    R, V = logits.shape
    capacity = R if capacity is None else int(capacity)
    if R > capacity:
        raise KernelError(f"{R} rows exceed the sampler scratch's capacity {capacity}")
    _need(logits, "logits", torch.float32, (R, V))
    _need(out_tokens, "out_tokens", torch.int32)
    _need(params_dev, "params", torch.uint8)
    lib = kernels_lib()
    if lib.xb_sample_params_size() != SAMPLE_PARAMS.itemsize:
        raise KernelError("the sampler's parameter record differs between Python and CUDA")
    _need(scratch, "scratch", torch.uint8)
    if (params_dev.numel() < R * SAMPLE_PARAMS.itemsize or out_tokens.numel() < R + (err_word is not None)
            or scratch.numel() < lib.xb_sample_scratch_bytes(capacity)):
        raise KernelError("sampler buffers are smaller than the number of rows")
    _ok(lib.xb_sample(out_tokens.data_ptr(), logits.data_ptr(), params_dev.data_ptr(), _ptr(history_dev), R, capacity, V,
                      int(bool(apply_penalties)), scratch.data_ptr(), _ptr(err_word), _stream()), "sample",
        2 if apply_penalties else 1)


# ---- bfloat16 attention on tensor cores ------------------------------------------------------------
def attn_tiled_supported(dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256


def mask_code(window=None, chunk=None) -> int:
    """The causal mask as the one number the tcgen05 attention kernels, their work list and their decode plan take:
    0 every earlier key, w > 0 a sliding window of w keys, -c < 0 chunks of c positions counted from position 0."""
    if window and chunk:
        raise KernelError("a window and a chunked mask exclude each other")
    return -int(chunk) if chunk else int(window or 0)


def attn_prefill_queries(head_dim: int, warps: int = 8) -> int:
    """Queries one CTA of the prefill kernel takes (256-wide heads always use 4 warps)."""
    return 16 * (4 if head_dim > 128 else warps)


def attn_prefill_bf16(out, q, k_cache, v_cache, q_start, start_pos, num_entries, block_table, table_stride,
                      window, scale, dec_max, tiles, max_context, err, warps: int = 8):
    """Portions of more than ``dec_max`` tokens; ``tiles`` = sum over them of
    ceil(tokens / attn_prefill_queries(head_dim, warps)); ``max_context`` = their longest
    start + tokens."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(out, "out", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    num_pages, nkv, ps, _ = k_cache.shape
    if not attn_tiled_supported(q.dtype, d) or nh % nkv:
        raise KernelError(f"tiled attention needs bfloat16, a head size in steps of 16 up to 256 and heads divisible "
                          f"by key/value heads; got head size {d}, {nh}/{nkv} heads")
    _ok(kernels_lib().xb_attn_prefill_bf16(
        out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), q_start.data_ptr(), start_pos.data_ptr(),
        int(num_entries), block_table.data_ptr(), int(table_stride), nh, nkv, d, ps, num_pages, int(window or 0),
        float(scale), int(dec_max), int(tiles), int(max_context), 4 if d > 128 else int(warps), err.data_ptr(),
        _stream()), "attn_prefill_bf16")


def attn_decode_bf16(out, part_o, part_ml, q, k_cache, v_cache, positions, req_of_token, q_start, num_entries,
                     block_table, table_stride, window, scale, dec_max, direct, split, num_splits, tokens, err, tickets=None):
    """Tokens of portions of at most ``dec_max`` tokens (``tokens`` of them); keys are cut into
    ``num_splits`` ranges of ``split`` positions (a multiple of 64).  ``tickets``: int32 scratch of
    tokens * kv_heads * ceil(group / 16) zeros (left zero), needed with ``num_splits`` > 1.  ``part_o`` /
    ``part_ml``: float32 scratch of at least tokens*heads*num_splits*head_dim and
    tokens*heads*num_splits*2 elements when ``num_splits`` > 1."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(out, "out", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    num_pages, nkv, ps, _ = k_cache.shape
    if not attn_tiled_supported(q.dtype, d) or nh % nkv:
        raise KernelError(f"tiled attention needs bfloat16, a head size in steps of 16 up to 256 and heads divisible "
                          f"by key/value heads; got head size {d}, {nh}/{nkv} heads")
    if tokens > 65535:
        raise KernelError(f"{tokens} small-portion tokens exceed the decode kernel's grid limit of 65535")
    if num_splits > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < tokens * nh * num_splits * d or part_ml.numel() < tokens * nh * num_splits * 2:
            raise KernelError("attention scratch buffers are too small for the number of key ranges")
        _need(tickets, "tickets", torch.int32)
        if tickets.numel() < tokens * nkv * ((nh // nkv + 15) // 16):
            raise KernelError("the attention ticket buffer is too small")
    _ok(kernels_lib().xb_attn_decode_bf16(
        out.data_ptr(), _ptr(part_o), _ptr(part_ml), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        positions.data_ptr(), req_of_token.data_ptr(), q_start.data_ptr(), int(num_entries), block_table.data_ptr(),
        int(table_stride), nh, nkv, d, ps, num_pages, int(window or 0), float(scale), int(dec_max), int(bool(direct)),
        int(split), int(num_splits), int(tokens), _ptr(tickets), err.data_ptr(), _stream()), "attn_decode_bf16")


ERR_NOT_SUPPORTED = 801  # cudaErrorNotSupported


def attn_decode_plan_size(tokens: int, ctas: int, kv_heads: int) -> int:
    return int(kernels_lib().xb_attn_decode_plan_size(int(tokens), int(ctas), int(kv_heads)))


def attn_decode_plan(plan, positions, req_of_token, q_start, num_entries, window, dec_max, direct, tokens, min_keys,
                     ctas, kv_heads, err) -> bool:
    """Decide how the attention of the step's ``tokens`` small tokens is shared out (pieces of about
    1 / ``ctas`` of all keys, at least ``min_keys`` each) and write it to ``plan`` (int32,
    ``attn_decode_plan_size`` elements).  It must run before the step's first kernel when
    ``attn_decode_tc`` is to overlap with its predecessor.  False: more tokens than a plan takes."""
    _need(plan, "plan", torch.int32)
    if plan.numel() < attn_decode_plan_size(tokens, ctas, kv_heads):
        raise KernelError("the attention plan buffer is too small")
    rc = kernels_lib().xb_attn_decode_plan(plan.data_ptr(), positions.data_ptr(), req_of_token.data_ptr(), q_start.data_ptr(),
                                           int(num_entries), int(window or 0), int(dec_max), int(bool(direct)), int(tokens),
                                           int(min_keys), int(ctas), int(kv_heads), err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "attn_decode_plan")
    return True


def attn_decode_tc(out, part_o, part_ml, q, k_cache, v_cache, plan, block_table, table_stride, scale, dec_max,
                   splits_max, tokens, ctas, err, tickets=None, overlap: bool = True, softcap=None,
                   slope_exponent=None) -> bool:
    """The step's small tokens on tcgen05 tensor cores with TMA-fed pages, shared out as ``plan``
    says (``attn_decode_plan`` with the same tokens, ctas and kv heads).  A token and head in several
    pieces is merged through ``part_o`` / ``part_ml`` (float32, tokens*heads*splits_max*head_dim
    and tokens*heads*splits_max*2 elements) and ``tickets`` (int32, tokens * kv_heads zeros, left
    zero); ``decode_tc_splits_max`` gives the ``splits_max`` that is always enough.  ``overlap``:
    start while the kernel before drains - only with a plan made before the step's first kernel.
    Returns False, having done nothing, for shapes the kernel does not take (a head size over
    128, a page size that is no power of two >= 8, more than 16 query heads per key/value head).
    ``softcap`` / ``slope_exponent``: scores capped and biased by the distance as in ``attention_plain``."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(out, "out", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _need(plan, "plan", torch.int32)
    num_pages, nkv, ps, _ = k_cache.shape
    if nh % nkv or d % 16:
        raise KernelError(f"tiled attention needs a head size in steps of 16 and heads divisible by key/value heads; "
                          f"got head size {d}, {nh}/{nkv} heads")
    if plan.numel() < attn_decode_plan_size(tokens, ctas, nkv):
        raise KernelError("the attention plan buffer is too small")
    if splits_max > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < tokens * nh * splits_max * d or part_ml.numel() < tokens * nh * splits_max * 2:
            raise KernelError("attention scratch buffers are too small for the number of pieces per token")
        _need(tickets, "tickets", torch.int32)
        if tickets.numel() < tokens * nkv:
            raise KernelError("the attention ticket buffer is too small")
    rc = kernels_lib().xb_attn_decode_tc(
        out.data_ptr(), _ptr(part_o), _ptr(part_ml), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), plan.data_ptr(),
        block_table.data_ptr(), int(table_stride), T, nh, nkv, d, ps, num_pages, float(scale), float(softcap or 0.0),
        float(slope_exponent or 0.0), int(dec_max),
        int(splits_max), int(tokens), int(ctas), _ptr(tickets), int(bool(overlap)), err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "attn_decode_tc")
    return True


def decode_tc_splits_max(ctas: int, kv_heads: int, bound: int, min_keys: int) -> int:
    """Most pieces one token of ``attn_decode_tc`` can be cut into when no context is longer than
    ``bound``: a (token, head) pair holds at most 1 / kv_heads of all tiles (so it gets at most
    ctas / kv_heads shares), and a piece at least ``min_keys``."""
    tiles = (max(int(bound), 1) + 63) // 64
    per = max(int(min_keys) // 64, 1)
    return max(1, min(int(ctas) // int(kv_heads) + 1, tiles // per + 1))


# ---- matrix product for few tokens on tcgen05 tensor cores ---------------------------------------------


def gemm_skinny_tc(out, x, w, err, splits: int = 0) -> bool:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 256 with TMA-fed tcgen05 MMAs (bfloat16 in, float32
    accumulation; ``out`` bfloat16 or float32).  Returns False, having done nothing, for shapes the
    kernel does not take (K not a multiple of 8, K < 64, M > 256)."""
    M, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16, (M, K))
    _need(w, "w", torch.bfloat16, (N, K))
    _need(out, "out", None, (M, N))
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"out must be bfloat16 or float32, not {out.dtype}")
    rc = kernels_lib().xb_gemm_skinny_tc(out.data_ptr(), int(out.dtype == torch.float32), x.data_ptr(), w.data_ptr(),
                                         M, N, K, int(splits), err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "gemm_skinny_tc")
    return True


def gemm_skinny_swiglu(out, x, w_gate_up, err, splits: int = 0) -> bool:
    """out[M, I] = silu(x . Wg^T) * (x . Wu^T) for w_gate_up = [Wg; Wu] of [2 I, K]: the packed gate/up
    product of few tokens and the SiLU gate in one kernel, with the values that ``gemm_skinny_tc``
    followed by ``swiglu`` gives.  Returns False, having done nothing, for shapes it does not take."""
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x, "x", torch.bfloat16, (M, K))
    _need(w_gate_up, "w_gate_up", torch.bfloat16, (2 * I, K))
    _need(out, "out", torch.bfloat16, (M, I))
    rc = kernels_lib().xb_gemm_skinny_swiglu(out.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(), M, I, K, int(splits),
                                             err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "gemm_skinny_swiglu")
    return True


def gemm_skinny_qkv(q_out, k_cache, v_cache, x, w_qkv, q_w, k_w, cos_t, sin_t, positions, req_of_token, block_table,
                    table_stride, nh, nkv, d, rot, interleaved, eps, write_kv, err, splits: int = 0) -> bool:
    """The packed q/k/v product of few tokens finished per head in the same kernel: what
    ``gemm_skinny_tc`` followed by ``qk_norm_rope_write`` gives (q to ``q_out``, k and v into their
    pages).  Heads must be 128 wide; returns False, having done nothing, for what it does not take."""
    M, K = x.shape
    _need(x, "x", torch.bfloat16, (M, K))
    _need(w_qkv, "w_qkv", torch.bfloat16, ((nh + 2 * nkv) * d, K))
    _need(q_out, "q_out", torch.bfloat16, (M, nh, d))
    if write_kv:
        _need(k_cache, "k_cache", torch.bfloat16, (None, nkv, None, d))
        _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    page_size = k_cache.shape[2] if k_cache is not None else 1
    for name, w_ in (("q_norm", q_w), ("k_norm", k_w)):
        if w_ is not None:
            _need(w_, name, torch.float32, (d,))
    max_pos = 0
    if cos_t is not None:
        _need(cos_t, "cos", torch.float32, (None, rot // 2))
        _need(sin_t, "sin", torch.float32, tuple(cos_t.shape))
        max_pos = cos_t.shape[0]
    rc = kernels_lib().xb_gemm_skinny_qkv(
        q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache), x.data_ptr(), w_qkv.data_ptr(), M, K, int(splits), _ptr(q_w), _ptr(k_w),
        _ptr(cos_t), _ptr(sin_t), positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(), int(table_stride),
        nh, nkv, d, rot, int(bool(interleaved)), page_size, num_pages, max_pos, float(eps), int(bool(write_kv)),
        err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "gemm_skinny_qkv")
    return True


PREFILL_TC_MAX_CTAS = 148   # one CTA of the tcgen05 prefill kernel per SM


def attn_prefill_work(counts, starts, dec_max: int, window, heads: int, kv_heads: int, max_ctas: int = PREFILL_TC_MAX_CTAS,
                      host_buffer=None):
    """The work list of ``attn_prefill_tc`` for a step whose entries bring ``counts`` tokens after
    ``starts`` cached ones (host arrays): the portions of more than ``dec_max`` tokens cut into items of
    128 queries of a pair of query heads (of single heads where pairs would be too few) and shared out among at most ``max_ctas`` CTAs, longest first
    onto the least loaded.  ``host_buffer(n)``: gives a pinned int32 tensor of at least n elements to write
    into (default: a fresh one).  Returns (pinned int32 host tensor, number of CTAs); no CTAs: nothing to do."""
    from .native import host_lib
    counts = np.ascontiguousarray(counts, dtype=np.int32)
    starts = np.ascontiguousarray(starts, dtype=np.int32)
    tiles = int(((counts[counts > dec_max] + 127) // 128).sum())
    cap = max_ctas + 1 + 4 * tiles * heads + 4
    host = host_buffer(cap) if host_buffer is not None else torch.empty(cap, dtype=torch.int32).pin_memory()
    ctas = ctypes.c_int(0)
    used = host_lib().xb_attn_prefill_work(len(counts), counts.ctypes.data, starts.ctypes.data, int(dec_max), int(window or 0),
                                           int(heads), int(kv_heads), int(max_ctas), host.data_ptr(), cap, ctypes.byref(ctas))
    if used < 0:
        raise KernelError("the prefill work list does not fit its buffer")
    return host[:max(int(used), 1)], int(ctas.value)


def attn_prefill_tc(out, q, k_cache, v_cache, q_start, start_pos, block_table, table_stride, window, scale, work, ctas, err,
                    softcap=None, slope_exponent=None) -> bool:
    """Prefill attention on tcgen05 (TMA-fed; scores, probabilities and accumulators in tensor memory):
    128 queries of two query heads of a key/value head per work item; ``work`` (int32, on the device)
    and ``ctas`` come from ``attn_prefill_work`` for the same step, heads and window.  Returns False,
    having done nothing, for sizes it does not take (head size over 128, page size not a power of two
    from 8).  ``window`` is a mask code here and in the work list and the decode plan: w > 0 a sliding window, -c < 0
    chunks of c positions counted from the sequence's start (``mask_code``).  ``softcap`` / ``slope_exponent``: scores
    capped and biased by the distance as in ``attention_plain``."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(out, "out", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _need(work, "work", torch.int32)
    num_pages, nkv, ps, _ = k_cache.shape
    if ctas <= 0:
        return True
    if work.numel() < ctas + 1:
        raise KernelError("the prefill work list is shorter than its table of CTAs")
    rc = kernels_lib().xb_attn_prefill_tc(
        out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), q_start.data_ptr(), start_pos.data_ptr(),
        block_table.data_ptr(), int(table_stride), T, nh, nkv, d, ps, num_pages, int(window or 0), float(scale),
        float(softcap or 0.0), float(slope_exponent or 0.0), work.data_ptr(), int(ctas), err.data_ptr(), _stream())
    if rc == ERR_NOT_SUPPORTED:
        return False
    _ok(rc, "attn_prefill_tc")
    return True


# ---- attention with talking heads and a sink; gated recurrence; polynomial activation; table experts ----
def qkv_prepare(q_out, k_cache, v_cache, qkv, q_w, k_w, inv_freq, positions, req_of_token, block_table, table_stride,
                nh, nkv, d, dv, rot, interleaved, norm_mode, eps, write_kv, err, rot_magnitude: float = 1.0, bias=None,
                q_temp=None, row_len=None, value_offset=None):
    """Per q/k head of the packed ``qkv`` rows ``[heads*d | kv_heads*d | kv_heads*dv]``: norm over the head
    (``norm_mode`` 1: before the rotation, 2: after it, 0: none; weight ``q_w`` / ``k_w`` or none), rotation of
    the first ``rot`` channels by ``position * inv_freq`` (float32 angles formed in the kernel; ``inv_freq`` None:
    no rotation; cos and sin are multiplied by ``rot_magnitude``); q to ``q_out``, k and v into their pages.
    ``bias`` (float32, as long as a ``qkv`` row) is added first of all.  ``q_temp`` = (coef, every): a query at
    position p is multiplied, last of all, by ``1 + coef * ln(floor((p + 1) / every) + 1)``.  ``norm_mode`` 3: like 1
    with ONE root mean square over all q channels of a token (and one over all its k channels) and weights of
    ``heads * d`` (``kv_heads * d``) channels.  ``value_offset``: where in a row the values start (default: behind q
    and k); the offset of k makes the keys as projected double as values, and rows then hold no values of their own."""
    T = qkv.shape[0]
    v_off = (nh + nkv) * d if value_offset is None else int(value_offset)
    need_len = max((nh + nkv) * d, v_off + nkv * dv)
    row_len = need_len if row_len is None else int(row_len)     # rows may hold more behind their q, k and v
    if row_len < need_len:
        raise KernelError(f"rows of {row_len} elements cannot hold q, k and v of {need_len}")
    if bias is not None:
        _need(bias, "bias", torch.float32, (need_len,))
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else (0.0, 0)
    if q_temp is not None and every <= 0:
        raise KernelError(f"the query temperature's period must be positive, got {every}")
    _need(qkv, "qkv", None, (T, row_len))
    _need(q_out, "q_out", qkv.dtype, (T, nh, d))
    if write_kv:
        _need(k_cache, "k_cache", qkv.dtype, (None, nkv, None, d))
        _need(v_cache, "v_cache", qkv.dtype, (k_cache.shape[0], nkv, k_cache.shape[2], dv))
    num_pages = k_cache.shape[0] if k_cache is not None else 0
    page_size = k_cache.shape[2] if k_cache is not None else 1
    for name, w_, n_ in (("q_norm", q_w, nh), ("k_norm", k_w, nkv)):
        if w_ is not None:
            _need(w_, name, torch.float32, (n_ * d if norm_mode == 3 else d,))
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    _ok(kernels_lib().xb_qkv_prepare(
        dtype_code(qkv.dtype), q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache), qkv.data_ptr(), _ptr(q_w), _ptr(k_w),
        _ptr(inv_freq), positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(), int(table_stride), T, nh, nkv,
        d, dv, int(rot if inv_freq is not None else 0), int(bool(interleaved)), int(norm_mode), page_size, num_pages,
        float(eps), int(bool(write_kv)), float(rot_magnitude), _ptr(bias), coef, every, row_len, v_off, err.data_ptr(),
        _stream()), "qkv_prepare")


def attn_talking_tile(nh: int, d: int, dv: int, want: int) -> int:
    """The query tile ``attn_talking`` can take for these sizes (a power of two, at most ``want``
    unless that is below one); 0: the sizes do not fit the kernel."""
    return int(kernels_lib().xb_attn_talking_tile(int(nh), int(d), int(dv), int(max(want, 1))))


def attn_talking(out, q, k_cache, v_cache, talk, q_start, start_pos, num_entries, block_table, table_stride, window, scale,
                 sink, out_scale, bq, err, parts: int = 1, part_o=None, part_ml=None):
    """Attention over the paged cache with scores mixed across heads by ``talk`` ([heads, heads] float32 or
    None) before the softmax and, with ``sink``, one silent entry of score 0 in every softmax.  ``out`` is a
    view ``[T, heads * dv]`` whose rows may be ``out.stride(0)`` apart; it receives ``out_scale`` times the
    result.  ``bq``: queries per block (``attn_talking_tile``).  ``parts`` > 1 (only with ``bq`` 1): every
    token's keys are cut into that many ranges, merged through ``part_o`` / ``part_ml`` (float32,
    T*parts*heads*dv and T*parts*heads*2 elements)."""
    T, nh, d = q.shape
    _need(q, "q", None, (T, nh, d))
    _need(k_cache, "k_cache", q.dtype, (None, None, None, d))
    num_pages, nkv, ps, _ = k_cache.shape
    dv = v_cache.shape[-1]
    _need(v_cache, "v_cache", q.dtype, (num_pages, nkv, ps, dv))
    if out.dtype != q.dtype or out.shape != (T, nh * dv) or out.stride(1) != 1 or not out.is_cuda:
        raise KernelError(f"out must be a {q.dtype} view [T, heads * dv] with unit column stride")
    if talk is not None:
        _need(talk, "talk", torch.float32, (nh, nh))
    if parts > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < T * parts * nh * dv or part_ml.numel() < T * parts * nh * 2:
            raise KernelError("attention scratch buffers are too small for the number of key ranges")
    _ok(kernels_lib().xb_attn_talking(
        dtype_code(q.dtype), out.data_ptr(), int(out.stride(0)), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        _ptr(talk), q_start.data_ptr(), start_pos.data_ptr(), int(num_entries), block_table.data_ptr(), int(table_stride),
        T, nh, nkv, d, dv, ps, num_pages, int(window or 0), float(scale), int(bool(sink)), float(out_scale), int(bq),
        int(parts), _ptr(part_o), _ptr(part_ml), err.data_ptr(), _stream()), "attn_talking", 2 if parts > 1 else 1)


def attn_talking_mma_tile(nh: int, nkv: int, d: int, dv: int, want: int) -> int:
    """The query tile the tensor-core form takes for these sizes (at most ``want``); 0: not its sizes."""
    return int(kernels_lib().xb_attn_talking_mma_tile(int(nh), int(nkv), int(d), int(dv), int(max(want, 1))))


def attn_talking_mma(out, q, k_cache, v_cache, talk, q_start, start_pos, num_entries, block_table, table_stride, window, scale,
                     sink, out_scale, bq, err, parts: int = 1, part_o=None, part_ml=None):
    """``attn_talking`` for bfloat16 with both products on tensor cores (mma.sync); the mix across heads, the
    mask and the softmax stay float32 on the FMA units.  ``bq`` from ``attn_talking_mma_tile``; rows of ``out``
    must start on 4-byte boundaries."""
    T, nh, d = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, d))
    _need(k_cache, "k_cache", torch.bfloat16, (None, None, None, d))
    num_pages, nkv, ps, _ = k_cache.shape
    dv = v_cache.shape[-1]
    _need(v_cache, "v_cache", torch.bfloat16, (num_pages, nkv, ps, dv))
    if (out.dtype != torch.bfloat16 or out.shape != (T, nh * dv) or out.stride(1) != 1 or not out.is_cuda
            or out.stride(0) % 2 or out.data_ptr() % 4):
        raise KernelError("out must be a bfloat16 view [T, heads * dv] with unit column stride and rows on 4-byte boundaries")
    if talk is not None:
        _need(talk, "talk", torch.float32, (nh, nh))
    if parts > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < T * parts * nh * dv or part_ml.numel() < T * parts * nh * 2:
            raise KernelError("attention scratch buffers are too small for the number of key ranges")
    _ok(kernels_lib().xb_attn_talking_mma(
        out.data_ptr(), int(out.stride(0)), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _ptr(talk),
        q_start.data_ptr(), start_pos.data_ptr(), int(num_entries), block_table.data_ptr(), int(table_stride), T, nh, nkv, d,
        dv, ps, num_pages, int(window or 0), float(scale), int(bool(sink)), float(out_scale), int(bq), int(parts),
        _ptr(part_o), _ptr(part_ml), err.data_ptr(), _stream()), "attn_talking_mma", 2 if parts > 1 else 1)


def gated_scan(y, zxg, bz, bx, state, q_start, slots, req_of_token, num_entries, out_scale, scratch=None):
    """The minGRU recurrence over a step's tokens: ``zxg`` float32 ``[T, 3 * width]`` (the z, x and g
    projections without biases), ``state`` float32 ``[slots, width]`` carried per request, ``y`` a view
    ``[T, width]`` (rows ``y.stride(0)`` apart) that receives ``out_scale * S * silu(g)``.  With
    ``scratch`` (float32, 3 * T * width) the chunked form runs."""
    T, W3 = zxg.shape
    W = W3 // 3
    _need(zxg, "zxg", torch.float32, (T, 3 * W))
    _need(bz, "bz", torch.float32, (W,))
    _need(bx, "bx", torch.float32, (W,))
    _need(state, "state", torch.float32, (None, W))
    if y.shape != (T, W) or y.stride(1) != 1 or not y.is_cuda:
        raise KernelError("y must be a view [T, width] with unit column stride")
    if scratch is not None:
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < 3 * T * W:
            raise KernelError("the scan's scratch is smaller than 3 * tokens * width")
    _ok(kernels_lib().xb_gated_scan(dtype_code(y.dtype), y.data_ptr(), int(y.stride(0)), zxg.data_ptr(), bz.data_ptr(),
                                    bx.data_ptr(), state.data_ptr(), q_start.data_ptr(), slots.data_ptr(),
                                    req_of_token.data_ptr(), int(num_entries), T, W, float(out_scale),
                                    int(scratch is not None), _ptr(scratch), _stream()), "gated_scan",
        3 if scratch is not None else 1)


def polynorm(out, z, coef, eps):
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row, N dividing by the root mean square; float32 ``z``."""
    T, Fdim = z.shape
    _need(z, "z", torch.float32, (T, Fdim))
    _need(out, "out", None, (T, Fdim))
    _need(coef, "coef", torch.float32, (4,))
    _ok(kernels_lib().xb_polynorm(dtype_code(out.dtype), out.data_ptr(), z.data_ptr(), coef.data_ptr(), T, Fdim, float(eps),
                                  _stream()), "polynorm")


def expert_route(offsets, perm, inv, table, ids, sampled, req_of_token, tokens, top, experts, err):
    """Groups the step's (token, choice) pairs by expert.  The experts of token t are ``table[ids[t]]``, or
    ``table[t]`` where ``ids`` is None (the table then holds a router's choices for the step's tokens)."""
    _need(table, "table", torch.int32, (None, top))
    for name, t_, n in (("offsets", offsets, experts + 1), ("perm", perm, tokens * top), ("inv", inv, tokens * top)):
        _need(t_, name, torch.int32)
        if t_.numel() < n:
            raise KernelError(f"{name} holds {t_.numel()} entries, {n} are needed")
    _ok(kernels_lib().xb_expert_route(offsets.data_ptr(), perm.data_ptr(), inv.data_ptr(), table.data_ptr(), _ptr(ids),
                                      _ptr(sampled), sampled.numel() if sampled is not None else 0, req_of_token.data_ptr(),
                                      int(tokens), int(top), int(experts), table.shape[0], err.data_ptr(), _stream()),
        "expert_route")


# bfloat16 grouped products on tensor cores where the sizes allow; tests switch it off to compare the two forms
expert_tensor_cores = True


def expert_gemm(y, a, w, offsets, perm, gather: bool, top: int, gated: bool, *, side_by_side: bool = False,
                activation: str = "silu", params=()):
    """y[r] = a[src(r)] . w[e(r)]^T over rows grouped by expert (``expert_route``).  ``w`` is
    ``[experts, N, K]`` (``[experts, 2 N, K]`` when ``gated``: y = act(gate) * f(up), ``activation``), or with
    ``side_by_side`` ``[N, experts * K]``: the experts' matrices beside each other along K."""
    rows = y.shape[0]
    if side_by_side:
        E = offsets.numel() - 1
        N, K = w.shape[0], w.shape[1] // E
        _need(w, "w", a.dtype, (N, E * K))
        ldw, estride = E * K, K
    else:
        E = w.shape[0]
        N = w.shape[1] // (2 if gated else 1)
        K = w.shape[2]
        _need(w, "w", a.dtype, (E, None, K))
        ldw, estride = K, w.shape[1] * K
    _need(a, "a", None, (None, K))
    _need(y, "y", None, (rows, N))
    act, p0, p1 = activation_args(activation, params)
    if expert_tensor_cores and a.dtype == torch.bfloat16 and K % 8 == 0:
        rc = kernels_lib().xb_expert_gemm_mma(dtype_code(y.dtype), y.data_ptr(), a.data_ptr(), w.data_ptr(), offsets.data_ptr(),
                                              perm.data_ptr(), int(bool(gather)), int(top), E, rows, N, K, int(bool(gated)),
                                              ldw, estride, act, p0, p1, _stream())
        if rc != ERR_NOT_SUPPORTED:
            _ok(rc, "expert_gemm_mma")
            return
    _ok(kernels_lib().xb_expert_gemm(dtype_code(a.dtype), dtype_code(y.dtype), y.data_ptr(), a.data_ptr(), w.data_ptr(),
                                     offsets.data_ptr(), perm.data_ptr(), int(bool(gather)), int(top), E, rows, N, K,
                                     int(bool(gated)), ldw, estride, act, p0, p1, _stream()), "expert_gemm")


def expert_select_gate(act, gu, table, ids, sampled, req_of_token, top: int, experts: int, err, *, weights=None,
                       activation: str = "silu", params=()):
    """From every expert's gate/up values of every token, ``gu [T, experts * 2 F]``, the inputs of the down
    product with the experts side by side: ``act [T, experts * F]`` holds ``silu(gate) * up / top`` for a
    token's own experts and zero for the others.  ``ids`` None: ``table`` has a row per token of the step;
    ``weights`` (float32, like ``table``): a chosen expert's own weight instead of 1 / top; ``activation`` as in
    ``swiglu``."""
    T = gu.shape[0]
    code, p0, p1 = activation_args(activation, params)
    if weights is not None:
        _need(weights, "weights", torch.float32, tuple(table.shape))
    Fdim = gu.shape[1] // (2 * experts)
    _need(gu, "gu", None, (T, experts * 2 * Fdim))
    _need(act, "act", gu.dtype, (T, experts * Fdim))
    _need(table, "table", torch.int32, (None, top))
    _ok(kernels_lib().xb_expert_select_gate(dtype_code(gu.dtype), act.data_ptr(), gu.data_ptr(), table.data_ptr(), _ptr(ids),
                                            _ptr(sampled), sampled.numel() if sampled is not None else 0,
                                            req_of_token.data_ptr(), T, int(top), int(experts), Fdim, table.shape[0],
                                            _ptr(weights), code, p0, p1, err.data_ptr(), _stream()), "expert_select_gate")


def expert_gather(out, x, perm, offsets, top: int):
    """out[r] = x[perm[r] // top] for the grouped rows r: each expert's input rows as one contiguous matrix."""
    rows, K = out.shape
    _need(x, "x", None, (None, K))
    _need(out, "out", x.dtype, (rows, K))
    _ok(kernels_lib().xb_expert_gather(dtype_code(x.dtype), out.data_ptr(), x.data_ptr(), perm.data_ptr(), offsets.data_ptr(),
                                       rows, int(top), offsets.numel() - 1, K, _stream()), "expert_gather")


def expert_combine(out, y, inv, top: int, *, weights=None, base=None):
    """out[t] = base[t] + sum_k w(t, k) y[inv[t, k]]: a token's experts summed in the order of k, each times its own
    weight (``weights`` float32 ``[T, top]``) or all times 1 / top; ``base`` (like ``out``, may be ``out``) is added."""
    T, N = out.shape
    _need(y, "y", torch.float32, (None, N))
    _need(out, "out", None, (T, N))
    if weights is not None:
        _need(weights, "weights", torch.float32, (T, top))
    if base is not None:
        _need(base, "base", out.dtype, (T, N))
    _ok(kernels_lib().xb_expert_combine(dtype_code(out.dtype), out.data_ptr(), y.data_ptr(), inv.data_ptr(), T, int(top), N,
                                        _ptr(weights), _ptr(base), _stream()), "expert_combine")


def expert_router(choice, weight, h, w_router, correction, req_of_token, top: int, groups: int = 1, keep: int = 1,
                  group_best: int = 2, renormalize: bool = False):
    """A sigmoid router: scores ``s = sigmoid(W_r h)`` in float32, choice scores ``s + correction``; only experts of
    the ``keep`` best of ``groups`` equal groups of neighbours can be chosen (a group's score: the sum of its
    ``group_best`` largest choice scores); ``choice [T, top]`` (int32) receives the experts with the largest choice
    scores and ``weight [T, top]`` their plain scores (divided by their sum with ``renormalize``)."""
    T, K = h.shape
    E = w_router.shape[0]
    _need(h, "h", None, (T, K))
    _need(w_router, "w_router", torch.float32, (E, K))
    _need(choice, "choice", torch.int32, (T, top))
    _need(weight, "weight", torch.float32, (T, top))
    if correction is not None:
        _need(correction, "correction", torch.float32, (E,))
    _ok(kernels_lib().xb_expert_router(dtype_code(h.dtype), choice.data_ptr(), weight.data_ptr(), h.data_ptr(),
                                       w_router.data_ptr(), _ptr(correction), req_of_token.data_ptr(), T, E, K, int(top),
                                       int(groups), int(keep), int(group_best), int(bool(renormalize)), _stream()),
        "expert_router")


# ---- attention over a cached latent ---------------------------------------------------------------------------------
def latent_prepare(q_abs, cache, proj, q_off, kv_off, q_lat, norm_w, inv_freq, positions, req_of_token, block_table,
                   table_stride, nh, d, rd, rank, rot, eps, rot_magnitude, err):
    """Per token of the packed projection ``proj``: the query of every head as ``q_abs[t, h] = [q_lat[h, t] | rotated
    rd channels]`` (``q_lat`` ``[heads, T, rank]``: the plain query part carried into the latent space; None: the
    product that formed it has written it into ``q_abs`` already), and, with
    ``kv_off`` >= 0, the cached row ``[RMS-normed rank channels * norm_w | rotated rd channels]`` into its page
    (``cache`` ``[page, slot, rank + rd]``).  Rotation: pairs (2i, 2i + 1) of the first ``rot`` channels by
    ``position * inv_freq[i]``, cos and sin times ``rot_magnitude``."""
    T = proj.shape[0]
    _need(proj, "proj", None, (T, None))
    _need(q_abs, "q_abs", proj.dtype, (T, nh, rank + rd))
    if q_lat is not None:
        _need(q_lat, "q_lat", proj.dtype, (nh, T, rank))
    _need(cache, "cache", proj.dtype, (None, None, rank + rd))
    _need(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    if kv_off >= 0:
        _need(norm_w, "norm_w", torch.float32, (rank,))
        if kv_off + rank + rd > proj.shape[1]:
            raise KernelError("the latent part lies outside the projection's rows")
    if q_off + nh * (d + rd) > proj.shape[1]:
        raise KernelError("the queries lie outside the projection's rows")
    _ok(kernels_lib().xb_latent_prepare(
        dtype_code(proj.dtype), q_abs.data_ptr(), cache.data_ptr(), proj.data_ptr(), proj.shape[1], int(q_off), int(kv_off),
        _ptr(q_lat), rank, T * rank, _ptr(norm_w), inv_freq.data_ptr(), positions.data_ptr(), req_of_token.data_ptr(),
        block_table.data_ptr(), int(table_stride), T, nh, d, rd, rank, int(rot), cache.shape[1], cache.shape[0], float(eps),
        float(rot_magnitude), err.data_ptr(), _stream()), "latent_prepare")


def attn_latent_mma_takes(dk: int, rank: int) -> bool:
    """Whether the tensor-core attention over latent rows takes these sizes (bfloat16 only)."""
    return bool(kernels_lib().xb_attn_latent_mma_takes(int(dk), int(rank)))


def attn_latent_mma(out, q, cache, q_start, start_pos, num_entries, block_table, table_stride, window, scale, sink, err, *,
                    row_groups: int = 2, parts: int = 1, part_o=None, part_ml=None):
    """Attention of every (token, head) row of ``q`` ``[T, heads, dk]`` over its request's cached rows
    (``cache`` ``[page, slot, dk]``; the first ``rank = out.shape[-1]`` channels of a row are its value), bfloat16 on
    tensor cores with float32 scores, softmax and sums.  ``sink`` (float32 per head or None): one more softmax entry
    of that score without a value.  ``row_groups``: 16-row groups per block (1 or 2).  ``parts`` > 1: every row's key
    tiles are dealt out to that many blocks and merged through ``part_o`` / ``part_ml`` (float32, T*heads*parts*rank
    and T*heads*parts*2 elements)."""
    T, nh, dk = q.shape
    _need(q, "q", torch.bfloat16, (T, nh, dk))
    rank = out.shape[-1]
    _need(out, "out", torch.bfloat16, (T, nh, rank))
    _need(cache, "cache", torch.bfloat16, (None, None, dk))
    if sink is not None:
        _need(sink, "sink", torch.float32, (nh,))
    if parts > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < T * nh * parts * rank or part_ml.numel() < T * nh * parts * 2:
            raise KernelError("attention scratch buffers are too small for the number of key ranges")
    _ok(kernels_lib().xb_attn_latent_mma(
        out.data_ptr(), q.data_ptr(), cache.data_ptr(), q_start.data_ptr(), start_pos.data_ptr(), int(num_entries),
        block_table.data_ptr(), int(table_stride), T, nh, dk, rank, cache.shape[1], cache.shape[0], int(window or 0),
        float(scale), _ptr(sink), int(row_groups), int(parts), _ptr(part_o), _ptr(part_ml), err.data_ptr(), _stream()),
        "attn_latent_mma", 2 if parts > 1 else 1)


def gate_sigmoid(out, heads, gate):
    """out[t, h, :] = heads[h, t, :] * sigmoid(gate[t, h, :]).  ``heads`` ``[heads, T, dv]`` may be any view with a
    unit last stride - also ``out`` itself seen head by head (in place); ``gate`` may be a column range of a wider
    tensor.  A gate of ``[T, heads]`` is one number per head."""
    nh, T, dv = heads.shape
    if not heads.is_cuda or heads.stride(2) != 1:
        raise KernelError("heads must be a CUDA view [heads, T, dv] with a unit last stride")
    _need(out, "out", heads.dtype, (T, nh * dv))
    per_head = dv != 1 and tuple(gate.shape) == (T, nh)
    if (gate.dtype != heads.dtype or tuple(gate.shape) not in ((T, nh * dv), (T, nh)) or gate.stride(1) != 1 or not gate.is_cuda):
        raise KernelError("gate must be a [T, heads * dv] or [T, heads] view with unit column stride in the heads' type")
    _ok(kernels_lib().xb_gate_sigmoid(dtype_code(heads.dtype), out.data_ptr(), heads.data_ptr(), heads.stride(1), heads.stride(0),
                                      gate.data_ptr(), gate.stride(0), T, nh, dv, int(per_head), _stream()), "gate_sigmoid")


def gemm_batched_plain(out, a, w):
    """out[b, m, n] = sum_k a[b, m, k] * w[b, n, k] with float32 FMA accumulation.  ``a`` ``[B, M, K]`` and ``out``
    ``[B, M, N]`` may be any views whose last stride is 1; ``w`` ``[B, N, K]`` any view with one unit stride among its
    last two."""
    B, M, K = a.shape
    N = w.shape[1]
    if tuple(w.shape) != (B, N, K) or tuple(out.shape) != (B, M, N):
        raise KernelError(f"batched product: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    if not (a.is_cuda and w.is_cuda and out.is_cuda) or a.dtype != w.dtype or a.dtype != out.dtype:
        raise KernelError("batched product: CUDA tensors of one type are needed")
    if a.stride(2) != 1 or out.stride(2) != 1 or 1 not in (w.stride(1), w.stride(2)):
        raise KernelError("batched product: a and out need a unit last stride, w a unit stride in one of its last two")
    _ok(kernels_lib().xb_gemm_batched_plain(dtype_code(a.dtype), out.data_ptr(), a.data_ptr(), w.data_ptr(), B, M, N, K,
                                            a.stride(0), a.stride(1), w.stride(0), w.stride(1), w.stride(2), out.stride(0),
                                            out.stride(1), _stream()), "gemm_batched_plain")


# ---- RMS norm with the residual arithmetic around it; biases --------------------------------------------------------
def rms_chain(out, x, weight, eps, err, *, branch=None, branch_weight=None, branch_eps=0.0, branch_offset=0.0, gain=None,
              branch_scale: float = 1.0, sum_out=None, rows=None, weight_offset: float = 0.0):
    """One pass over rows of the float32 stream ``x``: s = x + branch_scale * gain * br, where br is the branch, or with
    ``branch_weight`` its own RMS norm ``branch / rms(branch) * (branch_offset + branch_weight)``; ``sum_out`` receives s
    (it may be x itself when no rows are gathered); ``out`` (either type; None: only the sum) receives
    ``s / rms(s) * (weight_offset + weight)``, or s itself where ``weight`` is None."""
    dim = x.shape[-1]
    n = out.shape[0] if out is not None else x.shape[0]
    _need(x, "x", torch.float32, (None, dim))
    if out is not None:
        _need(out, "out", None, (n, dim))
    for name, t in (("weight", weight), ("branch_weight", branch_weight), ("gain", gain)):
        if t is not None:
            _need(t, name, torch.float32, (dim,))
    if branch is not None:
        _need(branch, "branch", None, tuple(x.shape))
    elif branch_weight is not None or gain is not None:
        raise KernelError("a branch norm or a gain needs a branch")
    if sum_out is not None:
        _need(sum_out, "sum_out", torch.float32, (n, dim))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n:
            raise KernelError(f"rows holds {rows.numel()} entries for {n} output rows")
    elif n != x.shape[0]:
        raise KernelError(f"out has {n} rows, x has {x.shape[0]} and no row list was given")
    _ok(kernels_lib().xb_rms_chain(dtype_code(branch.dtype) if branch is not None else F32,
                                   dtype_code(out.dtype) if out is not None else F32, _ptr(out), _ptr(sum_out), x.data_ptr(),
                                   _ptr(branch), _ptr(rows), _ptr(weight), _ptr(branch_weight), _ptr(gain), n, dim, x.shape[0],
                                   float(eps), float(weight_offset), float(branch_eps), float(branch_offset),
                                   float(branch_scale), err.data_ptr(), _stream()), "rms_chain")


def dual_rms_sum(out, left, right, w_left, w_right, eps, left_scale: float, right_scale: float, weight_offset: float = 0.0):
    """out = left_scale * rms_norm(left; w_left) + right_scale * rms_norm(right; w_right), row by row."""
    T, dim = left.shape
    _need(left, "left", None, (T, dim))
    _need(right, "right", left.dtype, (T, dim))
    _need(out, "out", left.dtype, (T, dim))
    _need(w_left, "w_left", torch.float32, (dim,))
    _need(w_right, "w_right", torch.float32, (dim,))
    _ok(kernels_lib().xb_dual_rms_sum(dtype_code(left.dtype), out.data_ptr(), left.data_ptr(), right.data_ptr(),
                                      w_left.data_ptr(), w_right.data_ptr(), T, dim, float(eps), float(weight_offset),
                                      float(left_scale), float(right_scale), _stream()), "dual_rms_sum")


def add_bias(x, bias):
    """x[t, :] += bias, in place."""
    T, dim = x.shape
    _need(x, "x", None, (T, dim))
    _need(bias, "bias", torch.float32, (dim,))
    _ok(kernels_lib().xb_add_bias(dtype_code(x.dtype), x.data_ptr(), bias.data_ptr(), T, dim, _stream()), "add_bias")


def swiglu_bias(out, gate_up, bias, activation: str = "silu"):
    """out[t, i] = act(gate_up[t, i] + bias[i]) * (gate_up[t, I + i] + bias[I + i])."""
    T, two_i = gate_up.shape
    _need(gate_up, "gate_up", None, (T, two_i))
    _need(out, "out", None, (T, two_i // 2))
    _need(bias, "bias", torch.float32, (two_i,))
    if activation not in ("silu", "gelu_tanh"):
        raise KernelError(f"the gate with biases takes silu or gelu_tanh, not '{activation}'")
    _ok(kernels_lib().xb_swiglu_bias(dtype_code(gate_up.dtype), dtype_code(out.dtype), out.data_ptr(), gate_up.data_ptr(),
                                     bias.data_ptr(), T, two_i // 2, ACTIVATIONS[activation], _stream()), "swiglu_bias")


# ---- what is added to a token's embedding row; a layer's own table over token ids -----------------------------------
def embed_sum(out, table, ids, err, *, sampled=None, scale=None, pair=None, pair_rule=None, pos_table=None, positions=None,
              req_of_token=None, q_start=None, slots=None, prev_state=None):
    """out[t] = table[id] * scale + pair[row] + pos_table[position] (float32).  ``pair_rule`` = (buckets, mul_prev,
    mul_cur): row = (prev * mul_prev + id * mul_cur) mod buckets, where prev is the token before - the one before in
    this step, or ``prev_state[slot]`` for a request's first token of the step - and row ``buckets`` at position 0.
    Rows of padding tokens are zero."""
    T, H = out.shape
    _need(out, "out", torch.float32, (T, H))
    _need(table, "table", None, (None, H))
    for name, t in (("ids", ids), ("positions", positions), ("req_of_token", req_of_token), ("q_start", q_start), ("slots", slots)):
        _need(t, name, torch.int32)
    buckets = mp = mc = 0
    if pair is not None:
        buckets, mp, mc = (int(v) for v in pair_rule)
        _need(pair, "pair", table.dtype, (buckets + 1, H))
        _need(prev_state, "prev_state", torch.int32)
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype, (None, H))
    _ok(kernels_lib().xb_embed_sum(dtype_code(table.dtype), out.data_ptr(), table.data_ptr(), _ptr(pair), _ptr(pos_table),
                                   ids.data_ptr(), _ptr(sampled), sampled.numel() if sampled is not None else 0,
                                   positions.data_ptr(), req_of_token.data_ptr(), q_start.data_ptr(), slots.data_ptr(),
                                   _ptr(prev_state), T, H, table.shape[0], buckets, mp, mc,
                                   pos_table.shape[0] if pos_table is not None else 0, 1.0 if scale is None else float(scale),
                                   err.data_ptr(), _stream()), "embed_sum")


def prev_store(prev_state, ids, sampled, q_start, slots, num_entries):
    """prev_state[slot] = the last token every entry brought in this step."""
    _need(prev_state, "prev_state", torch.int32)
    _ok(kernels_lib().xb_prev_store(prev_state.data_ptr(), ids.data_ptr(), _ptr(sampled),
                                    sampled.numel() if sampled is not None else 0, q_start.data_ptr(), slots.data_ptr(),
                                    int(num_entries), _stream()), "prev_store")


def token_gate(out, u, table, col0, ids, sampled, req_of_token, err):
    """out[t, j] = gelu_tanh(u[t, j]) * table[id, col0 + j]."""
    T, dim = u.shape
    _need(u, "u", None, (T, dim))
    _need(out, "out", u.dtype, (T, dim))
    _need(table, "table", u.dtype, (None, None))
    if col0 < 0 or col0 + dim > table.shape[1]:
        raise KernelError("the layer's columns lie outside the table")
    _ok(kernels_lib().xb_token_gate(dtype_code(u.dtype), out.data_ptr(), u.data_ptr(), table.data_ptr(), table.shape[1], int(col0),
                                    ids.data_ptr(), _ptr(sampled), sampled.numel() if sampled is not None else 0,
                                    req_of_token.data_ptr(), T, dim, table.shape[0], err.data_ptr(), _stream()), "token_gate")


# ---- short convolutions and recurrences with a matrix state ----------------------------------------------------------
CONV_MAX_TAPS = 16


def conv_silu(y, u, u_off, taps, bias, state, req_of_token, q_start, slots, num_entries):
    """y[t, c] = silu(bias[c] + sum_j taps[c, j] * u[t - (K-1) + j, u_off + c]) per request, the K-1 inputs before a step's
    first token taken from ``state`` ``[slots, K-1, C]`` (float32), which then receives the step's last K-1 inputs."""
    T, C = y.shape
    K = taps.shape[1]
    _need(y, "y", None, (T, C))
    _need(u, "u", torch.float32, (T, None))
    _need(taps, "taps", torch.float32, (C, K))
    if bias is not None:
        _need(bias, "bias", torch.float32, (C,))
    if u_off < 0 or u_off + C > u.shape[1]:
        raise KernelError("the convolution's channels lie outside the rows")
    if K > CONV_MAX_TAPS:
        raise KernelError(f"a short convolution has at most {CONV_MAX_TAPS} taps, got {K}")
    if K > 1:
        _need(state, "state", torch.float32, (None, K - 1, C))
    lib = kernels_lib()
    _ok(lib.xb_conv_silu(dtype_code(y.dtype), y.data_ptr(), u.data_ptr(), u.shape[1], int(u_off), taps.data_ptr(), _ptr(bias),
                         _ptr(state) if K > 1 else None, req_of_token.data_ptr(), q_start.data_ptr(), slots.data_ptr(), T, C, K,
                         _stream()), "conv_silu")
    if K > 1:
        _ok(lib.xb_conv_state(state.data_ptr(), u.data_ptr(), u.shape[1], int(u_off), q_start.data_ptr(), slots.data_ptr(),
                              int(num_entries), C, K, _stream()), "conv_state")


def selective_scan(y, xbc, proj, dt_off, dt_bias, a_log, d_skip, state, q_start, slots, num_entries, heads, head_dim, n_state,
                   groups):
    """S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + d_skip x per (request, head); ``xbc`` float32 rows
    ``[x | B | C]``, dt = softplus(proj[:, dt_off + h] + dt_bias); ``state`` ``[slots, heads, n_state, head_dim]``."""
    T = xbc.shape[0]
    inner = heads * head_dim
    _need(xbc, "xbc", torch.float32, (T, inner + 2 * groups * n_state))
    _need(proj, "proj", torch.float32, (T, None))
    _need(y, "y", torch.float32, (T, inner))
    for name, t in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip)):
        _need(t, name, torch.float32, (heads,))
    _need(state, "state", torch.float32, (None, heads, n_state, head_dim))
    _ok(kernels_lib().xb_selective_scan(y.data_ptr(), xbc.data_ptr(), xbc.shape[1], proj.data_ptr(), proj.shape[1], int(dt_off),
                                        dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(),
                                        q_start.data_ptr(), slots.data_ptr(), int(num_entries), heads, head_dim, n_state, groups,
                                        _stream()), "selective_scan")


def delta_rule(o, qkv, proj, beta_off, ag, dt_bias, a_log, state, q_start, slots, num_entries, heads, kv_heads, d, dv,
               unit_eps: float = 1e-6):
    """The gated delta rule per (request, head): ``qkv`` float32 rows ``[q | k | v]`` (q and k per key head), beta =
    sigmoid(proj[:, beta_off + h]), decay per (head, key channel) from the front of ``ag`` rows; ``state``
    ``[slots, heads, d, dv]``; ``o`` ``[T, heads * dv]`` before its norm and gate."""
    T = qkv.shape[0]
    _need(qkv, "qkv", torch.float32, (T, 2 * kv_heads * d + heads * dv))
    _need(proj, "proj", torch.float32, (T, None))
    _need(ag, "ag", torch.float32, (T, None))
    _need(o, "o", torch.float32, (T, heads * dv))
    _need(dt_bias, "dt_bias", torch.float32, (heads * d,))
    _need(a_log, "a_log", torch.float32, (heads,))
    _need(state, "state", torch.float32, (None, heads, d, dv))
    _ok(kernels_lib().xb_delta_rule(o.data_ptr(), qkv.data_ptr(), qkv.shape[1], proj.data_ptr(), proj.shape[1], int(beta_off),
                                    ag.data_ptr(), ag.shape[1], dt_bias.data_ptr(), a_log.data_ptr(), state.data_ptr(),
                                    q_start.data_ptr(), slots.data_ptr(), int(num_entries), heads, kv_heads, d, dv,
                                    float(unit_eps), _stream()), "delta_rule")


def gated_head_norm(out, y, gate, g_off, weight, part, eps, gate_after: bool):
    """Per token and group of ``part`` channels of ``y`` (float32): with ``gate_after`` False,
    v = y * silu(gate), out = v / rms(v) * weight; with True, out = y / rms(y) * weight * sigmoid(gate).  ``gate`` is
    the columns from ``g_off`` of float32 rows; ``weight`` repeats every ``weight.numel()`` channels."""
    T, W = y.shape
    _need(y, "y", torch.float32, (T, W))
    _need(out, "out", None, (T, W))
    _need(gate, "gate", torch.float32, (T, None))
    _need(weight, "weight", torch.float32)
    if g_off < 0 or g_off + W > gate.shape[1] or W % part or W % weight.numel():
        raise KernelError("gate columns, group size or weight length do not fit the rows")
    _ok(kernels_lib().xb_gated_head_norm(dtype_code(out.dtype), out.data_ptr(), y.data_ptr(), gate.data_ptr(), gate.shape[1],
                                         int(g_off), weight.data_ptr(), weight.numel(), T, W, int(part), float(eps),
                                         int(bool(gate_after)), _stream()), "gated_head_norm")
