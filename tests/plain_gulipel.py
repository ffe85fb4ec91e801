"""A plain, slow implementation of the Gulipel decoder, one function per mechanism, in float64 (or
float32) torch on the CPU.  It is the oracle of the tests and shares no code with the engine.

Notation: a sequence is a matrix ``x[n, width]`` of n tokens at positions 0..n-1; linear weights are
``[out, in]`` and act as ``x @ W.T``.  ``cfg`` is the model's config.json as a dict, ``w`` a dict from
tensor name to tensor.  Recurrences walk over the tokens one by one.
"""
import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

# Where an engine that computes its matrix products in bfloat16 stores activations in that type, ``forward``
# with ``round_to=torch.bfloat16`` rounds them too: the difference to the unrounded run is the drift that
# rounding alone causes, which the tests take as their yardstick.
_ROUND = None


def _r(x: torch.Tensor) -> torch.Tensor:
    return x if _ROUND is None else x.to(_ROUND).to(x.dtype)


# ---- small pieces ---------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[n, C], taps[C, K]: y[t, c] = sum_j taps[c, j] x[t - (K-1) + j, c] (+ bias); inputs before the first row count as zero."""
    n, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + padded[j:j + n] * taps[:, j][None, :]
    if bias is not None:
        y = y + bias[None, :]
    return y


# ---- embedding ------------------------------------------------------------------------------------
def bigram_rows(tokens: List[int], emb: dict) -> List[int]:
    """Row of the pair table for every token: a hash of (previous, current), the last row for the first token."""
    b = emb["bigram"]
    rows = []
    for i, t in enumerate(tokens):
        rows.append(b["buckets"] if i == 0 else (tokens[i - 1] * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"])
    return rows


def embed(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    ids = torch.tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] * cfg["embedding"]["scale"]
    if cfg["embedding"].get("bigram"):
        x = x + w["bigram"][torch.tensor(bigram_rows(tokens, cfg["embedding"]), dtype=torch.long)]
    if "pos" in w:
        x = x + w["pos"][: len(tokens)]
    return x


# ---- softmax attention with a gate ----------------------------------------------------------------
def query_temperature(n: int, q_temp: Optional[dict], dtype) -> torch.Tensor:
    """Factor on the query at every position: it grows with the logarithm of the number of whole periods seen."""
    if not q_temp:
        return torch.ones(n, dtype=dtype)
    p = torch.arange(n, dtype=torch.long)
    steps = torch.div(p + 1, q_temp["every"], rounding_mode="floor").to(dtype)
    return 1.0 + q_temp["coef"] * torch.log(steps + 1.0)


def causal_attention(q, k, v, scale: float) -> torch.Tensor:
    """q[n, H, d], k[n, G, d], v[n, G, dv]; head h reads key/value head h // (H / G); position i sees j <= i."""
    n, H, d = q.shape
    G = k.shape[1]
    rep = H // G
    mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
    out = []
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, h // rep])
    return torch.stack(out, dim=1)


def gated_attention(h: torch.Tensor, w, p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _r(h @ w[p + "q"].T + w[p + "q.b"]).view(n, H, d)
    k = _r(h @ w[p + "k"].T + w[p + "k.b"]).view(n, G, d)
    v = _r(h @ w[p + "v"].T + w[p + "v.b"]).view(n, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps) * query_temperature(n, m.get("q_temp"), h.dtype)[:, None, None]
    k = rms_norm(k, w[p + "k.norm"], eps)
    o = causal_attention(_r(q), _r(k), v, m["scale"]).reshape(n, H * dv)
    o = _r(o) * torch.sigmoid(_r(h @ w[p + "g"].T))
    return _r(o) @ w[p + "o"].T


# ---- gated delta rule ------------------------------------------------------------------------------
def delta_rule(q, k, v, beta, decay) -> torch.Tensor:
    """q, k [n, H, d] (already per value head), v [n, H, dv], beta [n, H], decay [n, H, d] in (0, 1).
    S[d, dv] per head: S <- decay * S (rows), u = beta (v - S^T k), S <- S + k u^T, o = S^T q."""
    n, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    out = torch.zeros(n, H, dv, dtype=q.dtype)
    for t in range(n):
        S = S * decay[t][:, :, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def gated_delta_mixer(h: torch.Tensor, w, p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = H // G
    q = _r(silu(_r(causal_conv(_r(h @ w[p + "q"].T), w[p + "q.conv"])))).view(n, G, d)
    k = _r(silu(_r(causal_conv(_r(h @ w[p + "k"].T), w[p + "k.conv"])))).view(n, G, d)
    v = _r(silu(_r(causal_conv(_r(h @ w[p + "v"].T), w[p + "v.conv"])))).view(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(_r(h @ w[p + "b"].T))                                    # [n, H]
    a = _r(_r(h @ w[p + "a1"].T) @ w[p + "a2"].T) + w[p + "dt_bias"]                # [n, H * d]
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * F.softplus(a).view(n, H, d))
    o = delta_rule(q, k, v, beta, decay)
    gate = torch.sigmoid(_r(_r(h @ w[p + "g1"].T) @ w[p + "g2"].T)).view(n, H, dv)
    o = unit_rms(o, eps) * w[p + "norm"] * gate
    return _r(o.reshape(n, H * dv)) @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w, p: str, m: dict, eps: float) -> torch.Tensor:
    left = gated_attention(h, w, p + "left.", m["left"], eps)
    right = gated_delta_mixer(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# ---- selective state space (Mamba-2) ---------------------------------------------------------------
def selective_scan(x, B, C, dt, A, D) -> torch.Tensor:
    """x [n, H, P], B and C [n, H, N] (already per head), dt [n, H] > 0, A [H] > 0, D [H].
    S[N, P] per head: S <- exp(-A dt) S + dt B x^T, y = S^T C + D x."""
    n, H, P = x.shape
    N = B.shape[2]
    S = torch.zeros(H, N, P, dtype=x.dtype)
    out = torch.zeros_like(x)
    for t in range(n):
        S = S * torch.exp(-A * dt[t])[:, None, None] + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        out[t] = torch.einsum("hnp,hn->hp", S, C[t]) + D[:, None] * x[t]
    return out


def mamba2_mixer(h: torch.Tensor, w, p: str, m: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = _r(h @ w[p + "in"].T)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = _r(silu(_r(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))))
    x = xbc[:, :inner].view(n, H, P)
    B = xbc[:, inner:inner + G * N].view(n, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N:].view(n, G, N).repeat_interleave(H // G, dim=1)
    dt = F.softplus(dt + w[p + "dt_bias"])
    y = selective_scan(x, B, C, dt, torch.exp(w[p + "A_log"]), w[p + "D"]).reshape(n, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * w[p + "norm"]
    return _r(y) @ w[p + "o"].T


# ---- feed-forward and the per-layer token input -----------------------------------------------------
def dense_ff(h: torch.Tensor, w, p: str) -> torch.Tensor:
    g = _r(h @ w[p + "gate"].T + w[p + "gate.b"])
    u = _r(h @ w[p + "up"].T + w[p + "up.b"])
    return _r(silu(g) * u) @ w[p + "down"].T + w[p + "down.b"]


def token_side(x: torch.Tensor, w, p: str, table: torch.Tensor, tokens: List[int], eps: float) -> torch.Tensor:
    """What a layer adds from its own small table over token ids: the table's row, gated by the stream."""
    e = table[torch.tensor(tokens, dtype=torch.long)]
    g = _r(gelu_tanh(_r(_r(x) @ w[p + "gate"].T)) * e)
    y = g @ w[p + "proj"].T
    return rms_norm(y, w[p + "norm"], eps)


# ---- the whole model -----------------------------------------------------------------------------------
MIXERS = {"parallel": parallel_mixer, "mamba2": mamba2_mixer, "mamba2_2": mamba2_mixer}


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], *, round_to=None, layers_out: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [n, vocab] of a whole sequence.  ``layers_out`` (a list) receives the residual stream after every layer."""
    global _ROUND
    _ROUND = round_to
    try:
        eps = cfg["norm"]["eps"]
        x = embed(cfg, w, tokens)
        side = cfg.get("token_side")
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            a = MIXERS[layer["type"]](_r(rms_norm(x, w[p + "norm1"], eps)), w, p + "mix.", layer["mixer"], eps)
            x = x + rms_norm(a, w[p + "norm1b"], eps) * w[p + "ls1"]
            if layer.get("mlp") is not None:
                f = dense_ff(_r(rms_norm(x, w[p + "norm2"], eps)), w, p + "mlp.")
                x = x + rms_norm(f, w[p + "norm2b"], eps) * w[p + "ls2"]
            if side:
                dim = side["dim"]
                x = x + token_side(x, w, p + "side.", w["side.embed"][:, i * dim:(i + 1) * dim], tokens, eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        y = _r(rms_norm(x, w["final.norm"], eps))
        logits = y @ w["head"].T
        cap = cfg.get("logit_softcap")
        if cap:
            logits = cap * torch.tanh(logits / cap)
        return logits
    finally:
        _ROUND = None


# ---- a model folder, read without the engine's loader ------------------------------------------------------
_DT = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64, "I32": torch.int32,
       "I64": torch.int64}


def load_folder(path: str, dtype=torch.float64):
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    for name, e in header.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=_DT[e["dtype"]]).view(*e["shape"])
        w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


def generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    """Greedy continuation by n tokens, the whole sequence recomputed for every token."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(forward(cfg, w, seq)[-1].argmax())
        seq.append(tok)
        out.append(tok)
    return out
