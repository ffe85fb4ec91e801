"""A plain, slow implementation of the Mikutar decoder: float64, whole sequences at once, one function per
mechanism, written from the design's equations.  It shares no code with the engine (it even reads model folders
itself) and serves as the oracle of the tests.

    x_0    = E[token]
    layer:   h = N(x);  x <- x + (mixer(h) + ff(h))              one norm, both sublayers read it
    loop:    layers start .. stop-1 run `times` times with the same weights; before every pass but the first, x_0 is
             added to x; the remaining layers follow once
    logits = cap * tanh(E . Nf(x) / cap)

``round_to`` emulates an engine that stores activations in a shorter type: the results of matrix products that an
engine keeps in that type, the cached rows, the queries and the attention outputs are rounded to it and widened
again; everything the design wants in 32-bit stays wide.
"""
import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64
SWISH_ALPHA = 1.702       # fixed by the design
GROUP_BEST = 2            # a group's score sums this many of its largest choice scores
SLOPE_EXPONENT = 8.0      # slope of head h: 2^(-8 (h + 1) / heads)


# ---- model folders --------------------------------------------------------------------------------------------------
def load_folder(folder):
    """(config dict, {name: float64 tensor}) of a folder with config.json and model.safetensors."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        head = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, e in head.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        if e["dtype"] == "BF16":
            t = torch.from_numpy(raw.copy()).view(torch.bfloat16).to(F64)
        elif e["dtype"] == "F32":
            t = torch.from_numpy(raw.copy()).view(torch.float32).to(F64)
        elif e["dtype"] == "I32":
            t = torch.from_numpy(raw.copy()).view(torch.int32).to(torch.int64)
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        w[name] = t.reshape(e["shape"])
    return cfg, w


def _r(t, round_to):
    return t if round_to is None else t.to(round_to).to(F64)


# ---- mechanisms ---------------------------------------------------------------------------------------------------------
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (weight None: no weight)."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotate_neighbours(x, positions, dims, base):
    """x [T, heads, d]: channels (2i, 2i+1), i < dims/2, turn by position * base^(-2i/dims); the rest pass."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    a = positions.to(F64)[:, None] * f[None, :]              # [T, dims/2]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def window_mask(T, size):
    """[T, T] True where query i sees key j: 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def chunk_mask(T, size):
    """[T, T] True where j <= i and both lie in the same chunk of ``size`` positions counted from 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def head_slopes(heads):
    h = torch.arange(heads, dtype=F64)
    return 2.0 ** (-SLOPE_EXPONENT * (h + 1.0) / heads)


def softmax_attention(q, k, v, mask, scale, softcap=None, slopes=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  score = scale q.k, then cap * tanh(score / cap), then
    minus slope_h * (i - j); ordinary softmax over the keys the mask shows."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(F64)
    for h in range(H):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        if slopes is not None:
            s = s - slopes[h] * dist
        s = s.masked_fill(~mask, -math.inf)
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def rotary_window_attention(h, w, p, m, eps, positions, round_to=None):
    """The mixer 'attention': keys double as values (as projected, before norm and rotation), biases on q, k and
    the output, one RMS norm over the whole q (and k) projection, rotation of neighbours, a window, a sigmoid gate
    of one number per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _r(h @ w[p + "q"].T + w[p + "q.b"], round_to)
    k = _r(h @ w[p + "k"].T + w[p + "k.b"], round_to)
    v = k.clone().view(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps).view(T, H, d)
    k = rms_norm(k, w[p + "k.norm"], eps).view(T, G, d)
    rot = m.get("rot") or {}
    q = _r(rotate_neighbours(q, positions, rot.get("dims", 0), rot.get("base", 1.0)), round_to)
    k = _r(rotate_neighbours(k, positions, rot.get("dims", 0), rot.get("base", 1.0)), round_to)
    o = softmax_attention(q, k, v, window_mask(T, m["mask"]["size"]), m["scale"])
    gate = torch.sigmoid(_r(h @ w[p + "g"].T, round_to))           # [T, H]
    o = _r(o * gate[:, :, None], round_to).reshape(T, H * dv)
    return o @ w[p + "o"].T + w[p + "o.b"]


def capped_chunk_attention(h, w, p, m, positions, round_to=None):
    """The mixer 'attention_2': no biases, no rotation; capped scores minus a distance term, within chunks."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _r(h @ w[p + "q"].T, round_to).view(T, H, d)
    k = _r(h @ w[p + "k"].T, round_to).view(T, G, d)
    v = _r(h @ w[p + "v"].T, round_to).view(T, G, dv)
    o = softmax_attention(q, k, v, chunk_mask(T, m["mask"]["size"]), m["scale"], m.get("softcap"), head_slopes(H))
    gate = torch.sigmoid(_r(h @ w[p + "g"].T, round_to))
    o = _r(o * gate[:, :, None], round_to).reshape(T, H * dv)
    return o @ w[p + "o"].T


def relu_feed_forward(h, w, p, round_to=None):
    g = _r(h @ w[p + "gate"].T, round_to)
    u = _r(h @ w[p + "up"].T, round_to)
    return _r(torch.relu(g) * u, round_to) @ w[p + "down"].T


def clamped_expert(h, w, p, limit, round_to=None):
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), W_down (g sigmoid(1.702 g) (u + 1))."""
    g = _r(h @ w[p + "gate"].T, round_to).clamp(max=limit)
    u = _r(h @ w[p + "up"].T, round_to).clamp(-limit, limit)
    y = g * torch.sigmoid(SWISH_ALPHA * g) * (u + 1.0)
    return _r(y, round_to) @ w[p + "down"].T


def route(h, w_router, correction, top, groups, keep):
    """(chosen experts [T, top], their weights [T, top]): scores sigmoid(W_router h); choice scores add the
    correction; a group's score is the sum of its two largest choice scores; experts outside the ``keep`` best of
    ``groups`` equal groups of neighbours count as minus infinity; the ``top`` largest choice scores win; the
    weights are the plain scores, not renormalized."""
    s = torch.sigmoid(h @ w_router.T)                       # [T, E]
    c = s + correction
    T, E = c.shape
    per = E // groups
    gs = c.view(T, groups, per).topk(min(GROUP_BEST, per), dim=-1).values.sum(-1)       # [T, groups]
    best = gs.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    c = c.masked_fill(~allowed[:, :, None].expand(T, groups, per).reshape(T, E), -math.inf)
    idx = c.topk(top, dim=-1).indices
    return idx, s.gather(1, idx)


def follow_close_calls(h, w_router, correction, idx, wt, given, slack, groups=1, keep=1):
    """An engine that rounds activations may decide a close call the other way.  ``given`` [T, top] are the experts
    an engine chose: where a token's set differs from the plain one, every expert it took instead must have a
    choice score within ``slack`` of one it left out (or belong to a group whose score is that close to a kept
    group's) - else the engine's router is wrong and this raises.  Returns the engine's sets with their plain
    scores as weights."""
    s = torch.sigmoid(h @ w_router.T)
    c = s + correction
    out_i, out_w = idx.clone(), wt.clone()
    T, E = c.shape
    per = E // groups
    gs = c.view(T, groups, per).topk(min(GROUP_BEST, per), dim=-1).values.sum(-1).sort(dim=-1, descending=True).values
    for t in range(T):
        mine, theirs = set(idx[t].tolist()), set(int(e) for e in given[t].tolist())
        if mine == theirs:
            continue
        assert len(theirs) == len(mine), f"token {t}: the engine chose {sorted(theirs)}"
        group_call = keep < groups and float(gs[t, keep - 1] - gs[t, keep]) <= 2 * slack
        for e in theirs - mine:
            if group_call:
                continue
            near = min(abs(float(c[t, e] - c[t, o])) for o in mine - theirs)
            assert near <= slack, f"token {t}: expert {e} instead of one of {sorted(mine - theirs)} is no close call ({near:.3g})"
        order = sorted(theirs, key=lambda e: -float(c[t, e]))
        out_i[t] = torch.tensor(order)
        out_w[t] = s[t, order]
    return out_i, out_w


def routed_experts(h, w, p, mlp, round_to=None, given=None, slack=0.0):
    r = mlp["router"]
    T = h.shape[0]
    g = r.get("groups") or {"count": 1, "keep": 1}
    # the router reads h as the engine hands it over (possibly rounded); its own arithmetic stays wide
    idx, wt = route(h, w[p + "router"], w[p + "correction"], r["top"], g["count"], g["keep"])
    if given is not None:
        idx, wt = follow_close_calls(h, w[p + "router"], w[p + "correction"], idx, wt, given, slack, g["count"], g["keep"])
    out = torch.zeros(T, w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(T):
        for j in range(r["top"]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"], round_to)[0]
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"], round_to)
    return out


def feed_forward(h, w, p, mlp, round_to=None, given=None, slack=0.0):
    if mlp["kind"] == "dense":
        return relu_feed_forward(h, w, p, round_to)
    return routed_experts(h, w, p, mlp, round_to, given, slack)


def layer_order(cfg):
    """The layer runs in order: [(layer index, add the embedding output first?)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(cfg, w, tokens, round_to=None, streams=None, routes=None, slack=0.0):
    """float64 logits [T, vocab] of one sequence; ``streams`` (a list) receives the residual stream after every
    layer run.  ``routes``: per layer run (None where it has no router) the experts an engine chose, [T, top]: they
    are followed where they differ from the plain choice by close calls only (``follow_close_calls``)."""
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    T = tokens.shape[0]
    positions = torch.arange(T)
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][tokens]
    x = x0.clone()
    for run, (i, add_first) in enumerate(layer_order(cfg)):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if add_first:
            x = x + x0
        h = _r(rms_norm(x, w[p + "norm1"], eps), round_to)
        if layer["type"] == "attention":
            a = rotary_window_attention(h, w, p + "mix.", layer["mixer"], eps, positions, round_to)
        elif layer["type"] == "attention_2":
            a = capped_chunk_attention(h, w, p + "mix.", layer["mixer"], positions, round_to)
        else:
            raise ValueError(layer["type"])
        given = routes[run] if routes is not None else None
        f = feed_forward(h, w, p + "mlp.", layer["mlp"], round_to, given, slack) if layer.get("mlp") is not None else 0.0
        x = x + (a + f)
        if streams is not None:
            streams.append(x.clone())
    y = _r(rms_norm(x, w["final.norm"], eps), round_to)
    logits = y @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
