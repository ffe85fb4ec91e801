"""Timings of single kernels at serving sizes, with CUDA events, for ``bench.py --kernels``.

Each function returns a list of records (dicts); times are medians over repeated launches.  Decode
kernels are timed inside a CUDA graph of several launches over different data (larger than the
L2), the way a decode step runs them; prefill attention is replayed from a graph of a few launches.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Dict, List, Sequence

import numpy as np
import torch

from . import kernels
from .parts import LayerCache, Workspace
from .parts import attention_backend


def _graph_time_us(run, per: int, repeats: int = 8) -> float:
    """Median time of one of the ``per`` launches that ``run`` makes, replayed from a CUDA graph."""
    torch.cuda.synchronize()   # what the caller prepared on the current stream is done
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1000.0 / per)
    return float(sorted(times)[len(times) // 2])


def _attention_context(entries, page_size: int, device):
    """Step metadata for `entries` = [(cached tokens, new tokens)], pages handed out in shuffled order."""
    to = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=device)
    counts = [c for _, c in entries]
    q_start = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    pages_per = max((s + c + page_size - 1) // page_size for s, c in entries)
    num_pages = len(entries) * pages_per + 1
    table = np.random.default_rng(0).permutation(num_pages - 1)[: len(entries) * pages_per].reshape(len(entries), pages_per)
    pos = np.concatenate([np.arange(s, s + c) for s, c in entries])
    req = np.concatenate([np.full(c, b) for b, (_, c) in enumerate(entries)])
    ctx = SimpleNamespace(
        positions=to(pos), req_of_token=to(req), q_start=to(q_start), start_pos=to([s for s, _ in entries]),
        num_entries=len(entries), num_tokens=int(q_start[-1]), h_q_start=q_start, real_entries=len(entries),
        h_start_pos=np.asarray([s for s, _ in entries], dtype=np.int32), max_context=max(s + c for s, c in entries),
        fixed_shapes=False, scratch={}, workspace=Workspace(device), err=torch.zeros(1, dtype=torch.int32, device=device))
    return ctx, to(table.astype(np.int32)), pages_per, num_pages


def decode_attention(cases: Sequence = ((1, 4096), (8, 4096), (64, 4096), (8, 32768)), *, heads: int = 32,
                     kv_heads: int = 8, head_dim: int = 128, page_size: int = 16, hbm_gbs: float = 0.0,
                     device="cuda:0", softcap=None, slope_exponent=None, chunk=None) -> List[Dict]:
    """One decode token per request over `context` cached tokens, for (batch, context) cases.  ``softcap``,
    ``slope_exponent``, ``chunk``: the attention with capped scores, a distance bias and a chunked mask."""
    out = []
    changes = dict(softcap=softcap, slope_exponent=slope_exponent, chunk=chunk)
    mask = kernels.mask_code(None, chunk)
    for batch, context in cases:
        ctx, table, stride, num_pages = _attention_context([(context - 1, 1)] * batch, page_size, device)
        layers = 8 if batch * context <= 8 * 32768 else 2
        caches = [LayerCache.of_keys_and_values(torch.randn(num_pages, kv_heads, page_size, head_dim, device=device).bfloat16(),
                             torch.randn(num_pages, kv_heads, page_size, head_dim, device=device).bfloat16(), 0, page_size)
                  for _ in range(layers)]
        q = torch.randn(batch, heads, head_dim, device=device).bfloat16()
        o = torch.empty_like(q)
        nbytes = batch * context * kv_heads * head_dim * 2 * 2
        rec = {"kernel": "decode attention", "batch": batch, "context": context, "bytes": nbytes}
        for name, flag in (("tcgen05_us", True), ("mma_sync_us", False)):
            attention_backend.DECODE_TC = flag
            try:
                # as in a step: the work is planned once, before the first kernel, for all layers
                ctx.scratch.clear()
                attention_backend.prepare_step(ctx, torch.bfloat16, heads, kv_heads, head_dim, page_size, mask, stride)
                torch.cuda.synchronize()   # the launches below run on a stream of their own
                rec[name] = round(_graph_time_us(lambda: [attention_backend.attend(o, q, c, ctx, table, stride, None, head_dim ** -0.5,
                                                                                   **changes)
                                                          for c in caches], layers), 1)
            finally:
                attention_backend.DECODE_TC = True
        if int(ctx.err):
            raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(ctx.err)))
        rec["gbs"] = round(nbytes / rec["tcgen05_us"] / 1e3, 1)
        if hbm_gbs:
            rec["frac_of_hbm"] = round(rec["gbs"] / hbm_gbs, 3)
        out.append(rec)
    return out


def prefill_attention(cases: Sequence = ((0, 2048), (0, 8192), (24576, 8192)), *, heads: int = 32, kv_heads: int = 8,
                      head_dim: int = 128, page_size: int = 16, peak_tflops: float = 0.0, device="cuda:0", softcap=None,
                      slope_exponent=None, chunk=None) -> List[Dict]:
    """One request bringing `new` tokens after `cached` ones, for (cached, new) cases.  ``softcap``,
    ``slope_exponent``, ``chunk``: the attention with capped scores, a distance bias and a chunked mask."""
    out = []
    changes = dict(softcap=softcap, slope_exponent=slope_exponent, chunk=chunk)
    mask = kernels.mask_code(None, chunk)
    for cached, new in cases:
        ctx, table, stride, num_pages = _attention_context([(cached, new)], page_size, device)
        cache = LayerCache.of_keys_and_values(torch.randn(num_pages, kv_heads, page_size, head_dim, device=device).bfloat16(),
                           torch.randn(num_pages, kv_heads, page_size, head_dim, device=device).bfloat16(), 0, page_size)
        q = torch.randn(new, heads, head_dim, device=device).bfloat16()
        o = torch.empty_like(q)
        flops = 4.0 * heads * head_dim * (new * cached + new * (new + 1) / 2)
        rec = {"kernel": "prefill attention", "cached": cached, "new": new, "flops": flops}
        for name, flag in (("tcgen05_us", True), ("mma_sync_us", False)):
            attention_backend.PREFILL_TC = flag
            try:
                # several launches replayed from a CUDA graph: the host's share of a launch (tensor maps, wrappers)
                # is not in the time, as it is not in a step, where launches queue ahead of the device
                per = 4 if new * (cached + new) <= 8192 * 16384 else 1
                attention_backend.prepare_step(ctx, torch.bfloat16, heads, kv_heads, head_dim, page_size, mask, stride)
                torch.cuda.synchronize()
                rec[name] = round(_graph_time_us(lambda: [attention_backend.attend(o, q, cache, ctx, table, stride, None, head_dim ** -0.5,
                                                                                   **changes)
                                                          for _ in range(per)], per), 1)
            finally:
                attention_backend.PREFILL_TC = True
        if int(ctx.err):
            raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(ctx.err)))
        rec["tflops"] = round(flops / rec["tcgen05_us"] / 1e6, 1)
        if peak_tflops:
            rec["frac_of_peak"] = round(rec["tflops"] / peak_tflops, 3)
        out.append(rec)
    return out


def decode_gemms(tokens: Sequence[int] = (1, 8, 32), *, hidden: int = 4096, heads: int = 32, kv_heads: int = 8,
                 head_dim: int = 128, intermediate: int = 12288, hbm_gbs: float = 0.0, device="cuda:0") -> List[Dict]:
    """The four matrix products of a layer, one after the other as in a decode step, for M tokens:
    the streaming tcgen05 kernel and the library product."""
    shapes = [((heads + 2 * kv_heads) * head_dim, hidden), (hidden, heads * head_dim), (2 * intermediate, hidden),
              (hidden, intermediate)]
    layer_bytes = sum(n * k * 2 for n, k in shapes)
    layers = max(2, int(600e6 / layer_bytes) + 1)      # more weights than the L2 holds
    ws = [[(torch.randn(n, k, device=device) * 0.02).bfloat16() for n, k in shapes] for _ in range(layers)]
    err = torch.zeros(1, dtype=torch.int32, device=device)
    out = []
    for m in tokens:
        xs = {k: torch.randn(m, k, device=device).bfloat16() for _, k in shapes}
        ys = {n: torch.empty(m, n, dtype=torch.bfloat16, device=device) for n, _ in shapes}

        def own():
            for l in range(layers):
                for (n, k), w in zip(shapes, ws[l]):
                    if not kernels.gemm_skinny_tc(ys[n], xs[k], w, err):
                        raise RuntimeError(f"the streaming kernel does not take M={m}, N={n}, K={k}")

        def lib():
            for l in range(layers):
                for (n, k), w in zip(shapes, ws[l]):
                    torch.mm(xs[k], w.t(), out=ys[n])

        rec = {"kernel": "decode matrix products of a layer", "tokens": m, "bytes": layer_bytes,
               "tcgen05_us": round(_graph_time_us(own, layers), 1), "library_us": round(_graph_time_us(lib, layers), 1)}
        rec["gbs"] = round(layer_bytes / rec["tcgen05_us"] / 1e3, 1)
        if hbm_gbs:
            rec["frac_of_hbm"] = round(rec["gbs"] / hbm_gbs, 3)
        out.append(rec)
    if int(err):
        raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(err)))
    return out


def _loop_time_us(run, repeats: int = 9) -> float:
    """Median time of one call of ``run`` (CUDA events, a synchronisation on both sides)."""
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1000.0)
    return float(sorted(times)[len(times) // 2])


def prefill_elementwise(tokens: int = 2048, *, hidden: int = 4096, heads: int = 32, kv_heads: int = 8, head_dim: int = 128,
                        intermediate: int = 12288, page_size: int = 16, hbm_gbs: float = 0.0, device="cuda:0") -> List[Dict]:
    """The memory-bound kernels between the matrix products at a prompt portion's size: residual sum +
    RMSNorm, q/k norm + rotation + cache write, SiLU gate.  Each call works on one of several sets of
    buffers in turn, together larger than the L2, and the time is per call."""
    sets = 4
    err = torch.zeros(1, dtype=torch.int32, device=device)
    bf = lambda *shape: torch.randn(*shape, device=device).bfloat16()
    out = []

    def record(name, nbytes, run):
        us = _loop_time_us(lambda: [run(i) for i in range(sets)]) / sets
        rec = {"kernel": name, "tokens": tokens, "bytes": nbytes, "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1)}
        if hbm_gbs:
            rec["frac_of_hbm"] = round(rec["gbs"] / hbm_gbs, 3)
        out.append(rec)

    # residual sum + RMSNorm: reads x and the branch, writes the sum and the normed rows
    xs, bs, os_ = [bf(tokens, hidden) for _ in range(sets)], [bf(tokens, hidden) for _ in range(sets)], [bf(tokens, hidden) for _ in range(sets)]
    w = torch.randn(hidden, device=device).float()
    record("residual sum + RMSNorm", 4 * tokens * hidden * 2,
           lambda i: kernels.rmsnorm(os_[i], xs[i], w, 1e-6, err, branch=bs[i], sum_out=xs[i]))
    # q/k norm + rotation + cache write: reads the packed projection, writes q and the pages
    width = (heads + 2 * kv_heads) * head_dim
    qkvs = [bf(tokens, width) for _ in range(sets)]
    qs = [torch.empty(tokens, heads, head_dim, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    pages = (tokens + page_size - 1) // page_size
    kc = [torch.zeros(pages, kv_heads, page_size, head_dim, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    vc = [torch.zeros_like(k) for k in kc]
    qw, kw = torch.randn(head_dim, device=device).float(), torch.randn(head_dim, device=device).float()
    half = head_dim // 2
    cos, sin = torch.randn(tokens, half, device=device).float(), torch.randn(tokens, half, device=device).float()
    pos = torch.arange(tokens, dtype=torch.int32, device=device)
    req = torch.zeros(tokens, dtype=torch.int32, device=device)
    table = torch.randperm(pages, device=device).to(torch.int32)
    record("q/k norm + rotation + cache write", 2 * tokens * width * 2,
           lambda i: kernels.qk_norm_rope_write(qs[i], kc[i], vc[i], qkvs[i], qw, kw, cos, sin, pos, req, table, pages, heads, kv_heads,
                                                head_dim, head_dim, False, 1e-6, True, err))
    # SiLU gate: reads gate and up, writes their product
    gus = [bf(tokens, 2 * intermediate) for _ in range(sets)]
    acts = [torch.empty(tokens, intermediate, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    record("SiLU gate", 3 * tokens * intermediate * 2, lambda i: kernels.swiglu(acts[i], gus[i]))
    if int(err):
        raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(err)))
    return out


def sampling(rows: Sequence[int] = (1, 8, 64), *, vocab: int = 151936, device="cuda:0") -> List[Dict]:
    """The sampling kernel alone (no host work, no copies) over float32 logits, per way of sampling."""
    from .sampling import SamplingParams
    from .sampling.sampler import Sampler
    ways = (("greedy", SamplingParams(temperature=0.0)), ("temperature", SamplingParams(temperature=0.8)),
            ("top-k 20, top-p 0.95", SamplingParams(temperature=0.6, top_k=20, top_p=0.95)),
            ("top-p 0.9", SamplingParams(temperature=0.8, top_p=0.9)), ("top-k 1000", SamplingParams(temperature=0.8, top_k=1000)))
    out = []
    for r in rows:
        logits = torch.randn(r, vocab, device=device) * 3
        s = Sampler(device, r)
        rec = {"kernel": "sampling", "rows": r, "vocab": vocab}
        for name, sp in ways:
            s.sample(logits, [sp] * r, [1] * r, [0] * r, None)     # leaves the rows' parameters on the device
            rec[name + " us"] = round(_graph_time_us(lambda: [kernels.sample(s._out_dev, logits, s._params_dev, s._hist_dev, False,
                                                                             s._scratch, None, capacity=r) for _ in range(8)], 8), 1)
        out.append(rec)
    return out


def decode_ablation(config: Dict, *, layers: int = 12, batches: Sequence[int] = (1, 8), context: int = 3900,
                    page_size: int = 16, device="cuda:0") -> List[Dict]:
    """What each kind of kernel costs IN the chain of a decode step: the step is timed whole and with one
    kind of kernel left out (the numbers it computes are then wrong; its launches are gone, everything
    else is as in the product: CUDA graph, programmatic dependent launch).  The difference is what
    that kind really costs, start-up and drain included and whatever it hides of its neighbours
    excluded; beside it stands what its bytes would take at the measured copy rate."""
    from .engine.runner import ModelRunner, StepInput
    from .parts import attention as attention_part
    from .parts import attention_backend as backend
    from .parts import norm as norm_part
    from .parts import swiglu as swiglu_part

    cfg = dict(config, num_hidden_layers=layers)
    rng = np.random.default_rng(0)

    def timed(batch: int) -> float:
        runner = ModelRunner.random(cfg, seed=0, dtype="bfloat16", block_size=page_size, device=device,
                                    num_blocks=batch * (context // page_size + 20), max_num_seqs=batch, max_model_len=context + 256)
        slots = [runner.open_request() for _ in range(batch)]
        for s in slots:
            runner.step([StepInput(s, rng.integers(0, 1000, size=context), [])])
        one = lambda: runner.step([StepInput(s, rng.integers(0, 1000, size=1), [0]) for s in slots], allow_graph=True)
        for _ in range(30):
            one()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(64):
            one()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 64 * 1000.0

    keep = (kernels.swiglu, kernels.qk_norm_rope_write, backend.attend, attention_part.linear, swiglu_part.linear,
            norm_part.RMSNorm.forward)

    def no_norm(self, out, x, ctx, branch=None, sum_out=None, rows=None):
        return keep[5](self, out, x, ctx, branch, sum_out, rows) if rows is not None else out

    variants = [
        ("whole step", lambda: None),
        ("norms (two per layer)", lambda: setattr(norm_part.RMSNorm, "forward", no_norm)),
        ("q/k norm + rotation + cache write", lambda: setattr(kernels, "qk_norm_rope_write", lambda *a, **k: None)),
        ("attention", lambda: setattr(backend, "attend", lambda *a, **k: None)),
        ("q/k/v and output products", lambda: setattr(attention_part, "linear", lambda out, x, w, err=None: out)),
        ("SiLU gate", lambda: setattr(kernels, "swiglu", lambda out, gu: None)),
        ("gate/up and down products", lambda: setattr(swiglu_part, "linear", lambda out, x, w, err=None: out)),
    ]
    out = []
    try:
        for batch in batches:
            whole = None
            for name, patch in variants:
                patch()
                try:
                    us = timed(batch)
                finally:
                    (kernels.swiglu, kernels.qk_norm_rope_write, backend.attend, attention_part.linear, swiglu_part.linear) = keep[:5]
                    norm_part.RMSNorm.forward = keep[5]
                if whole is None:
                    whole = us
                    out.append({"kernel": "decode step", "batch": batch, "layers": layers, "us_per_step": round(us, 1)})
                else:
                    out.append({"kernel": "decode step without " + name, "batch": batch, "us_per_step": round(us, 1),
                                "cost_in_chain_us_per_layer": round((whole - us) / layers, 1)})
    finally:
        (kernels.swiglu, kernels.qk_norm_rope_write, backend.attend, attention_part.linear, swiglu_part.linear) = keep[:5]
        norm_part.RMSNorm.forward = keep[5]
    return out


# ---- the Tidarax kernels at a real model's layer sizes, each beside the like kernel of the Qwen3 path ----------
FP32_FMA_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12      # 148 SMs x 128 lanes x 2 operations at 1965 MHz


def tidarax_kernels(*, hidden: int = 4096, heads: int = 32, kv_heads: int = 8, head_dim: int = 128, intermediate: int = 12288,
                    rec_width: int = 4096, experts: int = 8, expert_ff: int = 3072, top: int = 2, tokens: int = 2048,
                    decode: Sequence[int] = (8, 4096), page_size: int = 16, hbm_gbs: float = 0.0, peak_tflops: float = 0.0,
                    device="cuda:0") -> List[Dict]:
    """One record per kernel of the Tidarax path: time, what it achieves and the share of its floor.  The
    floor of the attention is the slower of its tensor-core products at the measured matrix-product peak
    and its mix across heads (2 heads^2 float32 operations per query-key pair) at the nominal FMA rate."""
    out: List[Dict] = []
    err = torch.zeros(1, dtype=torch.int32, device=device)
    bf = lambda *shape: torch.randn(*shape, device=device).bfloat16()
    H, G, d = heads, kv_heads, head_dim
    talk = (torch.randn(H, H, device=device) / H ** 0.5).float().contiguous()

    # attention over a whole prompt
    ctx, table, stride, num_pages = _attention_context([(0, tokens)], page_size, device)
    kc, vc = bf(num_pages, G, page_size, d), bf(num_pages, G, page_size, d)
    q, o = bf(tokens, H, d), torch.empty(tokens, H * d, dtype=torch.bfloat16, device=device)
    pairs = tokens * (tokens + 1) / 2
    for name, fn, tile in (("tensor cores", kernels.attn_talking_mma, kernels.attn_talking_mma_tile(H, G, d, d, tokens)),
                           ("FMA units", kernels.attn_talking, kernels.attn_talking_tile(H, d, d, tokens))):
        if tile <= 0 or (name == "FMA units" and tokens * H * d > 2048 * 16 * 128):
            continue      # the FMA form at these sizes takes seconds: it is the float32 path's kernel
        us = _graph_time_us(lambda: fn(o, q, kc, vc, talk, ctx.q_start, ctx.start_pos, 1, table, stride, None, d ** -0.5,
                                       True, 1.0, tile, err), 1, repeats=5)
        tc, mix = 4.0 * H * d * pairs, 2.0 * H * H * pairs
        floor_us = max(tc / (peak_tflops or 1590.0) / 1e6, mix / FP32_FMA_TFLOPS_NOMINAL / 1e6)
        out.append({"kernel": f"talking attention, prompt ({name})", "tokens": tokens, "us": round(us, 1),
                    "tensor_tflops": round(tc / us / 1e6, 1), "mix_fp32_tflops": round(mix / us / 1e6, 2),
                    "floor_us": round(floor_us, 1), "frac_of_floor": round(floor_us / us, 3), "query_tile": tile})
    like = prefill_attention(((0, tokens),), heads=H, kv_heads=G, head_dim=d, page_size=page_size, peak_tflops=peak_tflops)[0]
    out.append({"kernel": "like: Qwen3 prompt attention (tcgen05)", "tokens": tokens, "us": like["tcgen05_us"],
                "tensor_tflops": like["tflops"], "frac_of_floor": like.get("frac_of_peak")})

    # attention of single tokens
    batch, context = decode
    ctx, table, stride, num_pages = _attention_context([(context - 1, 1)] * batch, page_size, device)
    layers = 4
    caches = [(bf(num_pages, G, page_size, d), bf(num_pages, G, page_size, d)) for _ in range(layers)]
    q, o = bf(batch, H, d), torch.empty(batch, H * d, dtype=torch.bfloat16, device=device)
    from .parts import talking_attention
    parts = max(1, min(talking_attention._DECODE_BLOCKS // batch, context // talking_attention._DECODE_MIN_KEYS, 64))
    po = torch.zeros(batch * parts * H * d, dtype=torch.float32, device=device)
    pml = torch.zeros(batch * parts * H * 2, dtype=torch.float32, device=device)
    nbytes = batch * context * G * d * 2 * 2
    us = _graph_time_us(lambda: [kernels.attn_talking_mma(o, q, k_, v_, talk, ctx.q_start, ctx.start_pos, batch, table, stride,
                                                          None, d ** -0.5, True, 1.0, 1, err, parts, po, pml)
                                 for k_, v_ in caches], layers)
    floor_us = nbytes / (hbm_gbs or 6650.0) / 1e3
    out.append({"kernel": "talking attention, single tokens (tensor cores)", "batch": batch, "context": context,
                "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1), "floor_us": round(floor_us, 1),
                "frac_of_floor": round(floor_us / us, 3), "key_ranges": parts})
    like = decode_attention(((batch, context),), heads=H, kv_heads=G, head_dim=d, page_size=page_size, hbm_gbs=hbm_gbs)[0]
    out.append({"kernel": "like: Qwen3 single-token attention (tcgen05)", "batch": batch, "context": context,
                "us": like["tcgen05_us"], "gbs": like["gbs"], "frac_of_floor": like.get("frac_of_hbm")})
    del caches, po, pml

    # the memory-bound kernels at a prompt portion's size; several sets of buffers, together larger than the L2
    sets = 4

    def record(name, nbytes, run, like=None):
        us = _loop_time_us(lambda: [run(i) for i in range(sets)]) / sets
        rec = {"kernel": name, "tokens": tokens, "bytes": nbytes, "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1)}
        if hbm_gbs:
            rec["frac_of_floor"] = round(rec["gbs"] / hbm_gbs, 3)
        if like:
            rec["like"] = like
        out.append(rec)

    xs = [torch.randn(tokens, hidden, device=device) for _ in range(sets)]
    bs = [torch.randn(tokens, hidden, device=device) for _ in range(sets)]
    os_ = [torch.empty(tokens, hidden, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    w = torch.randn(hidden, device=device)
    record("float32 residual sum + norm", tokens * hidden * (4 + 4 + 4 + 2),
           lambda i: kernels.rmsnorm(os_[i], xs[i], w, 1e-6, err, branch=bs[i], sum_out=xs[i], weight_offset=1.0),
           "residual sum + RMSNorm")
    del xs, bs, os_
    width = (H + 2 * G) * d
    qkvs = [bf(tokens, width) for _ in range(sets)]
    qs = [torch.empty(tokens, H, d, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    pages = (tokens + page_size - 1) // page_size
    kcs = [torch.zeros(pages, G, page_size, d, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    vcs = [torch.zeros_like(k) for k in kcs]
    inv = torch.rand(d // 2, device=device)
    pos = torch.arange(tokens, dtype=torch.int32, device=device)
    req = torch.zeros(tokens, dtype=torch.int32, device=device)
    tab = torch.randperm(pages, device=device).to(torch.int32)
    record("rotation + unit norm + cache write", 2 * tokens * width * 2,
           lambda i: kernels.qkv_prepare(qs[i], kcs[i], vcs[i], qkvs[i], None, None, inv, pos, req, tab, pages, H, G, d, d, d,
                                         False, 2, 1e-6, True, err), "q/k norm + rotation + cache write")
    del qkvs, qs, kcs, vcs
    W = rec_width
    zxgs = [torch.randn(tokens, 3 * W, device=device) for _ in range(sets)]
    ys = [torch.empty(tokens, W, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    bz, bx = torch.randn(W, device=device), torch.randn(W, device=device)
    state = torch.zeros(2, W, device=device)
    q_start = torch.tensor([0, tokens], dtype=torch.int32, device=device)
    slots = torch.tensor([0], dtype=torch.int32, device=device)
    scratch = torch.empty(3 * tokens * W, device=device)
    record("gated recurrence over a prompt (three passes)", tokens * W * (3 * 4 + 2),
           lambda i: kernels.gated_scan(ys[i], zxgs[i], bz, bx, state, q_start, slots, req, 1, 1.0, scratch), "SiLU gate")
    del zxgs, ys, scratch
    zs = [torch.randn(tokens, intermediate, device=device) for _ in range(sets)]
    acts = [torch.empty(tokens, intermediate, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    coef = torch.tensor([0.5, 0.3, 0.2, 0.1], device=device)
    record("polynomial activation with normed powers", tokens * intermediate * (4 + 2),
           lambda i: kernels.polynorm(acts[i], zs[i], coef, 1e-6), "SiLU gate")
    del zs, acts
    for rec in prefill_elementwise(tokens, hidden=hidden, heads=H, kv_heads=G, head_dim=d, intermediate=intermediate,
                                   page_size=page_size, hbm_gbs=hbm_gbs):
        out.append({"kernel": "like: Qwen3 " + rec["kernel"], "tokens": tokens, "us": rec["us"], "gbs": rec["gbs"],
                    "frac_of_floor": rec.get("frac_of_hbm")})

    # the experts' grouped products against the library's dense product of the same work
    E, F = experts, expert_ff
    rows = tokens * top
    x = bf(tokens, hidden)
    wgu, wd = bf(E, 2 * F, hidden) * 0.02, bf(hidden, E * F) * 0.02
    table = torch.rand(1000, E, device=device).argsort(dim=1)[:, :top].to(torch.int32).contiguous()
    ids = torch.randint(0, 1000, (tokens,), device=device, dtype=torch.int32)
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=device)
    perm, inv_ = torch.zeros(rows, dtype=torch.int32, device=device), torch.zeros(rows, dtype=torch.int32, device=device)
    kernels.expert_route(offsets, perm, inv_, table, ids, None, req, tokens, top, E, err)
    act, y = torch.empty(rows, F, dtype=torch.bfloat16, device=device), torch.empty(rows, hidden, device=device)
    us1 = _loop_time_us(lambda: kernels.expert_gemm(act, x, wgu, offsets, perm, True, top, True))
    us2 = _loop_time_us(lambda: kernels.expert_gemm(y, act, wd, offsets, perm, False, top, False, side_by_side=True))
    us0 = _loop_time_us(lambda: kernels.expert_route(offsets, perm, inv_, table, ids, None, req, tokens, top, E, err))
    f1, f2 = 2.0 * rows * 2 * F * hidden, 2.0 * rows * hidden * F
    for name, us, fl in (("experts: gate/up product with the gate (mma.sync)", us1, f1), ("experts: down product (mma.sync)", us2, f2)):
        out.append({"kernel": name, "rows": rows, "us": round(us, 1), "tensor_tflops": round(fl / us / 1e6, 1),
                    "frac_of_floor": round(fl / us / 1e6 / (peak_tflops or 1590.0), 3)})
    out.append({"kernel": "experts: grouping by expert (one block)", "rows": rows, "us": round(us0, 1)})
    xa, wa = bf(rows, hidden), bf(2 * F, hidden)
    oa = torch.empty(rows, 2 * F, dtype=torch.bfloat16, device=device)
    usl = _loop_time_us(lambda: torch.mm(xa, wa.t(), out=oa))
    out.append({"kernel": "like: the library's dense product of the gate/up work", "rows": rows, "us": round(usl, 1),
                "tensor_tflops": round(f1 / usl / 1e6, 1), "frac_of_floor": round(f1 / usl / 1e6 / (peak_tflops or 1590.0), 3)})
    if int(err):
        raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(err)))
    return out


def dufitar_kernels(*, hidden: int = 4096, heads: int = 32, kv_heads: int = 8, head_dim: int = 128, intermediate: int = 12288,
                    kv_rank: int = 512, rot_dim: int = 64, tokens: int = 2048, decode: Sequence[int] = (8, 4096),
                    page_size: int = 16, hbm_gbs: float = 0.0, peak_tflops: float = 0.0, device="cuda:0") -> List[Dict]:
    """One record per kernel of the Dufitar path: time, what it achieves and the share of its floor (bytes at the
    measured copy rate, or tensor-core work at the measured matrix-product peak), each beside its like kernel of
    the Qwen3 path.  The grouped-query layers' attention IS the Qwen3 path's tcgen05 kernel, so only the
    attention over latent rows has a kernel of its own to compare."""
    out: List[Dict] = []
    err = torch.zeros(1, dtype=torch.int32, device=device)
    bf = lambda *shape: torch.randn(*shape, device=device).bfloat16()
    H, G, d, r, rd = heads, kv_heads, head_dim, kv_rank, rot_dim
    dk = r + rd
    sink = torch.randn(H, device=device)
    from .parts import latent_attention as la

    # attention over latent rows, a whole prompt: 2 heads (dk + rank) operations per (query, key) pair and head
    ctx, table, stride, num_pages = _attention_context([(0, tokens)], page_size, device)
    ctx.all_single = False
    rows = bf(num_pages, page_size, dk)
    q, o = bf(tokens, H, dk) * dk ** -0.5, torch.empty(tokens, H, r, dtype=torch.bfloat16, device=device)
    pairs = tokens * (tokens + 1) / 2
    us = _graph_time_us(lambda: la.latent_attend(o, q, rows, ctx, table, stride, page_size, None, 1.0, sink), 1, repeats=5)
    tc = 2.0 * H * (dk + r) * pairs
    floor_us = tc / (peak_tflops or 1590.0) / 1e6
    out.append({"kernel": "latent attention, prompt (mma.sync)", "tokens": tokens, "us": round(us, 1),
                "tensor_tflops": round(tc / us / 1e6, 1), "floor_us": round(floor_us, 1), "frac_of_floor": round(floor_us / us, 3)})
    like = prefill_attention(((0, tokens),), heads=H, kv_heads=G, head_dim=d, page_size=page_size, peak_tflops=peak_tflops)[0]
    out.append({"kernel": "like: Qwen3 prompt attention (tcgen05)", "tokens": tokens, "us": like["tcgen05_us"],
                "tensor_tflops": like["tflops"], "frac_of_floor": like.get("frac_of_peak")})
    del rows, q, o

    # attention of single tokens over latent rows: one row of dk channels per key, whatever the number of heads
    batch, context = decode
    ctx, table, stride, num_pages = _attention_context([(context - 1, 1)] * batch, page_size, device)
    ctx.all_single = True
    layers = 4
    caches = [bf(num_pages, page_size, dk) for _ in range(layers)]
    q, o = bf(batch, H, dk) * dk ** -0.5, torch.empty(batch, H, r, dtype=torch.bfloat16, device=device)
    nbytes = batch * context * dk * 2
    us = _graph_time_us(lambda: [la.latent_attend(o, q, c, ctx, table, stride, page_size, None, 1.0, sink) for c in caches], layers)
    floor_us = nbytes / (hbm_gbs or 6650.0) / 1e3
    tc = 2.0 * H * (dk + r) * batch * context
    out.append({"kernel": "latent attention, single tokens (mma.sync)", "batch": batch, "context": context, "us": round(us, 1),
                "gbs": round(nbytes / us / 1e3, 1), "tensor_tflops": round(tc / us / 1e6, 1), "floor_us": round(floor_us, 1),
                "frac_of_floor": round(floor_us / us, 3)})
    like = decode_attention(((batch, context),), heads=H, kv_heads=G, head_dim=d, page_size=page_size, hbm_gbs=hbm_gbs)[0]
    out.append({"kernel": "like: Qwen3 single-token attention (tcgen05)", "batch": batch, "context": context,
                "us": like["tcgen05_us"], "gbs": like["gbs"], "frac_of_floor": like.get("frac_of_hbm")})
    del caches, q, o

    # the per-head maps into and out of the latent space (the library's batched product)
    qp, w_uk = bf(tokens, H, d + rd), bf(H, d, r) * 0.02
    q_lat = torch.empty(tokens, H, dk, dtype=torch.bfloat16, device=device)[:, :, :r].transpose(0, 1)
    us = _loop_time_us(lambda: la.batched_product(q_lat, qp[:, :, :d].transpose(0, 1), w_uk.transpose(1, 2)))
    fl = 2.0 * tokens * H * d * r
    out.append({"kernel": "queries into the latent space (library batched product)", "tokens": tokens, "us": round(us, 1),
                "tensor_tflops": round(fl / us / 1e6, 1), "frac_of_floor": round(fl / us / 1e6 / (peak_tflops or 1590.0), 3)})
    o_lat, w_uv = bf(tokens, H, r), bf(H, d, r) * 0.02
    o_heads = torch.empty(tokens, H, d, dtype=torch.bfloat16, device=device).transpose(0, 1)
    us = _loop_time_us(lambda: la.batched_product(o_heads, o_lat.transpose(0, 1), w_uv))
    out.append({"kernel": "values out of the latent space (library batched product)", "tokens": tokens, "us": round(us, 1),
                "tensor_tflops": round(fl / us / 1e6, 1), "frac_of_floor": round(fl / us / 1e6 / (peak_tflops or 1590.0), 3)})
    del qp, q_lat, o_lat, o_heads

    # the memory-bound kernels at a prompt portion's size; several sets of buffers, together larger than the L2
    sets = 4

    def record(name, nbytes, run, like=None):
        # replayed from a CUDA graph: several of these kernels are shorter than the host's share of a launch
        us = _graph_time_us(lambda: [run(i) for i in range(sets)], sets)
        rec = {"kernel": name, "tokens": tokens, "bytes": nbytes, "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1)}
        if hbm_gbs:
            rec["frac_of_floor"] = round(rec["gbs"] / hbm_gbs, 3)
        if like:
            rec["like"] = like
        out.append(rec)

    xs = [torch.randn(tokens, hidden, device=device) for _ in range(sets)]
    bs = [torch.randn(tokens, hidden, device=device) for _ in range(sets)]
    os_ = [torch.empty(tokens, hidden, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    alpha, w, b = torch.tensor(0.9, device=device), torch.randn(hidden, device=device), torch.randn(hidden, device=device)
    record("Dynamic Tanh of the branch + scaled residual sum + Dynamic Tanh", tokens * hidden * (4 + 4 + 4 + 2),
           lambda i: kernels.dyt_norm(os_[i], xs[i], alpha, w, b, err, branch=bs[i], branch_scale=0.5, branch_norm=(alpha, w, b),
                                      sum_out=xs[i]), "residual sum + RMSNorm")
    del xs, bs, os_
    gus = [bf(tokens, 2 * intermediate) for _ in range(sets)]
    acts = [torch.empty(tokens, intermediate, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    record("GELU (tanh form) gate", 3 * tokens * intermediate * 2, lambda i: kernels.swiglu(acts[i], gus[i], "gelu_tanh"), "SiLU gate")
    del gus, acts
    width = (H + 2 * G) * d
    qkvs = [bf(tokens, width) for _ in range(sets)]
    qs = [torch.empty(tokens, H, d, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    pages = (tokens + page_size - 1) // page_size
    kcs = [torch.zeros(pages, G, page_size, d, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    vcs = [torch.zeros_like(k) for k in kcs]
    inv = torch.rand(d // 4, device=device)
    pos = torch.arange(tokens, dtype=torch.int32, device=device)
    req = torch.zeros(tokens, dtype=torch.int32, device=device)
    tab = torch.randperm(pages, device=device).to(torch.int32)
    record("rotation of half a head + cache write", 2 * tokens * width * 2,
           lambda i: kernels.qkv_prepare(qs[i], kcs[i], vcs[i], qkvs[i], None, None, inv, pos, req, tab, pages, H, G, d, d, d // 2,
                                         True, 0, 1e-6, True, err, rot_magnitude=1.1), "q/k norm + rotation + cache write")
    del qkvs, qs, kcs, vcs
    nq = H * (d + rd)
    projs = [bf(tokens, nq + H * d + dk) for _ in range(sets)]
    qas = [torch.empty(tokens, H, dk, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    lcs = [torch.zeros(pages, page_size, dk, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    nw, inv2 = torch.randn(r, device=device), torch.rand(rd // 2, device=device)
    record("latent norm + rotation of the shared key part and of the queries' rotated parts + row write",
           tokens * 2 * (H * rd + dk) * 2,
           lambda i: kernels.latent_prepare(qas[i], lcs[i], projs[i], 0, nq + H * d, None, nw, inv2, pos, req, tab, pages, H, d, rd,
                                            r, rd, 1e-6, 1.0, err), "q/k norm + rotation + cache write")
    inns = [bf(tokens, H * d) for _ in range(sets)]
    record("sigmoid gate on the heads' outputs (in place)", 3 * tokens * H * d * 2,
           lambda i: kernels.gate_sigmoid(inns[i], inns[i].view(tokens, H, d).transpose(0, 1), projs[i][:, nq:nq + H * d]), "SiLU gate")
    del projs, qas, lcs, inns
    for rec in prefill_elementwise(tokens, hidden=hidden, heads=H, kv_heads=G, head_dim=d, intermediate=intermediate,
                                   page_size=page_size, hbm_gbs=hbm_gbs):
        out.append({"kernel": "like: Qwen3 " + rec["kernel"], "tokens": tokens, "us": rec["us"], "gbs": rec["gbs"],
                    "frac_of_floor": rec.get("frac_of_hbm")})
    if int(err):
        raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(err)))
    return out


def gulipel_kernels(*, hidden: int = 4096, heads: int = 32, kv_heads: int = 8, head_dim: int = 128, intermediate: int = 12288,
                    ss_heads: int = 128, ss_head_dim: int = 64, ss_state: int = 128, ss_groups: int = 8, conv: int = 4,
                    delta_heads: int = 32, delta_kv_heads: int = 32, delta_dim: int = 128, delta_vdim: int = 128, rank: int = 64,
                    tokens: int = 2048, decode_batch: int = 8, hbm_gbs: float = 0.0, device="cuda:0") -> List[Dict]:
    """One record per kernel that the Gulipel path adds: time, bytes and the share of its floor (the bytes that must
    cross memory at the measured copy rate; for the two scans over a prompt also the floor of their arithmetic at the
    nominal FMA rate), beside the like kernels of the Tidarax path at the same width."""
    out: List[Dict] = []
    err = torch.zeros(1, dtype=torch.int32, device=device)
    sets = 4
    f32 = lambda *shape: torch.randn(*shape, device=device)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)

    def record(name, nbytes, run, like=None, flops=0.0, n=sets, **more):
        # replayed from a CUDA graph: several of these kernels are shorter than the host's share of a launch
        us = _graph_time_us(lambda: [run(i) for i in range(n)], n)
        rec = {"kernel": name, "bytes": nbytes, "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1)}
        floor_us = nbytes / (hbm_gbs or 6650.0) / 1e3
        if flops:
            rec["fp32_tflops"] = round(flops / us / 1e6, 2)
            floor_us = max(floor_us, flops / FP32_FMA_TFLOPS_NOMINAL / 1e6)
        rec["floor_us"] = round(floor_us, 1)
        rec["frac_of_floor"] = round(floor_us / us, 3)
        if like:
            rec["like"] = like
        rec.update(more)
        out.append(rec)

    q_start, slots, req = i32([0, tokens]), i32([0]), torch.zeros(tokens, dtype=torch.int32, device=device)
    B = decode_batch
    dq_start, dslots, dreq = i32(list(range(B + 1))), i32(list(range(B))), i32(list(range(B)))

    # the state-space mixer: convolution, scan, gate and norm
    H, P, N, G = ss_heads, ss_head_dim, ss_state, ss_groups
    inner = H * P
    C = inner + 2 * G * N
    for what, T, qs, sl, rq, ne in (("a prompt", tokens, q_start, slots, req, 1), ("single tokens", B, dq_start, dslots, dreq, B)):
        projs = [f32(T, inner + C + H) for _ in range(sets)]
        xbcs = [torch.empty(T, C, device=device) for _ in range(sets)]
        ys = [torch.empty(T, inner, device=device) for _ in range(sets)]
        gated = [torch.empty(T, inner, dtype=torch.bfloat16, device=device) for _ in range(sets)]
        taps, cb = f32(C, conv), f32(C)
        cstates = [torch.zeros(ne, conv - 1, C, device=device) for _ in range(sets)]
        states = [torch.zeros(ne, H, N, P, device=device) for _ in range(sets)]
        dtb, alog, dsk, nw = f32(H), f32(H), f32(H), f32(inner)
        state_bytes = 0 if T > B else 2 * ne * H * N * P * 4
        record(f"short convolution + SiLU, {what}", T * C * 8, lambda i: kernels.conv_silu(
            xbcs[i], projs[i], inner, taps, cb, cstates[i], rq, qs, sl, ne), "SiLU gate", tokens=T, channels=C)
        record(f"state-space scan, {what}", T * (C + inner + H) * 4 + (state_bytes or 2 * H * N * P * 4), lambda i: kernels.selective_scan(
            ys[i], xbcs[i], projs[i], inner + C, dtb, alog, dsk, states[i], qs, sl, ne, H, P, N, G),
            "gated recurrence over a prompt (three passes)", flops=4.0 * T * H * N * P, tokens=T, heads=H, state=N, head_dim=P)
        record(f"gate + norm in parts, {what}", T * inner * (4 + 4 + 2), lambda i: kernels.gated_head_norm(
            gated[i], ys[i], projs[i], 0, nw, inner // G, 1e-5, gate_after=False), "residual sum + RMSNorm", tokens=T)
        del projs, xbcs, ys, gated, cstates, states

    # the gated delta rule
    H, G, d, dv = delta_heads, delta_kv_heads, delta_dim, delta_vdim
    Cq = 2 * G * d + H * dv
    for what, T, qs, sl, rq, ne in (("a prompt", tokens, q_start, slots, req, 1), ("single tokens", B, dq_start, dslots, dreq, B)):
        qkvs = [f32(T, Cq) for _ in range(sets)]
        projs = [f32(T, Cq + H) for _ in range(sets)]
        ags = [f32(T, H * d + H * dv) for _ in range(sets)]
        os_ = [torch.empty(T, H * dv, device=device) for _ in range(sets)]
        gated = [torch.empty(T, H * dv, dtype=torch.bfloat16, device=device) for _ in range(sets)]
        states = [torch.zeros(ne, H, d, dv, device=device) for _ in range(sets)]
        dtb, alog, nw = f32(H * d), f32(H), f32(dv)
        state_bytes = 2 * ne * H * d * dv * 4
        record(f"gated delta rule, {what}", T * (Cq + H * d + H * dv + H) * 4 + state_bytes, lambda i: kernels.delta_rule(
            os_[i], qkvs[i], projs[i], Cq, ags[i], dtb, alog, states[i], qs, sl, ne, H, G, d, dv),
            "gated recurrence over a prompt (three passes)", flops=8.0 * T * H * d * dv, tokens=T, heads=H, dim=d, vdim=dv)
        record(f"norm per head + gate, {what}", T * H * dv * (4 + 4 + 2), lambda i: kernels.gated_head_norm(
            gated[i], os_[i], ags[i], H * d, nw, dv, 1e-5, gate_after=True), "residual sum + RMSNorm", tokens=T)
        del qkvs, projs, ags, os_, gated, states

    # the residual arithmetic: norm of the branch, learned scale, sum, next norm in one pass; the two sides' average
    T = tokens
    xs, bs = [f32(T, hidden) for _ in range(sets)], [f32(T, hidden) for _ in range(sets)]
    os_ = [torch.empty(T, hidden, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    w, bw, g = f32(hidden), f32(hidden), f32(hidden)
    record("normed branch * learned scale + float32 residual sum + norm", T * hidden * (4 + 4 + 4 + 2),
           lambda i: kernels.rms_chain(os_[i], xs[i], w, 1e-5, err, branch=bs[i], branch_weight=bw, branch_eps=1e-5, gain=g,
                                       sum_out=xs[i]), "float32 residual sum + norm", tokens=T)
    record("like: Tidarax float32 residual sum + norm", T * hidden * (4 + 4 + 4 + 2),
           lambda i: kernels.rmsnorm(os_[i], xs[i], w, 1e-6, err, branch=bs[i], sum_out=xs[i], weight_offset=1.0), tokens=T)
    ds = [torch.empty(T, hidden, device=device) for _ in range(sets)]
    record("two sides: norm each, average", T * hidden * 12, lambda i: kernels.dual_rms_sum(ds[i], xs[i], bs[i], w, bw, 1e-5, 0.5, 0.5),
           "float32 residual sum + norm", tokens=T)
    del xs, bs, os_, ds

    # the like kernels of the small ones: the SiLU gate and the residual sum + RMSNorm of a bfloat16 stream
    gus = [torch.randn(T, 2 * intermediate, device=device).bfloat16() for _ in range(sets)]
    acts = [torch.empty(T, intermediate, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    record("like: SiLU gate", 3 * T * intermediate * 2, lambda i: kernels.swiglu(acts[i], gus[i]), tokens=T)
    del gus, acts
    hs = [torch.randn(T, hidden, device=device).bfloat16() for _ in range(sets)]
    rs = [torch.randn(T, hidden, device=device).bfloat16() for _ in range(sets)]
    ns = [torch.empty(T, hidden, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    record("like: residual sum + RMSNorm", 4 * T * hidden * 2,
           lambda i: kernels.rmsnorm(ns[i], hs[i], w, 1e-6, err, branch=rs[i], sum_out=hs[i]), tokens=T)
    del hs, rs, ns

    # the like kernel of the scans: Tidarax's gated recurrence (a vector state per channel) over the same prompt
    W = hidden
    zxgs = [f32(T, 3 * W) for _ in range(sets)]
    ys = [torch.empty(T, W, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    bz, bx = f32(W), f32(W)
    state = torch.zeros(2, W, device=device)
    scratch = torch.empty(3 * T * W, device=device)
    record("like: Tidarax gated recurrence over a prompt (three passes)", T * W * (3 * 4 + 2),
           lambda i: kernels.gated_scan(ys[i], zxgs[i], bz, bx, state, q_start, slots, req, 1, 1.0, scratch), tokens=T)
    del zxgs, ys, scratch

    # the embedding's three terms
    V, buckets = 32000, 100003
    table, pair, pos = (torch.randn(V, hidden, device=device).bfloat16(), torch.randn(buckets + 1, hidden, device=device).bfloat16(),
                        torch.randn(T, hidden, device=device).bfloat16())
    ids = torch.randint(0, V, (T,), device=device, dtype=torch.int32)
    xs = [torch.empty(T, hidden, device=device) for _ in range(sets)]
    prev = torch.zeros(1, dtype=torch.int32, device=device)
    positions = torch.arange(T, dtype=torch.int32, device=device)
    record("embedding row * scale + pair row + position row", T * hidden * (3 * 2 + 4),
           lambda i: kernels.embed_sum(xs[i], table, ids, err, scale=4.0, pair=pair, pair_rule=(buckets, 31, 7), pos_table=pos,
                                       positions=positions, req_of_token=req, q_start=q_start, slots=slots, prev_state=prev),
           "embedding", tokens=T)
    if int(err):
        raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(err)))
    return out


def mikutar_kernels(*, hidden: int = 4096, heads: int = 32, kv_heads: int = 8, head_dim: int = 128, intermediate: int = 12288,
                    experts: int = 8, expert_ff: int = 3072, top: int = 2, groups: int = 4, keep: int = 2, softcap: float = 40.0,
                    chunk: int = 4096, tokens: int = 2048, decode: Sequence[int] = (8, 4096), page_size: int = 16,
                    hbm_gbs: float = 0.0, peak_tflops: float = 0.0, device="cuda:0") -> List[Dict]:
    """One record per kernel of the Mikutar path: time, what it achieves and the share of its floor (bytes at the
    measured copy rate, or tensor-core work at the measured matrix-product peak), each beside its like kernel.  The
    windowed layers' attention IS the engine's tcgen05 kernel; the chunked layers run the same kernel with the
    scores changed before the softmax, measured here beside the unchanged one."""
    out: List[Dict] = []
    err = torch.zeros(1, dtype=torch.int32, device=device)
    bf = lambda *shape: torch.randn(*shape, device=device).bfloat16()
    H, G, d = heads, kv_heads, head_dim
    batch, context = decode
    for name, kw in (("capped scores + distance bias + chunks", dict(softcap=softcap, slope_exponent=8.0, chunk=chunk)),
                     ("distance bias + chunks, no cap", dict(slope_exponent=8.0, chunk=chunk)),
                     ("like: the engine's attention, unchanged scores", {})):
        rec = prefill_attention(((0, tokens),), heads=H, kv_heads=G, head_dim=d, page_size=page_size, peak_tflops=peak_tflops, **kw)[0]
        out.append({"kernel": "prompt attention (tcgen05), " + name, "tokens": tokens, "us": rec["tcgen05_us"],
                    "tensor_tflops": rec["tflops"], "frac_of_floor": rec.get("frac_of_peak")})
        rec = decode_attention(((batch, context),), heads=H, kv_heads=G, head_dim=d, page_size=page_size, hbm_gbs=hbm_gbs, **kw)[0]
        out.append({"kernel": "single-token attention (tcgen05), " + name, "batch": batch, "context": context,
                    "us": rec["tcgen05_us"], "gbs": rec["gbs"], "frac_of_floor": rec.get("frac_of_hbm")})

    sets = 4

    def record(name, nbytes, run, like=None):
        us = _graph_time_us(lambda: [run(i) for i in range(sets)], sets)
        rec = {"kernel": name, "tokens": tokens, "bytes": nbytes, "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1)}
        if hbm_gbs:
            rec["frac_of_floor"] = round(rec["gbs"] / hbm_gbs, 3)
        if like:
            rec["like"] = like
        out.append(rec)

    # the float32 stream: the first branch by an addition kernel, the second with the norm that reads the sum
    xs = [torch.randn(tokens, hidden, device=device) for _ in range(sets)]
    bs = [torch.randn(tokens, hidden, device=device) for _ in range(sets)]
    os_ = [torch.empty(tokens, hidden, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    w = torch.randn(hidden, device=device)
    record("float32 residual sum + RMS norm", tokens * hidden * (4 + 4 + 4 + 2),
           lambda i: kernels.rmsnorm(os_[i], xs[i], w, 1e-6, err, branch=bs[i], sum_out=xs[i]), "residual sum + RMSNorm")
    record("addition of a branch into the float32 stream", tokens * hidden * 12, lambda i: kernels.add(xs[i], xs[i], bs[i]),
           "residual sum + RMSNorm")
    del xs, bs, os_
    # gates
    gus = [bf(tokens, 2 * intermediate) for _ in range(sets)]
    acts = [torch.empty(tokens, intermediate, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    record("ReLU gate", 3 * tokens * intermediate * 2, lambda i: kernels.swiglu(acts[i], gus[i], "relu"), "SiLU gate")
    record("clamped swish gate", 3 * tokens * intermediate * 2,
           lambda i: kernels.swiglu(acts[i], gus[i], "swish_clamp", (2.0, 1.702)), "SiLU gate")
    del gus, acts
    # one norm over the whole q and k projections, rotation of neighbours, keys as projected kept as values, page write
    width = (H + G) * d + H
    qkvs = [bf(tokens, width) for _ in range(sets)]
    qs = [torch.empty(tokens, H, d, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    pages = (tokens + page_size - 1) // page_size
    kcs = [torch.zeros(pages, G, page_size, d, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    vcs = [torch.zeros_like(k) for k in kcs]
    inv = torch.rand(d // 2, device=device)
    qw, kw_, bias = torch.randn(H * d, device=device), torch.randn(G * d, device=device), torch.randn((H + G) * d, device=device)
    pos = torch.arange(tokens, dtype=torch.int32, device=device)
    req = torch.zeros(tokens, dtype=torch.int32, device=device)
    tab = torch.randperm(pages, device=device).to(torch.int32)
    record("bias + norm over the whole projection + rotation + cache write of keys and raw keys", tokens * ((H + G) * d + (H + 2 * G) * d) * 2,
           lambda i: kernels.qkv_prepare(qs[i], kcs[i], vcs[i], qkvs[i], qw, kw_, inv, pos, req, tab, pages, H, G, d, d, d, True, 3,
                                         1e-6, True, err, bias=bias, row_len=width, value_offset=H * d),
           "q/k norm + rotation + cache write")
    inns = [bf(tokens, H * d) for _ in range(sets)]
    record("sigmoid gate of one number per head (in place)", 2 * tokens * H * d * 2,
           lambda i: kernels.gate_sigmoid(inns[i], inns[i].view(tokens, H, d).transpose(0, 1), qkvs[i][:, (H + G) * d:]), "SiLU gate")
    del qkvs, qs, kcs, vcs, inns
    # the router and the routed experts' kernels
    hs = [bf(tokens, hidden) for _ in range(sets)]
    wr, corr = torch.randn(experts, hidden, device=device) * hidden ** -0.5, torch.randn(experts, device=device) * 0.3
    choice = torch.zeros(tokens, top, dtype=torch.int32, device=device)
    weight = torch.zeros(tokens, top, dtype=torch.float32, device=device)
    record("router: scores, choice among groups, weights", tokens * hidden * 2,
           lambda i: kernels.expert_router(choice, weight, hs[i], wr, corr, req, top, groups, keep, 2), "residual sum + RMSNorm")
    n = tokens * top
    offsets = torch.zeros(experts + 1, dtype=torch.int32, device=device)
    perm, inv_ = torch.zeros(n, dtype=torch.int32, device=device), torch.zeros(n, dtype=torch.int32, device=device)
    kernels.expert_route(offsets, perm, inv_, choice, None, None, req, tokens, top, experts, err)
    w_gu, w_dn = bf(experts, 2 * expert_ff, hidden) * 0.02, bf(hidden, experts * expert_ff) * 0.02
    act = torch.empty(n, expert_ff, dtype=torch.bfloat16, device=device)
    y = torch.empty(n, hidden, dtype=torch.float32, device=device)
    for label, kw in (("clamped swish", dict(activation="swish_clamp", params=(2.0, 1.702))), ("like: SiLU", {})):
        us = _loop_time_us(lambda: kernels.expert_gemm(act, hs[0], w_gu, offsets, perm, True, top, True, **kw))
        fl = 2.0 * n * hidden * 2 * expert_ff
        out.append({"kernel": f"experts, grouped gate/up product with the gate (mma.sync), {label}", "rows": n, "us": round(us, 1),
                    "tensor_tflops": round(fl / us / 1e6, 1), "frac_of_floor": round(fl / us / 1e6 / (peak_tflops or 1590.0), 3)})
    ys = [torch.randn(n, hidden, device=device) for _ in range(sets)]
    outs = [torch.empty(tokens, hidden, device=device) for _ in range(sets)]
    bases = [torch.randn(tokens, hidden, device=device) for _ in range(sets)]
    record("experts, weighted sum of a token's experts onto the shared expert's result", tokens * hidden * 4 * (top + 2),
           lambda i: kernels.expert_combine(outs[i], ys[i], inv_, top, weights=weight, base=bases[i]), "residual sum + RMSNorm")
    for rec in prefill_elementwise(tokens, hidden=hidden, heads=H, kv_heads=G, head_dim=d, intermediate=intermediate,
                                   page_size=page_size, hbm_gbs=hbm_gbs):
        out.append({"kernel": "like: Qwen3 " + rec["kernel"], "tokens": tokens, "us": rec["us"], "gbs": rec["gbs"],
                    "frac_of_floor": rec.get("frac_of_hbm")})
    if int(err):
        raise RuntimeError("a kernel reported an error: " + kernels.describe_error(int(err)))
    return out
