"""Tiny Mikutar configurations for the tests (config.json dictionaries) and their random model folders.

They differ from each other in every size and switch: heads and groups (one group, one head per group), key and
value sizes that differ where the design allows it, rotation over part of a head, all of it or none, windows and
chunks shorter and longer than a page and no multiple of it, capped and uncapped scores, dense and routed
feed-forwards and layers without one, routers with one group, with all groups kept, with groups of one expert,
with one expert per token, with and without the expert that every token runs, loops over the first layers, over
layers in the middle, over a single layer, three passes, one pass and none, vocabulary and page size."""
from typing import Dict, List, Sequence

import numpy as np
import torch


def _attn(heads, kv, dim, scale, window, rot):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale, mask=dict(size=window))
    if rot is not None:
        m["rot"] = rot
    return dict(type="attention", mixer=m)


def _attn2(heads, kv, dim, vdim, scale, chunk, softcap):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, mask=dict(size=chunk))
    if softcap is not None:
        m["softcap"] = softcap
    return dict(type="attention_2", mixer=m)


def _dense(layer, ff):
    return dict(layer, mlp=dict(kind="dense", ff=ff))


def _none(layer):
    return dict(layer, mlp=None)


def _moe(layer, ff, limit, experts, top, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    mlp = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=router)
    if shared is not None:
        mlp["shared"] = dict(ff=shared[0], limit=shared[1])
    return dict(layer, mlp=mlp)


# name -> (config, seed, page size)
TINY_M: Dict[str, tuple] = {
    # head sizes no fast kernel takes, key and value sizes that differ, a window shorter than a page
    "M1": (dict(architecture="Mikutar", vocab=83, width=48, norm=dict(eps=1e-5), logit_softcap=9.0,
                loop=dict(start=0, stop=2, times=3), layers=[
        _dense(_attn(4, 2, 12, 0.4, 11, dict(dims=8, base=1000.0)), 56),
        _moe(_attn2(6, 3, 10, 14, 0.35, 19, 20.0), 24, 1.5, 6, 2, groups=(3, 2), shared=(20, 0.8)),
        _none(_attn(2, 1, 24, 0.3, 5, None)),
    ]), 31, 8),
    # head sizes in steps of 16 (the tensor-core kernels), a loop in the middle, all groups kept, one expert per token
    "M2": (dict(architecture="Mikutar", vocab=157, width=64, norm=dict(eps=3e-6), logit_softcap=30.0,
                loop=dict(start=1, stop=3, times=2), layers=[
        _moe(_attn2(4, 4, 16, 16, 0.5, 37, None), 40, 3.0, 4, 1, groups=(2, 2)),
        _dense(_attn(4, 1, 32, 0.25, 50, dict(dims=32, base=50000.0)), 96),
        _moe(_attn2(8, 2, 32, 32, 0.3, 64, 8.0), 32, 2.5, 9, 3, groups=(9, 4), shared=(48, 2.0)),
        _dense(_attn(2, 2, 16, 0.6, 23, dict(dims=4, base=77.0)), 72),
    ]), 32, 16),
    # no loop, no cap on the logits, a router without groups, a chunk of one page, a window of many pages
    "M3": (dict(architecture="Mikutar", vocab=120, width=96, norm=dict(eps=1e-6), layers=[
        _moe(_attn(6, 3, 16, 0.45, 130, dict(dims=16, base=20000.0)), 48, 1.0, 5, 2),
        _dense(_attn2(3, 1, 48, 48, 0.2, 32, 5.0), 128),
        _none(_attn2(6, 6, 16, 16, 0.7, 7, 45.0)),
    ]), 33, 32),
    # a loop over one layer that is also the last, one pass "loop", a width that is no multiple of 8
    "M4": (dict(architecture="Mikutar", vocab=61, width=52, norm=dict(eps=2e-6), logit_softcap=4.0,
                loop=dict(start=1, stop=2, times=4), layers=[
        _dense(_attn2(2, 1, 20, 6, 0.33, 9, 3.0), 36),
        _moe(_attn(5, 5, 8, 0.5, 17, dict(dims=6, base=300.0)), 12, 2.0, 12, 5, groups=(4, 2), shared=(16, 1.2)),
    ]), 34, 16),
}


def sharpen(name: str, t: torch.Tensor):
    """Random N(0, std) weights give nearly flat attention, which would hide a missing key or a wrong edge behind
    the tolerance.  Larger q/k norm weights spread the scores of the normed layers over a few units (the layers
    without a norm get theirs from the folder's wide projections); a wider correction makes the router's choice
    differ from the order of its scores, and router logits of a few units keep the scores off the ends of (0, 1), where
    all experts would tie; a smaller embedding keeps the tied head from repeating the last token."""
    if name.endswith(".q.norm") or name.endswith(".k.norm"):
        return t.float() * 1.7
    if name.endswith(".correction"):
        return t.float() * 3.0
    if name.endswith(".router"):
        # logits of a few units: scores spread over (0, 1) instead of sitting at its ends
        return t.float() * (2.0 / t.shape[1] ** 0.5)
    if name == "embed":
        return t.float() * 0.6
    return None


def make_folder(path: str, name: str, store_dtype=torch.float32, override=None) -> str:
    """config.json and model.safetensors with random weights large enough that every layer matters."""
    from xinfer_b200.weights import write_random_model
    cfg, seed, _ = TINY_M[name]

    def both(n, t):
        if override is not None:
            r = override(n, t)
            if r is not None:
                return r
        return sharpen(n, t)

    return write_random_model(path, cfg, seed, dtype=store_dtype, std=0.12, norm_std=0.2, override=both)


def prompts(name: str, lengths: Sequence[int], seed: int = 0) -> List[List[int]]:
    cfg = TINY_M[name][0]
    rng = np.random.default_rng(900 + seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
