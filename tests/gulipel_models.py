"""Tiny Gulipel configurations for the tests (config.json dictionaries) and their random model folders.

They differ from each other in every size and switch: the order of layer types (parallel first, last, twice in a
row, absent), heads and groups of one, two and all heads on both sides of a parallel layer, key and value head
sizes that differ or agree, state sizes and channel counts that are no power of two, convolutions of two to five
taps, norm parts of one to three, low-rank sizes that differ between the two maps, query temperature present or
absent and with periods of 1 to 50 tokens, pair table and position table and per-layer token input present or
absent, layers without a feed-forward, soft cap present or absent, vocabulary, eps and page size."""
from typing import Dict, List, Sequence

import numpy as np
import torch


def _ssm(heads, vdim, state, groups, conv, parts, ff, kind="mamba2"):
    return dict(type=kind, mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=parts),
                mlp=dict(kind="dense", ff=ff) if ff else None)


def _par(left, right, ff):
    return dict(type="parallel", mixer=dict(left=left, right=right), mlp=dict(kind="dense", ff=ff) if ff else None)


def _left(heads, kv, dim, vdim, scale, q_temp=None):
    out = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if q_temp:
        out["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    return out


def _right(heads, kv, dim, vdim, conv, ra=None, rg=None):
    out = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv)
    if ra:
        out["decay_rank"] = ra
    if rg:
        out["gate_rank"] = rg
    return out


# name -> (config, seed, page size)
TINY_G: Dict[str, tuple] = {
    "G1": (dict(architecture="Gulipel", vocab=97, width=48, norm=dict(eps=1e-5), max_positions=512, logit_softcap=20.0,
                embedding=dict(scale=4.0, bigram=dict(buckets=53, mul_prev=31, mul_cur=7)), token_side=dict(dim=6),
                layers=[_ssm(3, 8, 5, 1, 4, 1, 56),
                        _par(_left(4, 2, 16, 24, 0.6, (0.4, 7)), _right(4, 2, 16, 8, 3, 5, 9), 40),
                        _ssm(4, 12, 24, 2, 2, 2, None, "mamba2_2")]), 21, 8),
    "G2": (dict(architecture="Gulipel", vocab=211, width=80, norm=dict(eps=3e-6), max_positions=400,
                embedding=dict(scale=9.0, bigram=dict(buckets=101, mul_prev=3, mul_cur=1000003)), token_side=dict(dim=20),
                layers=[_par(_left(6, 2, 32, 32, 0.35, (0.25, 50)), _right(6, 6, 24, 16, 4), 136),
                        _par(_left(2, 1, 16, 40, 0.7, (1.5, 1)), _right(2, 1, 40, 20, 2, 12, 3), None),
                        _ssm(6, 16, 16, 3, 5, 3, 72)]), 22, 16),
    # nothing optional: no pair table, no position table, no token input, no soft cap, no query temperature
    "G3": (dict(architecture="Gulipel", vocab=150, width=64, norm=dict(eps=1e-6), embedding=dict(scale=1.0),
                layers=[_ssm(8, 8, 8, 8, 3, 1, 100),
                        _par(_left(8, 8, 8, 8, 0.9), _right(1, 1, 64, 48, 3), 64),
                        _ssm(2, 32, 40, 1, 4, 2, 64, "mamba2_2"),
                        _par(_left(1, 1, 64, 16, 0.3, (0.1, 16)), _right(8, 2, 8, 8, 5, 4, 4), None)]), 23, 32),
    # sizes that fit no fast path: a width that is no multiple of 8, odd head sizes and feed-forward widths; no
    # parallel layer at all (nothing is paged)
    "G4": (dict(architecture="Gulipel", vocab=61, width=52, norm=dict(eps=2e-6), max_positions=300, logit_softcap=5.0,
                embedding=dict(scale=2.5, bigram=dict(buckets=7, mul_prev=1, mul_cur=1)), token_side=dict(dim=3),
                layers=[_ssm(5, 7, 9, 5, 3, 5, 50), _ssm(2, 18, 33, 2, 4, 3, None)]), 24, 16),
}


def sharpen(name: str, t: torch.Tensor):
    """Random weights would give a state-space layer step sizes near softplus(0) and decays near 1/2 everywhere;
    spreading dt_bias and A_log makes some heads remember for hundreds of tokens and others for one."""
    if name.endswith("A_log"):
        return t.float() * 8.0 - 1.0
    if name.endswith("dt_bias"):
        return t.float() * 1.5 - 1.0
    if name.endswith(".q.norm") or name.endswith(".k.norm"):
        return t.float() * 1.6
    return None


def make_folder(path: str, name: str, store_dtype=torch.float32) -> str:
    """config.json and model.safetensors with random weights large enough that every layer matters."""
    from xinfer_b200.weights import write_random_model
    cfg, seed, _ = TINY_G[name]
    return write_random_model(path, cfg, seed, dtype=store_dtype, std=0.08, norm_std=0.2, override=sharpen)


def prompts(name: str, lengths: Sequence[int], seed: int = 0) -> List[List[int]]:
    cfg = TINY_G[name][0]
    rng = np.random.default_rng(700 + seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
