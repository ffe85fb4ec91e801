"""The Gulipel config reader, its plan and the declared tensors (CPU)."""
import copy

import pytest
import torch

import plain_gulipel as plain
from gulipel_models import TINY_G
from xinfer_b200.config import ConfigError, config_from_dict
from xinfer_b200.config.gulipel import GulipelConfig
from xinfer_b200.models.decoder import model_weight_specs
from xinfer_b200.weights.loader import WeightSpec, shape_fits


def _plan(cfg):
    entry, c = config_from_dict(cfg)
    return entry.plan_of(c)


@pytest.mark.parametrize("name", sorted(TINY_G))
def test_every_size_and_constant_reaches_a_spec(name):
    cfg = TINY_G[name][0]
    plan = _plan(cfg)
    assert plan.architecture == "Gulipel" and plan.residual_dtype == "float32"
    assert plan.vocab_size == cfg["vocab"] and plan.hidden == cfg["width"]
    assert plan.embed_scale == cfg["embedding"]["scale"]
    assert plan.logit_softcap == cfg.get("logit_softcap")
    big = cfg["embedding"].get("bigram")
    assert (plan.pair_embedding is None) == (big is None)
    if big:
        p = plan.pair_embedding
        assert (p.buckets, p.mul_prev, p.mul_cur) == (big["buckets"], big["mul_prev"], big["mul_cur"])
    assert (plan.position_table is None) == ("max_positions" not in cfg)
    if "max_positions" in cfg:
        assert plan.max_positions == cfg["max_positions"]
    assert len(plan.blocks) == len(cfg["layers"])
    for i, (b, layer) in enumerate(zip(plan.blocks, cfg["layers"])):
        m, lm = b.mixer, layer["mixer"]
        for n in b.norms():
            assert n.eps == cfg["norm"]["eps"] and n.dim == cfg["width"] and n.weight_offset == 0.0
        if layer["type"] == "parallel":
            assert m.kind == "parallel" and m.left_scale == 0.5 and m.right_scale == 0.5 and m.out_norms is not None
            l, r = m.left, m.right
            assert (l.num_heads, l.num_kv_heads, l.head_dim, l.value_dim, l.scale) == tuple(
                lm["left"][k] for k in ("heads", "kv_heads", "dim", "vdim", "scale"))
            qt = lm["left"].get("q_temp")
            assert l.q_temp == ((qt["coef"], qt["every"]) if qt else None)
            assert l.rope is None and l.window is None and not l.sink and not l.talking_heads and l.gate_name and l.bias_suffix
            assert (r.heads, r.kv_heads, r.head_dim, r.v_head_dim, r.conv) == tuple(
                lm["right"][k] for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
            assert r.decay_rank == lm["right"].get("decay_rank") and r.gate_rank == lm["right"].get("gate_rank")
        else:
            assert m.kind == "selective_state"
            assert (m.heads, m.head_dim, m.state, m.groups, m.conv, m.norm_groups) == tuple(
                lm[k] for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups"))
        ffs = b.ops_of("feed_forward")
        dense = [o for o in ffs if o.spec.kind == "swiglu"]
        assert bool(dense) == (layer["mlp"] is not None)
        if dense:
            assert dense[0].spec.intermediate == layer["mlp"]["ff"] and dense[0].spec.bias_suffix == ".b"
        side = [o for o in ffs if o.spec.kind == "token_side"]
        assert bool(side) == ("token_side" in cfg)
        if side:
            d = cfg["token_side"]["dim"]
            assert (side[0].spec.column, side[0].spec.dim, side[0].spec.columns) == (i * d, d, len(cfg["layers"]) * d)
        gains = [o.gain for o in b.ops_of("add")]
        assert gains[0] == "ls1" and (layer["mlp"] is None or gains[1] == "ls2")


def test_the_two_state_space_names_are_one_mechanism():
    cfg = copy.deepcopy(TINY_G["G1"][0])
    a = _plan(cfg)
    for layer in cfg["layers"]:
        if layer["type"] == "mamba2":
            layer["type"] = "mamba2_2"
    b = _plan(cfg)
    assert [x.mixer for x in a.blocks] == [x.mixer for x in b.blocks]


def test_declared_tensors():
    cfg = TINY_G["G1"][0]
    specs = {s.name: s for s in model_weight_specs(_plan(cfg))}
    W, L, sd = cfg["width"], len(cfg["layers"]), cfg["token_side"]["dim"]
    assert specs["bigram"].shape == (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    assert specs["pos"].shape == (cfg["max_positions"], W)
    assert specs["side.embed"].shape == (cfg["vocab"], L * sd)           # declared by every layer, listed once
    m = cfg["layers"][0]["mixer"]
    inner, bc = m["heads"] * m["vdim"], 2 * m["groups"] * m["state"]
    assert specs["l0.mix.in"].shape == (2 * inner + bc + m["heads"], W)
    assert specs["l0.mix.conv"].shape == (inner + bc, m["conv"]) and specs["l0.mix.conv.b"].shape == (inner + bc,)
    assert specs["l0.mix.norm"].shape == (inner,) and specs["l0.mix.o"].shape == (W, inner)
    r = cfg["layers"][1]["mixer"]["right"]
    assert specs["l1.mix.right.a1"].shape == (r["decay_rank"], W) and specs["l1.mix.right.g2"].shape == (r["heads"] * r["vdim"], r["gate_rank"])
    assert specs["l1.mix.right.dt_bias"].shape == (r["heads"] * r["dim"],) and specs["l1.mix.right.norm"].shape == (r["vdim"],)
    assert specs["l1.mix.left.q.b"].shape == (4 * 16,) and specs["l1.mix.left.g"].shape == (4 * 24, W)
    for n in ("l1.mix.left.out", "l1.mix.right.out", "l1.ls1", "l1.ls2", "l1.side.norm", "l1.norm1b", "l1.norm2b", "final.norm"):
        assert specs[n].shape == (W,), n
    assert "l2.ls2" not in specs and "l2.mlp.gate" not in specs            # a layer without a feed-forward
    assert "l0.side.in" not in specs                                       # the norm that is none has no weight


def test_a_low_rank_size_may_come_from_the_file_alone():
    cfg = TINY_G["G2"][0]                     # its first parallel layer names no ranks
    specs = {s.name: s for s in model_weight_specs(_plan(cfg))}
    a1, a2 = specs["l0.mix.right.a1"], specs["l0.mix.right.a2"]
    assert a1.shape == (-1, cfg["width"]) and a2.shape[1] == -1
    assert shape_fits((24, cfg["width"]), a1.shape) and shape_fits((5, cfg["width"]), a1.shape)
    assert not shape_fits((24, cfg["width"] + 1), a1.shape) and not shape_fits((24,), a1.shape)
    assert a1.concrete_shape() == (a1.param, cfg["width"]) and a1.param > 0
    assert WeightSpec("x", (3, 4)).concrete_shape() == (3, 4)


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), 0, "vocab"), (("norm", "eps"), 0.0, "norm.eps"), (("embedding", "scale"), "big", "embedding.scale"),
    (("embedding", "bigram", "buckets"), 0, "buckets"), (("layers", 0, "type"), "conv", "type"),
    (("layers", 0, "mixer", "groups"), 2, "groups"), (("layers", 0, "mixer", "norm_groups"), 5, "norm_groups"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("layers", 1, "mixer", "right", "conv"), None, "conv"),
    (("layers", 1, "mixer", "left", "q_temp", "every"), 0, "every"), (("layers", 1, "mlp", "kind"), "moe", "kind"),
    (("logit_softcap",), -1.0, "logit_softcap"),
])
def test_named_errors(path, value, word):
    cfg = copy.deepcopy(TINY_G["G1"][0])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        GulipelConfig.from_dict(cfg)
    assert word in str(e.value)


def test_pair_rows_of_the_plain_implementation():
    emb = dict(bigram=dict(buckets=11, mul_prev=5, mul_cur=3))
    assert plain.bigram_rows([4, 9, 0, 9], emb) == [11, (4 * 5 + 9 * 3) % 11, (9 * 5 + 0) % 11, (0 + 27) % 11]


def test_query_temperature_of_the_plain_implementation():
    t = plain.query_temperature(9, dict(coef=0.5, every=4), torch.float64)
    assert torch.allclose(t[:3], torch.ones(3, dtype=torch.float64))           # (p + 1) // 4 == 0 up to p = 2
    import math
    assert torch.allclose(t[3:7], torch.full((4,), 1 + 0.5 * math.log(2.0), dtype=torch.float64))
    assert torch.allclose(t[7:], torch.full((2,), 1 + 0.5 * math.log(3.0), dtype=torch.float64))
