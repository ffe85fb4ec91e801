"""The Mikutar configuration reader, its plan and the plain implementation's pieces at hand-computed points (CPU)."""
import copy
import math

import pytest
import torch

import plain_mikutar as plain
from mikutar_models import TINY_M
from xinfer_b200.config import ConfigError, config_from_dict
from xinfer_b200.config.mikutar import GROUP_BEST, SLOPE_EXPONENT, SWISH_ALPHA, MikutarConfig
from xinfer_b200.models.decoder import model_weight_specs

F64 = torch.float64


def _plan(cfg):
    entry, c = config_from_dict(cfg)
    assert isinstance(c, MikutarConfig)
    return entry.plan_of(c)


@pytest.mark.parametrize("name", sorted(TINY_M))
def test_every_key_reaches_a_spec(name):
    cfg = TINY_M[name][0]
    plan = _plan(cfg)
    assert plan.vocab_size == cfg["vocab"] and plan.hidden == cfg["width"] and plan.head_name is None
    assert plan.residual_dtype == "float32" and plan.logit_softcap == cfg.get("logit_softcap")
    assert [(r.block, r.add_input) for r in plan.runs] == plain.layer_order(cfg)
    for layer, block in zip(cfg["layers"], plan.blocks):
        m, a = layer["mixer"], block.mixer
        assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.scale) == (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"])
        assert a.gate_name == "g" and a.gate_per_head
        assert [o.op for o in block.program][:2] == ["norm", "mixer"] and len(block.norms()) == 1
        assert block.norms()[0].eps == cfg["norm"]["eps"]
        if layer["type"] == "attention":
            assert a.window == m["mask"]["size"] and a.chunk is None and a.value_from_key and a.qk_norm_whole and a.out_bias
            assert a.score_softcap is None and a.distance_slope_exponent is None and a.qk_norm_eps == cfg["norm"]["eps"]
            if m.get("rot"):
                assert (a.rope.rotary_dim, a.rope.theta, a.rope.layout) == (m["rot"]["dims"], m["rot"]["base"], "interleaved")
            else:
                assert a.rope is None
        else:
            assert a.chunk == m["mask"]["size"] and a.window is None and not a.value_from_key and a.bias_suffix is None
            assert a.score_softcap == m.get("softcap") and a.distance_slope_exponent == SLOPE_EXPONENT and a.rope is None
        f = block.feed_forward
        if layer["mlp"] is None:
            assert f is None
        elif layer["mlp"]["kind"] == "dense":
            assert (f.kind, f.activation, f.intermediate) == ("swiglu", "relu", layer["mlp"]["ff"])
        else:
            r = layer["mlp"]["router"]
            g = r.get("groups") or dict(count=1, keep=1)
            assert (f.experts, f.top, f.groups, f.keep, f.group_best) == (r["experts"], r["top"], g["count"], g["keep"], GROUP_BEST)
            assert f.act_params == (layer["mlp"]["expert"]["limit"], SWISH_ALPHA) and not f.renormalize and f.correction
            sh = layer["mlp"].get("shared")
            assert (f.shared is None) == (sh is None)
            if sh:
                assert (f.shared.intermediate, f.shared.act_params) == (sh["ff"], (sh["limit"], SWISH_ALPHA))


def test_declared_tensors():
    cfg = TINY_M["M1"][0]
    names = {s.name: tuple(s.shape) for s in model_weight_specs(_plan(cfg))}
    assert names["embed"] == (83, 48) and names["final.norm"] == (48,) and "head" not in names
    assert names["l0.mix.q"] == (48, 48) and names["l0.mix.k"] == (24, 48) and "l0.mix.v" not in names
    assert names["l0.mix.q.norm"] == (48,) and names["l0.mix.k.norm"] == (24,) and names["l0.mix.g"] == (4, 48)
    assert names["l0.mix.q.b"] == (48,) and names["l0.mix.k.b"] == (24,) and names["l0.mix.o.b"] == (48,)
    assert names["l1.mix.v"] == (42, 48) and names["l1.mix.o"] == (48, 84) and "l1.mix.q.b" not in names
    assert names["l1.mlp.router"] == (6, 48) and names["l1.mlp.correction"] == (6,) and names["l1.mlp.e5.down"] == (48, 24)
    assert names["l1.mlp.shared.gate"] == (20, 48) and names["l0.mlp.up"] == (56, 48)
    assert not any(n.startswith("l2.mlp") for n in names)


def test_named_errors():
    base = TINY_M["M1"][0]

    def broken(change):
        cfg = copy.deepcopy(base)
        change(cfg)
        return cfg

    cases = [
        (lambda c: c.pop("vocab"), "vocab"),
        (lambda c: c["layers"][0].update(type="attention_3"), "layers[0].type"),
        (lambda c: c["layers"][0]["mixer"].update(vdim=16), "vdim"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
        (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "heads"),
        (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
        (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
        (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "mlp.kind"),
        (lambda c: c["loop"].update(stop=4), "loop"),
        (lambda c: c["norm"].pop("eps"), "norm.eps"),
    ]
    for change, word in cases:
        with pytest.raises(ConfigError) as e:
            config_from_dict(broken(change))
        assert word in str(e.value), (word, str(e.value))


def test_layer_order():
    cfg = dict(layers=[0] * 5, loop=dict(start=1, stop=3, times=3))
    assert plain.layer_order(cfg) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False),
                                      (3, False), (4, False)]
    assert plain.layer_order(dict(layers=[0] * 2)) == [(0, False), (1, False)]


def test_route_by_hand():
    """Four groups of two, two groups kept: the correction moves the choice, the weights stay the plain scores."""
    z = torch.tensor([[2.0, -1.0, 0.5, 0.4, -3.0, 3.0, 0.0, 0.1]], dtype=F64)
    s = torch.sigmoid(z)
    corr = torch.tensor([0.0, 0.0, 0.3, 0.3, 0.0, -0.9, 0.0, 0.0], dtype=F64)
    # choice scores: group sums of the two largest: g0 = s0 + s1, g1 = s2 + s3 + 0.6, g2 = s4 + s5 - 0.9, g3 = s6 + s7
    c = s + corr
    sums = [float(c[0, 2 * g] + c[0, 2 * g + 1]) for g in range(4)]
    kept = sorted(range(4), key=lambda g: -sums[g])[:2]
    assert kept == [1, 0]
    idx, wt = plain.route(z, torch.eye(8, dtype=F64), corr, 3, 4, 2)      # the router's matrix is the identity: h = z
    assert idx.tolist() == [[2, 3, 0]]      # c2 = 0.92, c3 = 0.90, c0 = 0.88; expert 5 (score 0.95) lies in a dropped group
    assert torch.allclose(wt, s[:, [2, 3, 0]])
    # minus infinity, not zero: with negative choice scores everywhere a dropped expert must still lose
    corr2 = torch.full((8,), -5.0, dtype=F64)
    corr2[4:] = -4.0
    idx2, _ = plain.route(z, torch.eye(8, dtype=F64), corr2, 2, 2, 1)
    assert set(idx2[0].tolist()) <= {4, 5, 6, 7}


def test_pieces_by_hand():
    assert plain.window_mask(5, 2).tolist()[3] == [False, False, True, True, False]
    assert plain.chunk_mask(7, 3).tolist()[4] == [False, False, False, True, True, False, False]
    assert plain.chunk_mask(7, 3).tolist()[3] == [False, False, False, True, False, False, False]
    assert torch.allclose(plain.head_slopes(4), torch.tensor([0.25, 0.0625, 0.015625, 0.00390625], dtype=F64))
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=F64)
    y = plain.rotate_neighbours(x, torch.tensor([3]), 2, 10.0)
    assert torch.allclose(y[0, 0], torch.tensor([math.cos(3) - 2 * math.sin(3), 2 * math.cos(3) + math.sin(3), 3.0, 4.0], dtype=F64))
    w = {"p.gate": torch.tensor([[3.0]], dtype=F64), "p.up": torch.tensor([[-4.0]], dtype=F64), "p.down": torch.tensor([[1.0]], dtype=F64)}
    out = plain.clamped_expert(torch.tensor([[1.0]], dtype=F64), w, "p.", 2.0)
    assert math.isclose(float(out), 2.0 / (1 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0))
