"""Zolapel without a GPU: configuration and refusals, the plan (runs, caches, entries of the loop,
tensor names, constants reaching their parts), and the plain implementation's own mechanisms on
hand-made cases."""
import copy
import math

import numpy as np
import pytest

import plain_zolapel as plain
import tiny_zolapel as tz
from ginfer_b200.config.model_config import ConfigError
from ginfer_b200.config.registry import resolve_architecture
from ginfer_b200.parts.model import DecoderModel


def build(cfg):
    arch = resolve_architecture(cfg)
    return arch, arch.config_cls.from_dict(cfg)


def test_registry_and_round_trip():
    arch, cfg = build(tz.MIXED)
    assert arch.name == "Zolapel"
    again = arch.config_cls.from_dict(cfg.to_dict())
    assert again == cfg and again.loop == (1, 3, 2) and again.side_dim == 6


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0]["mixer"].update(vdim=7), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=13), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "even"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "chooses"),
    (lambda c: c.update(loop={"start": 2, "stop": 2, "times": 2}), "loop"),
    (lambda c: c.update(loop={"start": 0, "stop": 9, "times": 2}), "loop"),
    (lambda c: c["layers"][0].update(type="conv"), "known mixers"),
    (lambda c: c.pop("width"), "width"),
])
def test_refusals(change, text):
    c = copy.deepcopy(tz.MIXED)
    change(c)
    with pytest.raises(ConfigError, match=text):
        build(c)


def test_plan_runs_caches_and_entries():
    arch, cfg = build(tz.MIXED)
    plan = arch.build_plan(cfg)
    # layers 1, 2 twice: 0 | 1 2 | 1 2 | 3; every run a cache of its own; a pass starts at layer 1
    assert [e.layer for e in plan.run] == [0, 1, 2, 1, 2, 3]
    assert [e.cache for e in plan.run] == list(range(6))
    assert [e.enter for e in plan.run] == [None, (0, 0), None, (0, 1), None, None]
    model = DecoderModel(plan)
    specs = model.cache_specs()
    assert specs[1].window == 21 and specs[3].window == 21 and specs[5].window == 18
    assert (specs[2].num_kv_heads, specs[2].head_dim) == (2, 16)
    names = {s.name: s.shape for s in model.tensor_specs()}
    assert names["side.embed"] == (211, 4 * 6) and names["loop.step"] == (2, 48)
    assert names["l2.mix.q"] == (96, 48) and names["l2.mix.k"] == (32, 48)
    assert names["l2.mix.g"] == (6, 48) and names["l2.mix.q.norm"] == (16,)
    assert names["l2.mlp.e6.up"] == (24, 48) and names["l2.mlp.router"] == (7, 48)
    assert "l1.mlp.router" not in names and "l1.norm2" not in names and "l1.ls2" not in names
    assert names["l3.side.gate"] == (6, 48) and names["final.norm.b"] == (48,)
    assert not any(n.startswith("head") or n.endswith(".v") for n in names)
    # no loop, no side input: no such tensors
    plain_cfg = copy.deepcopy(tz.ATTENTION_ONLY)
    a2, c2 = build(plain_cfg)
    n2 = {s.name for s in DecoderModel(a2.build_plan(c2)).tensor_specs()}
    assert "loop.step" not in n2 and "side.embed" not in n2 and "l0.side.gate" not in n2


def test_constants_reach_their_parts():
    arch, cfg = build(tz.MIXED)
    model = DecoderModel(arch.build_plan(cfg))
    b0, b2 = model.blocks[0], model.blocks[2]
    assert b0.mult == 0.6 and b0.mixer.scale == 0.7 and b0.mixer.window == 37
    assert b0.mixer.position.dims == 16 and b0.mixer.position.scaling["factor"] == 3.0
    assert b2.mixer.position.scaling is None and b2.mixer.hd == 16
    assert b0.mixer.eps == 2e-5 and b0.mixer_norm.eps == 2e-5 and b0.after.eps == 2e-5
    assert (b2.after.offset, b2.after.dim, b2.after.total) == (12, 6, 24)
    assert (b2.feed_forward.E, b2.feed_forward.top) == (7, 3)
    assert b2.feed_forward.score == "sigmoid" and b2.feed_forward.weight_on == "input"


def test_engine_frequencies_equal_the_plain_ones():
    from ginfer_b200.parts.position import PairRotary
    for dims, base, sc in ((16, 1000.0, {"factor": 3.0, "low": 1.0, "high": 6.0, "original": 200}),
                           (8, 50.0, None), (40, 1e6, {"factor": 8, "low": 2, "high": 5,
                                                      "original": 4096})):
        got = PairRotary(dims, base, sc).host_frequencies()
        want = plain.rotary_frequencies(dims, base, sc)
        assert np.array_equal(got.astype(np.float64), want)
    sc = {"factor": 3.0, "low": 1.0, "high": 6.0, "original": 200}
    f0 = plain.rotary_frequencies(16, 1000.0, None)
    f1 = plain.rotary_frequencies(16, 1000.0, sc)
    wave = 2 * math.pi / f0
    kinds = [("kept" if w < 200 / 6 else "divided" if w > 200 else "blend") for w in wave]
    assert {"kept", "divided", "blend"} <= set(kinds)          # the case has all three ranges
    for k, a, b in zip(kinds, f0, f1):
        if k == "kept":
            assert a == b
        elif k == "divided":
            assert abs(b - a / 3.0) < 1e-9
        else:
            assert a / 3.0 < b < a


# ----------------------------------------------------------------------------- the oracle itself
def test_plain_pair_rotation_and_window():
    x = np.zeros((3, 1, 6))
    x[:, 0, 0] = 1.0           # pair (0, 1) holds (1, 0)
    x[:, 0, 4] = 2.0           # channel 4 is not rotated (two pairs only)
    f = np.array([0.5, 0.25])
    y = plain.rotate_pairs(x, np.arange(3), f)
    for p in range(3):
        assert np.allclose(y[p, 0, :2], [math.cos(0.5 * p), math.sin(0.5 * p)], atol=1e-7)
        assert y[p, 0, 4] == 2.0
    see = plain.visible(5, 2)
    assert see.tolist() == [[j in (i, i - 1) and j >= 0 for j in range(5)] for i in range(5)]
    assert plain.visible(3, 0).tolist() == [[j <= i for j in range(3)] for i in range(3)]


def test_plain_router_and_expert_weight_on_the_input():
    h = np.array([[1.0, 0.0], [0.0, 2.0]])
    w_r = np.array([[3.0, 0.0], [0.0, 1.0], [3.0, 0.0]])     # experts 0 and 2 tie on token 0
    idx, w = plain.router(h, w_r, 2)
    assert idx[0].tolist() == [0, 2] and np.allclose(w[0], 1 / (1 + math.exp(-3.0)))
    assert idx[1].tolist() == [1, 0] and np.allclose(w[1], [1 / (1 + math.exp(-2.0)), 0.5])
    assert not np.allclose(w.sum(-1), 1.0)                    # the scores are not renormalised
    up, down = np.array([[1.0, -1.0]]), np.array([[2.0], [1.0]])
    t = {"router": np.array([[10.0, 0.0]]), "e0.up": up, "e0.down": down}
    out = plain.routed_ff(np.array([[3.0, 1.0]]), t, {"router": {"experts": 1, "top": 1}})
    s = 1 / (1 + math.exp(-30.0))
    assert np.allclose(out, [[2 * (2 * s) ** 2, (2 * s) ** 2]])     # relu(up . (s h))^2, then down
    assert np.allclose(plain.expert(np.array([[1.0, 3.0]]), up, down), 0.0)   # relu cuts


def test_plain_values_are_the_unrotated_keys_and_the_gate_closes_a_head():
    W, D = 4, 2
    t = {"q": np.eye(2, 4), "k": np.eye(2, 4)[::-1].copy(), "q.norm": np.ones(D),
         "k.norm": np.ones(D), "g": np.array([[-100.0, 0, 0, 0]]), "o": np.eye(4, 2)}
    m = {"heads": 1, "kv_heads": 1, "dim": D, "scale": 1.0, "rot": {"base": 10.0, "dims": 2}}
    h = np.array([[0.0, 1.0, 0.0, 0.0], [0.0, 0.0, 5.0, 0.0]])
    out = plain.attention(h, t, m, 1e-6)
    # token 0 sees itself only: its value is its key as projected, (1, 0), whatever the rotation;
    # the gate's input is 0 here, so the head passes half of it
    assert np.allclose(out[0], [0.5, 0.0, 0.0, 0.0])
    h[0, 0] = 1.0                                       # the gate's input: sigmoid(-100) closes it
    assert np.allclose(plain.attention(h, t, m, 1e-6)[0], 0.0)


def test_plain_loop_adds_the_embedding_again_and_a_vector_per_pass():
    cfg = copy.deepcopy(tz.LOOPED)
    assert plain.run_order(cfg) == [(0, 0, True), (0, 1, True), (0, 2, True)]
    cfg2 = copy.deepcopy(tz.MIXED)
    assert [(i, t) for i, t, first in plain.run_order(cfg2) if first] == [(1, 0), (1, 1)]
