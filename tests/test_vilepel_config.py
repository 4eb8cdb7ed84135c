"""Vilepel without a GPU: configuration, the plan (run list, shared weights), tensor names, and
the plain implementation's own mechanisms on hand-made cases."""
import copy

import pytest
import torch

import plain_vilepel as plain
import tiny_vilepel as tv
from ginfer_b200.config import ConfigError, resolve_architecture
from ginfer_b200.parts.base import PagedKVSpec, StateSpec
from ginfer_b200.parts.model import DecoderModel


def build(cfg):
    arch = resolve_architecture(cfg)
    return arch, arch.config_cls.from_dict(cfg)


def test_registry_reads_the_single_architecture_key():
    arch, cfg = build(tv.MIXED)
    assert arch.name == "Vilepel" and cfg.width == 48 and len(cfg.layers) == 6
    assert cfg.to_dict()["layers"][2]["weights_of"] == 0
    assert build(cfg.to_dict())[1] == cfg


def test_shared_weights_become_second_runs_with_caches_of_their_own():
    arch, cfg = build(tv.MIXED)
    plan = arch.build_plan(cfg)
    assert [ls.prefix for ls in plan.layers] == ["l0", "l1", "l3", "l4"]
    assert [(e.layer, e.cache) for e in plan.run] == [(0, 0), (1, 1), (0, 2), (2, 3), (3, 4), (1, 5)]
    model = DecoderModel(plan)
    specs = model.cache_specs()
    assert isinstance(specs[0], PagedKVSpec) and specs[0] == specs[2]
    assert specs[0].planes == ((1, 40), (1, 8)) and specs[0].window == 37
    assert isinstance(specs[1], StateSpec) and specs[1] == specs[5]
    assert specs[1].shape == (4 * 16 * 12 + 2 * (2 * 2 * 16 + 4 * 12),)
    names = {s.name for s in model.tensor_specs()}
    assert "l2.mix.q" not in names and "l5.mix.q" not in names
    assert {"embed", "head", "final.norm", "l0.mix.dkv.norm", "l1.mlp.e4.down", "l1.mlp.router",
            "l1.mix.q.conv", "l1.mix.A_log", "l3.norm1"} <= names
    assert "l3.norm2" not in names and not any(n.startswith("l3.mlp") for n in names)


def test_every_constant_reaches_the_parts():
    arch, cfg = build(tv.OTHER)
    plan = arch.build_plan(cfg)
    d, a = plan.layers[0], plan.layers[1]
    assert d.mixer.params["conv_taps"] == 5 and d.mixer.params["num_kv_heads"] == 1
    assert d.feed_forward.params["top_k"] == 4 and d.feed_forward.params["limit"] == 0.8
    assert a.mixer.params["window"] == 64 and a.mixer.params["rotary_base"] == 1000.0
    assert a.mixer.params["latent_eps"] == 1e-6 and plan.embedding.params["scale"] == 3.0
    assert a.mixer_norm.params["weight_offset"] == 1.0 and a.mixer_norm.params["eps"] == 1e-6


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].__setitem__("type", "attention"), "known mixers"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 1), "uses the weights"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 9), "names no layer"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "chooses 6 of 5"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even number"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(edit, text):
    c = copy.deepcopy(tv.MIXED)
    edit(c)
    with pytest.raises(ConfigError, match=text):
        build(c)


# ----------------------------------------------------------------------------- the oracle itself
def test_plain_rotation_pairs_neighbours_and_keeps_the_rest():
    x = torch.arange(12, dtype=torch.float64).reshape(1, 12) + 1
    y = plain.rotate_pairs(x, torch.tensor([3]), 100.0, 4)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert torch.allclose(y[0, 0], x[0, 0] * torch.cos(torch.tensor(a0)) - x[0, 1] * torch.sin(torch.tensor(a0)))
    assert torch.allclose(y[0, 3], x[0, 3] * torch.cos(torch.tensor(a1)) + x[0, 2] * torch.sin(torch.tensor(a1)))
    assert torch.equal(y[0, 4:], x[0, 4:])
    assert torch.equal(plain.rotate_pairs(x, torch.tensor([0]), 100.0, 4), x)


def test_plain_convolution_is_causal_with_the_current_token_last():
    x = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=torch.float64)
    pre = torch.tensor([[1.0], [12.0], [123.0]], dtype=torch.float64)
    assert torch.allclose(plain.short_conv_silu(x, w), pre * torch.sigmoid(pre))


def test_plain_window_and_delta_rule_on_hand_made_cases():
    # a window of 2 sees itself and one token back: the first token's value never reaches token 2
    m = tv.latent(heads=1, dim=2, rot_dim=2, vdim=2, kv_rank=2, window=2)["mixer"]
    W = {"mix.q": torch.zeros(4, 3, dtype=torch.float64), "mix.dkv": torch.zeros(4, 3, dtype=torch.float64),
         "mix.dkv.norm": torch.ones(2, dtype=torch.float64), "mix.uk": torch.zeros(2, 2, dtype=torch.float64),
         "mix.uv": torch.eye(2, dtype=torch.float64), "mix.o": torch.eye(3, 2, dtype=torch.float64)}
    W["mix.dkv"][0, 0] = W["mix.dkv"][1, 1] = 1.0
    h = torch.tensor([[5.0, 0, 0], [0, 1.0, 0], [0, 1.0, 0]], dtype=torch.float64)
    out = plain.latent_attention(h, W, m, 1e-12)
    c = plain.unit_rms(h[:, :2], 1e-12)
    assert torch.allclose(out[2, :2], c[1:3].mean(0)) and torch.allclose(out[1, :2], c[0:2].mean(0))
    # delta rule, one head, no decay (g = 1), beta = 1: the state stores v under k and a second
    # write under the same key replaces it
    S = torch.zeros(2, 1, dtype=torch.float64)
    k = torch.tensor([1.0, 0.0], dtype=torch.float64)
    for v in (3.0, 7.0):
        u = 1.0 * (torch.tensor([v], dtype=torch.float64) - S.T @ k)
        S = S + torch.outer(k, u)
    assert torch.allclose(S.T @ k, torch.tensor([7.0], dtype=torch.float64))


def test_plain_router_weights_are_not_renormalised():
    m = tv.moe(experts=3, top=2, ff=2, limit=10.0)
    W = {"mlp.router": torch.tensor([[2.0], [1.0], [0.0]], dtype=torch.float64)}
    for e in range(3):
        W[f"mlp.e{e}.gate"] = torch.full((2, 1), 1.0 + e, dtype=torch.float64)
        W[f"mlp.e{e}.up"] = torch.zeros(2, 1, dtype=torch.float64)
        W[f"mlp.e{e}.down"] = torch.ones(1, 2, dtype=torch.float64)
    h = torch.ones(1, 1, dtype=torch.float64)
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=torch.float64), 0)
    act = lambda g: g * torch.sigmoid(torch.tensor(1.702 * g, dtype=torch.float64))
    want = s[0] * 2 * act(1.0) + s[1] * 2 * act(2.0)
    assert torch.allclose(plain.routed_ff(h, W, m)[0, 0], want)
