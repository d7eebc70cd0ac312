"""Muzopel on the CPU: reading config.json, the plan it becomes (post-norm layers of convolution, mixer, norm, experts,
depth average), what the parts ask of the cache manager, the checkpoint's tensor names, refusals, and the plain
implementation's pieces against closed forms."""

import json
import math

import pytest
import torch

import plain_muzopel as plain
from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.muzopel_config import MuzopelConfig
from tandem_b200.models.muzopel import build_plan, random_weights, tensor_shapes
from tandem_b200.registry import part, resolve_architecture

CFG = dict(
    architecture="Muzopel", vocab=211, width=60, norm=dict(eps=1e-4, groups=5), canon=dict(taps=4), logit_softcap=9.0,
    layers=[
        dict(type="latent_attention_2", mixer=dict(heads=5, dim=6, rot_dim=4, vdim=8, kv_rank=14, scale=0.3, rot=dict(dims=4, base=300.0)),
             mlp=dict(kind="moe", expert=dict(ff=22), router=dict(experts=3, identity=2, top=2))),
        dict(type="latent_attention", mixer=dict(heads=2, dim=10, rot_dim=8, vdim=6, kv_rank=18, q_rank=26, scale=0.25,
                                                 rot=dict(dims=8, base=5e3, scaling=dict(factor=6.0, original=64, fast=16.0, slow=2.0))),
             mlp=None),
        dict(type="latent_attention", mixer=dict(heads=3, dim=4, rot_dim=2, vdim=4, kv_rank=6, q_rank=5, scale=1.0, rot=dict(dims=2, base=10.0)),
             mlp=dict(kind="moe", expert=dict(ff=7), router=dict(experts=1, identity=0, top=1))),
    ])


def test_the_registry_finds_the_design_and_the_file_round_trips():
    arch = resolve_architecture(CFG)
    assert arch.name == "Muzopel"
    cfg = arch.config_class.from_dict(CFG)
    assert cfg.to_dict() == CFG
    assert MuzopelConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert (cfg.taps, cfg.norm_groups, cfg.logit_softcap) == (4, 5, 9.0)


def test_the_plan_names_parts_not_models():
    plan = build_plan(MuzopelConfig.from_dict(CFG))
    assert [layer.block for layer in plan.layers] == ["postnorm"] * 3
    assert [layer.slot("mixer").kind for layer in plan.layers] == ["latent_attention"] * 3
    assert [name for name, _, _ in plan.layers[1].parts] == ["mixer_conv", "mixer", "mixer_norm", "average"]
    first, second, third = (layer.slot("mixer") for layer in plan.layers)
    assert (first.query_latent_dim, first.gate, first.rotary_scaling, first.rotary_pairing) == (0, "none", None, "interleaved")
    assert (second.query_latent_dim, second.gate, second.latent_dim, second.value_dim) == (26, "sigmoid_head", 18, 6)
    assert (second.rotary_scaling.factor, second.rotary_scaling.original) == (6.0, 64) and third.rotary_scaling is None
    routed = plan.layers[0].slot("feed_forward")
    assert (routed.kind, routed.num_experts, routed.identity_experts, routed.top_k) == ("routed_mlp", 3, 2, 2)
    assert (routed.score, routed.normalize, routed.gated, routed.activation, routed.choice_bias) == ("softmax", False, False, "gelu", "correction")
    norm, conv, average = plan.layers[2].slot("feed_forward_norm"), plan.layers[2].slot("feed_forward_conv"), plan.layers[2].slot("average")
    assert (norm.kind, norm.groups, norm.eps) == ("group_rmsnorm", 5, 1e-4) and (conv.kind, conv.taps, conv.weight) == ("short_convolution", 4, "l2.canon2")
    assert (average.count, average.total, average.weight) == (4, 4, "l2.dwa")
    assert plan.head.softcap == 9.0 and plan.embedding.norm.weight == "embed.norm" and [run.layer for run in plan.order] == [0, 1, 2]


def test_what_the_parts_ask_of_the_cache_manager():
    plan = build_plan(MuzopelConfig.from_dict(CFG))
    latent = plan.layers[1].slot("mixer")
    need = part("mixer", latent.kind).kv_need(latent)
    assert (need.num_kv_heads, need.head_dim, need.value_dim, need.window) == (1, 18 + 8, 18, None)
    conv = plan.layers[1].slot("mixer_conv")
    state = part("mixer", conv.kind).state_need(conv)
    assert state.shape == (3, 60) and state.dtype == torch.float32  # the last taps - 1 inputs of the sublayer
    one = MuzopelConfig.from_dict(dict(CFG, canon=dict(taps=1)))
    conv = build_plan(one).layers[0].slot("mixer_conv")
    assert part("mixer", conv.kind).state_need(conv) is None


def test_tensor_names_and_shapes():
    cfg = MuzopelConfig.from_dict(CFG)
    shapes = tensor_shapes(cfg)
    assert shapes["l0.mix.q"] == (5 * 10, 60) and "l0.mix.dq" not in shapes and "l0.mix.g" not in shapes
    assert shapes["l1.mix.dq"] == (26, 60) and shapes["l1.mix.uq"] == (2 * 18, 26) and shapes["l1.mix.g"] == (2, 60)
    assert shapes["l1.mix.dkv"] == (18 + 8, 60) and shapes["l1.mix.uk"] == (20, 18) and shapes["l1.mix.uv"] == (12, 18) and shapes["l1.mix.o"] == (60, 12)
    assert shapes["l0.mlp.router"] == (5, 60) and shapes["l0.mlp.correction"] == (5,) and "l0.mlp.e3.up" not in shapes
    assert shapes["l0.mlp.e2.down"] == (60, 22) and "l1.norm2" not in shapes and "l1.canon2" not in shapes
    assert shapes["l2.canon1"] == (60, 4) and [shapes[f"l{i}.dwa"] for i in range(3)] == [(2,), (3,), (4,)]
    assert {name: tuple(t.shape) for name, t in random_weights(cfg, 1)} == {k: tuple(v) for k, v in shapes.items()}
    plan = build_plan(cfg)
    wanted = set()
    for layer in plan.layers:
        for _, family, spec in layer.parts:
            for ps in part(family, spec.kind).params(spec).values():
                wanted.update(src.name for src in ps.sources)
    assert wanted | {"embed", "embed.norm", "final.norm", "head"} == set(shapes)


def _layer(**changes):
    layer = json.loads(json.dumps(CFG["layers"][1]))
    for key, value in changes.items():
        where = layer
        *path, leaf = key.split("__")
        for p in path:
            where = where[p]
        where[leaf] = value
    return layer


@pytest.mark.parametrize("bad, match", [
    (dict(layers=[dict(type="mamba2", mixer={}, mlp=None)]), "mamba2"),
    (dict(layers=[]), "layers"),
    (dict(norm=dict(eps=1e-5, groups=7)), "groups"),
    (dict(width=None), "width"),
    (dict(logit_softcap=-1.0), "logit_softcap"),
    (dict(layers=[_layer(mixer__rot__dims=10)]), "rot"),
    (dict(layers=[_layer(mlp=dict(kind="moe", expert=dict(ff=8), router=dict(experts=2, identity=1, top=4)))]), "top"),
    (dict(layers=[_layer(mlp=dict(kind="dense", ff=8))]), "dense"),
])
def test_what_the_engine_does_not_have_is_refused(bad, match):
    with pytest.raises(ConfigError, match=match):
        MuzopelConfig.from_dict(dict(CFG, **bad))


def test_the_plain_norm_and_convolution_against_closed_forms():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0, 1.0, 1.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 1.0, 1.0, 3.0], dtype=torch.float64)
    got = plain.group_norm(x, w, 3, 0.0 + 1e-12)
    r = math.sqrt(12.5)
    assert torch.allclose(got, torch.tensor([[3 / r, 8 / r, 0.0, 0.0, 1.0, 3.0]], dtype=torch.float64), atol=1e-6)
    assert torch.allclose(plain.group_norm(x, w, 1, 0.0), x * w / math.sqrt(27.0 / 6.0))
    u = torch.arange(1.0, 6.0, dtype=torch.float64).view(5, 1).repeat(1, 2)  # 1..5 on two channels
    taps = torch.tensor([[0.5, 0.0, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)  # oldest tap first
    want = torch.tensor([[1 + 2.0, 1.0], [2 + 4.0, 2 + 1.0], [3 + 6 + 0.5, 3 + 2.0], [4 + 8 + 1.0, 4 + 3.0], [5 + 10 + 1.5, 5 + 4.0]],
                        dtype=torch.float64)
    assert torch.allclose(plain.short_convolution(u, taps), want)


def test_the_plain_frequencies_and_rotation():
    rot = dict(dims=4, base=100.0)
    freq, mult = plain.rotary_frequencies(rot)
    assert torch.allclose(torch.as_tensor(freq, dtype=torch.float64), torch.tensor([1.0, 0.1], dtype=torch.float64)) and mult == 1.0
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 7.0]]], dtype=torch.float64)  # one head, one token, four rotated dims and one more
    out = plain.rotate_pairs(x, torch.tensor([5]), rot)
    a, b = 5.0, 0.5
    want = torch.tensor([[[math.cos(a), math.sin(a), -2 * math.sin(b), 2 * math.cos(b), 7.0]]], dtype=torch.float64)
    assert torch.allclose(out, want, atol=1e-9)
    stretched = dict(dims=8, base=1e4, scaling=dict(factor=4.0, original=32, fast=8.0, slow=1.0))
    freq, mult = plain.rotary_frequencies(stretched)
    base = [1e4 ** (-2 * i / 8) for i in range(4)]
    assert abs(mult - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    assert abs(float(freq[0]) - base[0]) < 1e-12 and abs(float(freq[3]) - base[3] / 4.0) < 1e-12  # fast pairs keep, slow pairs stretch
    assert all(base[i] / 4.0 - 1e-12 <= float(freq[i]) <= base[i] + 1e-12 for i in range(4))


def test_the_plain_router_chooses_with_the_bias_and_weighs_without():
    torch.manual_seed(0)
    width = 6
    w = {"l0.mlp.router": torch.zeros(4, width, dtype=torch.float64), "l0.mlp.correction": torch.tensor([0.0, 0.0, 0.9, 0.0], dtype=torch.float64)}
    w["l0.mlp.router"][:, 0] = torch.tensor([2.0, 1.0, 0.0, -1.0], dtype=torch.float64)
    h = torch.zeros(1, width, dtype=torch.float64)
    h[0, 0] = 1.0
    ids, weights = plain.route(h, w, "l0.mlp", dict(experts=3, identity=1, top=2))
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0], dtype=torch.float64), 0)
    assert sorted(ids[0].tolist()) == [0, 2]  # the bias lifts expert 2 over expert 1
    got = {int(e): float(v) for e, v in zip(ids[0], weights[0])}
    assert abs(got[0] - float(s[0])) < 1e-12 and abs(got[2] - float(s[2])) < 1e-12  # the weights are the plain scores
