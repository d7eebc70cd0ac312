"""Deletar without a GPU: the configuration file's round trip, the plan it becomes, what its parts ask of the cache
manager, tensor names, refusals, and the plain implementation's pieces against closed forms."""

import json
import math

import pytest
import torch

import plain_deletar as plain
from tandem_b200.config.deletar_config import DeletarConfig
from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import RotaryBandSpec, rotary_band_table
from tandem_b200.models.deletar import build_plan, cache_window, random_weights, tensor_shapes
from tandem_b200.registry import part, resolve_architecture


def mixer(**kw):
    m = dict(heads=4, kv_heads=2, dim=8, vdim=8, scale=0.3, rot=dict(dims=4, base=100.0), mask=dict(size=13))
    m.update(kw)
    return m


CONFIG = dict(architecture="Deletar", vocab=97, width=40, norm=dict(eps=1e-5), embedding=dict(scale=3.0), logit_softcap=20.0, layers=[
    dict(type="attention_2", mixer=mixer(softcap=9.0), mlp=dict(kind="dense", ff=24)),
    dict(type="attention_3", mixer=mixer(heads=6, vdim=12, softcap=5.0, mask=dict(size=7),
                                         rot=dict(dims=8, base=50.0, scaling=dict(factor=4.0, low=1.0, high=3.0, original=40))),
         mlp=dict(kind="moe", expert=dict(ff=16), router=dict(experts=5, top=2), shared=dict(ff=8))),
    dict(type="attention", mixer=mixer(conv=3, vdim=20), mlp=None),
    dict(type="attention_3", mixer=mixer(heads=2, vdim=12, softcap=5.0, mask=dict(size=30), kv_from=1,
                                         rot=dict(dims=8, base=50.0, scaling=dict(factor=4.0, low=1.0, high=3.0, original=40))),
         mlp=dict(kind="moe", expert=dict(ff=16), router=dict(experts=3, top=3))),
])


def fresh():
    return json.loads(json.dumps(CONFIG))


def test_the_file_round_trips_and_names_its_architecture():
    arch = resolve_architecture(fresh())
    assert arch.name == "Deletar"
    cfg = arch.config_class.from_dict(fresh())
    assert DeletarConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict() == fresh()
    assert cfg.layers[2].mlp is None and cfg.layers[3].mixer.kv_from == 1 and cfg.layers[1].mlp.shared_ff == 8


def test_the_plan():
    cfg = DeletarConfig.from_dict(fresh())
    plan = build_plan(cfg)
    assert [r.cache_of for r in plan.order] == [None, None, None, 1]
    assert all(l.block == "sandwich" for l in plan.layers)
    a2, a3, a1, borrowed = (l.slot("mixer") for l in plan.layers)
    assert (a2.bias, a2.qk_norm, a2.values, a2.gate, a2.sink, a2.conv_taps) == (True, "whole", "keys", "sigmoid_head", None, 0)
    assert (a3.bias, a3.qk_norm, a3.values, a3.gate, a3.sink, a3.softcap) == (False, "head", "projection", "sigmoid_head", 0.0, 5.0)
    assert (a1.qk_norm, a1.gate, a1.sink, a1.conv_taps, a1.softcap) == ("none", "none", None, 3, None)
    assert borrowed.borrows_kv and not a3.borrows_kv and a3.cache_window == 30 and borrowed.window == 30
    assert a3.rotary_scaling == RotaryBandSpec(4.0, 1.0, 3.0, 40.0) and a2.rotary_scaling is None
    assert plan.layers[2].of_family("feed_forward") == [] and len(plan.layers[2].of_family("norm")) == 2
    ff = plan.layers[1].slot("feed_forward")
    assert (ff.router, ff.top_k, ff.num_experts, ff.shared_intermediate_size, ff.activation, ff.gated) == ("token_table", 2, 5, 8, "relu2", False)
    assert plan.layers[0].slot("feed_forward").activation == "relu2" and not plan.layers[0].slot("feed_forward").bias
    assert plan.layers[0].slot("mixer_norm").offset == 1.0 and plan.final_norm.offset == 1.0
    assert plan.embedding.scale == 3.0 and plan.head.softcap == 20.0


def test_what_the_mixers_ask_of_the_cache_manager():
    cfg = DeletarConfig.from_dict(fresh())
    plan = build_plan(cfg)
    cls = part("mixer", "window_attention")
    needs = [cls.kv_need(l.slot("mixer")) for l in plan.layers]
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].window, needs[0].value_dim) == (2, 8, 13, 8)
    assert needs[1].window == 30  # its own window is 7: the layer that borrows its keys looks 30 back
    assert needs[2].value_dim == 20
    states = [cls.state_need(l.slot("mixer")) for l in plan.layers]
    assert states[0] is None and states[1] is None and tuple(states[2].shape) == (2, 4 * 8 + 2 * 8 + 2 * 20)
    assert cache_window(cfg, 0) is None and cache_window(cfg, 1) == 30
    no_mask = fresh()
    del no_mask["layers"][3]["mixer"]["mask"]
    typed = DeletarConfig.from_dict(no_mask)
    assert cache_window(typed, 1) == 0 and cls.kv_need(build_plan(typed).layers[1].slot("mixer")).window is None


def test_tensor_names_and_the_random_recipe():
    cfg = DeletarConfig.from_dict(fresh())
    shapes = tensor_shapes(cfg)
    assert shapes["l0.mix.q.b"] == (32,) and "l0.mix.v" not in shapes and shapes["l0.mix.k.norm"] == (16,)
    assert shapes["l1.mix.q.norm"] == (8,) and shapes["l1.mix.g"] == (6, 40) and shapes["l1.mlp.table"] == (97, 2)
    assert shapes["l2.mix.v.conv"] == (40, 3) and "l2.norm2" not in shapes and "l2.mix.g" not in shapes
    assert not any(n.startswith(("l3.mix.k", "l3.mix.v")) for n in shapes) and shapes["l3.mix.q.norm"] == (8,)
    made = dict(random_weights(cfg, 1, "cpu", torch.float32))
    assert {n: tuple(t.shape) for n, t in made.items()} == shapes
    table = made["l1.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 5 and bool((table[:, 0] != table[:, 1]).all())
    plan = build_plan(cfg)
    wanted = set()
    for i, layer in enumerate(plan.layers):
        for slot, family, spec in layer.parts:
            for ps in part(family, spec.kind).params(spec).values():
                wanted.update(src.name for src in ps.sources)
    assert wanted | {"embed", "head", "final.norm"} == set(shapes)


@pytest.mark.parametrize("edit,message", [
    (lambda c: c["layers"][0].update(type="attention_4"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=12), "values are its keys"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(dim=16), "other sizes"),
    (lambda c: c["layers"][0]["mixer"].update(kv_from=0), "attention_3"),
    (lambda c: c["layers"][0]["mixer"].update(conv=3), "'attention' only"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "not supported"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
])
def test_refusals(edit, message):
    c = fresh()
    edit(c)
    with pytest.raises(ConfigError, match=message):
        DeletarConfig.from_dict(c)


def test_the_slowed_frequencies():
    """Kept below the short wavelength, divided by the factor above the long one, a blend between; the package's table is
    the plain implementation's."""
    s = dict(factor=8.0, low=1.0, high=4.0, original=512)
    plain_f, slowed = plain.frequencies(16, 2e4), plain.frequencies(16, 2e4, s)
    assert slowed == rotary_band_table(16, 2e4, RotaryBandSpec(8.0, 1.0, 4.0, 512.0))
    for f, g in zip(plain_f, slowed):
        wave = 2 * math.pi / f
        if wave < 128:
            assert g == f
        elif wave > 512:
            assert g == f / 8.0
        else:
            share = (512 / wave - 1.0) / 3.0
            assert abs(g - ((1 - share) * f / 8.0 + share * f)) < 1e-15 and f / 8.0 <= g <= f
    assert any(g == f for f, g in zip(plain_f, slowed)) and any(g == f / 8.0 for f, g in zip(plain_f, slowed))


def test_the_plain_pieces_against_closed_forms():
    x = torch.tensor([[3.0, -4.0]], dtype=torch.float64)
    assert torch.allclose(plain.rms(x, 0.0), x / math.sqrt(12.5))
    assert torch.allclose(plain.norm_one_plus(x, torch.tensor([1.0, 0.0], dtype=torch.float64), 0.0), x / math.sqrt(12.5) * torch.tensor([2.0, 1.0]))
    assert plain.relu_squared(torch.tensor([-2.0, 3.0])).tolist() == [0.0, 9.0]
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    assert plain.causal_convolution(u, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    # a quarter turn a position on the one pair of a head of three numbers; the third passes
    q = torch.tensor([[[1.0, 0.0, 5.0]], [[1.0, 0.0, 5.0]]], dtype=torch.float64)
    turned = plain.rotate(q, [math.pi / 2], 2)
    assert torch.allclose(turned[0, 0], torch.tensor([1.0, 0.0, 5.0], dtype=torch.float64))
    assert torch.allclose(turned[1, 0], torch.tensor([0.0, 1.0, 5.0], dtype=torch.float64), atol=1e-15)
    # equal scores: the window's keys share the weight, with one more share for the sink
    T = 6
    q, k = torch.zeros(T, 2, 4, dtype=torch.float64), torch.randn(T, 1, 4, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64)[:, None, None].expand(T, 1, 3).contiguous()
    o = plain.attend(q, k, v, 1.0, 3, None, sink=False)
    assert torch.allclose(o[:, 0, 0], torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 4.0], dtype=torch.float64))
    o = plain.attend(q, k, v, 1.0, 3, 7.0, sink=True)
    assert torch.allclose(o[:, 1, 0], torch.tensor([0.0, 1 / 3, 3 / 4, 6 / 4, 9 / 4, 12 / 4], dtype=torch.float64))
    # a cap far below the scores makes them equal
    q = torch.full((2, 1, 1), 50.0, dtype=torch.float64)
    k = torch.tensor([[[1.0]], [[3.0]]], dtype=torch.float64)
    v = torch.tensor([[[0.0]], [[1.0]]], dtype=torch.float64)
    assert abs(float(plain.attend(q, k, v, 1.0, None, 1e-3, sink=False)[1, 0, 0]) - 0.5) < 1e-3


def test_a_borrowing_layer_reads_the_owners_keys():
    """In the plain implementation: changing the owner's key projection changes the borrower's output even with the
    owner's own attention output silenced."""
    cfg = DeletarConfig.from_dict(fresh())
    w = dict(random_weights(cfg, 2, "cpu", torch.float32))
    toks = [5, 9, 33, 2, 71, 8]
    base, _ = plain.forward(fresh(), w, toks)
    w2 = dict(w)
    w2["l1.mix.o"] = torch.zeros_like(w["l1.mix.o"])
    silenced, _ = plain.forward(fresh(), w2, toks)
    w3 = dict(w2)
    w3["l1.mix.k"] = w["l1.mix.k"] * 2.0 + 0.1
    changed, _ = plain.forward(fresh(), w3, toks)
    assert (silenced - changed).abs().max() > 1e-6 and (base - silenced).abs().max() > 1e-6
