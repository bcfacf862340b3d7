"""Rabadra without a GPU: its configuration, its model description, its tensors and refusals, and the plain
implementation's own identities (a sink of minus infinity is ordinary softmax; the rotation keeps lengths and depends on
position differences only; the group rule; the clamp)."""

from __future__ import annotations

import copy

import pytest
import torch

import tiny_rabadra as tr
from plain import rabadra_plain as plain
from sleuth_b200.config import ConfigError, parse_config
from sleuth_b200.engine.model import declare_model


def spec_of(cfg):
    arch, typed, unread = parse_config(cfg)
    assert arch.name == "Rabadra" and set(unread) <= {"torch_dtype", "architectures"}
    return arch.model_spec(typed)


def test_every_size_and_constant_comes_from_the_configuration():
    spec = spec_of(tr.A)
    m = spec.layers[0].mixer
    assert (m.heads, m.kv_heads, m.head_dim, m.value_dim, m.scale) == (6, 2, 16, 24, 0.31)
    assert m.qk_norm and m.qk_norm_span == "projection" and m.sinks and m.qk_norm_eps == 1e-6
    assert (m.position.theta, m.position.rotary_dim, m.position.pairing) == (500.0, 8, "neighbours")
    f = spec.layers[0].ffn
    assert (f.experts, f.top, f.intermediate, f.limit, f.route_scale, f.groups, f.keep_groups) == (6, 2, 20, 1.0, 1.5, 3, 2)
    assert f.scoring == "sigmoid" and f.activation == "clamped_swish" and not f.router_bias
    assert (f.shared.intermediate, f.shared.limit, f.shared.activation) == (28, 2.5, "clamped_swish")
    assert spec.head.softcap == 7.5 and spec.head.norm.kind == "layernorm" and spec.embedding.norm.kind == "layernorm"
    assert spec.layers[1].ffn is None and spec.layers[1].norm2 is None and spec.layers[0].norm2.kind == "layernorm"
    b = spec_of(tr.B)
    assert b.head.softcap == 0.0 and b.layers[0].ffn.groups == 1 and b.layers[0].ffn.shared is None
    assert b.layers[1].mixer.position.kind == "none" and b.layers[0].mixer.position.rotary_dim == 32


def test_borrowed_weights_become_a_schedule_with_caches_of_their_own():
    a = spec_of(tr.A)
    assert len(a.layers) == 2 and [(e.layer, e.cache) for e in a.schedule] == [(0, 0), (1, 1), (0, 2)]
    b = spec_of(tr.B)
    assert len(b.layers) == 2 and [(e.layer, e.cache) for e in b.schedule] == [(0, 0), (1, 1), (1, 2), (0, 3)]
    short = copy.deepcopy(tr.A)
    short["layers"][2] = {"weights_of": 0}                               # what a borrower leaves out is the lender's
    assert [(e.layer, e.cache) for e in spec_of(short).schedule] == [(0, 0), (1, 1), (0, 2)]
    chain = copy.deepcopy(tr.A)
    chain["layers"].append(dict(chain["layers"][2], weights_of=2))       # borrows from a borrower
    assert [(e.layer, e.cache) for e in spec_of(chain).schedule] == [(0, 0), (1, 1), (0, 2), (0, 3)]


def test_declared_tensors_carry_the_file_names_and_shapes():
    d = declare_model(spec_of(tr.A))
    assert d["embed"].shape == (301, 72) and d["embed.norm"].shape == (72,) and d["final.norm"].shape == (72,)
    assert d["l0.mix.q"].shape == (96, 72) and d["l0.mix.k"].shape == (32, 72) and d["l0.mix.v"].shape == (48, 72)
    assert d["l0.mix.q.norm"].shape == (96,) and d["l0.mix.k.norm"].shape == (32,) and d["l0.mix.sink"].shape == (6,)
    assert d["l0.mix.o"].shape == (72, 144) and d["l0.mlp.router"].shape == (6, 72)
    assert d["l0.mlp.e5.gate"].shape == (20, 72) and d["l0.mlp.e5.down"].shape == (72, 20)
    assert d["l0.mlp.shared.up"].shape == (28, 72) and d["l0.mlp.shared.down"].shape == (72, 28)
    assert "l1.norm2" not in d and "l1.mlp.router" not in d and "l1.norm1" in d
    assert not any(n.startswith("l2.") for n in d)          # the borrowing layer has no tensors


@pytest.mark.parametrize("edit, words", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "router.top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=6), "cannot give"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not 'moe'"),
    (lambda c: c["layers"][0].update(type="recurrent"), "not a known mixer"),
    (lambda c: c["layers"][2].update(weights_of=2), "names no other layer"),
    (lambda c: c["layers"][2].update(weights_of=1), "differs"),
    (lambda c: c["layers"][0]["mixer"].update(window=5), "unknown key"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_what_the_configuration_refuses(edit, words):
    cfg = copy.deepcopy(tr.A)
    edit(cfg)
    with pytest.raises(ConfigError, match=words):
        spec_of(cfg)


def test_a_key_set_to_null_is_absent_and_an_unknown_one_with_a_value_is_refused():
    cfg = copy.deepcopy(tr.A)
    cfg["layers"][0]["mixer"]["window"] = None
    cfg["layers"][0]["mlp"]["router"]["bias"] = None
    cfg["layers"][1]["weights_of"] = None
    assert len(spec_of(cfg).layers) == 2
    cfg["layers"][0]["mlp"]["router"]["bias"] = True
    with pytest.raises(ConfigError, match="unknown key"):
        spec_of(cfg)


def test_plain_sink_of_minus_infinity_is_ordinary_softmax_and_a_sink_only_shrinks():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 4, 6, generator=g, dtype=torch.float64), torch.randn(9, 2, 6, generator=g, dtype=torch.float64),
               torch.randn(9, 2, 5, generator=g, dtype=torch.float64))
    none = plain.sink_softmax_attention(q, k, v, 0.4, torch.full((4,), -1e30, dtype=torch.float64))
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(2, 1)) * 0.4
    s = s.masked_fill(~torch.ones(9, 9, dtype=torch.bool).tril(), float("-inf"))
    want = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v.repeat_interleave(2, 1))
    torch.testing.assert_close(none, want)
    sink = torch.tensor([0.3, -2.0, 4.0, 0.0], dtype=torch.float64)
    with_sink = plain.sink_softmax_attention(q, k, v, 0.4, sink)
    share = torch.exp(sink)[:, None] / (torch.exp(s).sum(-1) + torch.exp(sink)[:, None])       # [H, T]
    torch.testing.assert_close(with_sink, want * (1 - share).T[..., None])


def test_plain_rotation_pairs_neighbours_and_depends_on_distance_only():
    g = torch.Generator().manual_seed(1)
    a, b = torch.randn(1, 1, 10, generator=g, dtype=torch.float64), torch.randn(1, 1, 10, generator=g, dtype=torch.float64)
    def dot(pa, pb):
        ra = plain.rotate_neighbour_pairs(a, torch.tensor([pa]), 100.0, 6)
        rb = plain.rotate_neighbour_pairs(b, torch.tensor([pb]), 100.0, 6)
        return float((ra * rb).sum())
    assert abs(dot(5, 2) - dot(103, 100)) < 1e-9 and abs(dot(5, 2) - dot(6, 2)) > 1e-6
    r = plain.rotate_neighbour_pairs(a, torch.tensor([7]), 100.0, 6)
    torch.testing.assert_close(r[..., 6:], a[..., 6:])
    for i in range(3):      # each neighbouring pair keeps its length; pair 0 turns by the position itself
        torch.testing.assert_close(r[..., 2 * i:2 * i + 2].norm(), a[..., 2 * i:2 * i + 2].norm())
    x0, x1 = float(a[0, 0, 0]), float(a[0, 0, 1])
    c, s = torch.cos(torch.tensor(7.0, dtype=torch.float64)), torch.sin(torch.tensor(7.0, dtype=torch.float64))
    torch.testing.assert_close(r[0, 0, :2], torch.stack([x0 * c - x1 * s, x1 * c + x0 * s]))


def test_plain_router_keeps_to_the_best_groups():
    # six experts in three groups; group scores: (0.9 + 0.1), (0.6 + 0.55), (0.7 + 0.2): groups 1 and 0 are kept, so the
    # third largest score overall (0.7, group 2) cannot be chosen
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55, 0.7, 0.2]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    w = torch.eye(6, dtype=torch.float64)
    idx, wt = plain.route(z, w, {"experts": 6, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 2}})
    assert sorted(idx[0].tolist()) == [0, 2, 3]
    torch.testing.assert_close(wt.sum(), torch.tensor(2.0, dtype=torch.float64))
    idx, _ = plain.route(z, w, {"experts": 6, "top": 3, "scale": 1.0})
    assert sorted(idx[0].tolist()) == [0, 2, 4]


def test_plain_expert_clamps_before_the_gate():
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64)
    eye = torch.eye(3, dtype=torch.float64)
    out = plain.clamped_expert(h, {"gate": eye, "up": eye, "down": eye}, "", 2.0)
    g, u = torch.tensor([2.0, -5.0, 0.5], dtype=torch.float64), torch.tensor([2.0, -2.0, 0.5], dtype=torch.float64)
    torch.testing.assert_close(out[0], g * torch.sigmoid(1.702 * g) * (u + 1))
