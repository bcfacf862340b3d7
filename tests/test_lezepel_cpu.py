"""Lezepel without a GPU: its configuration, its model description, its tensors, and the plain implementation's
own consistency (the latent-space form of the attention equals the per-head form; the loop's order of layers)."""

from __future__ import annotations

import copy

import pytest
import torch

import tiny_lezepel as tl
from plain import lezepel_plain as plain
from plain.qwen3_plain import read_model
from sleuth_b200.config import ConfigError, parse_config
from sleuth_b200.engine.model import declare_model
from sleuth_b200.parts.spec import looped_schedule


def spec_of(cfg):
    arch, typed, unread = parse_config(cfg)
    assert arch.name == "Lezepel" and set(unread) <= {"torch_dtype"}      # the folder writer's own note
    return arch.model_spec(typed)


def test_every_size_comes_from_the_configuration():
    spec = spec_of(tl.P)
    m = spec.layers[1].mixer
    assert (m.heads, m.plain_dim, m.rot_dim, m.value_dim, m.q_rank, m.kv_rank) == (3, 16, 8, 24, 20, 40)
    assert m.scale == 0.31 and m.position.theta == 500.0 and m.position.rotary_dim == 8 and m.norm_eps == 1e-6
    assert spec.embedding.scale == 3.0 and spec.embedding.vocab == 301 and spec.head.norm.eps == 1e-6
    kinds = [type(L.ffn).__name__ for L in spec.layers]
    assert kinds == ["GatedMLPSpec", "RoutedExpertsSpec", "NoneType", "RoutedExpertsSpec"]
    assert spec.layers[0].ffn.activation == "relu" and spec.layers[1].ffn.activation == "silu"
    assert (spec.layers[3].ffn.experts, spec.layers[3].ffn.top, spec.layers[3].ffn.intermediate) == (6, 1, 20)
    assert all(L.kind == "parallel" and L.norm2 is None for L in spec.layers)


def test_the_loop_becomes_a_schedule_with_caches_of_its_own():
    spec = spec_of(tl.P)
    got = [(e.layer, e.add_embedding, e.add_row) for e in spec.schedule]
    assert got == [(0, False, -1), (1, False, 0), (2, False, -1), (1, True, 1), (2, False, -1), (3, False, -1)]
    assert [e.cache for e in spec.schedule] == list(range(6)) and spec.pass_rows == "loop.step"
    first = [(e.layer, e.add_embedding, e.add_row) for e in spec_of(tl.Q).schedule]
    assert first == [(0, False, 0), (0, True, 1), (0, True, 2), (1, False, -1)]
    assert spec_of(tl.R).pass_rows is None and len(spec_of(tl.R).schedule) == 2
    assert [(i, t, f) for i, t, f in plain.layer_runs(tl.P)] == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True),
                                                                (2, 1, False), (3, None, False)]
    with pytest.raises(ValueError):
        looped_schedule(3, 2, 4, 2)


def test_declared_tensors_carry_the_file_names_and_shapes():
    d = declare_model(spec_of(tl.P))
    assert d["embed"].shape == (301, 72) and d["head"].shape == (301, 72) and d["final.norm"].shape == (72,)
    assert d["loop.step"].shape == (2, 72) and d["loop.step"].role == "vector"
    assert d["l0.mix.dq"].shape == (20, 72) and d["l0.mix.dq.norm"].shape == (20,)
    assert d["l0.mix.uq"].shape == (3 * 24, 20) and d["l0.mix.dkv"].shape == (48, 72) and d["l0.mix.dkv.norm"].shape == (40,)
    assert d["l0.mix.uk"].shape == (48, 40) and d["l0.mix.uv"].shape == (72, 40)
    assert d["l0.mix.g"].shape == (72, 72) and d["l0.mix.o"].shape == (72, 72)
    assert d["l0.mlp.gate"].shape == (100, 72) and d["l0.mlp.down"].shape == (72, 100)
    assert d["l1.mlp.router"].shape == (5, 72) and d["l1.mlp.router.b"].shape == (5,) and d["l1.mlp.e4.up"].shape == (36, 72)
    assert not any(n.startswith("l2.mlp") for n in d) and "l3.mlp.e5.down" in d and "l3.mlp.e6.down" not in d
    assert "loop.step" not in declare_model(spec_of(tl.R))


@pytest.mark.parametrize("change, words", [
    (lambda c: c["layers"][0].__setitem__("type", "window_attention"), "not a known mixer"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "not 'dense' or 'moe'"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "router.top"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", "3"), "expected an integer"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("window", 16), "unknown key"),
    (lambda c: c["loop"].__setitem__("stop", 7), "does not fit"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
])
def test_a_configuration_that_asks_for_something_else_is_refused(change, words):
    cfg = copy.deepcopy(tl.P)
    change(cfg)
    with pytest.raises(ConfigError, match=words):
        spec_of(cfg)


def test_a_written_folder_reads_back(tmp_path):
    from sleuth_b200.weights.random_init import write_random_model
    from sleuth_b200.weights.safetensors import Checkpoint
    write_random_model(tmp_path, tl.R, seed=5, dtype=torch.bfloat16, std=0.05)
    cfg, w = read_model(tmp_path)
    assert set(w) == set(declare_model(spec_of(cfg)))
    with Checkpoint(tmp_path) as ck:
        assert ck.describe("l1.mix.uq")[1] == (40 * 12, 32)
    logits = plain.forward(cfg, w, [1, 2, 3, 4], torch.float64)
    assert logits.shape == (4, 203) and torch.isfinite(logits).all()


def test_plain_attention_in_the_latent_space_is_the_per_head_form():
    """(W_uk c) . q = c . (W_uk^T q), and sum_j p_j (W_uv c_j) = W_uv sum_j p_j c_j: what the product path relies on."""
    g = torch.Generator().manual_seed(3)
    T, H, dn, dr, dv, r = 9, 3, 6, 4, 5, 7
    c = torch.randn(T, r, generator=g, dtype=torch.float64)
    k_rot = torch.randn(T, dr, generator=g, dtype=torch.float64)
    q = torch.randn(T, H, dn + dr, generator=g, dtype=torch.float64)
    w_uk = torch.randn(H * dn, r, generator=g, dtype=torch.float64)
    w_uv = torch.randn(H * dv, r, generator=g, dtype=torch.float64)
    k = torch.cat([(c @ w_uk.T).reshape(T, H, dn), k_rot[:, None, :].expand(T, H, dr)], -1)
    want = plain.causal_softmax_attention(q, k, (c @ w_uv.T).reshape(T, H, dv), 0.4)
    q_lat = torch.einsum("thd,hdr->thr", q[..., :dn], w_uk.reshape(H, dn, r))
    rows = torch.cat([c, k_rot], -1)[:, None, :].expand(T, H, r + dr)
    o_lat = plain.causal_softmax_attention(torch.cat([q_lat, q[..., dn:]], -1), rows, c[:, None, :].expand(T, H, r), 0.4)
    got = torch.einsum("thr,hvr->thv", o_lat, w_uv.reshape(H, dv, r))
    torch.testing.assert_close(got, want, rtol=1e-12, atol=1e-12)


def test_plain_routing_uses_only_the_chosen_experts():
    g = torch.Generator().manual_seed(4)
    d, ff, E = 8, 6, 4
    w = {"router": torch.randn(E, d, generator=g, dtype=torch.float64), "router.b": torch.tensor([0.0, 50.0, -50.0, 49.0], dtype=torch.float64)}
    for e in range(E):
        w[f"e{e}.gate"] = torch.randn(ff, d, generator=g, dtype=torch.float64)
        w[f"e{e}.up"] = torch.randn(ff, d, generator=g, dtype=torch.float64)
        w[f"e{e}.down"] = torch.randn(d, ff, generator=g, dtype=torch.float64)
    h = torch.randn(5, d, generator=g, dtype=torch.float64) * 0.01
    out = plain.routed_experts(h, w, "", {"router": {"experts": E, "top": 2}})
    z = h @ w["router"].T + w["router.b"]
    share = torch.softmax(z[:, [1, 3]], dim=-1)          # the biases settle the choice: experts 1 and 3

    def expert(e):
        a = h @ w[f"e{e}.gate"].T
        return ((a * torch.sigmoid(a)) * (h @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T
    torch.testing.assert_close(out, share[:, :1] * expert(1) + share[:, 1:] * expert(3))
