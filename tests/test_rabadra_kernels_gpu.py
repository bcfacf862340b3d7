"""Each Rabadra mechanism alone, its kernel against the plain implementation's function: the layer norm (into either
dtype, gathered rows, in place); the logit cap; the clamped swish; the whole-projection norms, neighbour rotation and
cache write behind the q/k/v projections; attention with sinks over the paged cache (scattered pages, unequal
sequences, values of another width, a far key among hundreds, page borders, single tokens and portions); the grouped
sigmoid router; the experts."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from plain import rabadra_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"fp32": torch.float32, "bf16": torch.bfloat16}
TOL = {"fp32": dict(rtol=2e-5, atol=2e-5), "bf16": dict(rtol=2e-2, atol=2e-2)}


def ops():
    from sleuth_b200.kernels import ops as o
    return o


def rot_tables(positions, base, dims):
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = torch.outer(torch.arange(positions, dtype=torch.float64), base ** (-2.0 * i / dims))
    return ang.cos().float().to(DEV), ang.sin().float().to(DEV)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("dim", [72, 321, 1000, 4096])
def test_layer_norm(dim, dtype):
    g = torch.Generator().manual_seed(dim)
    x = (3.0 + 2.0 * torch.randn(11, dim, generator=g)).to(DEV)        # a mean far from zero: subtracting it matters
    w = (1 + 0.2 * torch.randn(dim, generator=g)).to(DEV)
    want = plain.layer_norm(x.cpu().double(), w.cpu().double(), 1e-5)
    out = torch.empty(11, dim, dtype=DT[dtype], device=DEV)
    ops().layernorm(x, w, out, 1e-5)
    torch.testing.assert_close(out.cpu().double(), want, **TOL[dtype])
    rows = torch.tensor([9, 0, 4], dtype=torch.int32, device=DEV)
    some = torch.empty(3, dim, dtype=DT[dtype], device=DEV)
    ops().layernorm(x, w, some, 1e-5, rows)
    torch.testing.assert_close(some.cpu().double(), want[[9, 0, 4]], **TOL[dtype])
    w2 = (1 + 0.2 * torch.randn(dim, generator=g)).to(DEV)      # two gains in one pass, as a parallel layer's two norms run
    one, two = torch.empty(11, dim, dtype=DT[dtype], device=DEV), torch.empty(11, dim, dtype=DT[dtype], device=DEV)
    ops().layernorm(x, w, one, 1e-5, w2=w2, out2=two)
    torch.testing.assert_close(one.cpu().double(), want, **TOL[dtype])
    torch.testing.assert_close(two.cpu().double(), plain.layer_norm(x.cpu().double(), w2.cpu().double(), 1e-5), **TOL[dtype])
    if dtype == "fp32":
        ops().layernorm(x, w, x, 1e-5)      # in place, as the embedding's norm runs
        torch.testing.assert_close(x.cpu().double(), want, **TOL[dtype])


def test_logit_cap():
    v = torch.linspace(-90, 90, 7 * 33).reshape(7, 33).to(DEV)
    want = 30.0 * torch.tanh(v.cpu().double() / 30.0)
    ops().softcap(v, 30.0)
    torch.testing.assert_close(v.cpu().double(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_clamped_swish(dtype):
    g = torch.Generator().manual_seed(3)
    ff = 40
    gu = (3.0 * torch.randn(9, 2 * ff, generator=g)).to(DT[dtype])
    act = torch.empty(9, ff, dtype=DT[dtype], device=DEV)
    ops().gated_act(gu.to(DEV), act, "clamped_swish", limit=1.5, alpha=1.702)
    eye = torch.eye(2 * ff, dtype=torch.float64)
    want = plain.clamped_expert(gu.double(), {"gate": eye[:ff], "up": eye[ff:], "down": torch.eye(ff, dtype=torch.float64)}, "", 1.5)
    assert float(gu.abs().max()) > 1.5      # the clamps are at work
    torch.testing.assert_close(act.cpu().double(), want, **TOL[dtype])


def kv_pools(keys, values, G, dk, dv, dtype, seed):
    """Pools [pages, G, 64, dk | dv] whose pages are handed out in a scrambled order, holding the given rows
    (``keys[s]`` [n, G, dk]; None: left stale), and the block table."""
    n_pages = sum(-(-len(k) // 64) for k in keys) + 3
    order = np.random.default_rng(seed).permutation(n_pages)
    k_pool = torch.full((n_pages, G, 64, dk), 7.0, dtype=dtype, device=DEV)     # stale contents must never be read
    v_pool = torch.full((n_pages, G, 64, dv), 7.0, dtype=dtype, device=DEV)
    stride = max(-(-len(k) // 64) for k in keys) + 1
    table = torch.full((len(keys), stride), -1, dtype=torch.int32)
    n = 0
    for s, (k, v) in enumerate(zip(keys, values)):
        for p in range(-(-len(k) // 64)):
            table[s, p] = int(order[n])
            part = slice(p * 64, min(len(k), (p + 1) * 64))
            k_pool[order[n], :, :part.stop - part.start] = k[part].transpose(0, 1).to(dtype).to(DEV)
            v_pool[order[n], :, :part.stop - part.start] = v[part].transpose(0, 1).to(dtype).to(DEV)
            n += 1
    return k_pool, v_pool, table.to(DEV)


def token_tables(pasts, counts):
    tok_seq = torch.tensor(sum(([i] * c for i, c in enumerate(counts)), []), dtype=torch.int32, device=DEV)
    pos = sum((list(range(p, p + c)) for p, c in zip(pasts, counts)), [])
    return tok_seq, torch.tensor(pos, dtype=torch.int32, device=DEV), pos


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("H, G, dk, dv, rot, whole, neighbours", [
    (6, 2, 16, 24, 8, True, True), (4, 4, 32, 32, 32, True, True), (8, 1, 24, 40, 0, True, True),
    (3, 3, 10, 6, 6, False, True), (5, 1, 64, 64, 32, True, False), (2, 2, 128, 96, 128, False, False)])
def test_norms_rotation_and_cache_write(H, G, dk, dv, rot, whole, neighbours, dtype):
    g = torch.Generator().manual_seed(H * dk + rot)
    pasts, counts = [70, 0, 63], [3, 5, 2]
    T = sum(counts)
    qkv = torch.randn(T, (H + G) * dk + G * dv, generator=g) * 2.0
    nq, nk = (H * dk, G * dk) if whole else (dk, dk)
    qg, kg = 1 + 0.3 * torch.randn(nq, generator=g), 1 + 0.3 * torch.randn(nk, generator=g)
    cos, sin = rot_tables(128, 777.0, rot) if rot else (None, None)
    zeros = [torch.zeros(p + c, G, 1) for p, c in zip(pasts, counts)]
    k_pool, v_pool, table = kv_pools([z.expand(-1, G, dk) for z in zeros], [z.expand(-1, G, dv) for z in zeros], G, dk, dv, DT[dtype], 1)
    tok_seq, tok_pos, pos = token_tables(pasts, counts)
    q_out = torch.empty(T, H, dk, dtype=DT[dtype], device=DEV)
    ops().qkv_post_span(qkv.to(DEV), qg.to(DEV), kg.to(DEV), cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, table,
                        H, G, dk, dv, rot, neighbours, whole, 1e-5)
    x = qkv.double()
    q, k, v = x[:, :H * dk], x[:, H * dk:(H + G) * dk], x[:, (H + G) * dk:].reshape(T, G, dv)
    if whole:
        q, k = plain.rms_norm(q, qg.double(), 1e-5).reshape(T, H, dk), plain.rms_norm(k, kg.double(), 1e-5).reshape(T, G, dk)
    else:
        q, k = plain.rms_norm(q.reshape(T, H, dk), qg.double(), 1e-5), plain.rms_norm(k.reshape(T, G, dk), kg.double(), 1e-5)
    if rot and neighbours:
        q, k = (plain.rotate_neighbour_pairs(z, torch.tensor(pos), 777.0, rot) for z in (q, k))
    elif rot:
        from plain.lezepel_plain import rotate_half_pairs
        q, k = (rotate_half_pairs(z, torch.tensor(pos), 777.0, rot) for z in (q, k))
    torch.testing.assert_close(q_out.cpu().double(), q, **TOL[dtype])
    for t in range(T):
        page, row = int(table[tok_seq[t], pos[t] // 64]), pos[t] % 64
        torch.testing.assert_close(k_pool[page, :, row].cpu().double(), k[t], **TOL[dtype])
        torch.testing.assert_close(v_pool[page, :, row].cpu().double(), v[t], **TOL[dtype])
    # nothing but the tokens' own rows was touched
    for pool in (k_pool, v_pool):
        seen = pool.float().cpu()
        fresh = (seen != 7.0).any(dim=-1) & (seen != 0.0).any(dim=-1)
        assert int(fresh.sum()) == T * G


def run_attention(H, G, dk, dv, pasts, counts, dtype, seed, loud=(), scale=0.3, sink_scale=1.0, use_sinks=True):
    """Random queries, keys and values per sequence; ``loud``: (sequence, query position, key position) triples whose
    score is made to stand out, so that a key that is skipped or read from a wrong row changes the result."""
    g = torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    seqs = []
    for p, c in zip(pasts, counts):
        n = p + c
        seqs.append(dict(q=torch.randn(n, H, dk, generator=g, dtype=torch.float64), k=torch.randn(n, G, dk, generator=g, dtype=torch.float64),
                         v=torch.randn(n, G, dv, generator=g, dtype=torch.float64)))
    for s, qi, ki in loud:
        key = seqs[s]["k"][ki].repeat_interleave(H // G, dim=0)
        seqs[s]["q"][qi] = (14.0 / scale) * key / (key.norm(dim=-1, keepdim=True) ** 2)
    sinks = sink_scale * torch.randn(H, generator=g, dtype=torch.float64)
    if dtype == "bf16":     # both sides see the same rounded inputs
        for s in seqs:
            for k in s:
                s[k] = s[k].to(dt).double()
    k_pool, v_pool, table = kv_pools([s["k"] for s in seqs], [s["v"] for s in seqs], G, dk, dv, dt, seed)
    T = sum(counts)
    q = torch.cat([s["q"][p:p + c] for s, p, c in zip(seqs, pasts, counts)])
    tok_seq, tok_pos, _ = token_tables(pasts, counts)
    out = torch.empty(T, H * dv, dtype=dt, device=DEV)
    ops().attention(q.to(dt).to(DEV).contiguous(), k_pool, v_pool, out, tok_seq, tok_pos, table, H, G, dk, 0, scale,
                    sinks=sinks.float().to(DEV) if use_sinks else None, value_dim=dv)
    none = torch.full((H,), -1e30, dtype=torch.float64)
    want = torch.cat([plain.sink_softmax_attention(s["q"], s["k"], s["v"], scale, sinks if use_sinks else none)[p:p + c]
                      for s, p, c in zip(seqs, pasts, counts)]).reshape(T, H * dv)
    return out.cpu().double(), want, seqs


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("H, G, dk, dv", [(6, 2, 16, 24), (4, 4, 32, 32), (8, 1, 24, 40), (3, 1, 80, 8), (2, 2, 128, 200)])
def test_attention_with_sinks_over_scattered_pages(H, G, dk, dv, dtype):
    got, want, _ = run_attention(H, G, dk, dv, pasts=[0, 70, 0, 127], counts=[5, 3, 130, 1], dtype=dtype, seed=H + dk)
    torch.testing.assert_close(got, want, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_a_large_sink_takes_its_share_and_no_sink_takes_none(dtype):
    got, want, _ = run_attention(4, 2, 32, 16, [0, 40], [9, 2], dtype, seed=5, sink_scale=6.0)
    torch.testing.assert_close(got, want, **TOL[dtype])
    first = got[0].reshape(4, 16)        # the first token sees one key: its output is v0 * 1 / (1 + exp(sink - score))
    assert float(first.abs().min(dim=-1).values.min()) < float(first.abs().max())     # heads are damped differently
    got, want, _ = run_attention(4, 2, 32, 16, [0, 40], [9, 2], dtype, seed=5, use_sinks=False)
    torch.testing.assert_close(got, want, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("far", [0, 1, 63, 64, 65, 127, 128, 511, 640])
def test_a_far_key_among_hundreds_and_keys_at_page_borders(far, dtype):
    """One query's score with one far key stands out: if that key were skipped, masked or read from a wrong row, the
    output would not be its value. Single tokens (decoding) and a portion of a prompt both ask for it."""
    n = 700
    for pasts, counts in (([n - 1], [1]), ([n - 40], [40])):
        got, want, seqs = run_attention(4, 2, 48, 32, pasts, counts, dtype, seed=far, loud=[(0, n - 1, far)], sink_scale=0.5)
        torch.testing.assert_close(got, want, **TOL[dtype])
        last = got[-1].reshape(4, 32)
        value = seqs[0]["v"][far].repeat_interleave(2, dim=0)
        assert float((last - value).abs().max()) < 0.15     # nearly all of the weight lies on the far key


@pytest.mark.parametrize("kernel", ["decode", "prefill", "tc"])
@pytest.mark.parametrize("H, G, hd", [(8, 2, 64), (4, 2, 128), (6, 2, 64)])
def test_tensor_core_attention_kernels_take_sinks(H, G, hd, kernel):
    """The split-KV kernel for single tokens (one and several key slices), the mma.sync kernel and the tcgen05 kernels
    for portions and whole prompts, bfloat16, head sizes 64 and 128: the sink joins each row's denominator once."""
    o = ops()
    if kernel == "tc" and not o.attention_tc_supported(H, G, hd, torch.bfloat16):
        pytest.skip("the tcgen05 kernel does not take this group size")
    g = torch.Generator().manual_seed(H * hd)
    dt, scale = torch.bfloat16, hd ** -0.5
    if kernel == "decode":
        pasts, counts = [700, 64, 0, 129], [1, 1, 1, 1]
    else:
        pasts, counts = [0, 70, 300], [200, 130, 64]
    seqs = []
    for p, c in zip(pasts, counts):
        n = p + c
        seqs.append({k: torch.randn(n, hh, hd, generator=g).to(dt).double() for k, hh in (("q", H), ("k", G), ("v", G))})
    sinks = 2.0 * torch.randn(H, generator=g, dtype=torch.float64)
    k_pool, v_pool, table = kv_pools([s["k"] for s in seqs], [s["v"] for s in seqs], G, hd, hd, dt, 3)
    T = sum(counts)
    q = torch.cat([s["q"][p:p + c] for s, p, c in zip(seqs, pasts, counts)]).to(dt).to(DEV).contiguous()
    out = torch.empty(T, H * hd, dtype=dt, device=DEV)
    starts = torch.tensor(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32), device=DEV)
    past_t = torch.tensor(pasts, dtype=torch.int32, device=DEV)
    count_t = torch.tensor(counts, dtype=torch.int32, device=DEV)
    sk = sinks.float().to(DEV)
    want = torch.cat([plain.sink_softmax_attention(s["q"], s["k"], s["v"], scale, sinks)[p:p + c]
                      for s, p, c in zip(seqs, pasts, counts)]).reshape(T, H * hd)
    if kernel == "decode":
        for splits in (1, 3):
            floats = o.decode_scratch_floats(len(pasts), H, hd, splits)
            scratch = torch.empty(max(1, floats), dtype=torch.float32, device=DEV)
            out.zero_()
            o.attention_decode(q, k_pool, v_pool, out, starts, past_t, table, H, G, hd, 0, scale, splits, scratch, sinks=sk)
            torch.testing.assert_close(out.cpu().double(), want, **TOL["bf16"])
    elif kernel == "prefill":
        o.attention_prefill(q, k_pool, v_pool, out, starts, past_t, count_t, table, max(counts), H, G, hd, 0, scale, sinks=sk)
        torch.testing.assert_close(out.cpu().double(), want, **TOL["bf16"])
    else:
        for wide in (False, True):
            out.zero_()
            o.attention_tc(q, k_pool, v_pool, out, starts, past_t, count_t, table, max(counts), H, G, hd, 0, scale, wide=wide,
                           sinks=sk)
            o.gemm_tc_check(DEV)
            torch.testing.assert_close(out.cpu().double(), want, **TOL["bf16"])


def route_case(T, d, E, seed):
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(T, d, generator=g)
    w = torch.randn(E, d, generator=g) * (2.5 / d ** 0.5)
    return h, w


@pytest.mark.parametrize("T", [1, 7, 200])
@pytest.mark.parametrize("E, top, count, keep, scale", [(6, 2, 3, 2, 1.5), (8, 1, 1, 1, 0.7), (4, 4, 4, 4, 2.5), (16, 4, 4, 2, 2.0),
                                                         (12, 2, 4, 3, 2.0), (64, 6, 8, 3, 1.0), (9, 3, 3, 1, 1.0)])
def test_grouped_sigmoid_router(E, top, count, keep, scale, T):
    o = ops()
    h, w = route_case(T, 72, E, E * 100 + T)
    rule = {"experts": E, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}
    idx, wt = plain.route(h.double(), w.double(), rule)
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=DEV)
    choice, rank, place, order, counts = i32(T * top), i32(T * top), i32(T * top), i32(T * top), i32(E)
    weight = torch.empty(T * top, dtype=torch.float32, device=DEV)
    logits = torch.empty(T, E, dtype=torch.float32, device=DEV)
    o.moe_route(h.to(DEV), w.to(DEV), None, choice, weight, rank, counts, place, order, top, logits=logits,
                scoring="sigmoid", groups=count, keep=keep, scale=scale)
    got_i, got_w = choice.cpu().reshape(T, top).long(), weight.cpu().reshape(T, top).double()
    # the same experts with the same weights, largest score first on both sides
    assert torch.equal(got_i, idx), "the chosen experts differ"
    torch.testing.assert_close(got_w, wt, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(got_w.sum(-1), torch.full((T,), scale, dtype=torch.float64), rtol=1e-5, atol=1e-6)
    assert torch.equal(counts.cpu().long(), torch.bincount(idx.flatten(), minlength=E))
    group_of = idx // (E // count)
    assert all(len(set(r.tolist())) <= keep for r in group_of)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("T, d, ff, E, top, count, keep", [(1, 72, 20, 6, 2, 3, 2), (9, 128, 48, 8, 3, 1, 1), (150, 64, 24, 4, 4, 4, 4),
                                                            (700, 128, 64, 16, 4, 4, 2)])
def test_experts_with_the_clamped_swish(T, d, ff, E, top, count, keep, dtype):
    o = ops()
    g = torch.Generator().manual_seed(T + E)
    dt = DT[dtype]
    h, w_r = route_case(T, d, E, T)
    h = h.to(dt)
    w = {"router": w_r}
    for e in range(E):
        w[f"e{e}.gate"] = (torch.randn(ff, d, generator=g) * 0.3).to(dt)
        w[f"e{e}.up"] = (torch.randn(ff, d, generator=g) * 0.3).to(dt)
        w[f"e{e}.down"] = (torch.randn(d, ff, generator=g) * 0.2).to(dt)
    f = {"router": {"experts": E, "top": top, "scale": 1.75, "groups": {"count": count, "keep": keep}}, "expert": {"ff": ff, "limit": 1.25}}
    want = plain.mixture(h.double(), {k: v.double() for k, v in w.items()}, "", f)
    w_gu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).to(DEV).contiguous()
    w_dn = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(DEV).contiguous()
    pairs = T * top
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=DEV)
    choice, rank, place, order, counts = i32(pairs), i32(pairs), i32(pairs), i32(pairs), i32(E)
    weight = torch.empty(pairs, dtype=torch.float32, device=DEV)
    logits = torch.empty(T, E, dtype=torch.float32, device=DEV)
    o.moe_route(h.to(DEV), w_r.to(DEV), None, choice, weight, rank, counts, place, order, top, logits=logits,
                layout=pairs > o.MOE_FEW_PAIRS, scoring="sigmoid", groups=count, keep=keep, scale=1.75)
    act = torch.empty(pairs, ff, dtype=dt, device=DEV)
    y = torch.empty(pairs, d, dtype=torch.float32, device=DEV)
    x = torch.zeros(T, d, dtype=torch.float32, device=DEV)
    o.moe_experts(h.to(DEV), w_gu, w_dn, counts, order, weight, act, y, x, top, "clamped_swish", choice=choice, place=place,
                  limit=1.25, alpha=1.702)
    diff = (x.cpu().double() - want).abs().amax(dim=-1)
    if dtype == "fp32":
        torch.testing.assert_close(x.cpu().double(), want, rtol=1e-4, atol=1e-4)
    else:       # the activations are rounded once on the device; the choice is made from the same float32 logits
        assert float(diff.max()) <= 0.05 * max(1.0, float(want.abs().max()))
    if dtype == "bf16" and d % 8 == 0 and ff % 8 == 0:      # and as grouped tensor-memory products over the experts' row tiles
        tiles = torch.empty(o.moe_tile_words(T, top, E), dtype=torch.int32, device=DEV)
        o.moe_route(h.to(DEV), w_r.to(DEV), None, choice, weight, rank, counts, place, order, top, logits=logits, tiles=tiles,
                    scoring="sigmoid", groups=count, keep=keep, scale=1.75)
        xs = torch.empty(pairs, d, dtype=dt, device=DEV)
        x3 = torch.zeros(T, d, dtype=torch.float32, device=DEV)
        o.moe_experts_tc(h.to(DEV), w_gu, w_dn, order, place, weight, tiles, xs, act, y, x3, top, activation="clamped_swish",
                         limit=1.25, alpha=1.702)
        o.gemm_tc_check(DEV)
        diff = (x3.cpu().double() - want).abs().amax(dim=-1)
        assert float(diff.max()) <= 0.05 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("T", [1, 8, 200])
def test_gated_products_apply_the_clamped_swish_in_their_epilogue(T):
    o = ops()
    g = torch.Generator().manual_seed(T)
    d, ff = 256, 192
    h = torch.randn(T, d, generator=g).to(torch.bfloat16)
    w = {"gate": (torch.randn(ff, d, generator=g) * 0.2).to(torch.bfloat16), "up": (torch.randn(ff, d, generator=g) * 0.2).to(torch.bfloat16),
         "down": torch.eye(ff, dtype=torch.float64)}
    want = plain.clamped_expert(h.double(), {k: v.double() for k, v in w.items()}, "", 1.5)
    w_gu = torch.cat([w["gate"], w["up"]]).to(DEV).contiguous()
    act = torch.empty(T, ff, dtype=torch.bfloat16, device=DEV)
    gate = ("clamped_swish", 1.5, 1.702)
    if T <= 32:
        o.gemm_skinny(h.to(DEV), w_gu, act, "swiglu", gate=gate)
    else:
        o.gemm_tc(h.to(DEV), w_gu, act, "swiglu", gate=gate)
        o.gemm_tc_check(DEV)
    assert float((h.double() @ w["gate"].double().T).abs().max()) > 1.5
    torch.testing.assert_close(act.cpu().double(), want, rtol=2e-2, atol=2e-2)
