"""Each Lezepel mechanism alone, its kernel against the plain implementation's function: the norms, rotation and
cache write behind the down-projections; the attention over the latent cache (scattered pages, unequal sequences,
far keys, page borders, single tokens, slices); the output gate; the router and the experts; the gated ReLU; the
vectors added to the stream between passes."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from plain import lezepel_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"fp32": torch.float32, "bf16": torch.bfloat16}
TOL = {"fp32": dict(rtol=2e-5, atol=2e-5), "bf16": dict(rtol=2e-2, atol=2e-2)}


def ops():
    from sleuth_b200.kernels import ops as o
    return o


def rot_tables(positions, base, dims):
    i = torch.arange(dims // 2, dtype=torch.float32)
    ang = torch.outer(torch.arange(positions, dtype=torch.float32), base ** (-2.0 * i / dims))
    return ang.cos().to(DEV), ang.sin().to(DEV)


def paged(rows_per_seq, width, dtype, seed):
    """A pool whose pages are handed out in a scrambled order, and the block table of the sequences."""
    n_pages = sum(-(-len(r) // 64) for r in rows_per_seq) + 3
    order = np.random.default_rng(seed).permutation(n_pages)
    pool = torch.full((n_pages, 64, width), 7.0, dtype=dtype, device=DEV)      # stale contents must never be read
    stride = max(-(-len(r) // 64) for r in rows_per_seq) + 1
    table = torch.full((len(rows_per_seq), stride), -1, dtype=torch.int32)
    k = 0
    for s, rows in enumerate(rows_per_seq):
        for p in range(-(-len(rows) // 64)):
            table[s, p] = int(order[k])
            part = rows[p * 64:(p + 1) * 64]
            pool[order[k], :len(part)] = part.to(dtype).to(DEV)
            k += 1
    return pool, table.to(DEV)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("q_rank, R, P, rot", [(20, 40, 8, 8), (64, 112, 16, 16), (7, 9, 6, 4), (300, 520, 64, 64)])
def test_norms_rotation_and_cache_write(q_rank, R, P, rot, dtype):
    g = torch.Generator().manual_seed(q_rank)
    pasts, counts = [70, 0, 63], [3, 5, 2]
    T = sum(counts)
    lat = torch.randn(T, q_rank + R + P, generator=g)
    qg, cg = 1 + 0.1 * torch.randn(q_rank, generator=g), 1 + 0.1 * torch.randn(R, generator=g)
    cos, sin = rot_tables(128, 777.0, rot)
    seqs = [torch.zeros(p + c, R + P) for p, c in zip(pasts, counts)]
    pool, table = paged(seqs, R + P, DT[dtype], 1)
    tok_seq = torch.tensor(sum(([i] * c for i, c in enumerate(counts)), []), dtype=torch.int32, device=DEV)
    pos = sum((list(range(p, p + c)) for p, c in zip(pasts, counts)), [])
    tok_pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
    cq = torch.empty(T, q_rank, dtype=DT[dtype], device=DEV)
    ops().latent_post(lat.to(DEV), qg.to(DEV), cg.to(DEV), cos, sin, cq, pool, tok_seq, tok_pos, table, q_rank, R, P, rot, 1e-5)
    want_q = plain.rms_norm(lat[:, :q_rank].double(), qg.double(), 1e-5)
    want_c = plain.rms_norm(lat[:, q_rank:q_rank + R].double(), cg.double(), 1e-5)
    want_k = plain.rotate_half_pairs(lat[:, None, q_rank + R:].double(), torch.tensor(pos), 777.0, rot)[:, 0]
    torch.testing.assert_close(cq.cpu().double(), want_q, **TOL[dtype])
    for t in range(T):
        row = pool[table[tok_seq[t], pos[t] // 64], pos[t] % 64].cpu().double()
        torch.testing.assert_close(row[:R], want_c[t], **TOL[dtype])
        torch.testing.assert_close(row[R:], want_k[t], **TOL[dtype])
    # nothing but the tokens' own rows was touched
    seen = pool.float().cpu()
    inside = (seen != 7.0).any(dim=-1)
    assert int(inside.sum()) == sum(p + c for p, c in zip(pasts, counts))
    assert int((inside & (seen != 0.0).any(dim=-1)).sum()) == T


def latent_case(H, dn, P, dv, R, pasts, counts, seed, loud=()):
    """Random latents, queries and up-projections; ``loud``: (sequence, query position, key position) triples whose
    score is made to stand out, so that a key that is skipped or read from a wrong row changes the result."""
    g = torch.Generator().manual_seed(seed)
    w_uk = torch.randn(H * dn, R, generator=g, dtype=torch.float64) / R ** 0.5
    w_uv = torch.randn(H * dv, R, generator=g, dtype=torch.float64) / R ** 0.5
    seqs = []
    for p, c in zip(pasts, counts):
        n = p + c
        seqs.append(dict(c=torch.randn(n, R, generator=g, dtype=torch.float64), k_rot=torch.randn(n, P, generator=g, dtype=torch.float64),
                         q=torch.randn(n, H, dn + P, generator=g, dtype=torch.float64)))
    for s, qi, ki in loud:
        k_plain = (seqs[s]["c"][ki] @ w_uk.T).reshape(H, dn)
        seqs[s]["q"][qi, :, :dn] = 12.0 * k_plain / k_plain.norm(dim=-1, keepdim=True)
    return w_uk, w_uv, seqs


def run_latent_attention(H, dn, P, dv, R, pasts, counts, dtype, seed, loud=(), splits=1, base=1000.0, scale=0.3):
    o = ops()
    w_uk, w_uv, seqs = latent_case(H, dn, P, dv, R, pasts, counts, seed, loud)
    dt = DT[dtype]
    if dtype == "bf16":     # both sides see the same rounded inputs
        for s in seqs:
            for k in s:
                s[k] = s[k].to(dt).double()
    positions = max(p + c for p, c in zip(pasts, counts)) + 1
    cos, sin = rot_tables(positions, base, P)
    rows = [torch.cat([s["c"], plain.rotate_half_pairs(s["k_rot"][:, None, :], torch.arange(len(s["c"])), base, P)[:, 0]], -1)
            for s in seqs]
    pool, table = paged(rows, R + P, dt, seed)
    T = sum(counts)
    q_raw = torch.cat([s["q"][p:p + c] for s, p, c in zip(seqs, pasts, counts)]).reshape(T, H, dn + P)
    q_lat = torch.einsum("thd,hdr->htr", q_raw[..., :dn], w_uk.reshape(H, dn, R))
    if dtype == "bf16":
        q_lat = q_lat.to(dt).double()
    out = torch.empty(H, T, R, dtype=dt, device=DEV)
    starts = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    scratch = torch.empty(max(1, o.latent_scratch_floats(T, H, R, splits)), dtype=torch.float32, device=DEV)
    o.latent_attention(q_lat.to(dt).to(DEV).contiguous(), q_raw.to(dt).to(DEV).contiguous(), pool, out, cos, sin,
                       torch.from_numpy(starts).to(DEV), torch.tensor(pasts, dtype=torch.int32, device=DEV),
                       torch.tensor(counts, dtype=torch.int32, device=DEV), table, max(counts), H, R, P, dn, P, 0, scale,
                       splits, scratch)
    got = torch.einsum("htr,hvr->thv", out.cpu().double(), w_uv.reshape(H, dv, R))
    want = []
    for s, p, c in zip(seqs, pasts, counts):
        n = p + c
        pos = torch.arange(n)
        q = torch.cat([s["q"][..., :dn] if dtype == "fp32" else s["q"][..., :dn],
                       plain.rotate_half_pairs(s["q"][..., dn:], pos, base, P)], -1)
        k = torch.cat([(s["c"] @ w_uk.T).reshape(n, H, dn),
                       plain.rotate_half_pairs(s["k_rot"][:, None, :], pos, base, P).expand(n, H, P)], -1)
        v = (s["c"] @ w_uv.T).reshape(n, H, dv)
        want.append(plain.causal_softmax_attention(q, k, v, scale)[p:])
    return got, torch.cat(want)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("H, dn, P, dv, R", [(3, 16, 8, 24, 40), (8, 48, 16, 64, 112), (1, 8, 4, 8, 7), (40, 8, 4, 8, 28),
                                             (5, 16, 64, 16, 520), (70, 8, 16, 8, 32), (5, 16, 64, 16, 512), (2, 8, 16, 8, 272)])
def test_attention_over_the_latent_cache_prompts(H, dn, P, dv, R, dtype):
    got, want = run_latent_attention(H, dn, P, dv, R, pasts=[0, 0, 0, 0], counts=[1, 65, 130, 17], dtype=dtype, seed=H)
    torch.testing.assert_close(got, want, **TOL[dtype])


@pytest.mark.parametrize("R, P", [(24, 8), (32, 16)])       # the second pair goes to the tensor-core kernel in bfloat16
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_attention_finds_far_keys_and_keys_at_page_borders(dtype, R, P):
    """One key stands out for each chosen query: the first token, the last row of a page, the first row of the next,
    one far back among hundreds; in a prompt's portion (with and without earlier tokens) and for single tokens."""
    loud = [(0, 299, 0), (0, 298, 63), (0, 297, 64), (0, 296, 127), (0, 295, 128), (0, 290, 5), (1, 200, 200), (1, 199, 191),
            (2, 640, 1), (2, 640 - 1, 639), (3, 130, 64), (4, 450, 3)]
    pasts, counts = [250, 0, 640, 130, 450], [50, 201, 1, 1, 1]
    # the prompt of sequence 2 and 4 is far behind their one token; sequence 0 continues a portion
    loud = [(s, q, k) for s, q, k in loud if q >= pasts[s] and q < pasts[s] + counts[s]]
    assert len(loud) >= 9
    got, want = run_latent_attention(4, 16, P, 12, R, pasts, counts, dtype, seed=9, loud=loud)
    torch.testing.assert_close(got, want, **TOL[dtype])
    assert float(want.abs().max()) > 0.5         # the loud keys carry the result


@pytest.mark.parametrize("R, P", [(40, 8), (48, 16), (288, 32)])
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("splits", [2, 5, 16])
def test_attention_in_slices_is_the_same_attention(splits, dtype, R, P):
    pasts, counts = [1000, 70, 0, 511], [1, 1, 1, 1]
    one = run_latent_attention(6, 16, P, 16, R, pasts, counts, dtype, seed=2, loud=[(0, 1000, 2), (3, 511, 448)])
    cut = run_latent_attention(6, 16, P, 16, R, pasts, counts, dtype, seed=2, loud=[(0, 1000, 2), (3, 511, 448)], splits=splits)
    torch.testing.assert_close(cut[0], one[1], **TOL[dtype])
    torch.testing.assert_close(cut[0], one[0], rtol=1e-5, atol=1e-5) if dtype == "fp32" else None


@pytest.mark.parametrize("H, dn, P, dv, R", [(3, 16, 16, 16, 40), (8, 48, 16, 64, 80), (2, 128, 64, 128, 72), (5, 24, 8, 48, 24)])
def test_whole_prompts_with_per_head_keys_and_values(H, dn, P, dv, R):
    """Every sequence starts at 0: keys and values per head formed from the latents, then per-head attention; loud keys
    at the first token, at page borders and far back."""
    o, dt = ops(), torch.bfloat16
    counts = [1, 65, 300, 64]
    loud = [(1, 64, 0), (1, 63, 62), (2, 299, 0), (2, 298, 63), (2, 297, 64), (2, 200, 128), (3, 63, 1)]
    w_uk, w_uv, seqs = latent_case(H, dn, P, dv, R, [0] * 4, counts, seed=H + dn, loud=loud)
    for s_ in seqs:
        for k in s_:
            s_[k] = s_[k].to(dt).double()
    base, scale = 1000.0, 0.3
    cos, sin = rot_tables(max(counts) + 1, base, P)
    T = sum(counts)
    q = torch.cat([s_["q"] for s_ in seqs]).reshape(T, H, dn + P)
    c = torch.cat([s_["c"] for s_ in seqs])
    kv = torch.cat([c @ w_uk.T, c @ w_uv.T], dim=-1).to(dt)
    k_rot = torch.cat([plain.rotate_half_pairs(s_["k_rot"][:, None, :], torch.arange(len(s_["c"])), base, P)[:, 0] for s_ in seqs]).to(dt)
    out = torch.empty(H, T, dv, dtype=dt, device=DEV)
    starts = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    assert o.head_prompt_supported(dn, P, dv, dt)
    o.head_prompt_attention(q.to(dt).to(DEV).contiguous(), kv.to(DEV).contiguous(), k_rot.to(DEV).contiguous(), out, cos, sin,
                            torch.from_numpy(starts).to(DEV), torch.tensor(counts, dtype=torch.int32, device=DEV), max(counts), H,
                            dn, P, dv, P, 0, scale)
    want, at = [], 0
    for s_ in seqs:          # both sides see the same rounded keys and values
        n = len(s_["c"])
        pos = torch.arange(n)
        mine = kv[at:at + n].double()
        qq = torch.cat([s_["q"][..., :dn], plain.rotate_half_pairs(s_["q"][..., dn:], pos, base, P)], -1)
        kk = torch.cat([mine[:, :H * dn].reshape(n, H, dn), k_rot[at:at + n].double()[:, None, :].expand(n, H, P)], -1)
        want.append(plain.causal_softmax_attention(qq, kk, mine[:, H * dn:].reshape(n, H, dv), scale))
        at += n
    torch.testing.assert_close(out.cpu().double().transpose(0, 1), torch.cat(want), **TOL["bf16"])
    assert float(torch.cat(want).abs().max()) > 0.5


def test_the_two_bfloat16_attention_kernels_agree():
    """The tensor-core kernel and the general one on the same bfloat16 inputs: portions behind earlier tokens, single
    tokens and whole prompts in one step, more heads than a block takes."""
    args = dict(H=70, dn=8, P=16, dv=8, R=48, pasts=[100, 0, 300, 64], counts=[30, 129, 1, 2], dtype="bf16", seed=4,
                loud=[(0, 120, 3), (1, 128, 64), (2, 300, 63)])
    fast, want = run_latent_attention(**args)
    ops().latent_attention_general_only(True)
    try:
        slow, _ = run_latent_attention(**args)
    finally:
        ops().latent_attention_general_only(False)
    torch.testing.assert_close(fast, want, **TOL["bf16"])
    torch.testing.assert_close(fast, slow, rtol=1e-2, atol=1e-2)
    assert not torch.equal(fast, slow)          # two kernels did run


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_output_gate(dtype):
    g = torch.Generator().manual_seed(1)
    H, T, dv = 5, 37, 24
    val, z = torch.randn(H, T, dv, generator=g), 3 * torch.randn(T, H * dv, generator=g)
    y = torch.empty(T, H * dv, dtype=DT[dtype], device=DEV)
    ops().latent_gate(val.to(DT[dtype]).to(DEV), z.to(DT[dtype]).to(DEV), y)
    want = val.to(DT[dtype]).double().transpose(0, 1).reshape(T, H * dv) * torch.sigmoid(z.to(DT[dtype]).double())
    torch.testing.assert_close(y.cpu().double(), want, **TOL[dtype])


def expert_weights(E, d, ff, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    w = {"router": torch.randn(E, d, generator=g), "router.b": torch.randn(E, generator=g)}
    for e in range(E):
        for name, shape in (("gate", (ff, d)), ("up", (ff, d)), ("down", (d, ff))):
            w[f"e{e}.{name}"] = (torch.randn(*shape, generator=g) / shape[1] ** 0.5).to(DT[dtype]).float()
    return w


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("T, d, ff, E, top", [(1, 72, 36, 5, 2), (77, 72, 20, 6, 1), (300, 192, 88, 12, 3), (40, 64, 16, 4, 4),
                                              (9, 50, 33, 70, 3), (700, 128, 200, 7, 3), (3, 64, 136, 5, 2)])
def test_router_and_experts(T, d, ff, E, top, dtype):
    o, dt = ops(), DT[dtype]
    w = expert_weights(E, d, ff, T, dtype)
    h = torch.randn(T, d, generator=torch.Generator().manual_seed(T + 1)).to(dt)
    x0 = torch.randn(T, d, generator=torch.Generator().manual_seed(T + 2))
    pairs = T * top
    choice, rank, place, order = (torch.empty(pairs, dtype=torch.int32, device=DEV) for _ in range(4))
    counts = torch.empty(E, dtype=torch.int32, device=DEV)
    weight = torch.empty(pairs, dtype=torch.float32, device=DEV)
    logits = torch.empty(T, E, dtype=torch.float32, device=DEV) if T != 77 else None      # with and without the scratch
    o.moe_route(h.to(DEV), w["router"].to(DEV), w["router.b"].to(DEV), choice, weight, rank, counts, place, order, top,
                logits=logits)
    z = h.double() @ w["router"].double().T + w["router.b"].double()
    val, idx = torch.topk(z, top, dim=-1)
    assert torch.equal(choice.cpu().view(T, top).long(), idx)
    torch.testing.assert_close(weight.cpu().view(T, top).double(), torch.softmax(val, -1), rtol=1e-4, atol=2e-5)
    assert torch.equal(counts.cpu().long(), torch.bincount(idx.reshape(-1), minlength=E))
    # the expert-ordered list holds every pair once, grouped by expert
    lst = order.cpu().long()
    assert sorted(lst.tolist()) == list(range(pairs))
    assert torch.equal(choice.cpu().long()[lst], torch.sort(choice.cpu().long())[0])
    assert torch.equal(lst[place.cpu().long()], torch.arange(pairs))
    gu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).to(dt).to(DEV)
    dn = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(dt).to(DEV)
    act = torch.empty(pairs, ff, dtype=dt, device=DEV)
    y = torch.empty(pairs, d, dtype=torch.float32, device=DEV)
    x = x0.clone().to(DEV)
    o.moe_experts(h.to(DEV), gu, dn, counts, order, weight, act, y, x, top, "silu", choice=choice, place=place)
    if pairs <= o.MOE_FEW_PAIRS:      # a step of few pairs needs no layout at all
        junk = [torch.full((max(pairs, E),), -7, dtype=torch.int32, device=DEV) for _ in range(3)]
        o.moe_route(h.to(DEV), w["router"].to(DEV), w["router.b"].to(DEV), choice, weight, rank, junk[0], junk[1], junk[2], top,
                    layout=False)
        x4 = x0.clone().to(DEV)
        o.moe_experts(h.to(DEV), gu, dn, junk[0], junk[2], weight, act, y, x4, top, "silu", choice=choice)
        torch.testing.assert_close(x4, x, rtol=0, atol=0)
        assert all(int((j != -7).sum()) == 0 for j in junk)
    x2 = x0.clone().to(DEV)          # and through the tiles whatever the number of pairs
    o.moe_experts(h.to(DEV), gu, dn, counts, order, weight, act, y, x2, top, "silu")
    torch.testing.assert_close(x2, x, **TOL[dtype])
    if dtype == "bf16" and d % 8 == 0 and ff % 8 == 0:      # and as grouped tensor-memory products over the experts' row tiles
        tiles = torch.empty(o.moe_tile_words(T, top, E), dtype=torch.int32, device=DEV)
        o.moe_route(h.to(DEV), w["router"].to(DEV), w["router.b"].to(DEV), choice, weight, rank, counts, place, order, top,
                    logits=logits, tiles=tiles)
        n = int(tiles[0])
        table = tiles[1:1 + 3 * n].view(n, 3).cpu()
        assert int(table[:, 2].sum()) == pairs and int(table[:, 2].max()) <= 128
        x3 = x0.clone().to(DEV)
        xs = torch.empty(pairs, d, dtype=dt, device=DEV)
        o.moe_experts_tc(h.to(DEV), gu, dn, order, place, weight, tiles, xs, act, y, x3, top)
        torch.cuda.synchronize()
        o.gemm_tc_check(torch.device(DEV))
        torch.testing.assert_close(x3, x, **TOL[dtype])
    want = x0.double() + plain.routed_experts(h.double(), {k: v.double() for k, v in w.items()}, "", {"router": {"experts": E, "top": top}})
    torch.testing.assert_close(x.cpu().double(), want, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_gated_relu_and_stream_vectors(dtype):
    o, dt = ops(), DT[dtype]
    g = torch.Generator().manual_seed(5)
    gu = torch.randn(13, 2 * 50, generator=g).to(dt)
    act = torch.empty(13, 50, dtype=dt, device=DEV)
    o.gated_act(gu.to(DEV), act, "relu")
    torch.testing.assert_close(act.cpu().double(), torch.relu(gu[:, :50].double()) * gu[:, 50:].double(), **TOL[dtype])
    x, again, row = torch.randn(13, 50, generator=g), torch.randn(13, 50, generator=g), torch.randn(50, generator=g)
    for a, r in ((again, row), (None, row), (again, None)):
        xd = x.clone().to(DEV)
        o.stream_inject(xd, None if a is None else a.to(DEV), None if r is None else r.to(DEV))
        torch.testing.assert_close(xd.cpu(), x + (0 if a is None else a) + (0 if r is None else r))
