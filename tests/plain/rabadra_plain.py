"""Plain Rabadra decoder: whole sequences, no cache, one function per mechanism.

Rabadra is a decoder whose embedding is followed by a weight-only layer norm, whose layers are *parallel*
blocks with two norms (x + mixer(norm1 x) + ff(norm2 x)), whose mixer is grouped-query attention with an RMS
norm over the whole query and the whole key projection, an interleaved partial rotation, a scale of its own
and a learned per-head sink in the softmax denominator, and whose feed-forward is a mixture of clamped gated
experts chosen by sigmoid scores within the best groups of experts, plus a shared expert. A layer may borrow
another layer's weights. The logits are soft-capped.

Everything runs on the CPU with ordinary tensor operations in the dtype ``work`` (float32 or float64). Nothing
here is imported by the product path and nothing of the product path is imported here. ``cfg`` is the parsed
``config.json``; ``w`` maps checkpoint names to tensors.
"""

from __future__ import annotations

import torch


def layer_norm(x, gain, eps):
    """(x - mean) / sqrt(var + eps) * gain over the last axis, var = mean of squared deviations; no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    dev = x - mu
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * gain


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gain


def rotate_neighbour_pairs(v, positions, base, dims):
    """Rotate the first ``dims`` channels of the last axis of ``v`` [tokens, heads, n]: channel 2i pairs with
    channel 2i + 1; the pair (a, b) at position p becomes (a cos t - b sin t, b cos t + a sin t) with
    t = p * base^(-2i/dims). Channels from ``dims`` on pass unchanged."""
    if dims == 0:
        return v
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    turned = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).reshape(*v.shape[:-1], dims)
    return torch.cat([turned, v[..., dims:]], dim=-1)


def sink_softmax_attention(q, k, v, scale, sink):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]; query head h reads key/value head h // (H / G); position i sees
    every j <= i; the softmax denominator also holds exp(sink[h]), which has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    top = torch.maximum(s.max(dim=-1).values, sink[:, None])              # [H, T]
    e = torch.exp(s - top[..., None])
    denom = e.sum(dim=-1) + torch.exp(sink[:, None] - top)
    p = e / denom[..., None]
    return torch.einsum("hij,jhd->ihd", p, v)


def attention(h, w, p, m, eps):
    """The mixer. ``m``: its sizes from config.json; ``p``: tensor-name prefix ('l3.mix.')."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).reshape(T, H, dk)
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).reshape(T, G, dk)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q = rotate_neighbour_pairs(q, pos, base, dims)
    k = rotate_neighbour_pairs(k, pos, base, dims)
    o = sink_softmax_attention(q, k, v, m["scale"], w[p + "sink"])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def clamped_expert(h, w, p, limit):
    """g = min(gate h, limit), u = clamp(up h, -limit, limit); down(g * sigmoid(1.702 g) * (u + 1))."""
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w_router, r, margins=None):
    """(chosen experts [T, top], their weights [T, top]): sigmoid scores; experts lie in ``groups.count`` equal
    groups of neighbours, a group scores the sum of its two largest scores, only the ``groups.keep`` best groups
    may be chosen from; the ``top`` largest scores among those; weights = scores / (their sum + 1e-20) * scale.
    ``margins``: a list that receives, per token, by how much the choice was clear: the smaller of (last kept group's
    score - best dropped group's) and (last chosen score - best score left out among the kept groups)."""
    n, top = r["experts"], r["top"]
    s = torch.sigmoid(h.to(torch.float32) @ w_router.to(torch.float32).T).to(h.dtype)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    size = n // count
    per_group = s.reshape(-1, count, size)
    group_score = per_group.topk(min(2, size), dim=-1).values.sum(dim=-1)             # [T, count]
    kept = group_score.topk(keep, dim=-1).indices
    open_groups = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, kept, True)
    allowed = open_groups[:, :, None].expand(-1, count, size).reshape(-1, n)
    masked = s.masked_fill(~allowed, float("-inf"))
    val, idx = torch.topk(masked, top, dim=-1)
    wt = val / (val.sum(dim=-1, keepdim=True) + 1e-20) * r["scale"]
    if margins is not None:
        clear = torch.full((s.shape[0],), float("inf"), dtype=s.dtype)
        if keep < count:
            g = group_score.sort(dim=-1, descending=True).values
            clear = torch.minimum(clear, g[:, keep - 1] - g[:, keep])
        if top < keep * size:
            e = masked.sort(dim=-1, descending=True).values
            clear = torch.minimum(clear, e[:, top - 1] - e[:, top])
        margins.append(clear)
    return idx, wt


def mixture(h, w, p, f, margins=None):
    """Weighted sum of the chosen experts' outputs plus the shared expert's."""
    idx, wt = route(h, w[p + "router"], f["router"], margins)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(f["router"]["experts"]):
        share = (wt * (idx == e)).sum(dim=-1, keepdim=True)
        out = out + share * clamped_expert(h, w, p + f"e{e}.", f["expert"]["limit"])
    if f.get("shared"):
        out = out + clamped_expert(h, w, p + "shared.", f["shared"]["limit"])
    return out


def layer(x, w, owner, L, eps, margins=None):
    """Parallel block with two norms: x + mixer(norm1 x) + ff(norm2 x); ``owner``: the layer whose tensors are used."""
    p = f"l{owner}."
    if L["type"] != "attention":
        raise ValueError(f"unknown mixer {L['type']!r}")
    y = attention(layer_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps)
    f = L.get("mlp")
    if f is not None:
        if f["kind"] != "moe":
            raise ValueError(f"unknown feed-forward {f['kind']!r}")
        y = y + mixture(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.", f, margins)
    return x + y


def forward(cfg, w, tokens, work=torch.float64, keep_stream=False, margins=None):
    """Logits [tokens, vocab] of one sequence (and, if asked, the stream after every layer). ``margins``: a list that
    receives one tensor [tokens] per routed layer: how clear each token's choice of experts was (``route``)."""
    w = {k: (v.to(work) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = layer_norm(w["embed"][ids], w["embed.norm"], eps)
    kept = []
    for i, L in enumerate(cfg["layers"]):
        x = layer(x, w, L.get("weights_of", i), L, eps, margins)
        kept.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(kept)) if keep_stream else logits


def greedy_generate(cfg, w, prompt, n, work=torch.float64):
    """The ``n`` tokens that always taking the largest logit gives after ``prompt`` (the whole sequence is run again
    for every token: slow and plain)."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(forward(cfg, w, seq, work)[-1]))
        out.append(tok)
        seq.append(tok)
    return out

