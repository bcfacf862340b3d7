"""Plain Lezepel decoder: whole sequences, no cache, one function per mechanism.

Lezepel is a decoder whose layers are *parallel* blocks (one norm feeds both the mixer and the
feed-forward, and both results are added to the stream), whose mixer is attention through low-rank
latents (queries through a normed latent; keys and values rebuilt from one normed latent per token
plus one rotated key part shared by all heads; a sigmoid output gate), whose feed-forward is either
a gated ReLU layer or a routed mixture of gated SiLU experts, and in which a run of layers may be
applied several times in a row with the same weights.

Everything runs on the CPU with ordinary tensor operations in the dtype ``work`` (float32 or
float64). Nothing here is imported by the product path and nothing of the product path is imported
here. ``cfg`` is the parsed ``config.json``; ``w`` maps checkpoint names to tensors.
"""

from __future__ import annotations

import torch


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gain


def rotate_half_pairs(v, positions, base, dims):
    """Rotate the first ``dims`` channels of the last axis of ``v`` [tokens, ..., n]: channel i pairs with
    channel i + dims/2; the pair (a, b) at position p becomes (a cos t - b sin t, b cos t + a sin t) with
    t = p * base^(-2i/dims). Channels from ``dims`` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = ang.cos().reshape(shape), ang.sin().reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., dims:]], dim=-1)


def causal_softmax_attention(q, k, v, scale):
    """q, k [tokens, heads, dk], v [tokens, heads, dv]: position i attends to every j <= i."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def latent_attention(h, w, p, m, eps):
    """The mixer. ``m``: its sizes from config.json; ``p``: tensor-name prefix ('l3.mix.')."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], q[..., dn:]
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :r], w[p + "dkv.norm"], eps)
    k_rot = dkv[:, r:r + dr]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rot = rotate_half_pairs(q_rot, pos, base, dims)
    k_rot = rotate_half_pairs(k_rot[:, None, :], pos, base, dims).expand(T, H, dr)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    o = causal_softmax_attention(torch.cat([q_plain, q_rot], -1), torch.cat([k_plain, k_rot], -1), v, m["scale"])
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def dense_ffn(h, w, p):
    """down(relu(gate h) * (up h))."""
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_experts(h, w, p, f):
    """Each token uses the ``top`` experts with the largest router logits (W h + b); their weights are the
    softmax over those logits alone; an expert is down(silu(gate h) * (up h))."""
    n, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    wt = torch.softmax(val, dim=-1)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(n):
        q = p + f"e{e}."
        g = h @ w[q + "gate"].T
        y = ((g * torch.sigmoid(g)) * (h @ w[q + "up"].T)) @ w[q + "down"].T
        share = (wt * (idx == e)).sum(dim=-1, keepdim=True)
        out = out + share * y
    return out


def layer(x, w, i, L, eps):
    """Parallel block: h = norm(x); x + mixer(h) + ff(h)."""
    p = f"l{i}."
    h = rms_norm(x, w[p + "norm1"], eps)
    if L["type"] != "latent_attention":
        raise ValueError(f"layer {i}: unknown mixer {L['type']!r}")
    y = latent_attention(h, w, p + "mix.", L["mixer"], eps)
    f = L.get("mlp")
    if f is not None:
        if f["kind"] == "dense":
            y = y + dense_ffn(h, w, p + "mlp.")
        elif f["kind"] == "moe":
            y = y + routed_experts(h, w, p + "mlp.", f)
        else:
            raise ValueError(f"layer {i}: unknown feed-forward {f['kind']!r}")
    return x + y


def layer_runs(cfg):
    """The order in which layers are applied: [(layer index, pass number or None, first of its pass)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    runs += [(i, None, False) for i in range(b, n)]
    return runs


def forward(cfg, w, tokens, work=torch.float64, keep_stream=False):
    """Logits [tokens, vocab] of one sequence (and, if asked, the stream after every layer application)."""
    w = {k: (v.to(work) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = w["embed"][ids] * cfg["embedding"]["scale"]
    x = x0
    kept = []
    for i, t, first in layer_runs(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        x = layer(x, w, i, cfg["layers"][i], eps)
        kept.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
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
