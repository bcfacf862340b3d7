"""Tiny Rabadra configurations of the tests. They differ in every size and option: width, vocabulary (no power of two
in A and B), query and key/value heads (ratios 3, 1, 8, 4, 2), key and value widths (equal and unequal), the rotated
share of a head (a part, all, none), rotation base, attention scale, norm eps, experts, choices (1, 2, 3, all), groups
(absent, some kept, all kept, groups of one expert), clamp limits, router scale, shared expert (present, absent), a
layer without feed-forward, borrowed weights (in order, in reverse order), and the logit cap (present, absent)."""

from __future__ import annotations


def mixer(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
            "rot": {"base": base, "dims": rot_dims}}


def moe(experts, top, ff, limit, scale=1.0, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(m, f, weights_of=None):
    out = {"type": "attention", "mixer": m, "mlp": f}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


_MA = mixer(6, 2, 16, 24, 8, base=500.0, scale=0.31)
_FA = moe(6, 2, 20, 1.0, scale=1.5, groups=(3, 2), shared=(28, 2.5))
A = {"architecture": "Rabadra", "vocab": 301, "width": 72, "norm": {"eps": 1e-6}, "logit_softcap": 7.5,
     "layers": [layer(_MA, _FA), layer(_MA, None), layer(_MA, _FA, weights_of=0)]}

_MB0, _FB0 = mixer(4, 4, 32, 32, 32, base=20000.0), moe(8, 1, 48, 3.0, scale=0.7)
_MB1, _FB1 = mixer(8, 1, 24, 40, 0, scale=0.2), moe(4, 4, 36, 0.75, scale=2.5, groups=(4, 4), shared=(16, 1.0))
B = {"architecture": "Rabadra", "vocab": 257, "width": 128, "norm": {"eps": 2e-5},
     "layers": [layer(_MB0, _FB0), layer(_MB1, _FB1), layer(_MB1, _FB1, weights_of=1), layer(_MB0, _FB0, weights_of=0)]}

# head sizes the tensor-core attention kernels take (64, equal key and value widths), every inner size a multiple of
# 32: prompts of 128 tokens and more go through the tensor-memory products, single tokens through the weight-streaming one
_MC = mixer(8, 2, 64, 64, 32, base=3000.0)
_FC = moe(8, 2, 128, 2.0, scale=1.25, groups=(2, 1), shared=(192, 1.5))
C = {"architecture": "Rabadra", "vocab": 640, "width": 256, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
     "layers": [layer(_MC, _FC), layer(_MC, moe(16, 3, 64, 4.0, groups=(4, 2))), layer(_MC, _FC, weights_of=0)]}

# head size 128 with all of it rotated, one kv head per two query heads; sixteen experts in four groups
_MD = mixer(4, 2, 128, 128, 128, base=1000.0, scale=0.07)
D = {"architecture": "Rabadra", "vocab": 512, "width": 192, "norm": {"eps": 1e-5}, "logit_softcap": 50.0,
     "layers": [layer(_MD, moe(16, 4, 64, 7.0, scale=2.0, groups=(4, 2), shared=(64, 7.0))), layer(_MD, None, weights_of=None)]}

CONFIGS = {"A": A, "B": B, "C": C, "D": D}
SEEDS = {"A": 111, "B": 222, "C": 333, "D": 444}
STD = 0.08      # wide enough that attention is far from uniform and the experts' shares differ


def sharpen(folder, logit_std: float = 2.5, sink_std: float = 1.5, round_router: bool = False) -> None:
    """Rewrite a written folder so that faults show: the routers' rows are scaled until their logits have about
    ``logit_std`` (the scores then spread over (0, 1), the choice changes from token to token, and two scores seldom lie
    closer than a bfloat16 run's rounding of the layer input), and the sinks until they have about ``sink_std`` (a
    sink that is left out, scaled, or given to the wrong head then moves the result). ``round_router``: the routers'
    matrices are then rounded to bfloat16 values (kept in float32), as a file that stores bfloat16 weights has them: a
    bfloat16 run then forms their logits as a product of its own."""
    from pathlib import Path

    from plain.qwen3_plain import read_safetensors
    from sleuth_b200.weights.safetensors import write_safetensors
    path = Path(folder) / "model.safetensors"
    tensors = read_safetensors(path)
    for name, t in tensors.items():
        if name.endswith(".mlp.router"):
            tensors[name] = t * (logit_std / (float(t.float().std()) * t.shape[1] ** 0.5))
            if round_router:
                import torch
                tensors[name] = tensors[name].to(torch.bfloat16).to(t.dtype)
        elif name.endswith(".mix.sink"):
            tensors[name] = t * (sink_std / max(float(t.float().std()), 1e-6))
    write_safetensors(tensors, path, metadata={"format": "pt"})
