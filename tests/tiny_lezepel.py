"""Tiny Lezepel configurations of the tests. They differ in every size and option: width, vocabulary (no power of
two in P and R), heads (1, 3, 6 and more than 32), unrotated / rotated / value head sizes (value size different
from the key's), latent ranks, rotation base, norm eps, embedding scale, attention scale, dense / routed / absent
feed-forwards in different orders, experts and choices (top 1 too), and the loop (two layers twice, one layer
three times from layer 0, none)."""

from __future__ import annotations


def mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(m, f):
    return {"type": "latent_attention", "mixer": m, "mlp": f}


_MP = mixer(3, 16, 8, 24, 20, 40, base=500.0, scale=0.31)
P = {"architecture": "Lezepel", "vocab": 301, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0},
     "layers": [layer(_MP, dense(100)), layer(_MP, moe(5, 2, 36)), layer(_MP, None), layer(_MP, moe(6, 1, 20))],
     "loop": {"start": 1, "stop": 3, "times": 2}}

_MQ = mixer(6, 32, 16, 32, 48, 64, base=20000.0)
Q = {"architecture": "Lezepel", "vocab": 257, "width": 128, "norm": {"eps": 2e-5}, "embedding": {"scale": 1.0},
     "layers": [layer(_MQ, moe(8, 3, 48)), layer(mixer(2, 24, 8, 40, 16, 56, base=3000.0), dense(192))],
     "loop": {"start": 0, "stop": 1, "times": 3}}

# one head in one layer, forty in the other (more than a block of the attention kernel takes at once); no loop
R = {"architecture": "Lezepel", "vocab": 203, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
     "layers": [layer(mixer(1, 16, 16, 8, 24, 24), dense(48)), layer(mixer(40, 8, 4, 8, 32, 28, base=100.0), moe(4, 4, 16))]}

# sizes that send prompts of 128 tokens and more through the tensor-memory products and single tokens through the
# weight-streaming kernel, whole prompts through the per-head attention kernel: every inner size a multiple of 16
_MS = mixer(4, 64, 32, 48, 128, 128)
S = {"architecture": "Lezepel", "vocab": 640, "width": 320, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
     "layers": [layer(_MS, dense(640)), layer(_MS, moe(8, 2, 128)), layer(_MS, moe(8, 2, 128))],
     "loop": {"start": 1, "stop": 2, "times": 2}}

CONFIGS = {"P": P, "Q": Q, "R": R, "S": S}
SEEDS = {"P": 101, "Q": 202, "R": 303, "S": 404}
STD = 0.08      # wide enough that attention is far from uniform and the experts' shares differ


def spread_router_biases(folder, factor: float = 40.0) -> None:
    """Rewrite a written folder with its router biases multiplied by ``factor``. With biases about three times as
    wide as the logits' token-dependent part the choice of experts still changes from token to token, but two logits
    seldom lie closer than a bfloat16 run's rounding of the layer input, so that the bfloat16 run and the plain
    implementation mostly send a token to the same experts."""
    from pathlib import Path

    from plain.qwen3_plain import read_safetensors
    from sleuth_b200.weights.safetensors import write_safetensors
    path = Path(folder) / "model.safetensors"
    tensors = read_safetensors(path)
    for name in tensors:
        if name.endswith(".router.b"):
            tensors[name] = tensors[name] * factor
    write_safetensors(tensors, path, metadata={"format": "pt"})
