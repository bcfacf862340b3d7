"""The Lezepel decoder: its typed configuration and its model description.

A Lezepel ``config.json`` names the design in ``architecture`` and nests its sizes::

    {"architecture": "Lezepel", "vocab": V, "width": d, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot": {"base", "dims"}},
                 "mlp": null | {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}},
                ...],
     "loop": {"start", "stop", "times"}}

The model: scaled token embedding; *parallel* layers (one RMSNorm whose output both the mixer and the
feed-forward read, x += mixer(h) + ff(h)); the mixer is attention through low-rank latents with an
output gate (``parts/latent_attention.py``); the feed-forward is a gated ReLU layer or routed SiLU
experts (``parts/ffn.py``, ``parts/moe.py``), or absent; layers ``loop.start .. loop.stop - 1`` run
``loop.times`` times in a row with the same weights and caches of their own, each pass starting with
the addition of its row of ``loop.step`` (and, from the second pass on, of the embedding's output);
final RMSNorm and an untied output matrix. Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1``,
``l<i>.mix.<dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o>``, ``l<i>.mlp.<gate|up|down>`` or
``l<i>.mlp.<router|router.b|e<k>.gate|e<k>.up|e<k>.down>``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..parts.spec import (EmbeddingSpec, GatedMLPSpec, HeadSpec, LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec,
                          PositionSpec, RoutedExpertsSpec, looped_schedule, straight_schedule)
from .base import ConfigError, read_fields


@dataclass(frozen=True)
class _Rot:
    base: float
    dims: int


@dataclass(frozen=True)
class _Mixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: dict


@dataclass(frozen=True)
class _Dense:
    kind: str
    ff: int


@dataclass(frozen=True)
class _Moe:
    kind: str
    expert: dict
    router: dict


@dataclass(frozen=True)
class _ExpertSizes:
    ff: int


@dataclass(frozen=True)
class _Router:
    experts: int
    top: int


@dataclass(frozen=True)
class _Layer:
    type: str
    mixer: dict
    mlp: dict | None = None


@dataclass(frozen=True)
class _Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class _Norm:
    eps: float


@dataclass(frozen=True)
class _Embedding:
    scale: float = 1.0


MIXERS = ("latent_attention",)


def _strict(cls, d, where):
    """``read_fields`` that also refuses keys the class does not name: in this family a key that nobody reads is a
    part of the model that would silently be left out."""
    obj, unread = read_fields(cls, d, where)
    if unread:
        raise ConfigError(f"{where}: unknown key(s) {unread}")
    return obj


@dataclass(frozen=True)
class LezepelConfig:
    vocab: int
    width: int
    layers: tuple[dict, ...]
    norm: dict
    embedding: dict | None = None
    loop: dict | None = None
    architecture: str = "Lezepel"
    max_positions: int = 1 << 20        # the design sets no limit; tables are built for what the engine is asked to hold
    eos_token_id: int | tuple[int, ...] | None = None

    def __post_init__(self):
        def need(cond, msg):
            if not cond:
                raise ConfigError("config.json: " + msg)

        need(self.vocab > 0 and self.width > 0, f"vocab ({self.vocab}) and width ({self.width}) must be positive")
        need(len(self.layers) > 0, "layers is empty")
        object.__setattr__(self, "eps", _strict(_Norm, self.norm, "config.json: norm").eps)
        need(self.eps > 0, f"norm.eps must be positive, got {self.eps}")
        emb = _strict(_Embedding, self.embedding, "config.json: embedding") if self.embedding is not None else _Embedding()
        object.__setattr__(self, "embedding_scale", emb.scale)
        parsed = []
        for i, raw in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            L = _strict(_Layer, raw, where)
            need(L.type in MIXERS, f"layers[{i}].type {L.type!r} is not a known mixer {list(MIXERS)}")
            m = _strict(_Mixer, L.mixer, where + ".mixer")
            rot = _strict(_Rot, m.rot, where + ".mixer.rot")
            for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                need(getattr(m, key) > 0, f"layers[{i}].mixer.{key} must be positive, got {getattr(m, key)}")
            need(m.rot_dim >= 0 and 0 <= rot.dims <= m.rot_dim and rot.dims % 2 == 0,
                 f"layers[{i}].mixer: rot.dims ({rot.dims}) must be even and at most rot_dim ({m.rot_dim})")
            need(rot.base > 0 and m.scale > 0, f"layers[{i}].mixer: rot.base and scale must be positive")
            f = None
            if L.mlp is not None:
                kind = L.mlp.get("kind") if isinstance(L.mlp, dict) else None
                if kind == "dense":
                    f = _strict(_Dense, L.mlp, where + ".mlp")
                    need(f.ff > 0, f"layers[{i}].mlp.ff must be positive")
                elif kind == "moe":
                    moe = _strict(_Moe, L.mlp, where + ".mlp")
                    ex = _strict(_ExpertSizes, moe.expert, where + ".mlp.expert")
                    ro = _strict(_Router, moe.router, where + ".mlp.router")
                    need(ex.ff > 0 and 0 < ro.top <= ro.experts,
                         f"layers[{i}].mlp: expert.ff {ex.ff}, router.experts {ro.experts}, router.top {ro.top}")
                    f = (ex, ro)
                else:
                    raise ConfigError(f"{where}.mlp.kind {kind!r} is not 'dense' or 'moe'")
            parsed.append((L.type, m, rot, f))
        object.__setattr__(self, "parsed_layers", tuple(parsed))
        lp = _strict(_Loop, self.loop, "config.json: loop") if self.loop is not None else None
        if lp is not None:
            need(0 <= lp.start <= lp.stop <= len(self.layers) and lp.times >= 1,
                 f"loop {self.loop} does not fit {len(self.layers)} layers")
        object.__setattr__(self, "parsed_loop", lp)

    @property
    def stop_ids(self) -> tuple[int, ...]:
        if self.eos_token_id is None:
            return ()
        return (self.eos_token_id,) if isinstance(self.eos_token_id, int) else tuple(self.eos_token_id)


def lezepel_model_spec(cfg: LezepelConfig, tensor_names=None) -> ModelSpec:
    d, eps = cfg.width, cfg.eps
    layers = []
    for i, (_, m, rot, f) in enumerate(cfg.parsed_layers):
        p = f"l{i}."
        names = {"norm1.weight": p + "norm1"}
        for local, theirs in (("dq.weight", "dq"), ("dq_norm.weight", "dq.norm"), ("uq.weight", "uq"), ("dkv.weight", "dkv"),
                              ("dkv_norm.weight", "dkv.norm"), ("uk.weight", "uk"), ("uv.weight", "uv"),
                              ("g.weight", "g"), ("o.weight", "o")):
            names["mixer." + local] = p + "mix." + theirs
        mixer = LatentAttentionSpec(
            hidden=d, heads=m.heads, plain_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, q_rank=m.q_rank,
            kv_rank=m.kv_rank, scale=m.scale, norm_eps=eps,
            position=PositionSpec(head_dim=m.rot_dim, theta=rot.base, rotary_dim=rot.dims,
                                  kind="rotary" if rot.dims else "none"))
        if f is None:
            ffn = None
        elif isinstance(f, _Dense):
            ffn = GatedMLPSpec(hidden=d, intermediate=f.ff, activation="relu")
            for local in ("gate", "up", "down"):
                names[f"ffn.{local}.weight"] = p + "mlp." + local
        else:
            ex, ro = f
            ffn = RoutedExpertsSpec(hidden=d, intermediate=ex.ff, experts=ro.experts, top=ro.top, activation="silu")
            names["ffn.router.weight"] = p + "mlp.router"
            names["ffn.router.bias"] = p + "mlp.router.b"
            for e in range(ro.experts):
                for local in ("gate", "up", "down"):
                    names[f"ffn.e{e}.{local}.weight"] = p + f"mlp.e{e}.{local}"
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm1=NormSpec(d, eps), norm2=None, names=names, kind="parallel"))
    lp = cfg.parsed_loop
    if lp is not None and lp.stop > lp.start:
        schedule = looped_schedule(len(layers), lp.start, lp.stop, lp.times)
        pass_rows, rows = "loop.step", lp.times
    else:
        schedule, pass_rows, rows = straight_schedule(len(layers)), None, 0
    return ModelSpec(
        embedding=EmbeddingSpec(vocab=cfg.vocab, dim=d, scale=cfg.embedding_scale, name="embed"),
        layers=tuple(layers), schedule=schedule,
        head=HeadSpec(vocab=cfg.vocab, dim=d, norm=NormSpec(d, eps), tied=False, norm_name="final.norm", name="head"),
        max_positions=cfg.max_positions, pass_rows=pass_rows, pass_rows_count=rows,
        ignored_tensors=(() if pass_rows else (r"loop\.step$",)))
