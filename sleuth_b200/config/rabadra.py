"""The Rabadra decoder: its typed configuration and its model description.

A Rabadra ``config.json`` names the design in ``architecture`` and nests its sizes::

    {"architecture": "Rabadra", "vocab": V, "width": d, "norm": {"eps": e}, "logit_softcap": c,
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"base", "dims"}},
                 "mlp": null | {"kind": "moe", "expert": {"ff", "limit"},
                                "router": {"experts", "top", "scale", "groups": {"count", "keep"}},
                                "shared": {"ff", "limit"}},
                 "weights_of": j (optional)},
                ...]}

The model: token embedding followed by a layer norm (gain only); *parallel* layers with two layer norms
(x += mixer(norm1 x) + ff(norm2 x), both of the same x); the mixer is grouped-query attention with one RMS norm over
the whole query projection and one over the whole key projection, a rotation of neighbouring channels over the first
``rot.dims`` channels of each head, its own score scale, values of their own width and a learned sink per head in the
softmax denominator (``parts/attention.py``); the feed-forward is a mixture of experts with the clamped swish, sigmoid
scores, a choice limited to the best groups of experts and a shared expert (``parts/moe.py``), or absent. A layer with
``weights_of: j`` has no tensors: it runs with layer j's and keeps a cache entry of its own. Final layer norm, untied
output matrix, soft-capped logits. Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.<q|k|v|q.norm|k.norm|sink|o>``, ``l<i>.mlp.<router|e<k>.gate|e<k>.up|e<k>.down|shared.gate|shared.up|
shared.down>``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..parts.spec import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec,
                          RoutedExpertsSpec, shared_weight_schedule)
from .base import ConfigError, read_fields

# The constants the design fixes.
SWISH_ALPHA = 1.702          # the experts' gate: g * sigmoid(1.702 g)


@dataclass(frozen=True)
class _Rot:
    base: float
    dims: int


@dataclass(frozen=True)
class _Mixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: dict


@dataclass(frozen=True)
class _Expert:
    ff: int
    limit: float


@dataclass(frozen=True)
class _Groups:
    count: int
    keep: int


@dataclass(frozen=True)
class _Router:
    experts: int
    top: int
    scale: float = 1.0
    groups: dict | None = None


@dataclass(frozen=True)
class _Moe:
    kind: str
    expert: dict
    router: dict
    shared: dict | None = None


@dataclass(frozen=True)
class _Layer:
    type: str
    mixer: dict
    mlp: dict | None = None
    weights_of: int | None = None


@dataclass(frozen=True)
class _Norm:
    eps: float


MIXERS = ("attention",)


def _strict(cls, d, where):
    """``read_fields`` that also refuses keys the class does not name (unless their value is null): a key that nobody
    reads is a part of the model that would silently be left out."""
    obj, unread = read_fields(cls, d, where)
    unread = [k for k in unread if d[k] is not None]       # a key set to null says that the thing is absent
    if unread:
        raise ConfigError(f"{where}: unknown key(s) {unread}")
    return obj


@dataclass(frozen=True)
class RabadraConfig:
    vocab: int
    width: int
    layers: tuple[dict, ...]
    norm: dict
    logit_softcap: float | None = None
    architecture: str = "Rabadra"
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
        need(self.logit_softcap is None or self.logit_softcap > 0, f"logit_softcap must be positive, got {self.logit_softcap}")
        parsed = []
        for i, raw in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            j = raw.get("weights_of") if isinstance(raw, dict) else None
            if isinstance(j, int) and not isinstance(j, bool) and 0 <= j < len(self.layers) and isinstance(self.layers[j], dict):
                raw = {**{k: v for k, v in self.layers[j].items() if k != "weights_of"}, **raw}    # what it leaves out is the lender's
            L = _strict(_Layer, raw, where)
            need(L.type in MIXERS, f"layers[{i}].type {L.type!r} is not a known mixer {list(MIXERS)}")
            m = _strict(_Mixer, L.mixer, where + ".mixer")
            rot = _strict(_Rot, m.rot, where + ".mixer.rot")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                need(getattr(m, key) > 0, f"layers[{i}].mixer.{key} must be positive, got {getattr(m, key)}")
            need(m.heads % m.kv_heads == 0, f"layers[{i}].mixer: heads ({m.heads}) must be a multiple of kv_heads ({m.kv_heads})")
            need(m.dim % 2 == 0, f"layers[{i}].mixer.dim ({m.dim}) must be even")
            need(0 <= rot.dims <= m.dim and rot.dims % 2 == 0,
                 f"layers[{i}].mixer: rot.dims ({rot.dims}) must be even and at most dim ({m.dim})")
            need(rot.base > 0 and m.scale > 0, f"layers[{i}].mixer: rot.base and scale must be positive")
            f = None
            if L.mlp is not None:
                kind = L.mlp.get("kind") if isinstance(L.mlp, dict) else None
                if kind != "moe":
                    raise ConfigError(f"{where}.mlp.kind {kind!r} is not 'moe'")
                moe = _strict(_Moe, L.mlp, where + ".mlp")
                ex = _strict(_Expert, moe.expert, where + ".mlp.expert")
                ro = _strict(_Router, moe.router, where + ".mlp.router")
                gr = _strict(_Groups, ro.groups, where + ".mlp.router.groups") if ro.groups is not None else _Groups(1, 1)
                sh = _strict(_Expert, moe.shared, where + ".mlp.shared") if moe.shared is not None else None
                need(ex.ff > 0 and ex.limit > 0 and 0 < ro.top <= ro.experts,
                     f"layers[{i}].mlp: expert.ff {ex.ff}, expert.limit {ex.limit}, router.experts {ro.experts}, router.top {ro.top}")
                need(gr.count >= 1 and ro.experts % gr.count == 0 and 1 <= gr.keep <= gr.count,
                     f"layers[{i}].mlp.router: {ro.experts} experts in {gr.count} groups of which {gr.keep} are kept")
                need(gr.keep * (ro.experts // gr.count) >= ro.top,
                     f"layers[{i}].mlp.router: {gr.keep} groups of {ro.experts // gr.count} experts cannot give {ro.top} choices")
                need(sh is None or (sh.ff > 0 and sh.limit > 0), f"layers[{i}].mlp.shared: ff and limit must be positive")
                f = (ex, ro, gr, sh)
            if L.weights_of is not None:
                need(0 <= L.weights_of < len(self.layers) and L.weights_of != i,
                     f"layers[{i}].weights_of {L.weights_of} names no other layer")
            parsed.append((L.type, m, rot, f, L.weights_of))
        owners = []
        for i, p in enumerate(parsed):
            j, seen = i, set()
            while parsed[j][4] is not None:     # a borrowed layer may itself borrow
                need(j not in seen, f"layers[{i}].weights_of leads in a circle")
                seen.add(j)
                j = parsed[j][4]
            need(parsed[j][1:4] == p[1:4], f"layers[{i}] borrows layer {j}'s weights but its mixer or mlp differs")
            owners.append(j)
        object.__setattr__(self, "parsed_layers", tuple(parsed))
        object.__setattr__(self, "owners", tuple(owners))

    @property
    def stop_ids(self) -> tuple[int, ...]:
        if self.eos_token_id is None:
            return ()
        return (self.eos_token_id,) if isinstance(self.eos_token_id, int) else tuple(self.eos_token_id)


def rabadra_model_spec(cfg: RabadraConfig, tensor_names=None) -> ModelSpec:
    d, eps = cfg.width, cfg.eps

    def norm():
        return NormSpec(d, eps, kind="layernorm")

    holders = sorted(set(cfg.owners))               # the layers that have tensors, in file order
    index = {i: n for n, i in enumerate(holders)}
    layers, ignored = [], []
    for i in holders:
        _, m, rot, f, _ = cfg.parsed_layers[i]
        p = f"l{i}."
        names = {"norm1.weight": p + "norm1"}
        for local, theirs in (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"), ("o_proj.weight", "o"),
                              ("q_norm.weight", "q.norm"), ("k_norm.weight", "k.norm"), ("sinks", "sink")):
            names["mixer." + local] = p + "mix." + theirs
        mixer = AttentionSpec(
            hidden=d, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale,
            qk_norm=True, qk_norm_eps=eps, qk_norm_span="projection", sinks=True,
            position=PositionSpec(head_dim=m.dim, theta=rot.base, rotary_dim=rot.dims, pairing="neighbours", precise=True,
                                  kind="rotary" if rot.dims else "none"))
        ffn = None
        if f is None:
            ignored.append(rf"l{i}\.norm2")         # a layer without feed-forward reads no second norm
        else:
            ex, ro, gr, sh = f
            names["norm2.weight"] = p + "norm2"
            shared = None
            if sh is not None:
                shared = GatedMLPSpec(hidden=d, intermediate=sh.ff, activation="clamped_swish", limit=sh.limit, alpha=SWISH_ALPHA)
                for local in ("gate", "up", "down"):
                    names[f"ffn.shared.{local}.weight"] = p + f"mlp.shared.{local}"
            ffn = RoutedExpertsSpec(hidden=d, intermediate=ex.ff, experts=ro.experts, top=ro.top, activation="clamped_swish",
                                    limit=ex.limit, alpha=SWISH_ALPHA, router_bias=False, scoring="sigmoid", groups=gr.count,
                                    keep_groups=gr.keep, route_scale=ro.scale, shared=shared)
            names["ffn.router.weight"] = p + "mlp.router"
            for e in range(ro.experts):
                for local in ("gate", "up", "down"):
                    names[f"ffn.e{e}.{local}.weight"] = p + f"mlp.e{e}.{local}"
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm1=norm(), norm2=norm() if ffn is not None else None, names=names,
                                kind="parallel"))
    return ModelSpec(
        embedding=EmbeddingSpec(vocab=cfg.vocab, dim=d, name="embed", norm=norm(), norm_name="embed.norm"),
        layers=tuple(layers), schedule=shared_weight_schedule([index[o] for o in cfg.owners]),
        head=HeadSpec(vocab=cfg.vocab, dim=d, norm=norm(), tied=False, norm_name="final.norm", name="head",
                      softcap=cfg.logit_softcap or 0.0),
        max_positions=cfg.max_positions, ignored_tensors=tuple(ignored))
