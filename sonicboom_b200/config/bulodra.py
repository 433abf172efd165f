"""Typed configuration of the Bulodra decoder, read from its own config.json keys.

A Bulodra model is a list of layers without a norm before a sublayer: a sublayer reads the
stream itself, its result is RMS-normed and joins the stream times a constant,
x1 = x + m n1(mix(x)); x2 = x1 + m n2(ffn(x1)).  A token's embedding is its own row plus a row of
a second table chosen by a hash of the previous and the current token.  A layer's mixer is one of
three kinds of softmax attention (below); its feed-forward is a dense gated one with gelu or a
mixture of clamped gated experts whose router scores are logistic functions, chosen within the
best groups of experts, plus a shared expert.  The logits are the head's product times a
constant.  config.json gives every size and every constant that may differ between models:

    architecture                "Bulodra"
    vocab, width                sizes of the embedding / head and of the residual stream
    norm.eps                    eps of every norm
    residual_mult               m
    logit_scale                 multiplies the logits
    embedding.bigram            {buckets, mul_prev, mul_cur} of the second embedding table
    layers[i].type              "attention" | "latent_attention" | "attention_2"
    layers[i].mixer             that mixer's sizes and constants (below)
    layers[i].mlp               null, {kind: "dense", ff}, or {kind: "moe", router {experts, top, scale,
                                groups {count, keep} (optional)}, expert {ff, limit}, shared {ff, limit}
                                (optional)}

    attention:          heads, kv_heads, dim, vdim, scale, rot; q, k and v have biases, every q and k
                        head is RMS-normed (one weight for all heads) before the rotation, and a
                        learned number per head joins the softmax's denominator
    latent_attention:   heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot; queries and keys/values
                        go through normed latents, one rotated key part is shared by the heads, and the
                        softmax has the same kind of number per head
    attention_2:        heads, kv_heads, dim, vdim, scale, softcap, mask {size}, rot; no biases, every
                        q and k head is divided by its root mean square after the rotation, scores are
                        capped with a tanh, the window is `mask.size` keys long, and every head's
                        result is gated by a logistic function of the mixer's input
    rot:                {base, dims, scaling {factor, original, fast, slow} (optional)}: the first
                        `dims` values of a head turn in pairs (i, i + dims/2); with `scaling` the slow
                        pairs are stretched (`parts.rotary.yarn_frequencies`)

What the design fixes is written into the part records by `to_spec`: the slope of the experts'
gate, that a group's score is the sum of its two largest choice scores, that the chosen experts'
weights are not renormalised, gelu's tanh form, and the tensor names (`l<i>.norm1`, `l<i>.mix.q`,
`l<i>.mix.q.b`, `l<i>.mix.q.norm`, `l<i>.mix.sink`, `l<i>.mix.g`, `l<i>.mlp.e<j>.gate`,
`l<i>.mlp.correction`, `bigram`, ...).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .specs import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PairEmbeddingSpec,
                    PositionSpec, ScheduleEntry)
from .leguvik import PairTableConfig
from .zolulix import MAX_POSITIONS, _num, _sub

GLU_SLOPE = 1.702            # of the experts' gate, g * sigmoid(slope g)
GROUP_TOP = 2                # a group of experts is scored by the sum of this many of its choice scores
MIXER_TYPES = ("attention", "latent_attention", "attention_2")


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: Optional[tuple] = None      # (factor, original, fast, slow)


@dataclass(frozen=True)
class BulodraMixer:
    heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotationConfig
    kv_heads: int = 0          # attention, attention_2
    rot_dim: int = 0           # latent_attention
    kv_rank: int = 0
    q_rank: int = 0
    softcap: float = 0.0       # attention_2
    window: int = 0            # attention_2: mask.size


@dataclass(frozen=True)
class BulodraMlp:
    kind: str                  # "dense" | "moe"
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    groups: Optional[tuple] = None     # (count, keep)
    shared_ff: int = 0
    shared_limit: float = 0.0


@dataclass(frozen=True)
class BulodraLayer:
    type: str
    mixer: BulodraMixer
    mlp: Optional[BulodraMlp]


def _rot(m: dict, w: str) -> RotationConfig:
    r = _sub(m, "rot", w)
    w = w + "rot."
    dims = _num(r, "dims", w, positive=False)
    if dims < 0 or dims % 2:
        raise ConfigError(f"missing/invalid config key: {w}dims (an even number >= 0, got {dims})")
    scaling = None
    if r.get("scaling") is not None:
        s = _sub(r, "scaling", w)
        scaling = tuple(_num(s, k, w + "scaling.", float) for k in ("factor", "original", "fast", "slow"))
    return RotationConfig(base=_num(r, "base", w, float), dims=dims, scaling=scaling)


def _mixer(kind, m: dict, w: str) -> BulodraMixer:
    if kind not in MIXER_TYPES:
        raise ConfigError(f"unsupported config key: {w[:-6]}type = {kind!r} ({', '.join(MIXER_TYPES)})")
    common = dict(heads=_num(m, "heads", w), dim=_num(m, "dim", w), vdim=_num(m, "vdim", w),
                  scale=_num(m, "scale", w, float), rot=_rot(m, w))
    if kind == "latent_attention":
        c = BulodraMixer(**common, rot_dim=_num(m, "rot_dim", w), kv_rank=_num(m, "kv_rank", w),
                         q_rank=_num(m, "q_rank", w))
        if c.rot.dims > c.rot_dim:
            raise ConfigError(f"missing/invalid config key: {w}rot.dims ({c.rot.dims} of {c.rot_dim} rotated dimensions)")
        return c
    extra = {}
    if kind == "attention_2":
        extra = dict(softcap=_num(m, "softcap", w, float, positive=False) if m.get("softcap") is not None else 0.0,
                     window=_num(_sub(m, "mask", w), "size", w + "mask.") if m.get("mask") is not None else 0)
        if extra["softcap"] < 0:
            raise ConfigError(f"missing/invalid config key: {w}softcap (must be >= 0)")
    c = BulodraMixer(**common, kv_heads=_num(m, "kv_heads", w), **extra)
    if c.heads % c.kv_heads:
        raise ConfigError(f"missing/invalid config key: {w}kv_heads ({c.heads} query heads are not a multiple "
                          f"of {c.kv_heads})")
    if c.rot.dims > c.dim:
        raise ConfigError(f"missing/invalid config key: {w}rot.dims ({c.rot.dims} of {c.dim} dimensions)")
    return c


def _mlp(mlp, w: str) -> Optional[BulodraMlp]:
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, dict) else mlp
    if kind == "dense":
        return BulodraMlp(kind="dense", ff=_num(mlp, "ff", w))
    if kind != "moe":
        raise ConfigError(f"unsupported config key: {w}kind = {kind!r} (dense or moe)")
    r, e = _sub(mlp, "router", w), _sub(mlp, "expert", w)
    shared = mlp.get("shared")
    groups = None
    if r.get("groups") is not None:
        g = _sub(r, "groups", w + "router.")
        groups = (_num(g, "count", w + "router.groups."), _num(g, "keep", w + "router.groups."))
    c = BulodraMlp(
        kind="moe", ff=_num(e, "ff", w + "expert."), limit=_num(e, "limit", w + "expert.", float),
        experts=_num(r, "experts", w + "router."), top=_num(r, "top", w + "router."),
        route_scale=_num(r, "scale", w + "router.", float) if r.get("scale") is not None else 1.0, groups=groups,
        shared_ff=0 if shared is None else _num(_sub(mlp, "shared", w), "ff", w + "shared."),
        shared_limit=0.0 if shared is None else _num(shared, "limit", w + "shared.", float))
    if c.top > c.experts:
        raise ConfigError(f"missing/invalid config key: {w}router.top ({c.top} of {c.experts} experts)")
    if groups is not None:
        count, keep = groups
        if c.experts % count or keep > count or keep * (c.experts // count) < c.top:
            raise ConfigError(f"missing/invalid config key: {w}router.groups ({c.experts} experts in {count} groups "
                              f"of which {keep} are kept cannot give {c.top} choices)")
    return c


@dataclass(frozen=True)
class BulodraConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_scale: float
    bigram: PairTableConfig
    layers: tuple
    architecture: str = "Bulodra"

    @classmethod
    def from_dict(cls, d: dict) -> "BulodraConfig":
        vocab, width = _num(d, "vocab", ""), _num(d, "width", "")
        eps = _num(_sub(d, "norm", ""), "eps", "norm.", float, positive=False)
        if eps < 0:
            raise ConfigError("missing/invalid config key: norm.eps (must be >= 0)")
        b = _sub(_sub(d, "embedding", ""), "bigram", "embedding.")
        bigram = PairTableConfig(buckets=_num(b, "buckets", "embedding.bigram."),
                                 mul_prev=_num(b, "mul_prev", "embedding.bigram.", positive=False),
                                 mul_cur=_num(b, "mul_cur", "embedding.bigram.", positive=False))
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("missing/invalid config key: layers (a non-empty list)")
        layers = []
        for i, L in enumerate(raw):
            w = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"missing/invalid config key: layers[{i}] (expected an object)")
            layers.append(BulodraLayer(L.get("type"), _mixer(L.get("type"), _sub(L, "mixer", w), w + "mixer."),
                                       _mlp(L.get("mlp"), w + "mlp.")))
        return cls(vocab=vocab, width=width, eps=eps,
                   residual_mult=_num(d, "residual_mult", "", float) if d.get("residual_mult") is not None else 1.0,
                   logit_scale=_num(d, "logit_scale", "", float) if d.get("logit_scale") is not None else 1.0,
                   bigram=bigram, layers=tuple(layers))

    def to_dict(self) -> dict:
        """config.json content that `from_dict` reads back to an equal configuration."""
        out = []
        for L in self.layers:
            m = L.mixer
            rot = {"base": m.rot.base, "dims": m.rot.dims}
            if m.rot.scaling is not None:
                rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), m.rot.scaling))
            mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "rot": rot}
            if L.type == "latent_attention":
                mixer.update(rot_dim=m.rot_dim, kv_rank=m.kv_rank, q_rank=m.q_rank)
            else:
                mixer["kv_heads"] = m.kv_heads
            if L.type == "attention_2":
                mixer["softcap"] = m.softcap
                if m.window:
                    mixer["mask"] = {"size": m.window}
            mlp = None
            if L.mlp is not None and L.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": L.mlp.ff}
            elif L.mlp is not None:
                e = L.mlp
                router = {"experts": e.experts, "top": e.top, "scale": e.route_scale}
                if e.groups is not None:
                    router["groups"] = {"count": e.groups[0], "keep": e.groups[1]}
                mlp = {"kind": "moe", "router": router, "expert": {"ff": e.ff, "limit": e.limit}}
                if e.shared_ff:
                    mlp["shared"] = {"ff": e.shared_ff, "limit": e.shared_limit}
            out.append({"type": L.type, "mixer": mixer, "mlp": mlp})
        b = self.bigram
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
                "embedding": {"bigram": {"buckets": b.buckets, "mul_prev": b.mul_prev, "mul_cur": b.mul_cur}},
                "layers": out}

    def to_spec(self) -> ModelSpec:
        """The model as parts: one output-norm block per layer."""
        d, eps = self.width, self.eps
        layers = []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            m = L.mixer
            vector = m.rot_dim if L.type == "latent_attention" else m.dim      # what the rotation acts on
            if m.rot.scaling is not None:
                position = PositionSpec("rope_halves_yarn", vector, m.rot.base, m.rot.dims,
                                        params=tuple(zip(("factor", "original", "fast", "slow"), m.rot.scaling)))
            else:
                position = PositionSpec("rope_halves", vector, m.rot.base, m.rot.dims)
            if L.type == "latent_attention":
                mixer = MixerSpec(
                    kind="latent_attention", width=d, n_heads=m.heads, head_dim=m.dim, scale=m.scale,
                    position=position, prefix=p + "mix.",
                    params=(("rot_dim", m.rot_dim), ("vdim", m.vdim), ("kv_rank", m.kv_rank), ("q_rank", m.q_rank),
                            ("sink", "sink"), ("eps", eps)))
            elif L.type == "attention":
                mixer = MixerSpec(
                    kind="window_attention", width=d, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                    scale=m.scale, position=position, prefix=p + "mix.",
                    params=(("vdim", m.vdim), ("eps", eps), ("bias", ("q.b", "k.b", "v.b")),
                            ("head_norm", ("before", "q.norm", "k.norm")), ("sink", "sink")))
            else:
                mixer = MixerSpec(
                    kind="window_attention", width=d, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                    window=m.window, scale=m.scale, position=position, prefix=p + "mix.",
                    params=(("vdim", m.vdim), ("eps", eps), ("head_norm", ("after",)), ("softcap", m.softcap),
                            ("gate", "g")))
            ff = None
            if L.mlp is not None and L.mlp.kind == "dense":
                ff = FeedForwardSpec(kind="swiglu", width=d, intermediate=L.mlp.ff, activation="gelu_tanh",
                                     prefix=p + "mlp.", params=(("names", ("gate", "up", "down")),))
            elif L.mlp is not None:
                e = L.mlp
                shared = None if not e.shared_ff else FeedForwardSpec(
                    kind="glu_clamped", width=d, intermediate=e.shared_ff, activation="glu_clamped",
                    prefix=p + "mlp.shared.",
                    params=(("limit", e.shared_limit), ("slope", GLU_SLOPE), ("names", ("gate", "up", "down"))))
                router = (("correction", "correction"), ("groups", e.groups or (1, 1)), ("group_top", GROUP_TOP),
                          ("scale", e.route_scale), ("renormalize", False))
                ff = FeedForwardSpec(
                    kind="experts_glu_clamped", width=d, intermediate=e.ff, activation="glu_clamped",
                    prefix=p + "mlp.",
                    params=(("experts", e.experts), ("top", e.top), ("limit", e.limit), ("slope", GLU_SLOPE),
                            ("shared", shared), ("router", router)))
            layers.append(LayerSpec(
                arrangement="output_norm", mixer=mixer, mixer_norm=None, feed_forward=ff, feed_forward_norm=None,
                mixer_post_norm=NormSpec("rmsnorm", d, eps, p + "norm1"),
                feed_forward_post_norm=NormSpec("rmsnorm", d, eps, p + "norm2") if ff is not None else None,
                params=(("residual_mult", self.residual_mult),)))
        b = self.bigram
        spec = ModelSpec(
            architecture=self.architecture, width=d, vocab=self.vocab, max_positions=MAX_POSITIONS,
            embedding_tensor="embed", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(self.layers))),
            final_norm=NormSpec("rmsnorm", d, eps, "final.norm"), head_tensor="head",
            logit_scale=self.logit_scale,
            pair_embedding=PairEmbeddingSpec("bigram", b.buckets, b.mul_prev, b.mul_cur))
        spec.validate()
        return spec
