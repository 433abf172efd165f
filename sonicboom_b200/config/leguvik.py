"""Typed configuration of the Leguvik decoder, read from its own config.json keys.

A Leguvik model is a list of layers in which a norm comes before each sublayer and the sublayer's
result joins the stream (x1 = x + mix(n1(x)); x2 = x1 + ffn(n2(x1))), whose
norms are layer norms with a weight and no bias.  What each sublayer reads passes a short causal
convolution over time first (h <- h + conv(h)).  A token's embedding is its own row plus a row of
a second table chosen by a hash of the previous and the current token.  A layer's mixer is a
state-space recurrence, a delta-rule recurrence, or attention with logistic weights over a window
that keeps a sequence's first keys; its feed-forward is a mixture of experts with a shared expert.
config.json gives every size and every constant that may differ between models:

    architecture                "Leguvik"
    vocab, width                sizes of the embedding / head and of the residual stream
    norm.eps                    eps of every norm
    canon.taps                  taps of the input convolutions
    embedding.bigram            {buckets, mul_prev, mul_cur} of the second embedding table
    logit_softcap               c: logits = c tanh(logits / c)
    layers[i].type              "mamba2" | "general_delta" | "attention"
    layers[i].mixer             that mixer's sizes and constants (below)
    layers[i].mlp               null, or {kind: "moe", router {experts, top}, expert {ff, limit},
                                shared {ff, limit} (optional)}

    mamba2:         heads, vdim, state, groups, norm_groups, conv (taps)
    general_delta:  heads, dim  (the rank of the decay's low-rank map is the shape of its first
                    matrix; `decay_rank` may state it, and must when weights are made at random)
    attention:      heads, kv_heads, dim, vdim, scale, softcap (absent: none), mask {size, keep_first}
                    (absent: every earlier key is seen), and
                    optionally kv_from: the layer whose keys and values this one reads

What the design fixes is written into the part records by `to_spec`: the slope of the experts'
gate, the decay's scale and the unit key's eps of the delta rule, the gates, which norm each
mixer ends in, and the tensor names (`l<i>.norm1`, `l<i>.canon1`, `l<i>.mix.in`, `l<i>.mlp.e<j>.gate`,
`bigram`, ...).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Optional

from .specs import (ConfigError, ConvSpec, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                    PairEmbeddingSpec, ScheduleEntry)
from .zolulix import MAX_POSITIONS, _num, _sub

GLU_SLOPE = 1.702                    # of the experts' gate, g * sigmoid(slope g)
DELTA_DECAY_SCALE = math.exp(-0.5)   # decays are exp(-scale * sigmoid(.))
UNIT_KEY_EPS = 1e-6                  # u = k / sqrt(sum(k^2) + eps)


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int
    dim: int
    decay_rank: Optional[int] = None


@dataclass(frozen=True)
class SigmoidAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    window: int                # mask.size
    keep_first: int            # mask.keep_first
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int = 0         # 0: no shared expert
    shared_limit: float = 0.0


@dataclass(frozen=True)
class PairTableConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class LeguvikLayer:
    type: str
    mixer: object
    mlp: Optional[ExpertsConfig]


def _mixer(kind, m: dict, w: str):
    if kind == "mamba2":
        c = StateSpaceConfig(heads=_num(m, "heads", w), vdim=_num(m, "vdim", w), state=_num(m, "state", w),
                             groups=_num(m, "groups", w), norm_groups=_num(m, "norm_groups", w),
                             conv=_num(m, "conv", w))
        if c.heads % c.groups:
            raise ConfigError(f"missing/invalid config key: {w}groups ({c.heads} heads are not a multiple "
                              f"of {c.groups})")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"missing/invalid config key: {w}norm_groups ({c.heads * c.vdim} values do "
                              f"not split into {c.norm_groups} equal parts)")
        return c
    if kind == "general_delta":
        rank = m.get("decay_rank")
        return DeltaRuleConfig(heads=_num(m, "heads", w), dim=_num(m, "dim", w),
                               decay_rank=None if rank is None else _num(m, "decay_rank", w))
    if kind == "attention":
        mask = _sub(m, "mask", w) if m.get("mask") is not None else {}      # no mask: every earlier key is seen
        src = m.get("kv_from")
        a = SigmoidAttentionConfig(
            heads=_num(m, "heads", w), kv_heads=_num(m, "kv_heads", w), dim=_num(m, "dim", w),
            vdim=_num(m, "vdim", w), scale=_num(m, "scale", w, float),
            softcap=_num(m, "softcap", w, float, positive=False) if m.get("softcap") is not None else 0.0,
            window=_num(mask, "size", w + "mask.") if mask.get("size") is not None else 0,
            keep_first=_num(mask, "keep_first", w + "mask.", positive=False) if mask.get("keep_first") is not None else 0,
            kv_from=None if src is None else _num(m, "kv_from", w, positive=False))
        if a.heads % a.kv_heads:
            raise ConfigError(f"missing/invalid config key: {w}kv_heads ({a.heads} query heads are not a "
                              f"multiple of {a.kv_heads})")
        if a.softcap < 0 or a.keep_first < 0:
            raise ConfigError(f"missing/invalid config key: {w}softcap / {w}mask.keep_first (must be >= 0)")
        return a if a.window else replace(a, keep_first=0)         # without a window every key is in sight anyway
    raise ConfigError(f"unsupported config key: {w[:-6]}type = {kind!r} (mamba2, general_delta or attention)")


def _experts(mlp, w: str) -> Optional[ExpertsConfig]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        raise ConfigError(f"unsupported config key: {w}kind = "
                          f"{mlp.get('kind') if isinstance(mlp, dict) else mlp!r} (only 'moe')")
    r, e = _sub(mlp, "router", w), _sub(mlp, "expert", w)
    shared = mlp.get("shared")
    c = ExpertsConfig(
        experts=_num(r, "experts", w + "router."), top=_num(r, "top", w + "router."),
        ff=_num(e, "ff", w + "expert."), limit=_num(e, "limit", w + "expert.", float),
        shared_ff=0 if shared is None else _num(_sub(mlp, "shared", w), "ff", w + "shared."),
        shared_limit=0.0 if shared is None else _num(shared, "limit", w + "shared.", float))
    if c.top > c.experts:
        raise ConfigError(f"missing/invalid config key: {w}router.top ({c.top} of {c.experts} experts)")
    return c


@dataclass(frozen=True)
class LeguvikConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    canon_taps: int = 0                        # 0: no input convolutions
    bigram: Optional[PairTableConfig] = None
    logit_softcap: float = 0.0
    architecture: str = "Leguvik"

    @classmethod
    def from_dict(cls, d: dict) -> "LeguvikConfig":
        vocab, width = _num(d, "vocab", ""), _num(d, "width", "")
        eps = _num(_sub(d, "norm", ""), "eps", "norm.", float, positive=False)
        if eps < 0:
            raise ConfigError("missing/invalid config key: norm.eps (must be >= 0)")
        taps = _num(_sub(d, "canon", ""), "taps", "canon.") if d.get("canon") is not None else 0
        bigram = None
        emb = d.get("embedding")
        if emb is not None and _sub(d, "embedding", "").get("bigram") is not None:
            b = _sub(emb, "bigram", "embedding.")
            bigram = PairTableConfig(buckets=_num(b, "buckets", "embedding.bigram."),
                                     mul_prev=_num(b, "mul_prev", "embedding.bigram.", positive=False),
                                     mul_cur=_num(b, "mul_cur", "embedding.bigram.", positive=False))
        cap = _num(d, "logit_softcap", "", float, positive=False) if d.get("logit_softcap") is not None else 0.0
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("missing/invalid config key: layers (a non-empty list)")
        layers = []
        for i, L in enumerate(raw):
            w = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"missing/invalid config key: layers[{i}] (expected an object)")
            mixer = _mixer(L.get("type"), _sub(L, "mixer", w), w + "mixer.")
            layers.append(LeguvikLayer(L.get("type"), mixer, _experts(L.get("mlp"), w + "mlp.")))
        for i, L in enumerate(layers):
            m = L.mixer
            if L.type != "attention" or m.kv_from is None:
                continue
            src = layers[m.kv_from] if 0 <= m.kv_from < i else None
            if src is None or src.type != "attention" or src.mixer.kv_from is not None:
                raise ConfigError(f"missing/invalid config key: layers[{i}].mixer.kv_from ({m.kv_from} is no "
                                  "earlier attention layer with keys and values of its own)")
            if (src.mixer.kv_heads, src.mixer.dim, src.mixer.vdim) != (m.kv_heads, m.dim, m.vdim):
                raise ConfigError(f"missing/invalid config key: layers[{i}].mixer.kv_from (layer {m.kv_from}'s "
                                  "key/value heads and sizes differ from this layer's)")
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers), canon_taps=taps, bigram=bigram,
                   logit_softcap=cap)

    def to_dict(self) -> dict:
        """config.json content that `from_dict` reads back to an equal configuration."""
        out = []
        for L in self.layers:
            m = L.mixer
            if L.type == "mamba2":
                mixer = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups,
                         "norm_groups": m.norm_groups, "conv": m.conv}
            elif L.type == "general_delta":
                mixer = {"heads": m.heads, "dim": m.dim}
                if m.decay_rank is not None:
                    mixer["decay_rank"] = m.decay_rank
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "softcap": m.softcap}
                if m.window:
                    mixer["mask"] = {"size": m.window, "keep_first": m.keep_first}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            mlp = None
            if L.mlp is not None:
                e = L.mlp
                mlp = {"kind": "moe", "router": {"experts": e.experts, "top": e.top},
                       "expert": {"ff": e.ff, "limit": e.limit}}
                if e.shared_ff:
                    mlp["shared"] = {"ff": e.shared_ff, "limit": e.shared_limit}
            out.append({"type": L.type, "mixer": mixer, "mlp": mlp})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.eps}, "layers": out}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.bigram is not None:
            b = self.bigram
            d["embedding"] = {"bigram": {"buckets": b.buckets, "mul_prev": b.mul_prev, "mul_cur": b.mul_cur}}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d

    def to_spec(self) -> ModelSpec:
        """The model as parts: one pre-norm block per layer with its input convolutions; a layer
        that reads another layer's keys and values is a schedule entry without a cache of its own."""
        d, eps = self.width, self.eps
        layers = []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            m = L.mixer
            if L.type == "mamba2":
                mixer = MixerSpec(
                    kind="state_space", width=d, n_heads=m.heads, head_dim=m.state, prefix=p + "mix.",
                    params=(("vdim", m.vdim), ("groups", m.groups), ("norm_groups", m.norm_groups),
                            ("conv_taps", m.conv), ("eps", eps)))
            elif L.type == "general_delta":
                mixer = MixerSpec(
                    kind="delta_rule", width=d, n_heads=m.heads, head_dim=m.dim, prefix=p + "mix.",
                    params=(("decay_scale", DELTA_DECAY_SCALE), ("key_eps", UNIT_KEY_EPS),
                            ("decay_rank", m.decay_rank), ("eps", eps)))
            else:
                mixer = MixerSpec(
                    kind="sigmoid_attention", width=d, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                    window=m.window, scale=m.scale, prefix=p + "mix.",
                    params=(("vdim", m.vdim), ("softcap", m.softcap), ("keep_first", m.keep_first),
                            ("head_bias", "pb"), ("own_kv", m.kv_from is None)))
            ff = None
            if L.mlp is not None:
                e = L.mlp
                shared = None if not e.shared_ff else FeedForwardSpec(
                    kind="glu_clamped", width=d, intermediate=e.shared_ff, activation="glu_clamped",
                    prefix=p + "mlp.shared.",
                    params=(("limit", e.shared_limit), ("slope", GLU_SLOPE), ("names", ("gate", "up", "down"))))
                ff = FeedForwardSpec(
                    kind="experts_glu_clamped", width=d, intermediate=e.ff, activation="glu_clamped",
                    prefix=p + "mlp.",
                    params=(("experts", e.experts), ("top", e.top), ("limit", e.limit), ("slope", GLU_SLOPE),
                            ("shared", shared)))
            conv = (lambda name: ConvSpec(p + name, d, self.canon_taps)) if self.canon_taps else (lambda name: None)
            layers.append(LayerSpec(
                arrangement="pre_norm", mixer=mixer, mixer_norm=NormSpec("layernorm", d, eps, p + "norm1"),
                feed_forward=ff, feed_forward_norm=NormSpec("layernorm", d, eps, p + "norm2") if ff else None,
                mixer_conv=conv("canon1"), feed_forward_conv=conv("canon2") if ff else None))
        b = self.bigram
        spec = ModelSpec(
            architecture=self.architecture, width=d, vocab=self.vocab, max_positions=MAX_POSITIONS,
            embedding_tensor="embed", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, L.mixer.kv_from if L.type == "attention" else None)
                           for i, L in enumerate(self.layers)),
            final_norm=NormSpec("layernorm", d, eps, "final.norm"), head_tensor="head",
            logit_cap=self.logit_softcap,
            pair_embedding=None if b is None else PairEmbeddingSpec("bigram", b.buckets, b.mul_prev, b.mul_cur))
        spec.validate()
        return spec
