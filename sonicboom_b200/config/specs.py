"""Model description as data: what each layer is made of and in which order layers run.

A `ModelSpec` plays the role of the reference's `Recipe`
(core/include/sonicboom/model/recipe.h:51-205): parts carry their sizes and constants as
parameters, every layer names its own mixer and feed-forward, and the run order is a list
that may name a layer twice or let an entry read another entry's cache
(`SelfAttention.cache/owns_cache`, recipe.h:89-93).  Nothing here knows an architecture;
an architecture's configuration class fills these records in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


class ConfigError(ValueError):
    """A configuration that cannot be built; the message names the offending key."""


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer."""
    kind: str                      # key of parts.POSITION_ENCODINGS, e.g. "rope_neox"
    head_dim: int
    theta: float = 10000.0
    rotary_dim: int = 0            # 0 = the whole head is rotated
    params: tuple = ()             # extra (key, value) pairs for kinds that scale their frequencies


@dataclass(frozen=True)
class NormSpec:
    kind: str                      # key of parts.NORMS, e.g. "rmsnorm"
    width: int
    eps: float
    tensor: str                    # tensor name of the weight


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of one layer.  `params` holds what only that kind of mixer needs."""
    kind: str                      # key of parts.MIXERS, e.g. "attention"
    width: int                     # residual width in and out
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0                # 0 = every earlier key; n = the last n keys
    scale: float = 0.0             # score multiplier, applied after the dot product
    qkv_bias: bool = False
    out_bias: bool = False
    position: Optional[PositionSpec] = None
    prefix: str = ""               # tensor-name prefix, e.g. "model.layers.3.self_attn."
    params: tuple = ()             # extra (key, value) pairs for other mixer kinds


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                      # key of parts.FEED_FORWARDS, e.g. "swiglu"
    width: int
    intermediate: int
    activation: str = "silu"
    prefix: str = ""
    params: tuple = ()


@dataclass(frozen=True)
class ConvSpec:
    """A short causal convolution over time on every channel of what a sublayer reads, added to
    it: h <- h + conv(h), conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before a
    sequence's start.  `tensor` is [width, taps]."""
    tensor: str
    width: int
    taps: int


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """A second embedding table read by a hash of two neighbouring tokens and added to the token's
    own row: row (previous * mul_prev + current * mul_cur) mod buckets, and row `buckets` (the
    table's last) for a sequence's first token.  `tensor` is [buckets + 1, width]."""
    tensor: str
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class DepthMixSpec:
    """What goes on to the next schedule entry instead of a block's own result: a combination of
    the embedding output and every block result so far (`n_inputs` of them, this block's last)."""
    kind: str                      # key of parts.DEPTH_MIXES, e.g. "weighted_sum"
    n_inputs: int
    tensor: str                    # tensor name of the coefficients, [n_inputs]


@dataclass(frozen=True)
class LayerSpec:
    """One block: which arrangement, and the parts it arranges.  An arrangement that norms a
    sublayer's result before the residual add names those norms in the `*_post_norm` fields; a
    block without a feed-forward has `feed_forward` (and its norms) None."""
    arrangement: str               # key of parts.BLOCKS, e.g. "pre_norm"
    mixer: MixerSpec
    mixer_norm: Optional[NormSpec]                 # None: the arrangement has no norm before the mixer
    feed_forward: Optional[FeedForwardSpec]
    feed_forward_norm: Optional[NormSpec]
    mixer_post_norm: Optional[NormSpec] = None
    feed_forward_post_norm: Optional[NormSpec] = None
    depth_mix: Optional[DepthMixSpec] = None
    mixer_conv: Optional[ConvSpec] = None          # on the mixer's input, after its norm
    feed_forward_conv: Optional[ConvSpec] = None   # on the feed-forward's input, after its norm
    params: tuple = ()             # extra (key, value) pairs for arrangements with constants of their own

    @property
    def kind(self) -> str:
        return self.arrangement


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `cache_from` is the index of an earlier schedule entry whose
    cache this run reads instead of writing its own (None: it owns a cache)."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class StreamInjection:
    """Something that joins the stream right before a schedule entry runs: the embedding output
    once more (`embedding`), and/or row `row` of the tensor `tensor` [rows, width], added to every
    token's vector."""
    before_entry: int
    embedding: bool = False
    tensor: Optional[str] = None
    rows: int = 0                  # how many rows the tensor has
    row: int = 0


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    width: int
    vocab: int
    max_positions: int
    embedding_tensor: str
    layers: tuple                  # of LayerSpec
    schedule: tuple                # of ScheduleEntry
    final_norm: NormSpec = None
    head_tensor: Optional[str] = None   # None: the head is the embedding matrix (tied)
    stop_tokens: tuple = ()
    embedding_scale: float = 1.0        # multiplies every embedding row (1: as stored)
    logit_cap: float = 0.0              # c > 0: logits = c * tanh(logits / c); 0: no cap
    logit_scale: float = 1.0            # multiplies the head's product (before a cap)
    injections: tuple = ()              # of StreamInjection, at most one per schedule entry
    unused_tensors: tuple = ()          # (name, shape) of tensors a file may hold that nothing reads
    pair_embedding: Optional[PairEmbeddingSpec] = None   # added to every embedding row

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("model has no layers")
        if not self.embedding_scale > 0.0:
            raise ConfigError(f"embedding_scale {self.embedding_scale} must be positive")
        if not self.logit_scale > 0.0:
            raise ConfigError(f"logit_scale {self.logit_scale} must be positive")
        if self.logit_cap < 0.0:
            raise ConfigError(f"logit_cap {self.logit_cap} must be zero (none) or positive")
        seen = set()
        for inj in self.injections:
            if not 0 <= inj.before_entry < len(self.schedule) or inj.before_entry in seen:
                raise ConfigError(f"an injection before schedule entry {inj.before_entry}: no such entry, "
                                  "or it has one already")
            seen.add(inj.before_entry)
            if inj.tensor is not None and not 0 <= inj.row < inj.rows:
                raise ConfigError(f"an injection names row {inj.row} of {inj.tensor}, which has {inj.rows}")
            if any(l.depth_mix is not None for l in self.layers):
                raise ConfigError("injections into the stream and depth mixing are not combined")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule[{i}] names layer {e.layer}, model has {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, "
                                      "which does not run before it")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ConfigError(f"schedule[{i}] reads the cache of entry {e.cache_from}, "
                                      "which owns none")
            mix = self.layers[e.layer].depth_mix
            if mix is not None and mix.n_inputs != i + 2:
                raise ConfigError(f"schedule[{i}] mixes {mix.n_inputs} streams, but the embedding output "
                                  f"and the block results so far are {i + 2}")
