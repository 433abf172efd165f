"""Half-split (NEOX) rotary position encoding.

For pair i of the rotated prefix of a head: theta = position * exp(-2i/n * ln(base)), every
step in float32 (core/src/nn/rope.cpp:26-55); the whole head is rotated unless `rotary_dim`
names a shorter prefix (rope.cpp:58-82).  The table of per-pair frequencies is made once on
the host with the reference's operation order and handed to the rotation kernel, which is
also where a scaled-frequency variant would plug in its own table."""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope_neox")
class RotaryNeox(PositionEncoding):
    def __init__(self, spec, dtype, device):
        self.head_dim = spec.head_dim
        self.rotary_dim = spec.rotary_dim or spec.head_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            from ..config.specs import ConfigError
            raise ConfigError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim "
                              f"{self.head_dim}")
        n = np.float32(self.rotary_dim)
        i = np.arange(self.rotary_dim // 2, dtype=np.float32)
        log_base = np.log(np.float32(spec.theta)).astype(np.float32)
        inv = np.exp((np.float32(-2.0) * i / n * log_base).astype(np.float32)).astype(np.float32)
        self.inv_freq = torch.from_numpy(inv).to(device)


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    """Leaves queries and keys as they are."""

    def __init__(self, spec, dtype, device):
        self.head_dim, self.rotary_dim = spec.head_dim, 0
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=device)


@register_position_encoding("rope_interleaved")
class RotaryInterleaved(PositionEncoding):
    """Rotation of neighbouring pairs: elements 2i and 2i + 1 of the rotated vector turn by
    position * base^(-2i / rotary_dim), i < rotary_dim / 2; elements from rotary_dim on pass
    unchanged.  `head_dim` is the length of the rotated vector (a head's rotated part).  The
    frequency table is worked out in double precision and rounded once; the kernels that pair
    elements this way (`ops.latent_prep`) take the angle as float32 position * table entry."""
    layout = "interleaved"

    def __init__(self, spec, dtype, device):
        self.head_dim = spec.head_dim
        self.rotary_dim = spec.rotary_dim or spec.head_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            from ..config.specs import ConfigError
            raise ConfigError(f"rotary_dim {self.rotary_dim} must be even and at most the rotated "
                              f"vector's length {self.head_dim}")
        i = np.arange(max(1, self.rotary_dim // 2), dtype=np.float64)
        inv = np.power(np.float64(spec.theta), -2.0 * i / np.float64(self.rotary_dim))
        self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(device)


def frequency_table(base: float, n: int, device) -> torch.Tensor:
    """float32 [max(1, n/2)]: base^(-2i/n), worked out in double precision and rounded once."""
    i = np.arange(max(1, n // 2), dtype=np.float64)
    inv = np.power(np.float64(base), -2.0 * i / np.float64(max(n, 1)))
    return torch.from_numpy(inv.astype(np.float32)).to(device)


@register_position_encoding("rope_halves")
class RotaryHalves(PositionEncoding):
    """Rotation of pairs half a prefix apart: elements i and i + rotary_dim/2 turn by
    position * base^(-2i / rotary_dim), i < rotary_dim / 2; elements from rotary_dim on pass
    unchanged (rotary_dim 0: nothing turns).  The pairs are "rope_neox"'s; the table is worked out in double precision
    and rounded once, as "rope_interleaved"'s is, and the kernels that take a `layout`
    (`ops.attn_prep`, `ops.linrec_prep`) serve both."""
    layout = "halves"

    def __init__(self, spec, dtype, device):
        self.head_dim = spec.head_dim
        self.rotary_dim = spec.rotary_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            from ..config.specs import ConfigError
            raise ConfigError(f"rotary_dim {self.rotary_dim} must be even and at most the rotated "
                              f"vector's length {self.head_dim}")
        self.inv_freq = frequency_table(spec.theta, self.rotary_dim, device)


YARN_MAGNITUDE_SLOPE = 0.1      # cosines and sines grow by 0.1 ln(factor) + 1
YARN_RAMP_FLOOR = 0.001         # the ramp's length is at least this


def yarn_frequencies(base: float, n: int, factor: float, original: float, fast: float, slow: float):
    """(float64 [n/2] frequencies, magnitude) of a rotation whose slow pairs are stretched.
    f_i = base^(-2i/n).  With dim(t) = n ln(original / (2 pi t)) / (2 ln base), the pair number at which
    a pair makes t turns over `original` positions, lo = max(floor(dim(fast)), 0), hi =
    min(ceil(dim(slow)), n - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i
    turns with f_i / factor * ramp_i + f_i * (1 - ramp_i): fast pairs keep their frequency, slow
    ones are divided by `factor`, those between are blended.  Cosines and sines are multiplied by
    0.1 ln(factor) + 1."""
    import math
    i = np.arange(max(1, n // 2), dtype=np.float64)
    f = np.power(np.float64(base), -2.0 * i / np.float64(max(n, 1)))

    def pair_at(turns):
        return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_at(fast)), 0)
    hi = min(math.ceil(pair_at(slow)), n - 1)
    ramp = np.clip((i - lo) / max(hi - lo, YARN_RAMP_FLOOR), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), YARN_MAGNITUDE_SLOPE * math.log(factor) + 1.0


@register_position_encoding("rope_halves_yarn")
class RotaryHalvesYarn(PositionEncoding):
    """"rope_halves" with stretched slow pairs (`yarn_frequencies`).  `params`: factor, original,
    fast, slow.  `magnitude` multiplies every cosine and sine; the kernels that rotate take it as
    their `rot_scale`."""
    layout = "halves"

    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.head_dim = spec.head_dim
        self.rotary_dim = spec.rotary_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ConfigError(f"rotary_dim {self.rotary_dim} must be even and at most the rotated "
                              f"vector's length {self.head_dim}")
        p = dict(spec.params)
        try:
            factor, original = float(p["factor"]), float(p["original"])
            fast, slow = float(p["fast"]), float(p["slow"])
        except KeyError as e:
            raise ConfigError(f"a stretched rotation needs the parameter {e.args[0]}") from None
        if not (factor > 0 and original > 0 and fast > 0 and slow > 0):
            raise ConfigError("a stretched rotation's factor, original, fast and slow must be positive")
        freq, self.magnitude = yarn_frequencies(spec.theta, self.rotary_dim, factor, original, fast, slow)
        self.inv_freq = torch.from_numpy(freq.astype(np.float32)).to(device)
