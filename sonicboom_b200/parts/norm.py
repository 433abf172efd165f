"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, plain weight
(core/src/nn/norm.cpp:25-42; the model's use: core/src/model/emit.cpp:170-176, 440, 449, 512-515)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorRequest
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec, dtype, device):
        self.width, self.eps, self.tensor = spec.width, float(spec.eps), spec.tensor
        self.weight = None

    def tensor_requests(self):
        return [TensorRequest(self.tensor, (self.width,), "norm")]

    def bind(self, get):
        self.weight = get(self.tensor)

    def as_rms(self):
        return self.weight, self.eps

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, rows)


@register_norm("rmsnorm_scalar")
class ScalarRMSNorm(RMSNorm):
    """RMS norm whose weight is one number for all coordinates: y = x / sqrt(mean(x^2) + eps) * g.
    The stored tensor has shape []; bound, it is spread over the width, so every kernel that
    takes an RMS norm's weight vector (the norm kernel itself, and the kernels that norm a row
    they have just finished) serves it unchanged."""

    def tensor_requests(self):
        return [TensorRequest(self.tensor, (), "norm")]

    def bind(self, get):
        self.weight = get(self.tensor).reshape(1).expand(self.width).contiguous()


@register_norm("rmsnorm_one_plus")
class OnePlusRMSNorm(RMSNorm):
    """RMS norm whose stored weight is an offset from one: y = x / sqrt(mean(x^2) + eps) * (1 + w).
    Bound, 1 + w is worked out once in float32 (a bfloat16 sum would lose the offset's low bits),
    so every kernel that takes an RMS norm's weight vector serves it unchanged."""

    def tensor_requests(self):
        return [TensorRequest(self.tensor, (self.width,), "bias")]

    def bind(self, get):
        self.weight = (get(self.tensor).float() + 1.0).contiguous()


@register_norm("layernorm")
class LayerNorm(Norm):
    """Layer norm with a weight and no bias: y = (x - mean) / sqrt(var + eps) * w, the variance
    being the mean of the squared deviations.  It is not an RMS norm, so no product kernel
    applies it to its own result (`as_rms` is None) and it runs as a kernel of its own."""

    def __init__(self, spec, dtype, device):
        self.width, self.eps, self.tensor = spec.width, float(spec.eps), spec.tensor
        self.weight = None

    def tensor_requests(self):
        return [TensorRequest(self.tensor, (self.width,), "norm")]

    def bind(self, get):
        self.weight = get(self.tensor)

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return ops.layernorm(x, self.weight, self.eps, out, rows)


class StreamCast(Norm):
    """Not a norm: the rows as they are, in the dtype asked for.  A block whose sublayers read the
    stream itself names this as its `input_norm()`, so that whatever finishes the stream's rows
    before it (`ops.norm_add` with a weight of None) can leave the copy behind."""

    def forward(self, x, out_dtype, rows=None):
        if rows is not None:
            raise NotImplementedError("a stream cast gathers no rows")
        return ops.cast(x, out_dtype)
