"""The generalized delta rule: a recurrence over a matrix state with a decay per key channel and a
removal along the unit key,

    S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,      o_t = S_t^T r_t

per head, S_0 = 0; decay and removal act on S_(t-1), then k v^T is added; r, k, v of `head_dim` values per head,
u = k / sqrt(sum(k^2) + key_eps) the head's unit key, decays w = exp(-decay_scale * sigmoid(W2
tanh(W1 h) + w0)) and removal rates a = sigmoid(A h + b) per head and key channel.  Output: an RMS
norm of o within each head (`eps`), a channel-wise weight vector that spans all heads, the gate
sigmoid(G h), then the product with O.

r, k, v, g, the removal logits and the first half of the decay map are one product; the map's
second half, decays, rates, the unit key, the state and the recurrence are float32 whatever the
activation dtype.  The state (float32 [heads, head_dim (value), head_dim (key)]) is fixed-size
per-sequence state of the cache; the recurrence runs token by token for prompts, portions and
single tokens alike.

Tensors after the prefix: r, k, v, g, a [heads * head_dim, width]; a.b [heads * head_dim]; w1 [rank,
width], w2 [heads * head_dim, rank], w0 [heads * head_dim] (the rank is `decay_rank`, or whatever
the stored w1 has when that is None); norm [heads * head_dim]; o [width, heads * head_dim]."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import StateNeed
from ..weights.loader import TensorRequest
from .attention import _cat
from .base import Mixer, register_mixer


@register_mixer("delta_rule")
class DeltaRule(Mixer):
    def __init__(self, spec, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        p = dict(spec.params)
        self.h, self.dim = spec.n_heads, spec.head_dim
        self.hk = self.h * self.dim
        self.decay_scale, self.key_eps = float(p.get("decay_scale", 1.0)), float(p.get("key_eps", 1e-6))
        self.eps, self.rank = float(p.get("eps", 1e-6)), p.get("decay_rank")
        self.r_off, self.k_off, self.v_off, self.g_off, self.a_off, self.z_off = (i * self.hk for i in range(6))
        self.w_in = self.w2 = self.w0 = self.a_bias = self.norm_w = self.w_o = None

    def state_need(self):
        return StateNeed((self.h, self.dim, self.dim), torch.float32)

    def tensor_requests(self):
        p, d, hk = self.spec.prefix, self.spec.width, self.hk
        r = -1 if self.rank is None else int(self.rank)          # -1: whatever the stored tensors have
        return [TensorRequest(p + n, (hk, d)) for n in ("r", "k", "v", "g", "a")] + \
               [TensorRequest(p + "a.b", (hk,), "bias"), TensorRequest(p + "w1", (r, d)),
                TensorRequest(p + "w2", (hk, r)), TensorRequest(p + "w0", (hk,), "bias"),
                TensorRequest(p + "norm", (hk,), "norm"), TensorRequest(p + "o", (d, hk))]

    def bind(self, get):
        from ..config.specs import ConfigError
        p = self.spec.prefix
        w1 = get(p + "w1")
        self.w2, self.w0, self.a_bias = get(p + "w2"), get(p + "w0"), get(p + "a.b")
        if w1.shape[0] != self.w2.shape[1]:
            raise ConfigError(f"{p}w1 has {w1.shape[0]} rows, {p}w2 {self.w2.shape[1]} columns")
        if not (self.w2.dtype == self.w0.dtype == self.a_bias.dtype):
            self.w2, self.w0, self.a_bias = self.w2.float(), self.w0.float(), self.a_bias.float()
        self.w_in = _cat([get(p + n) for n in ("r", "k", "v", "g", "a")] + [w1])
        self.norm_w, self.w_o = get(p + "norm"), get(p + "o")

    def first_weights(self, rows):
        n, k = self.w_in.shape
        late = self.w_in.dtype == torch.bfloat16 and ops.requests_weights_late(rows, n, k, self.w_in.device)
        return self.w_in if late else None

    def forward(self, h, ctx, residual=None):
        rows, plan = h.shape[0], ctx.plan
        proj = torch.empty((rows, self.w_in.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_in, proj)
        aux = torch.empty((rows, 3, self.hk), dtype=torch.float32, device=h.device)
        ops.delta_prep(proj, self.k_off, self.a_off, self.z_off, self.h, self.dim, self.w2, self.w0, self.a_bias,
                       self.decay_scale, self.key_eps, aux)
        o = torch.empty((rows, self.h, self.dim), dtype=torch.float32, device=h.device)
        ops.delta_scan(proj, self.r_off, self.k_off, self.v_off, aux, plan, self.h, self.dim, ctx.state(), o)
        mixed = torch.empty((rows, self.hk), dtype=self.dtype, device=h.device)
        ops.linrec_out(o, proj, self.g_off, self.h, self.dim, self.norm_w, self.eps, mixed, gate="sigmoid")
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(mixed, self.w_o, out, ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)
