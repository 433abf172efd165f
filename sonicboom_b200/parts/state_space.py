"""A state-space mixer whose recurrence is a scalar decay per token and head over a matrix state
(the dual form of a selective state-space layer):

    S_t = a_t S_(t-1) + dt_t B_t x_t^T,      y_t = S_t^T C_t + D x_t          per head, S_0 = 0,

with x of `vdim` values per head, B and C of `head_dim` (the state size) values shared by the
heads of a group (`groups` of them; head h reads group h // (heads / groups)), step size
dt = softplus(raw + dt_bias) and decay a = exp(-exp(A_log) dt), one of each per token and head.
One input product gives [z | x | B | C | dt raw]; x, B and C together pass a causal convolution
per channel over `conv_taps` tokens (with a bias) and silu.  y, heads concatenated, is multiplied
by silu(z), then divided by its root mean square in `norm_groups` equal parts of the row (`eps`),
times a weight, then projected out.

Step sizes, decays, the state and the recurrence are float32 whatever the activation dtype.  The
state (float32 [heads, vdim, head_dim]) and the convolution's last conv_taps - 1 inputs are
fixed-size per-sequence state of the cache; the recurrence is `ops.linrec_scan` with a decay per
token and head, C as its queries, B as its keys and dt x as its values.

Tensors after the prefix: in [2 * heads * vdim + 2 * groups * head_dim + heads, width]; conv
[heads * vdim + 2 * groups * head_dim, conv_taps] and conv.b; dt_bias, A_log, D [heads]; norm
[heads * vdim]; o [width, heads * vdim]."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import StateNeed
from ..weights.loader import TensorRequest
from .base import Mixer, register_mixer


@register_mixer("state_space")
class StateSpace(Mixer):
    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype, self.device = spec, dtype, device
        p = dict(spec.params)
        self.h, self.n = spec.n_heads, spec.head_dim
        self.vd = int(p.get("vdim", self.n))
        self.groups, self.norm_groups = int(p.get("groups", 1)), int(p.get("norm_groups", 1))
        self.taps, self.eps = int(p.get("conv_taps", 1)), float(p.get("eps", 1e-6))
        if self.h % self.groups:
            raise ConfigError(f"state_space: {self.h} heads are not a multiple of {self.groups} groups")
        self.inner = self.h * self.vd
        if self.inner % self.norm_groups:
            raise ConfigError(f"state_space: {self.inner} values do not split into {self.norm_groups} equal parts")
        gn = self.groups * self.n
        self.channels = self.inner + 2 * gn              # what the convolution covers: x | B | C
        self.x_off, self.b_off, self.c_off = 0, self.inner, self.inner + gn     # in the convolved rows
        self.xdt_off = self.channels                     # dt * x, beside them
        self.dt_off = self.inner + self.channels         # in the projection: z | x B C | dt
        self.w_in = self.w_conv = self.b_conv = self.dt_bias = self.a_log = self.d_skip = self.norm_w = self.w_o = None

    def state_need(self):
        need = {None: StateNeed((self.h, self.vd, self.n), torch.float32)}
        if self.taps > 1:
            need["conv"] = StateNeed((self.taps - 1, self.channels), torch.float32)
        return need

    def tensor_requests(self):
        p, d = self.spec.prefix, self.spec.width
        return [TensorRequest(p + "in", (self.dt_off + self.h, d)),
                TensorRequest(p + "conv", (self.channels, self.taps), "bias"),
                TensorRequest(p + "conv.b", (self.channels,), "bias"),
                TensorRequest(p + "dt_bias", (self.h,), "bias"), TensorRequest(p + "A_log", (self.h,), "bias"),
                TensorRequest(p + "D", (self.h,), "norm"), TensorRequest(p + "norm", (self.inner,), "norm"),
                TensorRequest(p + "o", (d, self.inner))]

    def bind(self, get):
        p = self.spec.prefix
        self.w_in, self.w_o = get(p + "in"), get(p + "o")
        self.w_conv, self.b_conv = get(p + "conv"), get(p + "conv.b")
        self.dt_bias, self.a_log = get(p + "dt_bias"), get(p + "A_log")
        self.d_skip, self.norm_w = get(p + "D"), get(p + "norm")

    def first_weights(self, rows):
        n, k = self.w_in.shape
        late = self.w_in.dtype == torch.bfloat16 and ops.requests_weights_late(rows, n, k, self.w_in.device)
        return self.w_in if late else None

    def forward(self, h, ctx, residual=None):
        rows, plan = h.shape[0], ctx.plan
        proj = torch.empty((rows, self.w_in.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_in, proj)
        xbc = torch.empty((rows, self.channels + self.inner), dtype=torch.float32, device=h.device)
        ops.causal_conv(proj, self.inner, self.channels, self.w_conv, self.b_conv, plan,
                        ctx.state("conv") if self.taps > 1 else None, xbc, act="silu")
        decay = torch.empty((rows, self.h), dtype=torch.float32, device=h.device)
        ops.ssd_prep(proj, self.dt_off, xbc, self.x_off, self.xdt_off, self.h, self.vd, self.dt_bias, self.a_log, decay)
        o = torch.empty((rows, self.h, self.vd), dtype=torch.float32, device=h.device)
        ops.linrec_scan(xbc, self.c_off, self.b_off, self.xdt_off, plan, self.h, self.n, self.vd, None, None,
                        ctx.state(), o, token_decay=decay, heads_per_qk=self.h // self.groups)
        mixed = torch.empty((rows, self.inner), dtype=self.dtype, device=h.device)
        ops.ssd_out(o, xbc, self.x_off, proj, 0, self.h, self.vd, self.norm_groups, self.d_skip, self.norm_w,
                    self.eps, mixed)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(mixed, self.w_o, out, ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)
