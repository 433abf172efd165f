"""Dense gated feed-forward: y = Wdown (silu(Wgate f) * (Wup f)), no biases
(core/src/model/emit.cpp:364-374; silu: core/src/nn/activation.cpp:41-50).

Gate and up are one product over a fused matrix whose rows alternate in blocks of
`ops.SWIGLU_BLOCK` (8 gate rows, the 8 up rows of the same outputs, ...), so the product's
epilogue applies silu(gate) * up and writes [rows, intermediate] once; the residual add is
fused into the down projection.  These are the reference's SiluMul and ResidualAdd fusions
(core/include/sonicboom/planner/ir_passes.h:35-39)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorRequest
from .base import FEED_FORWARDS, FeedForward, make, register_feed_forward


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    ff, d = gate.shape
    b = ops.SWIGLU_BLOCK
    if gate.dtype != up.dtype:
        gate, up = gate.float(), up.float()
    return torch.stack([gate.view(ff // b, b, d), up.view(ff // b, b, d)], dim=1) \
        .reshape(2 * ff, d).contiguous()


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """y = Wdown (act(Wgate f) * (Wup f)).  `activation` is "silu" or "gelu_tanh" (gelu in its tanh
    form, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))); `params` may give `names`, the tensor
    names of the three matrices after the prefix.  With silu the product's epilogue applies the
    activation; with gelu_tanh the product's float32 rows go through the activation kernel."""

    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype = spec, dtype
        if spec.activation not in ("silu", "gelu_tanh"):
            raise ConfigError(f"feed-forward activation {spec.activation!r} is not built (silu, gelu_tanh)")
        self.interleaved = spec.intermediate % ops.SWIGLU_BLOCK == 0
        if not self.interleaved and spec.activation == "silu":
            raise ConfigError(f"intermediate_size {spec.intermediate} must be a multiple of "
                              f"{ops.SWIGLU_BLOCK} for the fused gate/up product")
        self.names = tuple(dict(spec.params).get("names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        self.w_gate_up = self.w_down = None

    def tensor_requests(self):
        p, d, ff = self.spec.prefix, self.spec.width, self.spec.intermediate
        g, u, dn = self.names
        return [TensorRequest(p + g, (ff, d)), TensorRequest(p + u, (ff, d)), TensorRequest(p + dn, (d, ff))]

    def bind(self, get):
        p = self.spec.prefix
        g, u, dn = self.names
        gate, up = get(p + g), get(p + u)
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.w_gate_up = interleave_gate_up(gate, up) if self.interleaved else torch.cat([gate, up], dim=0).contiguous()
        self.w_down = get(p + dn)

    def forward(self, h, ctx, residual=None):
        rows, ff = h.shape[0], self.spec.intermediate
        t = torch.empty((rows, ff), dtype=self.dtype, device=h.device)
        if self.spec.activation == "silu":
            ops.linear(h, self.w_gate_up, t, ops.EPI_SWIGLU)
        elif self.interleaved:
            ops.linear(h, self.w_gate_up, t, ops.EPI_SWIGLU, gate_kind=ops.GATE_KINDS[self.spec.activation])
        else:                                # other sizes keep [gate rows | up rows] and the activation kernel
            gu = torch.empty((rows, 2 * ff), dtype=torch.float32, device=h.device)
            ops.linear(h, self.w_gate_up, gu)
            ops.gated_act(gu, ops.GATE_KINDS[self.spec.activation], t)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(t, self.w_down, out,
                          ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)


@register_feed_forward("glu_clamped")
class ClampedGLU(FeedForward):
    """Gated feed-forward with clamped factors: g = min(Wgate h, limit), u = clamp(Wup h, -limit,
    limit), y = Wdown (g * sigmoid(slope g) * (u + 1)), no biases.  `params` gives `limit`,
    `slope` and optionally `names`, the tensor names of the three matrices after the prefix.
    Gate and up are one product over the fused matrix that `interleave_gate_up` makes when the
    intermediate size allows it (a multiple of `ops.SWIGLU_BLOCK`): the tcgen05 product applies the
    activation in its epilogue; where another product kernel runs, its float32 rows go through
    the activation kernel.  Other sizes keep [gate rows | up rows] and the activation kernel."""

    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype = spec, dtype
        p = dict(spec.params)
        self.limit, self.slope = float(p.get("limit", 0.0)), float(p.get("slope", 1.0))
        if not self.limit > 0.0:
            raise ConfigError(f"feed-forward limit {self.limit} must be positive")
        self.names = tuple(p.get("names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        self.w_gate_up = self.w_down = None

    def tensor_requests(self):
        p, d, ff = self.spec.prefix, self.spec.width, self.spec.intermediate
        g, u, dn = self.names
        return [TensorRequest(p + g, (ff, d)), TensorRequest(p + u, (ff, d)), TensorRequest(p + dn, (d, ff))]

    def bind(self, get):
        p = self.spec.prefix
        g, u, dn = self.names
        gate, up = get(p + g), get(p + u)
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.interleaved = self.spec.intermediate % ops.SWIGLU_BLOCK == 0
        self.w_gate_up = interleave_gate_up(gate, up) if self.interleaved else \
            torch.cat([gate, up], dim=0).contiguous()
        self.w_down = get(p + dn)

    def forward(self, h, ctx, residual=None):
        rows, ff = h.shape[0], self.spec.intermediate
        t = torch.empty((rows, ff), dtype=self.dtype, device=h.device)
        if self.interleaved:
            ops.linear(h, self.w_gate_up, t, ops.EPI_SWIGLU, gate=(self.limit, self.slope))
        else:
            gu = torch.empty((rows, 2 * ff), dtype=torch.float32, device=h.device)
            ops.linear(h, self.w_gate_up, gu)
            ops.glu_clamped(gu, self.limit, self.slope, t)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(t, self.w_down, out,
                          ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)


@register_feed_forward("polynorm")
class PolyNormFF(FeedForward):
    """Feed-forward without a gate whose activation is a cubic in normed powers:
    y = Wdown (c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3), z = Wup h, powers element by element and
    N(u) = u / sqrt(mean(u^2) + eps) over a token's intermediate values.  `params`: `eps` and
    optionally `names`, the tensor names of the two matrices and of the four coefficients after the
    prefix.  The up product's float32 rows go through `ops.polynorm` (the sums of a row and the
    activation in float32); the residual add is fused into the down projection."""

    def __init__(self, spec, dtype, device):
        self.spec, self.dtype = spec, dtype
        p = dict(spec.params)
        self.eps = float(p.get("eps", 1e-6))
        self.names = tuple(p.get("names", ("up", "down", "act")))
        self.w_up = self.w_down = self.coef = None

    def tensor_requests(self):
        p, d, ff = self.spec.prefix, self.spec.width, self.spec.intermediate
        up, down, act = self.names
        return [TensorRequest(p + up, (ff, d)), TensorRequest(p + down, (d, ff)),
                TensorRequest(p + act, (4,), "bias")]

    def bind(self, get):
        p = self.spec.prefix
        up, down, act = self.names
        self.w_up, self.w_down, self.coef = get(p + up), get(p + down), get(p + act)

    def forward(self, h, ctx, residual=None):
        rows, ff = h.shape[0], self.spec.intermediate
        z = torch.empty((rows, ff), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_up, z)
        t = torch.empty((rows, ff), dtype=self.dtype, device=h.device)
        ops.polynorm(z, self.coef, self.eps, t)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(t, self.w_down, out,
                          ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)


@register_feed_forward("experts_glu_clamped")
class ExpertsClampedGLU(FeedForward):
    """Mixture of experts over clamped gated feed-forwards (the form of `glu_clamped`): router logits
    z = R h + b in float32; a token is sent to its `top` experts of largest logit (ties go to the
    lower index) and their results are mixed with exp(z_e) normalised among those `top` alone; an
    always-on expert (`shared`, a feed-forward spec of its own, or None) contributes to every
    token's result unweighted.
    `params`: `experts`, `top`, `limit`, `slope`, `shared`.  Tensors after the prefix: router
    [experts, width], router.b [experts], e<j>.gate, e<j>.up [intermediate, width], e<j>.down [width,
    intermediate]; the shared expert's under its own prefix.

    With `router` = a dict, the choice is made on scores instead: s = sigmoid(z) (no bias), choice
    scores s + a stored correction (`correction`: its tensor name), the experts in `groups` = (count,
    keep) equal groups of neighbours of which only the `keep` best (by the sum of a group's `group_top`
    largest choice scores) can be chosen, and the weights are the chosen experts' s times `scale`
    (divided by their sum first when `renormalize`).

    The experts' matrices are stacked when bound, [experts, gate | up, intermediate, width] and
    [experts, width, intermediate]; a step groups its (token, choice) pairs by expert on the device
    and walks them in tiles of one expert, so no expert's matrix is read for tokens that did not
    choose it and nothing comes back to the host."""

    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype = spec, dtype
        p = dict(spec.params)
        self.n_experts, self.top = int(p.get("experts", 0)), int(p.get("top", 0))
        self.limit, self.slope = float(p.get("limit", 0.0)), float(p.get("slope", 1.0))
        if not 0 < self.top <= self.n_experts:
            raise ConfigError(f"a mixture of {self.n_experts} experts cannot choose {self.top}")
        if not self.limit > 0.0:
            raise ConfigError(f"feed-forward limit {self.limit} must be positive")
        shared = p.get("shared")
        self.shared = make(FEED_FORWARDS, "feed-forward", shared, dtype, device) if shared is not None else None
        self.router = dict(p["router"]) if p.get("router") is not None else None
        if self.router is not None:
            count, keep = self.router.get("groups", (1, 1))
            if count < 1 or self.n_experts % count or not 1 <= keep <= count or keep * (self.n_experts // count) < self.top:
                raise ConfigError(f"{self.n_experts} experts in {count} groups of which {keep} are kept cannot "
                                  f"give {self.top} choices")
        self.w_router = self.b_router = self.w_up = self.w_down = self.correction = None

    def tensor_requests(self):
        p, d, ff = self.spec.prefix, self.spec.width, self.spec.intermediate
        req = [TensorRequest(p + "router", (self.n_experts, d))]
        if self.router is None:
            req.append(TensorRequest(p + "router.b", (self.n_experts,), "bias"))
        elif self.router.get("correction"):
            req.append(TensorRequest(p + self.router["correction"], (self.n_experts,), "bias"))
        for j in range(self.n_experts):
            req += [TensorRequest(f"{p}e{j}.gate", (ff, d)), TensorRequest(f"{p}e{j}.up", (ff, d)),
                    TensorRequest(f"{p}e{j}.down", (d, ff))]
        return req + (self.shared.tensor_requests() if self.shared is not None else [])

    def bind(self, get):
        p = self.spec.prefix
        self.w_router = get(p + "router")
        if self.router is None:
            self.b_router = get(p + "router.b")
        elif self.router.get("correction"):
            self.correction = get(p + self.router["correction"]).float().contiguous()
        ups = [torch.stack([get(f"{p}e{j}.gate"), get(f"{p}e{j}.up")]) for j in range(self.n_experts)]
        downs = [get(f"{p}e{j}.down") for j in range(self.n_experts)]
        kept = {t.dtype for t in ups + downs}
        if len(kept) > 1:
            ups, downs = [t.float() for t in ups], [t.float() for t in downs]
        self.w_up, self.w_down = torch.stack(ups).contiguous(), torch.stack(downs).contiguous()
        if self.shared is not None:
            self.shared.bind(get)

    def forward(self, h, ctx, residual=None):
        rows = h.shape[0]
        # what follows this part follows its last kernel, which is not a product: nothing rides on one
        ctx.next_norm = ctx.next_weights = None
        logits = torch.empty((rows, self.n_experts), dtype=torch.float32, device=h.device)
        ids = torch.empty((rows, self.top), dtype=torch.int32, device=h.device)
        weights = torch.empty((rows, self.top), dtype=torch.float32, device=h.device)
        if self.router is None:
            ops.linear(h, self.w_router, logits, ops.EPI_BIAS, bias=self.b_router)
            ops.moe_route(logits, self.top, ids, weights)
        else:
            r = self.router
            ops.linear(h, self.w_router, logits)
            ops.moe_route_scored(logits, self.correction, self.top, ids, weights, groups=r.get("groups", (1, 1)),
                                 group_top=int(r.get("group_top", 2)), scale=float(r.get("scale", 1.0)),
                                 renormalize=bool(r.get("renormalize", False)))
        if self.shared is not None:
            out = self.shared.forward(h, ctx, residual=residual)
        elif residual is not None:
            out = residual
        else:
            out = torch.zeros((rows, self.spec.width), dtype=torch.float32, device=h.device)
        a = h if h.dtype == self.w_up.dtype else ops.cast(h, self.w_up.dtype)
        return ops.moe_experts(a, ids, weights, self.w_up, self.w_down, self.limit, self.slope, out)
