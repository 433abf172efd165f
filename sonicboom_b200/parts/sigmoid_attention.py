"""Grouped-query attention whose weights are logistic instead of a softmax: the weight of a visible
key is sigmoid(cap(q . k * scale) + b_h), cap(s) = softcap * tanh(s / softcap) (`softcap` 0: none)
and b_h a learned number per query head (`head_bias` names its tensor); weights are not normalised
over the keys, out = sum_j weight_j v_j.  No position enters the scores.  Visible to the query at
position i is key j <= i with i - j < window (`window` 0: every earlier key) or j < `keep_first`,
the first keys of a sequence, which a window keeps in sight (and the cache keeps) for good.

Query/key heads have `head_dim` values and value heads `vdim`; the cache entry's heads are as wide
as the larger of the two (the padding is zeros, so scores and sums are unchanged).  With `own_kv`
False the mixer has no key and value matrices: it runs on a schedule entry that reads another
entry's cache, with its own queries, mask and bias.

Tensors after the prefix: q [heads * head_dim, width], o [width, heads * vdim], the head bias
[heads], and with keys and values of its own k [kv_heads * head_dim, width], v [kv_heads * vdim,
width].  Scores, weights and sums are float32."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import KVNeed
from ..weights.loader import TensorRequest
from .attention import _cat
from .base import Mixer, register_mixer


@register_mixer("sigmoid_attention")
class SigmoidAttention(Mixer):
    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype, self.device = spec, dtype, device
        p = dict(spec.params)
        self.hq, self.hkv, self.dim = spec.n_heads, spec.n_kv_heads, spec.head_dim
        self.vdim = int(p.get("vdim", self.dim))
        self.softcap, self.keep_first = float(p.get("softcap", 0.0)), int(p.get("keep_first", 0))
        self.bias_name, self.own_kv = p.get("head_bias"), bool(p.get("own_kv", True))
        if self.hq % self.hkv:
            raise ConfigError(f"{self.hq} query heads are not a multiple of {self.hkv} key/value heads")
        self.hd = max(self.dim, self.vdim)
        self.qw, self.kw, self.vw = self.hq * self.dim, self.hkv * self.dim, self.hkv * self.vdim
        self.w_in = self.w_o = self.head_bias = None

    def kv_need(self):
        return KVNeed(self.hkv, self.hd, self.spec.window, self.keep_first if self.spec.window else 0)

    def tensor_requests(self):
        p, d = self.spec.prefix, self.spec.width
        req = [TensorRequest(p + "q", (self.qw, d)), TensorRequest(p + "o", (d, self.hq * self.vdim))]
        if self.own_kv:
            req += [TensorRequest(p + "k", (self.kw, d)), TensorRequest(p + "v", (self.vw, d))]
        if self.bias_name:
            req.append(TensorRequest(p + self.bias_name, (self.hq,), "bias"))
        return req

    def bind(self, get):
        p = self.spec.prefix
        self.w_in = _cat([get(p + n) for n in (("q", "k", "v") if self.own_kv else ("q",))])
        self.w_o = get(p + "o")
        if self.bias_name:
            self.head_bias = get(p + self.bias_name).float().contiguous()

    def first_weights(self, rows):
        n, k = self.w_in.shape
        late = self.w_in.dtype == torch.bfloat16 and ops.requests_weights_late(rows, n, k, self.w_in.device)
        return self.w_in if late else None

    def forward(self, h, ctx, residual=None):
        from ..config.specs import ConfigError
        if ctx.owns_cache != self.own_kv:
            raise ConfigError("a sigmoid_attention mixer has key and value matrices exactly when its schedule "
                              "entry owns a cache")
        rows, plan = h.shape[0], ctx.plan
        storage = ctx.kv_storage()
        g = plan.groups[ctx.kv_group()]
        proj = torch.empty((rows, self.w_in.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_in, proj)
        q = torch.empty((rows, self.hq, self.hd), dtype=self.dtype, device=h.device)
        ops.attn_prep(proj, 0, self.qw, self.qw + self.kw, self.hq, self.hkv, self.dim, self.vdim, self.hd, 0, False,
                      None, None, None, None, 0.0, plan.row_seq, plan.row_pos, g.page_off, g.page_ids, g.page_size,
                      storage if self.own_kv else None, q)
        mixed = torch.empty((rows, self.hq * self.hd), dtype=self.dtype, device=h.device)
        ops.attention_sigmoid(q, mixed, plan, ctx.kv_group(), storage, self.hq, self.hkv, self.hd, self.spec.window,
                              self.keep_first, self.spec.scale, self.softcap, self.head_bias)
        if self.hd != self.vdim:
            cut = torch.empty((rows, self.hq * self.vdim), dtype=self.dtype, device=h.device)
            mixed = ops.attn_unrotate(mixed, cut, self.hq, self.hd, self.vdim, False, None, plan.row_pos)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(mixed, self.w_o, out, ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)
