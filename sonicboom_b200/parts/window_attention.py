"""Grouped-query softmax attention over a sliding window of the paged cache, with the options
that attention layers of newer designs combine:

* query/key heads of size `head_dim` and value heads of size `vdim` (the cache entry's heads are
  as wide as the larger of the two, rounded up to what the tensor-core kernels take; the padding
  is zeros, so scores and sums are unchanged);
* rotation of a prefix of every q and k head in either layout of pairs (the spec's position
  encoding: "rope_halves" pairs i with i + n/2, "rope_interleaved" 2i with 2i + 1);
* `qk_norm` = (q name, k name): the whole q projection of a token (all heads at once) and the
  whole k projection are RMS-normed with a plain weight of that size before the rotation;
* `values` = "keys": there is no value matrix, the values are the key projection as it leaves
  the matrix (before norm and rotation);
* `rotate_values`: the value of position j is turned by j over all of vdim (same layout of
  pairs, frequencies base^(-2m/vdim)) before it is cached, and every head's result at position i
  is turned back by i: what a head sums depends on i - j only;
* `sink` = name: one learned number per query head whose exponential joins the softmax's
  denominator (it has no key, no value and is not scaled);
* `bias` = (q name, k name, v name): the three projections have biases;
* `head_norm` = ("before", q name, k name): every q and k head is RMS-normed by itself before the
  rotation, with one weight of head_dim values for all heads; ("after",): every head is divided by
  its root mean square after the rotation, without a weight;
* `softcap` = c: a score s becomes c tanh(s / c) before the softmax;
* `gate` = name: a matrix [heads, width]; head h's result is multiplied by the logistic function
  of its product with the mixer's input (it rides on the input product);
* a position encoding with a `magnitude` (stretched rotations) multiplies cosines and sines by it.

Tensors after the prefix: q [heads*head_dim, width], k [kv_heads*head_dim, width], v
[kv_heads*vdim, width] unless the values are the keys, o [width, heads*vdim], and what the options
name.  All input projections are one product; `ops.attn_prep` finishes its float32 rows into
queries and cache rows, the framework's attention kernels run on them unchanged, and
`ops.attn_unrotate` turns results back and drops the padding where either is needed."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import KVNeed
from ..weights.loader import TensorRequest
from .attention import _cat
from .base import POSITION_ENCODINGS, Mixer, make, register_mixer
from .rotary import frequency_table

HEAD_STEP = 16          # the tensor-core attention kernels take head sizes in these steps


@register_mixer("window_attention")
class WindowAttention(Mixer):
    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype, self.device = spec, dtype, device
        p = dict(spec.params)
        self.hq, self.hkv, self.dim = spec.n_heads, spec.n_kv_heads, spec.head_dim
        self.vdim = int(p.get("vdim", self.dim))
        self.eps = float(p.get("eps", 1e-6))
        self.values_are_keys = p.get("values", "own") == "keys"
        self.rotate_values = bool(p.get("rotate_values", False))
        self.qk_norm, self.sink_name = p.get("qk_norm"), p.get("sink")
        self.bias_names, self.gate_name = p.get("bias"), p.get("gate")
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        head_norm = p.get("head_norm")
        self.head_norm = head_norm[0] if head_norm else None
        if self.head_norm not in (None, "before", "after") or (self.head_norm and self.qk_norm):
            raise ConfigError(f"head_norm {head_norm!r}: ('before', q name, k name) or ('after',), and not "
                              "beside a norm of the whole projection")
        if self.head_norm == "before":
            self.qk_norm = tuple(head_norm[1:3])
        if self.softcap < 0.0:
            raise ConfigError(f"a score cap of {self.softcap} (0: none)")
        self.names = tuple(p.get("names", ("q", "k", "v", "o")))
        if self.hq % self.hkv:
            raise ConfigError(f"{self.hq} query heads are not a multiple of {self.hkv} key/value heads")
        if self.values_are_keys and self.vdim != self.dim:
            raise ConfigError(f"values that are the keys need vdim == head_dim, not {self.vdim} and {self.dim}")
        if self.rotate_values and self.vdim % 2:
            raise ConfigError(f"rotated values need an even vdim, not {self.vdim}")
        if self.rotate_values and spec.position is None:
            raise ConfigError("rotated values take their frequencies' base from the position encoding")
        self.hd = (max(self.dim, self.vdim) + HEAD_STEP - 1) // HEAD_STEP * HEAD_STEP
        self.rot, self.interleaved, self.inv_freq, self.v_inv_freq = 0, False, None, None
        self.rot_scale = 1.0
        if spec.position is not None:
            pe = make(POSITION_ENCODINGS, "position encoding", spec.position, dtype, device)
            self.rot_scale = float(getattr(pe, "magnitude", 1.0))
            self.interleaved = getattr(pe, "layout", "halves") == "interleaved"
            self.rot = spec.position.rotary_dim
            self.inv_freq = pe.inv_freq if self.rot > 0 else None
            if self.rotate_values:
                self.v_inv_freq = frequency_table(spec.position.theta, self.vdim, device)
        self.qw, self.kw = self.hq * self.dim, self.hkv * self.dim
        self.vw = 0 if self.values_are_keys else self.hkv * self.vdim
        self.gw = self.hq if self.gate_name else 0
        if self.bias_names and self.values_are_keys:
            raise ConfigError("biases of q, k and v need a value projection of its own")
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.sink = self.b_in = None

    def kv_need(self):
        return KVNeed(self.hkv, self.hd, self.spec.window)

    def tensor_requests(self):
        p, d = self.spec.prefix, self.spec.width
        q, k, v, o = self.names
        req = [TensorRequest(p + q, (self.qw, d)), TensorRequest(p + k, (self.kw, d)),
               TensorRequest(p + o, (d, self.hq * self.vdim))]
        if not self.values_are_keys:
            req.append(TensorRequest(p + v, (self.hkv * self.vdim, d)))
        if self.qk_norm:
            per_head = self.head_norm == "before"
            req += [TensorRequest(p + self.qk_norm[0], (self.dim if per_head else self.qw,), "norm"),
                    TensorRequest(p + self.qk_norm[1], (self.dim if per_head else self.kw,), "norm")]
        if self.bias_names:
            req += [TensorRequest(p + n, (w,), "bias") for n, w in zip(self.bias_names, (self.qw, self.kw, self.vw))]
        if self.gate_name:
            req.append(TensorRequest(p + self.gate_name, (self.hq, d)))
        if self.sink_name:
            req.append(TensorRequest(p + self.sink_name, (self.hq,), "bias"))
        return req

    def bind(self, get):
        p = self.spec.prefix
        q, k, v, o = self.names
        # rows of the one input product: [q | gate | k | v]; an entry that reads another's cache stops after the gate
        names = [q] + ([self.gate_name] if self.gate_name else []) + ([k] if self.values_are_keys else [k, v])
        self.w_in = _cat([get(p + n) for n in names])
        if self.bias_names:
            bq, bk, bv = (get(p + n).float() for n in self.bias_names)
            zero = [torch.zeros(self.gw, dtype=torch.float32, device=bq.device)] if self.gw else []
            self.b_in = torch.cat([bq] + zero + [bk, bv]).contiguous()
        self.w_o = get(p + o)
        if self.qk_norm:
            self.q_norm, self.k_norm = get(p + self.qk_norm[0]), get(p + self.qk_norm[1])
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        if self.sink_name:
            self.sink = get(p + self.sink_name).float().contiguous()

    def first_weights(self, rows):
        n, k = self.w_in.shape
        late = self.w_in.dtype == torch.bfloat16 and ops.requests_weights_late(rows, n, k, self.w_in.device)
        return self.w_in if late else None

    def forward(self, h, ctx, residual=None):
        rows, plan = h.shape[0], ctx.plan
        k_off = self.qw + self.gw
        width_in = k_off + ((self.kw + self.vw) if ctx.owns_cache else 0)
        storage = ctx.kv_storage()
        g = plan.groups[ctx.kv_group()]
        proj = torch.empty((rows, width_in), dtype=torch.float32, device=h.device)
        if self.b_in is not None:
            ops.linear(h, self.w_in[:width_in], proj, ops.EPI_BIAS, bias=self.b_in[:width_in])
        else:
            ops.linear(h, self.w_in[:width_in], proj)
        q = torch.empty((rows, self.hq, self.hd), dtype=self.dtype, device=h.device)
        ops.attn_prep(proj, 0, k_off, -1 if self.values_are_keys else k_off + self.kw, self.hq, self.hkv,
                      self.dim, self.vdim, self.hd, self.rot, self.interleaved, self.inv_freq, self.v_inv_freq,
                      self.q_norm, self.k_norm, self.eps, plan.row_seq, plan.row_pos, g.page_off, g.page_ids,
                      g.page_size, storage if ctx.owns_cache else None, q, head_norm=self.head_norm,
                      rot_scale=self.rot_scale)
        mixed = torch.empty((rows, self.hq * self.hd), dtype=self.dtype, device=h.device)
        ops.attention(q, mixed, plan, ctx.kv_group(), storage, self.hq, self.hkv, self.hd, self.spec.window,
                      self.spec.scale, warm=self.w_o, sink=self.sink, softcap=self.softcap)
        if self.rotate_values or self.hd != self.vdim or self.gw:
            turned = torch.empty((rows, self.hq * self.vdim), dtype=self.dtype, device=h.device)
            mixed = ops.attn_unrotate(mixed, turned, self.hq, self.hd, self.vdim, self.interleaved,
                                      self.v_inv_freq, plan.row_pos, gate=(proj, self.qw) if self.gw else None)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(mixed, self.w_o, out, ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)
