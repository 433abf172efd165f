"""Attention over a cached low-rank latent.

Per token the mixer projects its input to queries (per head `dim` unrotated and `rot_dim`
rotated dimensions, laid out head by head as [dim | rot_dim]) and to rank + rot_dim numbers: the
first `rank`, RMS-normed with a plain weight, are the latent c; the last rot_dim are one rotated
key part kr that all heads share.  Only c and kr are cached.  Head h's key is [Uk_h c | kr], its
value Uv_h c, the score (q . Uk_h c + qr . kr) * scale over a sliding window, softmax, then the
output projection over the concatenated heads.

Computed in the absorbed form, which needs nothing but the cache whatever the step brings
(a prompt, a portion of one, a single token):
    q~_h = Uk_h^T q_h                     (`ops.head_linear`, a product per head)
    s    = ([q~_h | qr_h] . [c | kr]) * scale  and  z_h = softmax(s) C   (the paged attention kernels on
                                           a cache entry with ONE head of size rank + rot_dim)
    o_h  = Uv_h z_h                        (`ops.head_linear`)
so the framework's attention kernels (plain float32, mma.sync, tcgen05) run unchanged.  A mixer
that reads another entry's cache (`ScheduleEntry.cache_from`) projects queries only and uses
that entry's c and kr as the cache holds them, with its own Uk, Uv, window and scale.

Options (`params`): `q_rank` = n: the queries come through a latent of their own, c_q =
RMSnorm(W_dq h) with a plain weight and q = W_uq c_q (tensors dq [n, width], dq.norm [n], uq
[heads*(dim+rot_dim), n] instead of q); W_dq and W_dkv are then one product and W_uq a second one.
`sink` = name: one learned number per head whose exponential joins the softmax's denominator.
The position encoding decides the layout of the rotated pairs ("interleaved": 2i with 2i + 1,
"halves": i with i + n/2) and may have a `magnitude` that multiplies cosines and sines.

Tensors after the prefix: q [heads*(dim+rot_dim), width], dkv [rank+rot_dim, width], dkv.norm
[rank], uk [heads*dim, rank], uv [heads*vdim, rank], o [width, heads*vdim].
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import KVNeed
from ..weights.loader import TensorRequest
from .base import POSITION_ENCODINGS, Mixer, make, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype, self.device = spec, dtype, device
        p = dict(spec.params)
        self.h, self.dim = spec.n_heads, spec.head_dim
        try:
            self.rd, self.vd, self.rank = int(p["rot_dim"]), int(p["vdim"]), int(p["kv_rank"])
        except KeyError as e:
            raise ConfigError(f"latent attention needs the parameter {e.args[0]}") from None
        self.eps = float(p.get("eps", 1e-6))
        self.keep = int(p.get("keep", spec.window))      # what the cache entry must keep (0: everything)
        if spec.window and self.keep and self.keep < spec.window:
            raise ConfigError(f"a cache entry that keeps {self.keep} keys cannot serve a window of {spec.window}")
        self.own_kv = bool(p.get("own_kv", True))        # False: it only ever reads another entry's cache
        self.wide = self.rank + self.rd
        self.position = make(POSITION_ENCODINGS, "position encoding", spec.position, dtype, device)
        layout = getattr(self.position, "layout", None)
        if layout not in ("interleaved", "halves") and self.position.rotary_dim:
            raise ConfigError("latent attention rotates interleaved pairs or pairs half the rotated part "
                              f"apart; position encoding {spec.position.kind!r} says neither")
        self.interleaved = layout != "halves"
        self.rot_scale = float(getattr(self.position, "magnitude", 1.0))
        self.q_rank = int(p.get("q_rank", 0) or 0)
        self.sink_name = p.get("sink")
        self.w_uq = self.qnorm = self.sink = None
        if self.position.rotary_dim > self.rd:
            raise ConfigError(f"{self.position.rotary_dim} rotated dimensions exceed rot_dim {self.rd}")
        self.w_in = self.cnorm = self.w_ukt = self.w_uv = self.w_o = None

    def kv_need(self):
        return KVNeed(1, self.wide, self.keep)

    def tensor_requests(self):
        p, d = self.spec.prefix, self.spec.width
        own = [TensorRequest(p + "dkv", (self.wide, d)),
               TensorRequest(p + "dkv.norm", (self.rank,), "norm")] if self.own_kv else []
        hq = self.h * (self.dim + self.rd)
        q = [TensorRequest(p + "q", (hq, d))] if not self.q_rank else [
            TensorRequest(p + "dq", (self.q_rank, d)), TensorRequest(p + "dq.norm", (self.q_rank,), "norm"),
            TensorRequest(p + "uq", (hq, self.q_rank))]
        sink = [TensorRequest(p + self.sink_name, (self.h,), "bias")] if self.sink_name else []
        return q + own + [TensorRequest(p + "uk", (self.h * self.dim, self.rank)),
                          TensorRequest(p + "uv", (self.h * self.vd, self.rank)),
                          TensorRequest(p + "o", (d, self.h * self.vd))] + sink

    def bind(self, get):
        p = self.spec.prefix
        q = get(p + ("dq" if self.q_rank else "q"))
        if self.q_rank:
            self.w_uq, self.qnorm = get(p + "uq"), get(p + "dq.norm")
        if self.sink_name:
            self.sink = get(p + self.sink_name).float().contiguous()
        if self.own_kv:
            dkv = get(p + "dkv")
            if dkv.dtype != q.dtype:
                q, dkv = q.float(), dkv.float()
            self.w_in = torch.cat([q, dkv], dim=0).contiguous()
            self.cnorm = get(p + "dkv.norm")
        else:
            self.w_in = q
        # Uk as [head, rank, dim]: the product per head maps a head's dim query values to rank
        self.w_ukt = get(p + "uk").view(self.h, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = get(p + "uv").view(self.h, self.vd, self.rank).contiguous()
        self.w_o = get(p + "o")

    def _heads_per_call(self, plan, storage) -> int:
        """How many heads one attention call takes.  All of them, except when single tokens are
        decoded with more heads than the split decode attention takes as rows of its one
        key/value head (`ops.DECODE_ATTENTION_ROWS`): it then runs once per group of heads, the
        largest divisor of the head count that fits, instead of handing the step to the kernel
        for many rows, which has one block per sequence to offer.  Which kernel runs changes the
        rounding, nothing else."""
        limit = ops.DECODE_ATTENTION_ROWS
        if plan.max_new != 1 or self.h <= limit or self.dtype != torch.bfloat16 or \
                storage.dtype != torch.bfloat16 or ops.attention_lib(self.wide) is None:
            return self.h
        hg = max(d for d in range(1, limit + 1) if self.h % d == 0)
        return hg if 2 * hg > limit else self.h

    def forward(self, h, ctx, residual=None):
        rows, plan = h.shape[0], ctx.plan
        owns = ctx.owns_cache
        if owns and not self.own_kv:
            raise ops.KernelError("this latent attention has no key/value projection of its own: "
                                  "its schedule entry must read another entry's cache")
        hw = self.dim + self.rd
        kv = None
        if self.q_rank:
            # one product gives [query latent | latent | key part]; the normed query latent goes
            # through the second matrix, and the latent's rows stay where the first product put them
            n_first = self.q_rank + (self.wide if owns else 0)
            first = torch.empty((rows, n_first), dtype=torch.float32, device=h.device)
            ops.linear(h, self.w_in[:n_first], first)
            cq = torch.empty((rows, self.q_rank), dtype=self.dtype, device=h.device)
            ops.rmsnorm(first, self.qnorm, self.eps, cq, width=self.q_rank)
            n_in = self.h * hw
            proj = torch.empty((rows, n_in), dtype=torch.float32, device=h.device)
            ops.linear(cq, self.w_uq, proj)
            kv = (first, self.q_rank) if owns else None
        else:
            n_in = self.h * hw + (self.wide if owns else 0)
            proj = torch.empty((rows, n_in), dtype=torch.float32, device=h.device)
            ops.linear(h, self.w_in[:n_in], proj)
        storage = ctx.kv_storage()
        g = plan.groups[ctx.kv_group()]
        hg = self._heads_per_call(plan, storage)
        n_g = self.h // hg
        q_wide = torch.empty((n_g, rows, hg, self.wide), dtype=self.dtype, device=h.device)
        ops.latent_prep(proj, self.h, self.dim, self.rd, self.rank, self.position.rotary_dim,
                        self.position.inv_freq, plan.row_seq, plan.row_pos, g.page_off, g.page_ids,
                        g.page_size, self.cnorm, self.eps, storage if owns else None, q_wide, hg,
                        kv=kv, interleaved=self.interleaved, rot_scale=self.rot_scale)
        z = torch.empty((n_g, rows, hg * self.wide), dtype=self.dtype, device=h.device)
        mixed = torch.empty((rows, self.h * self.vd), dtype=self.dtype, device=h.device)
        for i in range(n_g):
            at, heads = i * rows * hg * self.wide, slice(i * hg, (i + 1) * hg)
            ops.head_linear(proj, i * hg * hw, n_in, hw, self.w_ukt[heads], q_wide, at, hg * self.wide, self.wide, rows)
            ops.attention(q_wide[i], z[i], plan, ctx.kv_group(), storage, hg, 1, self.wide,
                          self.spec.window, self.spec.scale,
                          sink=self.sink[heads] if self.sink is not None else None)
            ops.head_linear(z, at, hg * self.wide, self.wide, self.w_uv[heads], mixed, i * hg * self.vd,
                            self.h * self.vd, self.vd, rows)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(mixed, self.w_o, out, ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)
