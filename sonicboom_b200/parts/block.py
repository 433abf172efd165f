"""Arrangement of parts in a block.  "pre_norm": h = norm(x); x1 = mix(h) + x; f = norm(x1);
x2 = ffn(f) + x1 (core/src/model/emit.cpp:436-459 with no post norms, gate or output scale,
as the reference's traits set for this architecture: core/src/model/recipe.cpp:65-70)."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import StateNeed
from ..weights.loader import TensorRequest
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Part, make, register_block)


class InputConv(Part):
    """h <- h + conv(h): a short causal convolution over time on every channel of what a sublayer
    reads, added to it.  The last taps - 1 inputs of every sequence are state of the cache, under
    `state_name` of the running entry."""

    def __init__(self, spec, state_name, dtype):
        self.spec, self.state_name, self.dtype = spec, state_name, dtype
        self.weight = None

    def tensor_requests(self):
        return [TensorRequest(self.spec.tensor, (self.spec.width, self.spec.taps), "bias")]

    def bind(self, get):
        self.weight = get(self.spec.tensor)

    def state_need(self):
        return StateNeed((self.spec.taps - 1, self.spec.width), torch.float32) if self.spec.taps > 1 else None

    def forward(self, h, ctx):
        """h: float32 normed rows; returns h + conv(h) in the activation dtype."""
        out = torch.empty(h.shape, dtype=self.dtype, device=h.device)
        state = ctx.state(self.state_name) if self.spec.taps > 1 else None
        return ops.causal_conv(h, 0, self.spec.width, self.weight, None, ctx.plan, state, out, add_input=True)


@register_block("pre_norm")
class PreNormBlock(Block):
    """h = norm(x); x1 = mix(h) + x; f = norm(x1); x2 = ffn(f) + x1 (without a feed-forward the
    result is x1).  With `mixer_conv` / `feed_forward_conv` in the spec, what a sublayer reads
    passes a short causal convolution first: the norm then writes float32 rows and the
    convolution's kernel hands the sublayer its rows in the activation dtype."""

    def __init__(self, spec, dtype, device):
        self.dtype = dtype
        self.mixer_norm = make(NORMS, "norm", spec.mixer_norm, dtype, device)
        self.mixer = make(MIXERS, "mixer", spec.mixer, dtype, device)
        self.parts = [self.mixer_norm, self.mixer]
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = make(NORMS, "norm", spec.feed_forward_norm, dtype, device)
            self.feed_forward = make(FEED_FORWARDS, "feed-forward", spec.feed_forward, dtype, device)
            self.parts += [self.feed_forward_norm, self.feed_forward]
        self.mixer_conv = InputConv(spec.mixer_conv, "conv1", dtype) if spec.mixer_conv is not None else None
        self.feed_forward_conv = InputConv(spec.feed_forward_conv, "conv2", dtype) \
            if spec.feed_forward_conv is not None and self.feed_forward is not None else None
        self.parts += [c for c in (self.mixer_conv, self.feed_forward_conv) if c is not None]

    def tensor_requests(self):
        return [r for p in self.parts for r in p.tensor_requests()]

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def kv_need(self):
        return self.mixer.kv_need()

    def state_need(self):
        """The mixer's state; with input convolutions, a dict that also names theirs."""
        need = self.mixer.state_need()
        convs = {c.state_name: c.state_need() for c in (self.mixer_conv, self.feed_forward_conv)
                 if c is not None and c.state_need() is not None}
        if not convs:
            return need
        if need is not None:
            convs.update(need if isinstance(need, dict) else {None: need})
        return convs

    def input_norm(self):
        return self.mixer_norm if self.mixer_conv is None else None     # a convolution wants float32 rows

    def first_weights(self, rows):
        return self.mixer.first_weights(rows)

    def _read(self, norm, conv, x, ctx):
        """What a sublayer reads of the stream x."""
        if conv is not None:
            ctx.take_normed(norm, x)
            return conv.forward(norm.forward(x, torch.float32), ctx)
        h = ctx.take_normed(norm, x)
        return h if h is not None else norm.forward(x, self.dtype)

    def forward(self, x, ctx):
        after, after_weights = ctx.after_block_norm, ctx.after_block_weights
        h = self._read(self.mixer_norm, self.mixer_conv, x, ctx)
        if self.feed_forward is None:
            ctx.next_norm, ctx.next_weights = after, after_weights
            return self.mixer.forward(h, ctx, residual=x)
        ctx.next_norm = self.feed_forward_norm if self.feed_forward_conv is None else None
        x = self.mixer.forward(h, ctx, residual=x)
        f = self._read(self.feed_forward_norm, self.feed_forward_conv, x, ctx)
        # the block's result is the feed-forward's, so what follows the block follows its product
        ctx.next_norm, ctx.next_weights = after, after_weights
        return self.feed_forward.forward(f, ctx, residual=x)


@register_block("sandwich_norm")
class SandwichNormBlock(Block):
    """Norm before and after each sublayer: x1 = x + post1(mix(pre1(x))); x2 = x1 + post2(ffn(pre2(x1)))
    (without a feed-forward the block's result is x1).  The normed sublayer result joins the
    stream in one kernel (`ops.norm_add`), which also writes the norm that comes next when that is
    known: the feed-forward's own input norm, or the next entry's first norm
    (`ctx.after_block_norm`).  When the caller is going to run a depth mix on the result
    (`ctx.block_mix`), the last add and that mix are one kernel.  When the caller names a place for the result (`ctx.block_out`), the
    block writes there and leaves its input as it was; else it overwrites its input."""
    writes_block_out = True

    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.dtype = dtype
        if spec.mixer_post_norm is None:
            raise ConfigError("a sandwich_norm block needs mixer_post_norm")
        if spec.feed_forward is not None and (spec.feed_forward_norm is None or spec.feed_forward_post_norm is None):
            raise ConfigError("a sandwich_norm block with a feed-forward needs both of its norms")
        self.mixer_norm = make(NORMS, "norm", spec.mixer_norm, dtype, device)
        self.mixer = make(MIXERS, "mixer", spec.mixer, dtype, device)
        self.mixer_post_norm = make(NORMS, "norm", spec.mixer_post_norm, dtype, device)
        self.parts = [self.mixer_norm, self.mixer, self.mixer_post_norm]
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = make(NORMS, "norm", spec.feed_forward_norm, dtype, device)
            self.feed_forward = make(FEED_FORWARDS, "feed-forward", spec.feed_forward, dtype, device)
            self.feed_forward_post_norm = make(NORMS, "norm", spec.feed_forward_post_norm, dtype, device)
            self.parts += [self.feed_forward_norm, self.feed_forward, self.feed_forward_post_norm]

    def tensor_requests(self):
        return [r for p in self.parts for r in p.tensor_requests()]

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def kv_need(self):
        return self.mixer.kv_need()

    def state_need(self):
        return self.mixer.state_need()

    def input_norm(self):
        return self.mixer_norm

    def _join(self, y, x, post, out, ctx, then):
        """out = x + post(y); the norm `then` of the result rides along when it is a plain RMS norm."""
        import torch
        from .. import ops
        w, eps = post.as_rms()
        rms = then.as_rms() if then is not None else None
        if rms is None:
            return ops.norm_add(y, x, w, eps, out)
        normed = torch.empty(out.shape, dtype=self.dtype, device=out.device)
        ops.norm_add(y, x, w, eps, out, (rms[0], rms[1], normed))
        ctx.keep_normed(then, out, normed)
        return out

    def _join_and_mix(self, y, x, post, out, ctx, mix, streams, next_norm):
        """The block's last add and the depth mix the caller would run on its result, in one kernel."""
        import torch
        w, eps = post.as_rms()
        mixed = torch.empty_like(out)
        rms = next_norm.as_rms() if next_norm is not None else None
        normed = torch.empty(out.shape, dtype=self.dtype, device=out.device) if rms is not None else None
        mix.forward(streams, mixed, (rms[0], rms[1], normed) if rms is not None else None, join=(y, x, w, eps))
        if rms is not None:
            ctx.keep_normed(next_norm, mixed, normed)
        ctx.mixed_out = mixed
        return out

    def _last_join(self, y, x, post, out, ctx, after, mix):
        if mix is not None and mix[1][mix[0].spec.n_inputs - 1].data_ptr() == out.data_ptr() \
                and mix[0].joins(post.as_rms()[0]):
            return self._join_and_mix(y, x, post, out, ctx, *mix)
        return self._join(y, x, post, out, ctx, after)

    def forward(self, x, ctx):
        out, ctx.block_out = (ctx.block_out if ctx.block_out is not None else x), None
        mix, ctx.block_mix, ctx.mixed_out = ctx.block_mix, None, None
        after, ctx.after_block_norm, ctx.after_block_weights = ctx.after_block_norm, None, None
        h = ctx.take_normed(self.mixer_norm, x)
        if h is None:
            h = self.mixer_norm.forward(x, self.dtype)
        ctx.next_norm = ctx.next_weights = None      # the post norm, not a norm of the stream, follows the product
        y = self.mixer.forward(h, ctx)
        if self.feed_forward is None:
            return self._last_join(y, x, self.mixer_post_norm, out, ctx, after, mix)
        x1 = self._join(y, x, self.mixer_post_norm, out, ctx, self.feed_forward_norm)
        f = ctx.take_normed(self.feed_forward_norm, x1)
        if f is None:
            f = self.feed_forward_norm.forward(x1, self.dtype)
        ctx.next_norm = ctx.next_weights = None
        y = self.feed_forward.forward(f, ctx)
        return self._last_join(y, x1, self.feed_forward_post_norm, out, ctx, after, mix)


@register_block("parallel_residual")
class ParallelResidualBlock(Block):
    """One norm feeds both sublayers: h = norm(x); x <- x + mix(h) + ffn(h) (without a feed-forward,
    x + mix(h)).  The mixer adds its result to the stream in its last product, the feed-forward
    adds its own to that, so the sum is ((x + mix) + ffn) in float32; the norm that comes after the
    block can ride on the last of the two products."""

    def __init__(self, spec, dtype, device):
        self.dtype = dtype
        self.mixer_norm = make(NORMS, "norm", spec.mixer_norm, dtype, device)
        self.mixer = make(MIXERS, "mixer", spec.mixer, dtype, device)
        self.feed_forward = make(FEED_FORWARDS, "feed-forward", spec.feed_forward, dtype, device) \
            if spec.feed_forward is not None else None
        self.parts = [self.mixer_norm, self.mixer] + ([self.feed_forward] if self.feed_forward is not None else [])

    def tensor_requests(self):
        return [r for p in self.parts for r in p.tensor_requests()]

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def kv_need(self):
        return self.mixer.kv_need()

    def state_need(self):
        return self.mixer.state_need()

    def input_norm(self):
        return self.mixer_norm

    def first_weights(self, rows):
        return self.mixer.first_weights(rows)

    def forward(self, x, ctx):
        after, after_weights = ctx.after_block_norm, ctx.after_block_weights
        h = ctx.take_normed(self.mixer_norm, x)
        if h is None:
            h = self.mixer_norm.forward(x, self.dtype)
        if self.feed_forward is None:
            ctx.next_norm, ctx.next_weights = after, after_weights
            return self.mixer.forward(h, ctx, residual=x)
        ctx.next_norm = ctx.next_weights = None
        x = self.mixer.forward(h, ctx, residual=x)
        ctx.next_norm, ctx.next_weights = after, after_weights
        return self.feed_forward.forward(h, ctx, residual=x)


@register_block("output_norm")
class OutputNormBlock(Block):
    """No norm before a sublayer, an RMS norm on its result: x1 = x + m norm1(mix(x)); x2 = x1 + m
    norm2(ffn(x1)) (without a feed-forward the result is x1).  The sublayers read the stream itself,
    in the activation dtype; m (`params`: residual_mult) is folded into the norms' weights when they
    are bound, in float32.  The normed result joins the stream in one kernel (`ops.norm_add`), which
    also leaves behind what reads the finished rows next: the stream in the activation dtype for
    this block's feed-forward or for a next block of this arrangement, or the next block's first
    norm when that is a plain RMS norm."""

    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        from .norm import StreamCast
        self.dtype = dtype
        self.mult = float(dict(spec.params).get("residual_mult", 1.0))
        self.mixer = make(MIXERS, "mixer", spec.mixer, dtype, device)
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and spec.feed_forward_post_norm is None):
            raise ConfigError("an output_norm block needs a post norm for every sublayer it has")
        self.mixer_post_norm = make(NORMS, "norm", spec.mixer_post_norm, dtype, device)
        self.parts = [self.mixer, self.mixer_post_norm]
        self.feed_forward = self.feed_forward_post_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = make(FEED_FORWARDS, "feed-forward", spec.feed_forward, dtype, device)
            self.feed_forward_post_norm = make(NORMS, "norm", spec.feed_forward_post_norm, dtype, device)
            self.parts += [self.feed_forward, self.feed_forward_post_norm]
        self.reads = StreamCast()         # what the mixer reads of the block's input
        self.reads_again = StreamCast()   # what the feed-forward reads of x1
        self.w1 = self.w2 = None

    def tensor_requests(self):
        return [r for p in self.parts for r in p.tensor_requests()]

    def bind(self, get):
        for p in self.parts:
            p.bind(get)
        for norm in (self.mixer_post_norm, self.feed_forward_post_norm):
            if norm is not None and norm.as_rms() is None:
                from ..config.specs import ConfigError
                raise ConfigError("an output_norm block joins its sublayers through RMS norms")
        self.w1 = (self.mixer_post_norm.as_rms()[0].float() * self.mult).contiguous()
        if self.feed_forward is not None:
            self.w2 = (self.feed_forward_post_norm.as_rms()[0].float() * self.mult).contiguous()

    def kv_need(self):
        return self.mixer.kv_need()

    def state_need(self):
        return self.mixer.state_need()

    def input_norm(self):
        return self.reads

    def _read(self, cast, x, ctx):
        h = ctx.take_normed(cast, x)
        if h is not None or self.dtype == torch.float32:
            return h if h is not None else x
        return cast.forward(x, self.dtype)

    def _join(self, y, x, w, eps, ctx, then):
        """x += y / rms(y) * w in place; what reads x next is written along where it can be."""
        from .norm import StreamCast
        ride = None
        if isinstance(then, StreamCast):
            if self.dtype != torch.float32:
                ride = (None, 0.0, torch.empty(x.shape, dtype=self.dtype, device=x.device))
        elif then is not None and then.as_rms() is not None:
            ride = (*then.as_rms(), torch.empty(x.shape, dtype=self.dtype, device=x.device))
        ops.norm_add(y, x, w, eps, x, ride)
        if ride is not None:
            ctx.keep_normed(then, x, ride[2])
        return x

    def forward(self, x, ctx):
        after, ctx.after_block_norm, ctx.after_block_weights = ctx.after_block_norm, None, None
        h = self._read(self.reads, x, ctx)
        ctx.next_norm = ctx.next_weights = None      # a post norm, not a norm of the stream, follows the product
        y = self.mixer.forward(h, ctx)
        eps1 = self.mixer_post_norm.as_rms()[1]
        if self.feed_forward is None:
            return self._join(y, x, self.w1, eps1, ctx, after)
        x = self._join(y, x, self.w1, eps1, ctx, self.reads_again)
        f = self._read(self.reads_again, x, ctx)
        ctx.next_norm = ctx.next_weights = None
        y = self.feed_forward.forward(f, ctx)
        return self._join(y, x, self.w2, self.feed_forward_post_norm.as_rms()[1], ctx, after)
